"""World-size-2 (and 3) CPU runs of the multi-GPU host logic over gloo: the nnz-balanced row
partition, the halo windows and the point-to-point exchange plan, and the two allreduces of a
PCG iteration.  The local compute is done by the CPU oracle here (the CUDA kernels need a GPU);
what is under test is that the distributed schedule reproduces the single-rank solve."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, grid, iters, out_dir, zhalo=False):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lapis_b200 import workloads as w
    from lapis_b200.dist import HaloExchanger, all_windows, local_block
    from oracle import oracle

    d = w.pcg_laplacian(grid)
    pos, crd, val, b, dinv = d["pos"], d["crd"], d["val"], d["b"], d["dinv"]
    bounds, lpos, lcrd, lval = local_block(pos, crd, val, rank, world)
    wins = all_windows(pos, crd, bounds)
    halo = HaloExchanger(bounds, wins, rank)
    r0, r1 = halo.r0, halo.r1
    n, off = r1 - r0, halo.own_offset
    lcrd = (lcrd.astype(np.int64) - halo.c0).astype(lcrd.dtype)

    def allsum(*vals):
        t = torch.tensor(vals, dtype=torch.float64)
        dist.all_reduce(t)
        return [float(v) for v in t]

    # examples/pcg_solve.py:52-101 in the LAPIS project, with every vector split by rows
    r = b[r0:r1].copy()
    z = oracle.mult(r, dinv[r0:r1])
    p_ext = torch.zeros(halo.window_len, dtype=torch.float64)
    p = p_ext.numpy()[off:off + n]
    p[:] = z
    x = np.zeros(n)
    rr0, rz = allsum(oracle.dot(r, r), oracle.dot(r, z))
    initres = np.sqrt(rr0)
    it = 1
    z_ext = torch.zeros(halo.window_len, dtype=torch.float64)
    halo.exchange(p_ext)  # the halo of the first p travels as p
    while True:
        if not zhalo:
            halo.exchange(p_ext)
        Ap = oracle.spmv(lpos, lcrd, lval, p_ext.numpy(), np.zeros(n))
        (pAp,) = allsum(oracle.dot(p, Ap))
        alpha = rz / pAp
        x = oracle.axpby(1.0, x, alpha, p)
        r = oracle.axpby(1.0, r, -alpha, Ap)
        z = oracle.mult(r, dinv[r0:r1])
        rr, rz_new = allsum(oracle.dot(r, r), oracle.dot(r, z))
        relres = np.sqrt(rr) / initres
        if not (relres > 0.0 and it != iters):
            break
        beta = rz_new / rz
        rz = rz_new
        if zhalo:
            # the schedule of the fused GPU passes: the neighbours' rows of z arrive with the second pair of sums,
            # and every rank updates its whole window of p, halo included, itself
            z_ext.numpy()[off:off + n] = z
            halo.exchange(z_ext)
            p_ext.numpy()[:] = oracle.axpby(1.0, z_ext.numpy(), beta, p_ext.numpy())
        else:
            p[:] = oracle.axpby(1.0, z, beta, p)
        it += 1
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), x=x, r0=r0, r1=r1, relres=relres, it=it)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("zhalo", [False, True], ids=["halo_of_p", "halo_from_z"])
@pytest.mark.parametrize("world", [2, 3])
def test_row_partitioned_pcg_reproduces_single_rank(tmp_path, world, zhalo):
    from lapis_b200 import workloads as w
    from oracle import oracle
    grid, iters = 24, 30
    mp.spawn(_worker, args=(world, _free_port(), grid, iters, str(tmp_path), zhalo), nprocs=world, join=True)
    d = w.pcg_laplacian(grid)
    xo, io, ro = oracle.pcg(d["pos"], d["crd"], d["val"], d["b"], d["dinv"], 0.0, iters)
    x = np.zeros(grid * grid)
    covered = 0
    for rank in range(world):
        g = np.load(tmp_path / f"rank{rank}.npz")
        x[int(g["r0"]):int(g["r1"])] = g["x"]
        covered += int(g["r1"]) - int(g["r0"])
        assert int(g["it"]) == io == iters
        assert abs(float(g["relres"]) - ro) <= 1e-10 * ro
    assert covered == grid * grid
    # the split dot products are summed in another order: agreement to rounding, amplified by CG
    assert np.max(np.abs(x - xo)) <= 1e-10 * np.max(np.abs(xo))


def _spmv_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lapis_b200 import workloads as w
    from lapis_b200.dist import local_block
    from oracle import oracle
    d = w.spmv_power_law(1 << 12)
    bounds, lpos, lcrd, lval = local_block(d["pos"], d["crd"], d["val"], rank, world)
    y = oracle.spmv(lpos, lcrd, lval, d["x"], np.zeros(len(lpos) - 1))   # x replicated, no exchange
    gathered = [None] * world
    dist.all_gather_object(gathered, (int(bounds[rank]), y))
    if rank == 0:
        full = np.concatenate([g[1] for g in sorted(gathered, key=lambda t: t[0])])
        np.save(os.path.join(out_dir, "y.npy"), full)
    dist.barrier()
    dist.destroy_process_group()


def test_row_partitioned_spmv_is_bit_identical(tmp_path):
    from lapis_b200 import workloads as w
    from oracle import oracle
    mp.spawn(_spmv_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    d = w.spmv_power_law(1 << 12)
    ref = oracle.spmv(d["pos"], d["crd"], d["val"], d["x"], np.zeros(1 << 12))
    assert np.array_equal(np.load(tmp_path / "y.npy"), ref)   # rows are independent: same bits


def _dropout_worker(rank, world, port, out_dir):
    """Rank 1 leaves between two steps; rank 0 learns of it from the short timeout of its next collective."""
    import datetime
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    t = torch.ones(2, dtype=torch.float64)
    dist.all_reduce(t)                       # step 1: both ranks take part
    assert float(t[0]) == world
    if rank == 1:
        os._exit(0)                          # leaves between steps, nothing in flight
    outcome = "completed"
    try:
        dist.all_reduce(t)                   # step 2: the peer never joins
    except Exception as exc:                 # the process-group timeout ends the collective with an error
        outcome = "peer lost: " + type(exc).__name__
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_a_rank_that_leaves_is_noticed_by_the_others(tmp_path):
    """Failure detection on the host side of the multi-rank solver, without a GPU and without a hang: a rank
    that exits between two steps makes the next collective of the remaining rank end with an error after the
    process group's (short) timeout, instead of blocking for ever."""
    mp.spawn(_dropout_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "rank0.txt").read().startswith("peer lost")
