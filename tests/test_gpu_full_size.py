"""The benchmark configurations at their full sizes against the CPU oracle (needs a B200).

Config 2 (SpMV) at full size is in tests/test_gpu_parity.py (every tunable kernel).  Here: config 3 (SpMM,
2^21 rows, k = 64), config 4a (4096 problems of 128^3), config 4b (one 8192^3 product) and config 5 (PCG on the
4096^2 Laplacian, 200 iterations).  The oracle cannot run these whole in seconds, so each case compares a sample
that it can (rows, problems, the first iterations) and adds a property of the whole result.
"""
import numpy as np
import pytest
import torch

from lapis_b200 import workloads as w
from oracle import oracle

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: the gpu-marked tests must run on a GPU box")
    return torch.device("cuda:0")


def _sub_csr(pos, crd, val, rows):
    lens = (pos[rows + 1] - pos[rows]).astype(np.int64)
    spos = np.zeros(len(rows) + 1, dtype=pos.dtype)
    np.cumsum(lens, out=spos[1:])
    idx = np.concatenate([np.arange(int(pos[r]), int(pos[r + 1])) for r in rows])
    return spos, np.ascontiguousarray(crd[idx]), np.ascontiguousarray(val[idx])


def test_spmm_config3_full_size():
    """2,097,152 rows, 32 entries per row, dense B of 64 columns: 4000 sampled rows of C bit for bit against the
    oracle's sequential row loop, the accumulate form on the same rows, and run-to-run identity of all of C."""
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    d = w.spmm_uniform()
    pos, crd, val, B = d["pos"], d["crd"], d["val"], d["B"]
    n = len(pos) - 1
    assert n == 1 << 21 and len(crd) == 32 * n and B.shape == (n, 64)
    A = CsrMatrix.from_host(pos, crd, val, (n, n), dev)
    Bd = torch.as_tensor(B).to(dev)
    C = torch.zeros((n, 64), dtype=torch.float64, device=dev)
    A.spmm(Bd, C, accumulate=False)
    C2 = torch.full((n, 64), 3.0, dtype=torch.float64, device=dev)
    A.spmm(Bd, C2, accumulate=False)
    assert torch.equal(C, C2)
    rows = np.sort(np.random.default_rng(3).choice(n, 4000, replace=False))
    spos, scrd, sval = _sub_csr(pos, crd, val, rows)
    ridx = torch.as_tensor(rows, device=dev)
    ref = oracle.spmm(spos, scrd, sval, B, np.zeros((len(rows), 64)))
    assert np.array_equal(C[ridx].cpu().numpy(), ref)
    # C = C_in + A B on the same rows
    Cin = np.random.default_rng(4).uniform(-1, 1, (len(rows), 64))
    C2[ridx] = torch.as_tensor(Cin).to(dev)
    A.spmm(Bd, C2, accumulate=True)
    assert np.array_equal(C2[ridx].cpu().numpy(), oracle.spmm(spos, scrd, sval, B, Cin))


def test_batched_gemm_config4a_full_size():
    """4096 problems of 128 x 128 x 128 in fp32 on the tensor-core path: 24 sampled problems against a product
    accumulated in double (norm-wise bar of the tensor-core tests), every problem's checksum against fp64 row
    sums, and run-to-run identity."""
    from lapis_b200.device import bgemm, bgemm_status
    dev = _dev()
    d = w.batched_gemm()
    A, B = d["A"], d["B"]
    assert A.shape == (4096, 128, 128)
    Ad, Bd = torch.as_tensor(A).to(dev), torch.as_tensor(B).to(dev)
    C = torch.zeros((4096, 128, 128), dtype=torch.float32, device=dev)
    bgemm(Ad, Bd, C)
    bgemm_status()
    C2 = torch.zeros_like(C)
    bgemm(Ad, Bd, C2)
    bgemm_status()
    assert torch.equal(C, C2)
    pick = np.unique(np.linspace(0, 4095, 24).astype(int))
    zero = np.zeros((len(pick), 128, 128), np.float32)
    As, Bs = np.ascontiguousarray(A[pick]), np.ascontiguousarray(B[pick])
    exact = oracle.bgemm_acc64(As, Bs, zero, nthreads=8)
    loop_err = np.max(np.abs(oracle.bgemm(As, Bs, zero, nthreads=8).astype(np.float64) - exact))
    got = C[torch.as_tensor(pick, device=dev)].cpu().numpy().astype(np.float64)
    err = np.max(np.abs(got - exact))
    assert err <= max(1e-5 * np.max(np.abs(exact)), loop_err), f"err {err:.3e}, fp32 loop {loop_err:.3e}"
    # checksum of every problem: sum_ij C[b,i,j] = sum_k (sum_i A[b,i,k]) (sum_j B[b,k,j]), in double
    check = np.einsum("bk,bk->b", A.astype(np.float64).sum(axis=1), B.astype(np.float64).sum(axis=2))
    sums = C.double().sum(dim=(1, 2)).cpu().numpy()
    mag = np.einsum("bk,bk->b", np.abs(A).astype(np.float64).sum(axis=1), np.abs(B).astype(np.float64).sum(axis=2))
    assert np.all(np.abs(sums - check) <= 1e-5 * mag)


def test_gemm_config4b_full_size():
    """One 8192 x 8192 x 8192 fp32 product: 64 sampled rows against fp64 dot products, norm-wise within 1e-5 of
    the result's largest entry (the tolerance stated for fp32), and the checksum of every row."""
    from lapis_b200.device import bgemm, bgemm_status
    dev = _dev()
    d = w.dense_gemm()
    A, B = d["A"], d["B"]
    assert A.shape == (8192, 8192)
    Ad, Bd = torch.as_tensor(A).to(dev), torch.as_tensor(B).to(dev)
    C = torch.zeros((8192, 8192), dtype=torch.float32, device=dev)
    bgemm(Ad, Bd, C)
    bgemm_status()
    rows = np.unique(np.linspace(0, 8191, 64).astype(int))
    ridx = torch.as_tensor(rows, device=dev)
    exact = (Ad[ridx].double() @ Bd.double()).cpu().numpy()            # fp64 on the device, checked against numpy below
    exact_np = A[rows[:4]].astype(np.float64) @ B.astype(np.float64)   # the yardstick itself, on the host
    assert np.max(np.abs(exact[:4] - exact_np)) <= 1e-10 * np.max(np.abs(exact_np))
    got = C[ridx].cpu().numpy().astype(np.float64)
    err = np.max(np.abs(got - exact)) / np.max(np.abs(exact))
    assert err <= 1e-5, f"max error / max |C| = {err:.3e}"
    # every row's checksum: sum_j C[i,j] = A[i,:] . (sum_j B[:,j])
    bsum = B.astype(np.float64).sum(axis=1)
    check = A.astype(np.float64) @ bsum
    mag = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64).sum(axis=1)
    assert np.all(np.abs(C.double().sum(dim=1).cpu().numpy() - check) <= 1e-5 * mag)


def test_pcg_config5_full_size():
    """5-point Laplacian on the 4096 x 4096 grid (16,777,216 rows): the relative residual after each of the first
    five iterations against the oracle's loop (the recurrences alpha, beta, r.r all enter it), x after five
    iterations element by element, and after 200 iterations the reported residual against the true residual
    b - A x computed by the oracle's SpMV on the host."""
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    d = w.pcg_laplacian(4096)
    pos, crd, val, b, dinv = d["pos"], d["crd"], d["val"], d["b"], d["dinv"]
    n = d["shape"][0]
    assert n == 4096 * 4096 and len(crd) == 83_869_696
    A = CsrMatrix.from_host(pos, crd, val, (n, n), dev)
    bd, dd = torch.as_tensor(b).to(dev), torch.as_tensor(dinv).to(dev)
    for k in (1, 2, 3, 5):
        x, iters, relres = A.pcg(bd, dd, 0.0, k)
        xo, io, ro = oracle.pcg(pos, crd, val, b, dinv, 0.0, k, 16)
        assert iters == io == k
        assert abs(relres - ro) <= 1e-11 * ro, f"iteration {k}: relres {relres!r} vs {ro!r}"
    assert np.max(np.abs(x.cpu().numpy() - xo)) <= 1e-11 * np.max(np.abs(xo))
    x, iters, relres = A.pcg(bd, dd, 0.0, 200)
    assert iters == 200
    xh = x.cpu().numpy()
    r_true = b - oracle.spmv(pos, crd, val, xh, np.zeros(n), 16)
    true_rel = np.linalg.norm(r_true) / np.linalg.norm(b)
    assert abs(true_rel - relres) <= 1e-8 * relres, f"reported {relres!r}, true {true_rel!r}"
    # the same solve again: identical bits
    x2, _, relres2 = A.pcg(bd, dd, 0.0, 200)
    assert relres2 == relres and torch.equal(x, x2)
