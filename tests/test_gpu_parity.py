"""Parity of the CUDA path with the CPU oracle, through the C ABI (needs a B200).

Tolerances.  Integer work (offsets, partition bounds) is bit-exact.  Kernels that keep
the reference's summation order -- SpMM, the general-shape matmul, axpby, mult -- are
compared bit for bit.  SpMV and dot sum a row / vector in a different (fixed) order than
the sequential CPU loop, so they are held to 1e-12 relative to the magnitude of the terms
that were summed, TOL_F64 below; every such kernel must also give identical bits when run
twice (no atomics anywhere).
"""
import os

import numpy as np
import pytest
import torch

from lapis_b200 import KokkosBackend as KB
from lapis_b200 import workloads as w
from oracle import oracle
from tests import mlir_modules as mm

pytestmark = pytest.mark.gpu

TOL_F64 = 1e-12


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: the gpu-marked tests must run on a GPU box")
    return torch.device("cuda:0")


def _spec(pos, crd, val, shape):
    return (shape, (len(pos), len(crd), len(val)))


def _row_scale(pos, crd, val, x, y_in):
    """|y_in| + sum_j |val_j x_j| per row: the magnitude the rounding errors scale with."""
    absprod = np.abs(val) * np.abs(x[crd])
    return oracle.spmv(pos, crd, absprod, np.ones_like(x), np.abs(y_in))


def _assert_spmv_close(y, ref, scale):
    err = np.abs(y - ref)
    bound = TOL_F64 * np.maximum(scale, np.finfo(np.float64).tiny)
    assert np.all(err <= bound), f"max err/scale = {np.max(err / np.maximum(scale, 1e-300)):.3e}"


def _random_csr(rng, lens, ncols, idx):
    pos, crd = w.random_csr_from_lengths(lens, ncols, rng, idx)
    return pos, crd, rng.uniform(-1, 1, crd.size)


# ---------------------------------------------------------------------------
# SpMV
# ---------------------------------------------------------------------------
def test_spmv_known_answer_through_backend(golden_dir):
    # examples/spmv_noalloc.py:16-37 in the LAPIS project
    _dev()
    g = np.load(os.path.join(golden_dir, "spmv_noalloc.npz"))
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmv(mm.CSR32))
    y = np.zeros(5)
    out = module.spmv(g["rowptrs"], g["colinds"], g["values"], ((5, 5), (6, 8, 8)), np.ones(5), y)
    assert np.allclose(y, g["ycorrect"]) and out is y
    assert np.array_equal(y, oracle.spmv(g["rowptrs"], g["colinds"], g["values"], np.ones(5), np.zeros(5)))
    # accumulates into y
    module.spmv(g["rowptrs"], g["colinds"], g["values"], ((5, 5), (6, 8, 8)), np.ones(5), y)
    assert np.allclose(y, 2 * g["ycorrect"])


@pytest.fixture(params=[(256, 4, 1), (-256, 3, 1), (-512, 2, 0), (2, 4, 1), (3, 4, 0), (4, 0, 0)],
                ids=["chunk", "pipe256", "pipe512", "scan", "scan512", "walk"])
def spmv_kernel(request):
    """Runs the test once per SpMV kernel variant and restores the default afterwards."""
    from lapis_b200._lib import check, load
    check(load().lapis_b200_spmv_select_kernel(*request.param))
    yield request.param
    check(load().lapis_b200_spmv_status(None))
    check(load().lapis_b200_spmv_select_kernel(0, 0, 0))


@pytest.mark.parametrize("idx", [np.int32, np.int64])
@pytest.mark.parametrize("case", ["uniform10", "powerlaw", "ragged", "empty_rows", "one_huge_row", "all_empty", "dense_rows"])
def test_spmv_matches_oracle(idx, case, spmv_kernel):
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    rng = np.random.default_rng(sum(map(ord, case)))
    if case == "uniform10":      # config 1 of the benchmark
        d = w.spmv_uniform(10_000, 10, idx)
        pos, crd, val, ncols = d["pos"], d["crd"], d["val"], 10_000
    elif case == "powerlaw":     # config 2 at 1/64 size
        d = w.spmv_power_law(1 << 17, idx_dtype=idx)
        pos, crd, val, ncols = d["pos"], d["crd"], d["val"], 1 << 17
    elif case == "ragged":       # rows % 32 != 0, lengths 0..70
        lens = rng.integers(0, 70, 1237)
        ncols = 999
        pos, crd, val = _random_csr(rng, lens, ncols, idx)
    elif case == "empty_rows":   # long runs of empty rows, also at both ends
        lens = rng.integers(0, 6, 50_000)
        lens[:3000] = 0
        lens[20_000:26_000] = 0
        lens[-2500:] = 0
        ncols = 50_000
        pos, crd, val = _random_csr(rng, lens, ncols, idx)
    elif case == "one_huge_row":  # a row spanning many tiles among short rows
        lens = rng.integers(1, 5, 3000)
        lens[1500] = 40_000
        lens[7] = 4096
        ncols = 50_000
        pos, crd, val = _random_csr(rng, lens, ncols, idx)
    elif case == "all_empty":
        lens = np.zeros(777, dtype=np.int64)
        ncols = 10
        pos, crd, val = _random_csr(rng, lens, ncols, idx)
    else:                        # every row longer than a tile's average threshold
        lens = np.full(300, 700)
        ncols = 4000
        pos, crd, val = _random_csr(rng, lens, ncols, idx)
    nrows = len(pos) - 1
    x = rng.uniform(-1, 1, ncols)
    y0 = rng.uniform(-1, 1, nrows)
    A = CsrMatrix.from_host(pos, crd, val, (nrows, ncols), dev)
    assert A.nnz == len(crd)
    xd = torch.as_tensor(x).to(dev)
    for accumulate in (True, False):
        yd = torch.as_tensor(y0).to(dev)
        A.spmv(xd, yd, accumulate=accumulate)
        y = yd.cpu().numpy()
        y_in = y0 if accumulate else np.zeros(nrows)
        ref = oracle.spmv(pos, crd, val, x, y_in)
        _assert_spmv_close(y, ref, _row_scale(pos, crd, val, x, y_in))
        yd2 = torch.as_tensor(y0).to(dev)
        A.spmv(xd, yd2, accumulate=accumulate)
        assert torch.equal(yd, yd2), "SpMV is not run-to-run deterministic"
    # rows of up to 32 entries inside one chunk of 2048 are summed in the CPU order: identical bits for all
    # but the (at most one per chunk) rows cut by a chunk boundary (the segmented-scan and warp-walk kernels sum
    # in scan order and are held to the tolerance above only)
    if case in ("uniform10", "empty_rows") and spmv_kernel[0] not in (2, 3, 4):
        yd = torch.as_tensor(y0).to(dev)
        A.spmv(xd, yd, accumulate=True)
        same = yd.cpu().numpy() == oracle.spmv(pos, crd, val, x, y0)
        assert np.count_nonzero(~same) <= len(crd) // 2048 + 1
    # rows with at most one entry involve no reordering: identical bits
    short = np.flatnonzero(np.diff(pos) <= 1)
    if short.size:
        yd = torch.as_tensor(y0).to(dev)
        A.spmv(xd, yd, accumulate=True)
        assert np.array_equal(yd.cpu().numpy()[short], oracle.spmv(pos, crd, val, x, y0)[short])


@pytest.mark.parametrize("forced", [None, (4, 0, 0)], ids=["default", "walk"])
def test_spmv_random_shapes_property(forced):
    """Random small CSR shapes (hypothesis): empty rows, rows longer than a warp's threshold, rows cut by the
    2048-entry chunk boundary, ncols == 1, int32 and int64 -- all against the oracle; once with the default
    kernel and once with the warp-walk kernel forced."""
    from hypothesis import given, settings, strategies as st
    from lapis_b200._lib import check, load
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    if forced is not None:
        check(load().lapis_b200_spmv_select_kernel(*forced))

    @settings(max_examples=40, deadline=None)
    @given(lens=st.lists(st.one_of(st.integers(0, 6), st.integers(0, 90), st.just(2500)), min_size=1, max_size=400),
           ncols=st.sampled_from([1, 7, 64, 3000]), wide=st.booleans(), seed=st.integers(0, 2 ** 16), acc=st.booleans())
    def run(lens, ncols, wide, seed, acc):
        rng = np.random.default_rng(seed)
        lens = np.minimum(np.array(lens, dtype=np.int64), ncols)
        idx = np.int64 if wide else np.int32
        pos, crd, val = _random_csr(rng, lens, ncols, idx)
        x = rng.uniform(-1, 1, ncols)
        y0 = rng.uniform(-1, 1, len(lens))
        A = CsrMatrix.from_host(pos, crd, val, (len(lens), ncols), dev)
        yd = torch.as_tensor(y0).to(dev)
        A.spmv(torch.as_tensor(x).to(dev), yd, accumulate=acc)
        y_in = y0 if acc else np.zeros(len(lens))
        _assert_spmv_close(yd.cpu().numpy(), oracle.spmv(pos, crd, val, x, y_in), _row_scale(pos, crd, val, x, y_in))

    try:
        run()
    finally:
        check(load().lapis_b200_spmv_select_kernel(0, 0, 0))


def test_spmv_tuning_keeps_the_bits():
    """Every kernel variant sums a row in the same order, so the tuned choice changes speed only."""
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    for d in (w.spmv_power_law(1 << 16, idx_dtype=np.int64), w.pcg_laplacian(200)):
        n = d["shape"][0]
        x = torch.as_tensor(np.random.default_rng(2).uniform(-1, 1, n)).to(dev)
        A = CsrMatrix.from_host(d["pos"], d["crd"], d["val"], (n, n), dev)
        y0 = torch.zeros(n, dtype=torch.float64, device=dev)
        A.spmv(x, y0, accumulate=False)
        threads, blocks = A.tune()
        assert (threads, blocks) in ((256, 4), (256, 6), (512, 3), (-256, 3), (-256, 4), (1, 0))
        y1 = torch.zeros(n, dtype=torch.float64, device=dev)
        A.spmv(x, y1, accumulate=False)
        assert torch.equal(y0, y1)


def test_spmv_relaxed_tuning_stays_within_the_tolerance():
    """The relaxed tuner may also pick the segmented-scan or the warp-walk kernel, which sum a row in scan order: the result
    stays within the bound of the other SpMV tests and repeats bit for bit; any other pick keeps the bits."""
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    d = w.spmv_power_law(1 << 16, idx_dtype=np.int64)
    pos, crd, val, x = d["pos"], d["crd"], d["val"], d["x"]
    n = d["shape"][0]
    xd = torch.as_tensor(x).to(dev)
    A = CsrMatrix.from_host(pos, crd, val, (n, n), dev)
    y0 = torch.zeros(n, dtype=torch.float64, device=dev)
    A.spmv(xd, y0, accumulate=False)
    threads, blocks = A.tune(relaxed=True)
    assert (threads, blocks) in ((256, 4), (256, 6), (512, 3), (-256, 3), (-256, 4), (1, 0), (2, 4), (2, 5), (3, 3), (3, 4), (4, 0))
    y1 = torch.zeros(n, dtype=torch.float64, device=dev)
    A.spmv(xd, y1, accumulate=False)
    y2 = torch.zeros(n, dtype=torch.float64, device=dev)
    A.spmv(xd, y2, accumulate=False)
    assert torch.equal(y1, y2)
    if threads not in (2, 3, 4):
        assert torch.equal(y0, y1)
    zero = np.zeros(n)
    _assert_spmv_close(y1.cpu().numpy(), oracle.spmv(pos, crd, val, x, zero), _row_scale(pos, crd, val, x, zero))


@pytest.mark.parametrize("idx", [np.int32, np.int64])
def test_spmv_one_thread_per_row_kernel_keeps_the_bits(idx):
    """Matrices whose rows have at most 32 entries may run with one thread per row; rows that cross a chunk
    boundary of the plan are joined as the chunk kernels join them, so y and the accumulate path are
    bit-identical.  Matrices with a longer row keep the chunk kernels even when the variant is forced."""
    from lapis_b200._lib import check, load
    from lapis_b200.device import CsrMatrix
    dev, lib = _dev(), load()
    rng = np.random.default_rng(77)
    cases = []
    lap = w.pcg_laplacian(300, idx_dtype=idx)
    cases.append((lap["pos"], lap["crd"], lap["val"], lap["shape"][0]))
    lens = rng.integers(0, 33, size=50_000)              # 0..32 entries, many rows crossing chunk boundaries
    pos, crd, val = _random_csr(rng, lens, 50_000, idx)
    cases.append((pos, crd, val, 50_000))
    for pos, crd, val, n in cases:
        x = rng.uniform(-1, 1, n)
        y_in = rng.uniform(-1, 1, n)
        A = CsrMatrix.from_host(pos, crd, val, (n, n), dev)
        xd = torch.as_tensor(x).to(dev)
        ref = [torch.zeros(n, dtype=torch.float64, device=dev), torch.as_tensor(y_in).to(dev)]
        A.spmv(xd, ref[0], accumulate=False)
        A.spmv(xd, ref[1], accumulate=True)
        A.tune()                                          # finds the longest row; may or may not pick (1, 0)
        check(lib.lapis_b200_spmv_select_kernel(1, 0, 1))
        try:
            got = [torch.zeros(n, dtype=torch.float64, device=dev), torch.as_tensor(y_in).to(dev)]
            A.spmv(xd, got[0], accumulate=False)
            A.spmv(xd, got[1], accumulate=True)
        finally:
            check(lib.lapis_b200_spmv_select_kernel(0, 0, 0))
        assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1])
        yo = oracle.spmv(pos, crd, val, x, y_in)
        _assert_spmv_close(got[1].cpu().numpy(), yo, _row_scale(pos, crd, val, x, y_in))
    # a matrix with one long row: the request is not honoured, the result is the chunk kernels'
    lens = rng.integers(0, 20, size=4000)
    lens[1234] = 700
    pos, crd, val = _random_csr(rng, lens, 4000, idx)
    A = CsrMatrix.from_host(pos, crd, val, (4000, 4000), dev)
    xd = torch.as_tensor(rng.uniform(-1, 1, 4000)).to(dev)
    y0 = torch.zeros(4000, dtype=torch.float64, device=dev)
    A.spmv(xd, y0, accumulate=False)
    assert A.tune()[0] != 1
    check(lib.lapis_b200_spmv_select_kernel(1, 0, 1))
    try:
        y1 = torch.zeros(4000, dtype=torch.float64, device=dev)
        A.spmv(xd, y1, accumulate=False)
    finally:
        check(lib.lapis_b200_spmv_select_kernel(0, 0, 0))
    assert torch.equal(y0, y1)


def test_spmv_row_block_in_place(spmv_kernel):
    """A handle over rows [r0, r1) of a larger matrix (non-zero pos[0]) gives that slice of y."""
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    d = w.spmv_power_law(1 << 14, idx_dtype=np.int64)
    pos, crd, val, x = d["pos"], d["crd"], d["val"], d["x"]
    n = len(pos) - 1
    ref = oracle.spmv(pos, crd, val, x, np.zeros(n))
    pos_d, crd_d, val_d = (torch.as_tensor(a).to(dev) for a in (pos, crd, val))
    xd = torch.as_tensor(x).to(dev)
    r0, r1 = 3001, 11_111
    A = CsrMatrix(pos_d[r0:r1 + 1], crd_d, val_d, (r1 - r0, n))
    assert A.nnz == pos[r1] - pos[r0]
    yd = torch.zeros(r1 - r0, dtype=torch.float64, device=dev)
    A.spmv(xd, yd, accumulate=False)
    scale = _row_scale(pos, crd, val, x, np.zeros(n))[r0:r1]
    _assert_spmv_close(yd.cpu().numpy(), ref[r0:r1], scale)


@pytest.fixture(scope="module")
def config2_full():
    """Config 2 at full size (2^23 rows, ~1.34e8 entries, int64 indices) on the device, with the host-side
    quantities the size-independent checks need (computed once for all kernel variants)."""
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    d = w.spmv_power_law()
    pos, crd, val, x = d["pos"], d["crd"], d["val"], d["x"]
    n = len(pos) - 1
    starts = pos[:-1].astype(np.int64)
    ref = {
        "absum_x": np.add.reduceat(np.abs(val * x[crd]), starts),
        "rowsum": np.add.reduceat(val, starts),
        "absum": np.add.reduceat(np.abs(val), starts),
        "rows": np.random.default_rng(5).integers(0, n, 2000),
    }
    ref["sample"] = np.array([
        oracle.spmv(np.array([0, int(pos[r + 1] - pos[r])], dtype=np.int64), crd[pos[r]:pos[r + 1]], val[pos[r]:pos[r + 1]], x,
                    np.zeros(1))[0] for r in ref["rows"]])
    A = CsrMatrix.from_host(pos, crd, val, (n, n), dev)
    yield {"A": A, "x": torch.as_tensor(x).to(dev), "n": n, "ref": ref, "dev": dev}
    del A
    torch.cuda.empty_cache()


_FULL_VARIANTS = ["default", "tuned", "tuned_relaxed"] + [(t, b, h) for (t, b) in ((2, 4), (2, 5), (3, 3), (3, 4)) for h in (0, 1)] + [(4, 0, 0)]


@pytest.mark.parametrize("variant", _FULL_VARIANTS, ids=[v if isinstance(v, str) else "k%d_%d_%d" % v for v in _FULL_VARIANTS])
def test_spmv_full_size_properties(config2_full, variant):
    """Config 2 at full size through every kernel the tuners can pick for it -- the default chunk kernel, the
    strict and the relaxed tuner's choice, each segmented-scan instantiation and the warp-walk kernel: exact
    linearity, the accumulate identity, row sums against numpy's reduceat, and 2000 rows against the oracle.
    None of these needs a CPU pass over the whole matrix per variant."""
    from lapis_b200._lib import check, load
    c = config2_full
    A, xd, n, ref, dev = c["A"], c["x"], c["n"], c["ref"], c["dev"]
    lib = load()
    if variant == "tuned":
        A.tune()
    elif variant == "tuned_relaxed":
        A.tune(relaxed=True)
    elif variant != "default":
        check(lib.lapis_b200_spmv_select_kernel(*variant))
    try:
        y1 = torch.zeros(n, dtype=torch.float64, device=dev)
        A.spmv(xd, y1, accumulate=False)
        y1b = torch.full((n,), 7.0, dtype=torch.float64, device=dev)
        A.spmv(xd, y1b, accumulate=False)
        assert torch.equal(y1, y1b), "not run-to-run identical / depends on the old contents of y"
        # A(2x) = 2 A x exactly (scaling by 2 is exact in binary floating point)
        y2 = torch.zeros(n, dtype=torch.float64, device=dev)
        A.spmv(2.0 * xd, y2, accumulate=False)
        assert torch.equal(y2, 2.0 * y1)
        # accumulate: y1 + A x == 2 A x up to the rounding of the final adds
        y3 = y1.clone()
        A.spmv(xd, y3, accumulate=True)
        assert np.all(np.abs((y3 - 2.0 * y1).cpu().numpy()) <= TOL_F64 * ref["absum_x"])
        # x = 1: y = row sums of val, checked against numpy's reduceat on the host
        ones = torch.ones(n, dtype=torch.float64, device=dev)
        ys = torch.zeros(n, dtype=torch.float64, device=dev)
        A.spmv(ones, ys, accumulate=False)
        assert np.all(np.abs(ys.cpu().numpy() - ref["rowsum"]) <= TOL_F64 * ref["absum"])
        # a sample of rows against the oracle
        yh = y1.cpu().numpy()
        rows = ref["rows"]
        err = np.abs(yh[rows] - ref["sample"])
        assert np.all(err <= TOL_F64 * ref["absum_x"][rows]), f"max err/scale {np.max(err / ref['absum_x'][rows]):.3e}"
    finally:
        check(lib.lapis_b200_spmv_select_kernel(0, 0, 0))


# ---------------------------------------------------------------------------
# SpMM
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("idx", [np.int32, np.int64])
@pytest.mark.parametrize("k", [64, 5, 130, 2])
def test_spmm_bit_exact(idx, k):
    from lapis_b200.device import CsrMatrix
    dev = _dev()
    rng = np.random.default_rng(k)
    lens = rng.integers(0, 80, 2001)
    lens[11] = 0
    lens[500] = 900
    ncols = 1500
    pos, crd, val = _random_csr(rng, lens, ncols, idx)
    B = rng.uniform(-1, 1, (ncols, k))
    C0 = rng.uniform(-1, 1, (2001, k))
    A = CsrMatrix.from_host(pos, crd, val, (2001, ncols), dev)
    Bd = torch.as_tensor(B).to(dev)
    for accumulate in (True, False):
        Cd = torch.as_tensor(C0).to(dev)
        A.spmm(Bd, Cd, accumulate=accumulate)
        ref = oracle.spmm(pos, crd, val, B, C0 if accumulate else np.zeros_like(C0))
        assert np.array_equal(Cd.cpu().numpy(), ref)


def test_spmm_config3_shape_through_backend():
    """Config 3 at 1/256 size (8192 rows, 32 per row, k = 64) through py_spmm with host buffers."""
    _dev()
    d = w.spmm_uniform(1 << 13)
    n = 1 << 13
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmm(mm.CSR64))
    C = np.zeros((n, 64))
    out = module.spmm(d["pos"], d["crd"], d["val"], _spec(d["pos"], d["crd"], d["val"], (n, n)), d["B"], C)
    assert out is C
    assert np.array_equal(C, oracle.spmm(d["pos"], d["crd"], d["val"], d["B"], np.zeros((n, 64))))


# ---------------------------------------------------------------------------
# dense / batched matmul
# ---------------------------------------------------------------------------
def test_matmul_examples_through_backend(golden_dir):
    _dev()
    g = np.load(os.path.join(golden_dir, "gemm.npz"))             # examples/gemm_no_alloc.py
    module = KB.KokkosBackend().compile(mm.MATMUL)
    c = torch.zeros((8, 9))
    module.forward(torch.as_tensor(g["a"]), torch.as_tensor(g["b"]), c)   # CPU torch tensors, updated in place
    assert np.allclose(c.numpy(), g["c"])
    assert np.array_equal(c.numpy(), oracle.gemm(g["a"], g["b"], np.zeros((8, 9), dtype=np.float32)))
    g = np.load(os.path.join(golden_dir, "batched_gemm.npz"))     # examples/batched_gemm_no_alloc.py
    module = KB.KokkosBackend().compile(mm.BATCH_MATMUL)
    c = np.zeros((64, 5, 5), dtype=np.float32)
    module.forward(g["a"], g["b"], c)
    assert np.array_equal(c, g["c"])
    with pytest.raises(Exception, match="contracting"):
        KB.KokkosBackend().compile(mm.MATMUL).forward(np.zeros((4, 3), np.float32), np.zeros((5, 2), np.float32),
                                                     np.zeros((4, 2), np.float32))


@pytest.mark.parametrize("shape", [(1, 33, 17, 65), (7, 31, 32, 33), (3, 64, 64, 8), (1, 1, 1, 1), (2, 100, 3, 257)])
def test_bgemm_general_shapes_bit_exact(shape):
    from lapis_b200.device import bgemm
    dev = _dev()
    b, M, N, K = shape
    rng = np.random.default_rng(M * N + K)
    A = rng.uniform(-1, 1, (b, M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (b, K, N)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (b, M, N)).astype(np.float32)
    Cd = torch.as_tensor(C0).to(dev)
    bgemm(torch.as_tensor(A).to(dev), torch.as_tensor(B).to(dev), Cd)
    assert np.array_equal(Cd.cpu().numpy(), oracle.bgemm(A, B, C0))


@pytest.mark.parametrize("shape", [(1, 128, 128, 32), (1, 128, 128, 256), (3, 128, 128, 128), (2, 256, 384, 96),
                                   (1, 512, 512, 1024),
                                   (1, 1024, 5120, 160), (2, 1280, 2048, 144)])  # enough 128 x 256 tiles: wide configuration
def test_bgemm_tensor_core_path(shape):
    """Tile-aligned shapes run on tcgen05 with fp32 emulated by three TF32 products.  The bar is
    norm-wise against a product accumulated in double: no worse than max(1e-5 * |C|_max, the error
    of the reference's own sequential fp32 loop)."""
    from lapis_b200.device import bgemm, bgemm_status
    dev = _dev()
    b, M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    A = rng.uniform(-1, 1, (b, M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (b, K, N)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (b, M, N)).astype(np.float32)
    Cd = torch.as_tensor(C0).to(dev)
    bgemm(torch.as_tensor(A).to(dev), torch.as_tensor(B).to(dev), Cd)
    bgemm_status()
    got = Cd.cpu().numpy().astype(np.float64)
    exact = oracle.bgemm_acc64(A, B, C0, nthreads=8)
    ref_err = np.max(np.abs(oracle.bgemm(A, B, C0, nthreads=8).astype(np.float64) - exact))
    err = np.max(np.abs(got - exact))
    scale = np.max(np.abs(exact))
    assert err <= max(1e-5 * scale, ref_err), f"err {err:.3e}, fp32 loop err {ref_err:.3e}, |C| {scale:.3e}"
    # identical bits from run to run
    Cd2 = torch.as_tensor(C0).to(dev)
    bgemm(torch.as_tensor(A).to(dev), torch.as_tensor(B).to(dev), Cd2)
    bgemm_status()
    assert torch.equal(Cd, Cd2)


def test_bgemm_unaligned_operands_take_the_general_kernel():
    """A tile-aligned shape whose device pointers are not 16-byte aligned (slices of larger tensors) cannot use
    the tensor-core kernel's TMA loads; it runs on the general-shape kernel instead of being refused, and that
    kernel is bit-exact against the sequential loop."""
    from lapis_b200.device import bgemm
    dev = _dev()
    rng = np.random.default_rng(9)
    M = N = 128
    K = 64
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    big = torch.zeros(M * K + 1, dtype=torch.float32, device=dev)
    Ad = big[1:].view(M, K)                      # 4 bytes past a 16-byte boundary
    assert Ad.data_ptr() % 16 == 4
    Ad.copy_(torch.as_tensor(A))
    Cd = torch.as_tensor(C0).to(dev)
    bgemm(Ad, torch.as_tensor(B).to(dev), Cd)
    assert np.array_equal(Cd.cpu().numpy(), oracle.bgemm(A, B, C0))


def test_bgemm_tensor_core_path_with_an_infinite_input():
    """x = hi + lo with lo = x - hi would give lo = NaN for an infinite x and turn a whole row of C into NaN;
    the split gives lo = 0 there, so the row is infinite with the sign of the other operand, as in the fp32
    loop (entries whose partner has an exactly zero low part may still be NaN: 0 * inf), and the other rows
    are untouched."""
    from lapis_b200.device import bgemm, bgemm_status
    dev = _dev()
    rng = np.random.default_rng(10)
    M, N, K = 128, 256, 64
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(0.1, 1, (K, N)).astype(np.float32) * np.where(rng.random((K, N)) < 0.5, -1, 1).astype(np.float32)
    A[5, 7] = np.inf
    Cd = torch.zeros((M, N), dtype=torch.float32, device=dev)
    bgemm(torch.as_tensor(A).to(dev), torch.as_tensor(B).to(dev), Cd)
    bgemm_status()
    C = Cd.cpu().numpy()
    row = C[5]
    assert np.mean(np.isinf(row)) > 0.98
    inf_at = np.isinf(row)
    assert np.array_equal(np.sign(row[inf_at]), np.sign(B[7][inf_at]))
    others = np.delete(C, 5, axis=0)
    exact = np.delete(A, 5, axis=0).astype(np.float64) @ B.astype(np.float64)
    assert np.all(np.isfinite(others)) and np.max(np.abs(others - exact)) <= 1e-5 * np.max(np.abs(exact))



# ---------------------------------------------------------------------------
# vector kernels and PCG
# ---------------------------------------------------------------------------
def test_vector_kernels():
    from lapis_b200 import device as D
    dev = _dev()
    rng = np.random.default_rng(1)
    for n in (1, 1000, 1 << 20, (1 << 20) + 77):
        x, y = rng.uniform(-1, 1, n), rng.uniform(-1, 1, n)
        xd, yd = torch.as_tensor(x).to(dev), torch.as_tensor(y).to(dev)
        dst = torch.empty_like(xd)
        assert np.array_equal(D.axpby(0.3, xd, -1.7, yd, dst).cpu().numpy(), oracle.axpby(0.3, x, -1.7, y))
        assert np.array_equal(D.mult(xd, yd, dst).cpu().numpy(), oracle.mult(x, y))
        got = float(D.dot(xd, yd).item())
        assert abs(got - oracle.dot(x, y)) <= TOL_F64 * float(np.sum(np.abs(x * y)))
        assert got == float(D.dot(xd, yd).item())


def test_pcg_nos4_through_backend(golden_dir):
    # examples/pcg_solve.py:106-141 in the LAPIS project
    _dev()
    g = np.load(os.path.join(golden_dir, "pcg_nos4.npz"))
    n = len(g["b"])
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.pcg(mm.CSR32))
    spec = ((n, n), (n + 1, len(g["indices"]), len(g["data"])))
    x, iters, relres = module.pcg(g["indptr"], g["indices"], g["data"], spec, g["b"], g["dinv"],
                                  float(g["reltol"]), int(g["maxiter"]))
    assert np.allclose(x, g["x_scipy"])                       # the reference's own check
    xo, io, ro = oracle.pcg(g["indptr"], g["indices"], g["data"], g["b"], g["dinv"], float(g["reltol"]),
                            int(g["maxiter"]))
    assert iters == io == 40
    assert np.max(np.abs(x - xo)) <= 1e-10 * np.max(np.abs(xo))
    assert abs(relres - ro) <= 1e-8 * ro
    # converges when allowed to
    x, iters, relres = module.pcg(g["indptr"], g["indices"], g["data"], spec, g["b"], g["dinv"], 1e-10, 400)
    xo, io, ro = oracle.pcg(g["indptr"], g["indices"], g["data"], g["b"], g["dinv"], 1e-10, 400)
    assert relres <= 1e-10 and abs(iters - io) <= 1
    assert np.max(np.abs(x - 1.0)) < 1e-8
    # iteration-count semantics (i starts at 1; tol = 0 runs exactly maxiter iterations)
    for m in (1, 2, 17):
        _, iters, _ = module.pcg(g["indptr"], g["indices"], g["data"], spec, g["b"], g["dinv"], 0.0, m)
        assert iters == m


def test_pcg_step_parity_laplacian(spmv_kernel):
    """One iteration from the oracle's state reproduces the oracle's next state: the passes are
    checked without CG's amplification of rounding differences (config 5 at 128x128)."""
    from lapis_b200.device import CsrMatrix
    from lapis_b200.dist import DistPcg
    dev = _dev()
    d = w.pcg_laplacian(128)
    n = d["shape"][0]
    pos, crd, val, b, dinv = d["pos"], d["crd"], d["val"], d["b"], d["dinv"]
    # the first k iterations: per-iteration scalars against the oracle's trace
    xo, io, ro, tr = oracle.pcg(pos, crd, val, b, dinv, 0.0, 25, trace=True)
    solver = DistPcg(pos, crd, val, (n, n), b, dinv, dev, use_graph=False)
    x, iters, relres = solver.solve(0.0, 25, check_every=1)
    assert iters == io == 25
    assert abs(relres - ro) <= 1e-9 * ro
    assert np.max(np.abs(x.cpu().numpy() - xo)) <= 1e-9 * np.max(np.abs(xo))
    # a single iteration (maxiter = 1) differs from the oracle only by the dot summation order
    x1o, _, r1o, tr1 = oracle.pcg(pos, crd, val, b, dinv, 0.0, 1, trace=True)
    A = CsrMatrix.from_host(pos, crd, val, (n, n), dev)
    x1, it1, r1 = A.pcg(torch.as_tensor(b).to(dev), torch.as_tensor(dinv).to(dev), 0.0, 1)
    assert it1 == 1
    assert np.max(np.abs(x1.cpu().numpy() - x1o)) <= 1e-13 * np.max(np.abs(x1o))
    assert abs(r1 - r1o) <= 1e-13 * r1o


def test_pcg_laplacian_converges_and_graph_matches_eager():
    from lapis_b200.dist import DistPcg
    dev = _dev()
    d = w.pcg_laplacian(96, idx_dtype=np.int64)
    n = d["shape"][0]
    args = (d["pos"], d["crd"], d["val"], (n, n), d["b"], d["dinv"], dev)
    # tune=False: both solvers run the default SpMV kernel (a timed choice could differ between the two
    # objects, and the kernels group the fused dot partials differently)
    xe, ie, re_ = DistPcg(*args, use_graph=False, tune=False).solve(1e-8, 2000, check_every=10)
    xg, ig, rg = DistPcg(*args, use_graph=True, tune=False).solve(1e-8, 2000, check_every=10)
    assert ie == ig and re_ == rg and torch.equal(xe, xg)     # same kernels, same order: same bits
    assert re_ <= 1e-8 and ie < 2000
    xo, io, ro = oracle.pcg(d["pos"], d["crd"], d["val"], d["b"], d["dinv"], 1e-8, 2000)
    assert abs(ie - io) <= 2
    assert np.max(np.abs(xe.cpu().numpy() - xo)) <= 1e-6 * np.max(np.abs(xo))
    # the solution satisfies the system
    res = oracle.spmv(d["pos"], d["crd"], d["val"], xe.cpu().numpy(), -d["b"])
    assert np.linalg.norm(res) <= 2e-8 * np.linalg.norm(d["b"])


def test_pcg_two_launches_per_iteration_repeat_the_three_launch_form():
    """On matrices served by the one-thread-per-row SpMV kernel the direction update is folded into the next
    SpMV pass (two launches per iteration): x, the iteration count and the residual are those of the
    three-launch form bit for bit -- without and with the exchange kernels in the loop (the rank as its own
    peer), eager and from captured graphs, for a solve that converges and for one that stops at maxiter."""
    from lapis_b200._lib import check, load
    from lapis_b200.dist import DistPcg
    dev = _dev()
    lib = load()
    for grid, idx in ((64, np.int32), (96, np.int64)):
        d = w.pcg_laplacian(grid, idx_dtype=idx)
        n = d["shape"][0]
        args = (d["pos"], d["crd"], d["val"], (n, n), d["b"], d["dinv"], dev)
        check(lib.lapis_b200_spmv_select_kernel(1, 0, 1))   # the one-thread-per-row kernel, whatever the tuner timed
        try:
            for transport in (False, True):
                kw = dict(comm="p2p", transport_on_one_rank=transport)
                three = DistPcg(*args, use_graph=False, two_pass=False, **kw)
                assert not three._two_pass()
                for tol, maxiter in ((1e-9, 500), (0.0, 37)):
                    xr, ir, rr = three.solve(tol, maxiter, check_every=8)
                    xr = xr.clone()
                    for use_graph in (False, True):
                        two = DistPcg(*args, use_graph=use_graph, **kw)
                        assert two._two_pass()
                        for _ in range(2):   # the second solve starts from the state the first one left
                            x, it, rel = two.solve(tol, maxiter, check_every=8)
                            assert it == ir and rel == rr and torch.equal(x, xr), (grid, transport, tol, use_graph)
                            assert two.comm_error() == 0.0
        finally:
            check(lib.lapis_b200_spmv_select_kernel(0, 0, 0))
    # the C-level solver takes the same form by itself
    from lapis_b200.device import CsrMatrix
    d = w.pcg_laplacian(64)
    n = d["shape"][0]
    A = CsrMatrix.from_host(d["pos"], d["crd"], d["val"], (n, n), dev)
    A.tune()
    bd, dd = torch.as_tensor(d["b"]).to(dev), torch.as_tensor(d["dinv"]).to(dev)
    x0, i0, r0 = A.pcg(bd, dd, 1e-9, 500)
    check(lib.lapis_b200_spmv_select_kernel(1, 0, 1))
    try:
        assert lib.lapis_b200_pcg_folds_direction(A._h) == 1
        x1, i1, r1 = A.pcg(bd, dd, 1e-9, 500)
    finally:
        check(lib.lapis_b200_spmv_select_kernel(0, 0, 0))
    xo, io, ro = oracle.pcg(d["pos"], d["crd"], d["val"], d["b"], d["dinv"], 1e-9, 500)
    assert abs(i1 - io) <= 2 and r1 <= 1e-9
    assert np.max(np.abs(x1.cpu().numpy() - xo)) <= 1e-6 * np.max(np.abs(xo))


def test_pcg_peer_transport_on_one_rank():
    """The peer-to-peer exchange kernels with the rank as its own only peer (push, then wait, in stream
    order: nothing waits on another launch): same bits as the fused single-rank scalar steps, over
    two solves (two epochs of the sequence numbers) with and without a captured graph."""
    from lapis_b200.dist import DistPcg
    dev = _dev()
    d = w.pcg_laplacian(64)
    n = d["shape"][0]
    args = (d["pos"], d["crd"], d["val"], (n, n), d["b"], d["dinv"], dev)
    # tune=False: every solver uses the default SpMV kernel (the timed choice may differ between objects,
    # and the kernels group the fused dot partials differently)
    xr, ir, rr = DistPcg(*args, use_graph=False, tune=False).solve(1e-9, 500, check_every=8)
    for use_graph in (False, True):
        solver = DistPcg(*args, use_graph=use_graph, comm="p2p", transport_on_one_rank=True, tune=False)
        assert solver.comm == "p2p"
        for _ in range(2):
            x, it, rel = solver.solve(1e-9, 500, check_every=8)
            assert it == ir and rel == rr and torch.equal(x, xr)
            assert solver.comm_error() == 0.0
