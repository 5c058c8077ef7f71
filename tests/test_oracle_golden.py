"""Pins the CPU oracle against the known answers of the reference's example tests
(fixtures made by tests/golden/make_golden.py) and against independent numpy /
scipy statements of the same operations."""
import os

import numpy as np
import pytest
from scipy.sparse import csr_matrix

from oracle import oracle


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_spmv_known_answer(golden_dir):
    # examples/spmv_noalloc.py:16-37: 5x5 CSR with an empty last row, x = 1, y = 0.
    g = _load(golden_dir, "spmv_noalloc.npz")
    y = oracle.spmv(g["rowptrs"], g["colinds"], g["values"], np.ones(5), np.zeros(5))
    assert np.allclose(y, g["ycorrect"])            # the reference's own check
    assert np.allclose(y, g["ycorrect"], rtol=1e-15, atol=1e-15)
    assert y[4] == 0.0                              # empty row keeps y_in
    # accumulate semantics: y_out = y_in + A x
    y2 = oracle.spmv(g["rowptrs"], g["colinds"], g["values"], np.ones(5), np.arange(5.0))
    assert np.allclose(y2, g["ycorrect"] + np.arange(5.0), rtol=1e-15)
    # int64 indices give the same bits
    y3 = oracle.spmv(g["rowptrs"].astype(np.int64), g["colinds"].astype(np.int64), g["values"],
                     np.ones(5), np.zeros(5))
    assert np.array_equal(y, y3)
    assert np.array_equal(y, oracle.spmv_numpy(g["rowptrs"], g["colinds"], g["values"], np.ones(5),
                                               np.zeros(5)))


def test_pcg_nos4_matches_scipy(golden_dir):
    # examples/pcg_solve.py:106-141
    g = _load(golden_dir, "pcg_nos4.npz")
    x, iters, relres = oracle.pcg(g["indptr"], g["indices"], g["data"], g["b"], g["dinv"],
                                  float(g["reltol"]), int(g["maxiter"]))
    assert np.allclose(x, g["x_scipy"])             # the reference's own check
    assert iters == int(g["maxiter"]) or relres <= float(g["reltol"])
    assert 1 <= iters <= int(g["maxiter"])
    # 40 iterations do not reach 1e-10 on nos4; both solvers stop at the same iterate
    assert iters == 40 and np.max(np.abs(x - g["x_scipy"])) < 1e-12
    # run to convergence: x_gold is all ones (b = A*1, pcg_solve.py:110-111)
    x, iters, relres = oracle.pcg(g["indptr"], g["indices"], g["data"], g["b"], g["dinv"], 1e-10, 400)
    assert relres <= 1e-10 and iters < 400 and np.max(np.abs(x - 1.0)) < 1e-8


def test_pcg_iteration_semantics(golden_dir):
    g = _load(golden_dir, "pcg_nos4.npz")
    args = (g["indptr"], g["indices"], g["data"], g["b"], g["dinv"])
    # tol = 0 never converges: exactly maxiter iterations (i starts at 1, pcg_solve.py:72,89)
    for m in (1, 2, 7):
        _, iters, _ = oracle.pcg(*args, 0.0, m)
        assert iters == m
    # a loose tolerance stops early
    _, iters, relres = oracle.pcg(*args, 1e-2, 40)
    assert iters < 40 and relres <= 1e-2
    # trace: relres of the last iteration equals the returned relres
    x, iters, relres, tr = oracle.pcg(*args, 1e-10, 40, trace=True)
    assert tr["relres"][iters - 1] == relres
    assert np.all(np.isfinite(tr["alpha"][:iters]))
    assert np.all(np.isfinite(tr["beta"][:iters - 1]))


def test_mht_golden_vectors(golden_dir):
    # examples/hitting_times.py:196-228: 17-digit vectors from the reference's own run.
    g = _load(golden_dir, "mht.npz")
    mom1, mom2 = oracle.mht(g["indptr"], g["indices"], g["data"], g["mask"], g["D"],
                            float(g["alpha"]), float(g["tol"]), int(g["maxiter"]))
    assert np.allclose(mom1, g["mom1_gold"]) and np.allclose(mom2, g["mom2_gold"])  # reference's check
    # The golden values are printed to 17 digits; the PCG inside stops at relres 1e-10, so the
    # restatement is held to a far tighter bound than np.allclose.
    assert np.allclose(mom1, g["mom1_gold"], rtol=1e-9, atol=1e-9)
    assert np.allclose(mom2, g["mom2_gold"], rtol=1e-9, atol=1e-9)


def test_gemm_examples(golden_dir):
    g = _load(golden_dir, "gemm.npz")
    c = oracle.gemm(g["a"], g["b"], np.zeros_like(g["c"]))
    assert np.allclose(c, g["c"])                  # examples/gemm_no_alloc.py:46
    g = _load(golden_dir, "batched_gemm.npz")
    c = oracle.bgemm(g["a"], g["b"], np.zeros_like(g["c"]))
    assert np.array_equal(c, g["c"])               # small integers: exact (batched_gemm_no_alloc.py:53)
    # accumulate semantics C = C_in + A B
    c2 = oracle.bgemm(g["a"], g["b"], np.ones_like(g["c"]))
    assert np.array_equal(c2, g["c"] + 1)


@pytest.mark.parametrize("idx", [np.int32, np.int64])
def test_spmv_spmm_random_vs_scipy(idx):
    rng = np.random.default_rng(7)
    n, m = 257, 301
    lens = rng.integers(0, 40, n)
    lens[5] = 0
    lens[100] = 300
    pos = np.zeros(n + 1, dtype=idx)
    pos[1:] = np.cumsum(lens)
    crd = np.concatenate([np.sort(rng.choice(m, l, replace=False)) for l in lens]).astype(idx)
    val = rng.uniform(-1, 1, len(crd))
    x = rng.uniform(-1, 1, m)
    y0 = rng.uniform(-1, 1, n)
    A = csr_matrix((val, crd, pos), shape=(n, m))
    y = oracle.spmv(pos, crd, val, x, y0)
    assert np.allclose(y, y0 + A @ x, rtol=1e-12, atol=1e-13)
    assert np.array_equal(y, oracle.spmv_numpy(pos, crd, val, x, y0))
    assert np.array_equal(y, oracle.spmv(pos, crd, val, x, y0, nthreads=4))  # rows are independent
    B = rng.uniform(-1, 1, (m, 64))
    C0 = rng.uniform(-1, 1, (n, 64))
    C = oracle.spmm(pos, crd, val, B, C0)
    assert np.allclose(C, C0 + A @ B, rtol=1e-12, atol=1e-13)
    # column c of SpMM is the SpMV with B[:, c], bit for bit
    assert np.array_equal(C[:, 3], oracle.spmv(pos, crd, val, np.ascontiguousarray(B[:, 3]), C0[:, 3]))
    B5 = rng.uniform(-1, 1, (m, 5))
    assert np.allclose(oracle.spmm(pos, crd, val, B5, np.zeros((n, 5))), A @ B5, rtol=1e-12, atol=1e-13)


def test_vector_kernels():
    rng = np.random.default_rng(3)
    x, y = rng.uniform(-1, 1, 1000), rng.uniform(-1, 1, 1000)
    acc = 0.0
    for a, b in zip(x, y):
        acc = acc + a * b
    assert oracle.dot(x, y) == acc
    assert abs(oracle.dot(x, y, nthreads=4) - acc) < 1e-12
    assert np.array_equal(oracle.axpby(0.3, x, -1.7, y), x * 0.3 + y * -1.7)
    assert np.array_equal(oracle.mult(x, y), x * y)


def test_gemm_order_and_yardstick():
    rng = np.random.default_rng(11)
    A = rng.uniform(-1, 1, (3, 17, 33)).astype(np.float32)
    B = rng.uniform(-1, 1, (3, 33, 9)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (3, 17, 9)).astype(np.float32)
    C = oracle.bgemm(A, B, C0)
    # sequential-k fp32 order with separate multiply and add
    ref = np.zeros_like(C0)
    for k in range(33):
        ref = ref + A[:, :, k:k + 1] * B[:, k:k + 1, :]
    assert np.array_equal(C, ref + C0)
    exact = oracle.bgemm_acc64(A, B, C0)
    assert np.allclose(exact, C0.astype(np.float64) + np.matmul(A.astype(np.float64), B.astype(np.float64)),
                       rtol=1e-13, atol=1e-13)
    assert np.max(np.abs(C - exact)) < 1e-5


@pytest.mark.parametrize("G", [1, 2, 3, 4, 8])
def test_partition_rows(G):
    rng = np.random.default_rng(G)
    lens = rng.integers(0, 50, 1000)
    lens[:40] = 0
    lens[500] = 5000
    for dt in (np.int32, np.int64):
        pos = np.zeros(1001, dtype=dt)
        pos[1:] = np.cumsum(lens)
        b = oracle.partition_rows(pos, G)
        assert np.array_equal(b, oracle.partition_rows_numpy(pos, G))
        assert b[0] == 0 and b[-1] == 1000 and np.all(np.diff(b) >= 0)
