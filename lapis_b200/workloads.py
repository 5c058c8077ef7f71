"""Seeded synthetic inputs with the shapes of the benchmark configurations.

The reference times SpMV on SuiteSparse / Galeri matrices and GEMMs on random
matrices (benchmarks/spmv/main.cpp, benchmarks/gemm/main.cpp,
benchmarks/batched_gemm/main.cpp in the LAPIS project).  The matrices are not
redistributed with it, so these generators stand in for them: same shape family
(rows, nonzeros per row and their distribution, index width, value range), all
reproducible from ``numpy.random.Generator(PCG64(seed))``.  Every generator takes
the size as a parameter so the tests can run the same distribution small.
"""
from __future__ import annotations

import numpy as np

SEED_BASE = 20240


def _rng(config_index: int, seed=None):
    return np.random.Generator(np.random.PCG64(SEED_BASE + config_index if seed is None else seed))


def random_csr_from_lengths(lens: np.ndarray, ncols: int, rng, idx_dtype=np.int64):
    """CSR pattern with ``lens[r]`` distinct, sorted, uniformly random columns in row r.

    Columns are drawn i.i.d. uniform, sorted per row with one global key sort, and the
    few within-row duplicates are redrawn until none is left.
    """
    lens = np.asarray(lens, dtype=np.int64)
    if lens.size and lens.max() > ncols:
        raise ValueError("a row cannot hold more distinct columns than the matrix has")
    nrows = lens.size
    pos = np.zeros(nrows + 1, dtype=np.int64)
    np.cumsum(lens, out=pos[1:])
    nnz = int(pos[-1])
    rows = np.repeat(np.arange(nrows, dtype=np.int64), lens)
    key = rows * np.int64(ncols) + rng.integers(0, ncols, nnz, dtype=np.int64)
    del rows
    key.sort()
    while True:
        dup = np.flatnonzero(key[1:] == key[:-1]) + 1
        if dup.size == 0:
            break
        bad_rows = np.unique(key[dup] // ncols)
        key[dup] = (key[dup] // ncols) * ncols + rng.integers(0, ncols, dup.size, dtype=np.int64)
        for r in bad_rows:  # a handful of rows: re-sort them in place
            key[pos[r]:pos[r + 1]].sort()
    crd = (key % ncols).astype(idx_dtype)
    return pos.astype(idx_dtype), crd


def power_law_lengths(nrows: int, rng, mean: float = 16.0, cap: int = 4096):
    """Row lengths with density ~ L^-2 on [x_min, cap], x_min solved so that E[L] = mean."""
    # E[L] = ln(cap/x) / (1/x - 1/cap): solve for x by bisection.
    lo, hi = 1e-6, float(cap)
    for _ in range(200):
        x = 0.5 * (lo + hi)
        e = np.log(cap / x) / (1.0 / x - 1.0 / cap)
        lo, hi = (x, hi) if e < mean else (lo, x)
    x_min = 0.5 * (lo + hi)
    u = rng.random(nrows)
    L = 1.0 / (1.0 / x_min - u * (1.0 / x_min - 1.0 / cap))
    return np.clip(np.rint(L), 1, cap).astype(np.int64)


def spmv_uniform(nrows: int = 10_000, per_row: int = 10, idx_dtype=np.int64, seed=None):
    """Config 1: square matrix with exactly ``per_row`` entries per row, values and x in [-1, 1)."""
    rng = _rng(1, seed)
    pos, crd = random_csr_from_lengths(np.full(nrows, per_row), nrows, rng, idx_dtype)
    val = rng.uniform(-1.0, 1.0, crd.size)
    x = rng.uniform(-1.0, 1.0, nrows)
    return {"pos": pos, "crd": crd, "val": val, "x": x, "shape": (nrows, nrows)}


def spmv_power_law(nrows: int = 1 << 23, mean: float = 16.0, cap: int = 4096, idx_dtype=np.int64, seed=None):
    """Config 2: square matrix, power-law row lengths (alpha = 2, mean 16, cap 4096)."""
    rng = _rng(2, seed)
    lens = power_law_lengths(nrows, rng, mean, min(cap, nrows))
    pos, crd = random_csr_from_lengths(lens, nrows, rng, idx_dtype)
    val = rng.uniform(-1.0, 1.0, crd.size)
    x = rng.uniform(-1.0, 1.0, nrows)
    return {"pos": pos, "crd": crd, "val": val, "x": x, "shape": (nrows, nrows)}


def spmm_uniform(nrows: int = 1 << 21, per_row: int = 32, k: int = 64, idx_dtype=np.int64, seed=None):
    """Config 3: square sparse A with ``per_row`` entries per row, dense row-major B [nrows, k]."""
    rng = _rng(3, seed)
    pos, crd = random_csr_from_lengths(np.full(nrows, min(per_row, nrows)), nrows, rng, idx_dtype)
    val = rng.uniform(-1.0, 1.0, crd.size)
    B = rng.uniform(-1.0, 1.0, (nrows, k))
    return {"pos": pos, "crd": crd, "val": val, "B": B, "shape": (nrows, nrows)}


def batched_gemm(batch: int = 4096, n: int = 128, seed=None):
    """Config 4a: ``batch`` problems of n x n x n in fp32, entries in [-1, 1)."""
    rng = _rng(4, seed)
    A = rng.uniform(-1.0, 1.0, (batch, n, n)).astype(np.float32)
    B = rng.uniform(-1.0, 1.0, (batch, n, n)).astype(np.float32)
    return {"A": A, "B": B}


def dense_gemm(n: int = 8192, seed=None):
    """Config 4b: one n x n x n fp32 product."""
    rng = _rng(4, (SEED_BASE + 4) * 7 if seed is None else seed)
    A = rng.uniform(-1.0, 1.0, (n, n)).astype(np.float32)
    B = rng.uniform(-1.0, 1.0, (n, n)).astype(np.float32)
    return {"A": A, "B": B}


def laplacian_2d(grid: int = 4096, idx_dtype=np.int32):
    """5-point Laplacian on a grid x grid mesh, Dirichlet boundary: diagonal 4, neighbours -1.

    Rows are ordered grid-row-major; columns ascend within a row.
    """
    g = int(grid)
    n = g * g
    ii, jj = np.divmod(np.arange(n, dtype=np.int64), g)
    # neighbour order by ascending column: (i-1,j), (i,j-1), (i,j), (i,j+1), (i+1,j)
    masks = [ii > 0, jj > 0, np.ones(n, dtype=bool), jj < g - 1, ii < g - 1]
    offs = [-g, -1, 0, 1, g]
    vals = [-1.0, -1.0, 4.0, -1.0, -1.0]
    lens = sum(m.astype(np.int64) for m in masks)
    pos = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(lens, out=pos[1:])
    crd = np.empty(int(pos[-1]), dtype=idx_dtype)
    val = np.empty(int(pos[-1]), dtype=np.float64)
    slot = pos[:-1].copy()
    rows = np.arange(n, dtype=np.int64)
    for m, o, v in zip(masks, offs, vals):
        dst = slot[m]
        crd[dst] = (rows[m] + o).astype(idx_dtype)
        val[dst] = v
        slot[m] += 1
    return pos.astype(idx_dtype), crd, val


def pcg_laplacian(grid: int = 4096, idx_dtype=np.int32, seed=None):
    """Config 5: the Laplacian above, b uniform in [0, 1), Jacobi preconditioner dinv = 1/4."""
    rng = _rng(5, seed)
    pos, crd, val = laplacian_2d(grid, idx_dtype)
    n = grid * grid
    return {"pos": pos, "crd": crd, "val": val, "b": rng.uniform(0.0, 1.0, n), "dinv": np.full(n, 0.25),
            "shape": (n, n)}


# ---- algorithmic traffic (the roofline numerators) ------------------------------------
def spmv_bytes(nrows: int, ncols: int, nnz: int, idx_bytes: int) -> int:
    """benchmarks/plots/plotSPMV.py:20 generalised to the index width: every stored entry and
    offset once, x read once, y written once."""
    return nnz * (8 + idx_bytes) + (nrows + 1) * idx_bytes + 8 * ncols + 8 * nrows


def spmm_bytes(nrows: int, ncols: int, nnz: int, k: int, idx_bytes: int) -> int:
    return nnz * (8 + idx_bytes) + (nrows + 1) * idx_bytes + 8 * ncols * k + 8 * nrows * k


def gemm_bytes(batch: int, M: int, N: int, K: int) -> int:
    return 4 * batch * (M * K + K * N + M * N)


def gemm_flops(batch: int, M: int, N: int, K: int) -> int:
    return 2 * batch * M * N * K


def pcg_bytes_per_iteration(n: int, nnz: int, idx_bytes: int) -> int:
    """Matrix once, plus the vector traffic of the three passes: A {p, Ap} 16n,
    B {x, p, r, Ap, dinv read; x, r, z written} 64n, C {z, p read; p written} 24n."""
    return nnz * (8 + idx_bytes) + (n + 1) * idx_bytes + 104 * n
