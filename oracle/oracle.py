"""ctypes face of the CPU oracle (``lapis_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the product package never does.  ``build()`` compiles the C file with
the Makefile beside it; ``lib()`` loads the portable build, ``lib(native=True)``
the ``-march=native`` one used for timing.

Parity status of the restatement: pinned against the reference's example known
answers (see the header of ``lapis_oracle.c`` and ``tests/golden``); the
reference's own Kokkos build is not available to run beside it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS: dict = {}

c_i64 = ctypes.c_int64
c_u64 = ctypes.c_uint64
c_dbl = ctypes.c_double
c_int = ctypes.c_int
c_vp = ctypes.c_void_p


def build(native: bool = False) -> str:
    target = "native" if native else "all"
    subprocess.run(["make", "-s", "-C", _HERE, target], check=True)
    return os.path.join(_HERE, "liblapis_oracle_native.so" if native else "liblapis_oracle.so")


def lib(native: bool = False) -> ctypes.CDLL:
    key = bool(native)
    if key not in _LIBS:
        name = "liblapis_oracle_native.so" if native else "liblapis_oracle.so"
        path = os.path.join(_HERE, name)
        if not os.path.isfile(path):
            build(native)
        L = ctypes.CDLL(path)
        L.oracle_dot_f64.restype = c_dbl
        L.oracle_pcg_f64_i32.restype = c_u64
        L.oracle_pcg_f64_i64.restype = c_u64
        L.oracle_max_threads.restype = c_int
        _LIBS[key] = L
    return _LIBS[key]


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def _p(a):
    return None if a is None else a.ctypes.data_as(c_vp)


def _f64(a):
    return np.require(a, dtype=np.float64, requirements=["C", "A"])


def _f32(a):
    return np.require(a, dtype=np.float32, requirements=["C", "A"])


def _idx(pos, crd):
    """Index arrays keep their width (int32 or int64); anything else is an error."""
    if pos.dtype != crd.dtype or pos.dtype not in (np.int32, np.int64):
        raise TypeError("pos/crd must both be int32 or both int64")
    suffix = "i32" if pos.dtype == np.int32 else "i64"
    return suffix, np.ascontiguousarray(pos), np.ascontiguousarray(crd)


def spmv(pos, crd, val, x, y_in, nthreads: int = 1, native: bool = False):
    """y = y_in + A x (returns a new array)."""
    s, pos, crd = _idx(pos, crd)
    val, x = _f64(val), _f64(x)
    y = np.array(y_in, dtype=np.float64, copy=True)
    fn = getattr(lib(native), f"oracle_spmv_f64_{s}")
    fn(c_i64(len(pos) - 1), _p(pos), _p(crd), _p(val), _p(x), _p(y), c_int(nthreads))
    return y


def spmv_inplace(pos, crd, val, x, y, nthreads: int = 1, native: bool = False):
    s, pos, crd = _idx(pos, crd)
    fn = getattr(lib(native), f"oracle_spmv_f64_{s}")
    fn(c_i64(len(pos) - 1), _p(pos), _p(crd), _p(val), _p(x), _p(y), c_int(nthreads))


def spmm(pos, crd, val, B, C_in, nthreads: int = 1, native: bool = False):
    s, pos, crd = _idx(pos, crd)
    val, B = _f64(val), _f64(B)
    C = np.array(C_in, dtype=np.float64, copy=True, order="C")
    fn = getattr(lib(native), f"oracle_spmm_f64_{s}")
    fn(c_i64(len(pos) - 1), c_i64(B.shape[1]), _p(pos), _p(crd), _p(val), _p(B), _p(C),
       c_int(nthreads))
    return C


def spmm_inplace(pos, crd, val, B, C, nthreads: int = 1, native: bool = False):
    s, pos, crd = _idx(pos, crd)
    fn = getattr(lib(native), f"oracle_spmm_f64_{s}")
    fn(c_i64(len(pos) - 1), c_i64(B.shape[1]), _p(pos), _p(crd), _p(val), _p(B), _p(C),
       c_int(nthreads))


def bgemm(A, B, C_in, nthreads: int = 1, native: bool = False):
    """C = C_in + A @ B in fp32, sequential-k order; A [b,M,K] or [M,K]."""
    A, B = _f32(A), _f32(B)
    C = np.array(C_in, dtype=np.float32, copy=True, order="C")
    if A.ndim == 2:
        batch, (M, K), N = 1, A.shape, B.shape[1]
    else:
        batch, M, K = A.shape
        N = B.shape[2]
    lib(native).oracle_bgemm_f32(c_i64(batch), c_i64(M), c_i64(N), c_i64(K), _p(A), _p(B), _p(C),
                                 c_int(nthreads))
    return C


gemm = bgemm


def bgemm_acc64(A, B, C_in, nthreads: int = 1):
    """Same product accumulated in double: the accuracy yardstick."""
    A, B, C_in = _f32(A), _f32(B), _f32(C_in)
    if A.ndim == 2:
        batch, (M, K), N = 1, A.shape, B.shape[1]
    else:
        batch, M, K = A.shape
        N = B.shape[2]
    out = np.empty(C_in.shape, dtype=np.float64)
    lib().oracle_bgemm_f32_acc64(c_i64(batch), c_i64(M), c_i64(N), c_i64(K), _p(A), _p(B),
                                 _p(C_in), _p(out), c_int(nthreads))
    return out


def dot(x, y, nthreads: int = 1):
    x, y = _f64(x), _f64(y)
    return float(lib().oracle_dot_f64(c_i64(len(x)), _p(x), _p(y), c_int(nthreads)))


def axpby(a, x, b, y, nthreads: int = 1):
    x, y = _f64(x), _f64(y)
    dst = np.empty_like(x)
    lib().oracle_axpby_f64(c_i64(len(x)), c_dbl(a), _p(x), c_dbl(b), _p(y), _p(dst), c_int(nthreads))
    return dst


def mult(x, y, nthreads: int = 1):
    x, y = _f64(x), _f64(y)
    dst = np.empty_like(x)
    lib().oracle_mult_f64(c_i64(len(x)), _p(x), _p(y), _p(dst), c_int(nthreads))
    return dst


def pcg(pos, crd, val, b, dinv, tol, maxiter, nthreads: int = 1, trace: bool = False,
        native: bool = False):
    """Returns (x, iters, relres) and, with trace=True, a dict of per-iteration scalars."""
    s, pos, crd = _idx(pos, crd)
    val, b, dinv = _f64(val), _f64(b), _f64(dinv)
    n = len(b)
    x = np.empty(n, dtype=np.float64)
    work = np.empty(4 * n, dtype=np.float64)
    relres = c_dbl(0.0)
    tr = {k: (np.full(maxiter, np.nan) if trace else None) for k in ("alpha", "beta", "relres")}
    fn = getattr(lib(native), f"oracle_pcg_f64_{s}")
    iters = fn(c_i64(n), _p(pos), _p(crd), _p(val), _p(b), _p(dinv), c_dbl(tol), c_u64(maxiter),
               _p(x), ctypes.byref(relres), _p(work), _p(tr["alpha"]), _p(tr["beta"]),
               _p(tr["relres"]), c_int(nthreads))
    if trace:
        return x, int(iters), float(relres.value), tr
    return x, int(iters), float(relres.value)


def mht(pos, crd, val, mask, d, alpha, tol, maxiter):
    """Hitting-time moments (mom1, normalised mom2); pins the PCG loop."""
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    crd = np.ascontiguousarray(crd, dtype=np.int32)
    val = np.array(val, dtype=np.float64, copy=True)
    mask, d = _f64(mask), _f64(d)
    n = len(d)
    mom1 = np.empty(n)
    mom2 = np.empty(n)
    work = np.empty(7 * n)
    lib().oracle_mht_f64_i32(c_i64(n), _p(pos), _p(crd), _p(val), _p(mask), _p(d), c_dbl(alpha),
                             c_dbl(tol), c_u64(maxiter), _p(mom1), _p(mom2), _p(work))
    return mom1, mom2


def bspmm(pos, crd, val, B, C_in=None):
    """Batched SpMM over a CSRV tensor (examples/bspmm.py:14-52), fp32: val [nnz*nh], B [n2, dh, nh]."""
    pos = np.ascontiguousarray(pos)
    crd = np.ascontiguousarray(crd, dtype=pos.dtype)
    s = "i32" if pos.dtype == np.int32 else "i64"
    val = np.ascontiguousarray(val, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    n1, (n2, dh, nh) = len(pos) - 1, B.shape
    C = np.zeros((n1, dh, nh), dtype=np.float32) if C_in is None else np.array(C_in, dtype=np.float32, copy=True, order="C")
    getattr(lib(), f"oracle_bspmm_f32_{s}")(c_i64(n1), c_i64(nh), c_i64(dh), _p(pos), _p(crd), _p(val), _p(B), _p(C))
    return C


def spmm_dcsr(i1, p2, i2, val, B, C_in):
    """C_in + A B with A in DCSR (examples/spmm_dcsr_opdsl.py:59-101), fp64."""
    p2 = np.ascontiguousarray(p2)
    i1 = np.ascontiguousarray(i1, dtype=p2.dtype)
    i2 = np.ascontiguousarray(i2, dtype=p2.dtype)
    s = "i32" if p2.dtype == np.int32 else "i64"
    val, B = _f64(val), _f64(B)
    C = np.array(C_in, dtype=np.float64, copy=True, order="C")
    getattr(lib(), f"oracle_spmm_dcsr_f64_{s}")(c_i64(len(i1)), c_i64(B.shape[1]), _p(i1), _p(p2), _p(i2), _p(val), _p(B), _p(C))
    return C


def partition_rows(pos, G: int):
    pos = np.ascontiguousarray(pos)
    s = "i32" if pos.dtype == np.int32 else "i64"
    bounds = np.empty(G + 1, dtype=np.int64)
    getattr(lib(), f"oracle_partition_rows_{s}")(c_i64(len(pos) - 1), _p(pos), c_int(G), _p(bounds))
    return bounds


# ---------------------------------------------------------------------------
# Pure-numpy second opinions (small cases only).
# ---------------------------------------------------------------------------
def spmv_numpy(pos, crd, val, x, y_in):
    y = np.array(y_in, dtype=np.float64, copy=True)
    for r in range(len(pos) - 1):
        acc = 0.0
        for j in range(int(pos[r]), int(pos[r + 1])):
            acc = acc + float(val[j]) * float(x[int(crd[j])])
        y[r] = acc + y[r]
    return y


def partition_rows_numpy(pos, G: int):
    pos = np.asarray(pos).astype(np.int64)
    n = len(pos) - 1
    base, nnz = int(pos[0]), int(pos[n] - pos[0])
    out = [int(np.searchsorted(pos[:n], base + (nnz * g) // G, side="left")) for g in range(G)]
    return np.array(out + [n], dtype=np.int64)
