"""Device-resident layer: the ``lapis_b200_*`` entry points over torch CUDA tensors.

torch is used for device memory and streams only; every operation below is one
call into ``liblapis_b200.so`` on torch's current stream.  This is the layer a
caller uses who keeps operands on the GPU between calls, as the C++ drivers of
the reference do with ``LAPIS::DualView`` (benchmarks/spmv/main.cpp:42-62).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ._lib import c_dbl, c_int, c_u64, c_vp, check, load


def _stream():
    return c_vp(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return c_vp(0 if t is None or t.numel() == 0 else t.data_ptr())


def _f64(t, name):
    if not (t.is_cuda and t.dtype == torch.float64 and t.is_contiguous()):
        raise TypeError(f"{name} must be a contiguous float64 CUDA tensor")
    return t


class CsrMatrix:
    """CSR matrix on the device with its streaming plan (``lapis_b200_csr_t``).

    ``pos``/``crd`` are int32 or int64 CUDA tensors, ``val`` float64; they are
    borrowed (kept referenced here) and must not be modified while in use.
    ``pos`` may be a slice of a larger offsets array (non-zero ``pos[0]``).
    """

    def __init__(self, pos: torch.Tensor, crd: torch.Tensor, val: torch.Tensor, shape, tune: bool = False):
        if pos.dtype != crd.dtype or pos.dtype not in (torch.int32, torch.int64):
            raise TypeError("pos/crd must both be int32 or both int64")
        for t in (pos, crd, val):
            if not (t.is_cuda and t.is_contiguous()):
                raise TypeError("pos/crd/val must be contiguous CUDA tensors")
        if val.dtype != torch.float64:
            raise TypeError("val must be float64")
        self.pos, self.crd, self.val = pos, crd, val
        self.nrows, self.ncols = int(shape[0]), int(shape[1])
        if pos.numel() != self.nrows + 1:
            raise ValueError("pos must have rows+1 entries")
        self._lib = load()
        h = c_vp()
        with torch.cuda.device(pos.device):
            check(self._lib.lapis_b200_csr_create(ctypes.byref(h), c_int(pos.element_size()), self.nrows, self.ncols,
                                                  _ptr(pos), _ptr(crd), _ptr(val), _stream()))
        self._h = h
        self.nnz = int(self._lib.lapis_b200_csr_nnz(h))
        if tune:
            self.tune()

    def tune(self, relaxed: bool = False):
        """Times the SpMV kernel candidates on this matrix and keeps the fastest; returns
        (threads, blocks_per_sm) of the winner (negative threads: the persistent kernel).
        ``relaxed=True`` adds the segmented-scan kernel (threads == 2 or 3), whose row sums agree with the
        others to 1e-12 of the row's magnitude but not bit for bit."""
        fn = self._lib.lapis_b200_csr_tune_relaxed if relaxed else self._lib.lapis_b200_csr_tune
        with torch.cuda.device(self.pos.device):
            check(fn(self._h, _stream()))
        t, b = c_int(0), c_int(0)
        self._lib.lapis_b200_csr_tuned_kernel(self._h, ctypes.byref(t), ctypes.byref(b))
        return int(t.value), int(b.value)

    def tuned_kernel(self):
        """(threads, blocks_per_sm) stored by the last :meth:`tune` ((0, 0): never tuned)."""
        t, b = c_int(0), c_int(0)
        self._lib.lapis_b200_csr_tuned_kernel(self._h, ctypes.byref(t), ctypes.byref(b))
        return int(t.value), int(b.value)

    @classmethod
    def from_host(cls, pos, crd, val, shape, device="cuda", tune: bool = False):
        return cls(torch.as_tensor(np.ascontiguousarray(pos)).to(device), torch.as_tensor(np.ascontiguousarray(crd)).to(device),
                   torch.as_tensor(np.ascontiguousarray(val, dtype=np.float64)).to(device), shape, tune=tune)

    @property
    def handle(self):
        return self._h

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.lapis_b200_csr_destroy(h)
            self._h = None

    def spmv(self, x: torch.Tensor, y: torch.Tensor, accumulate: bool = True) -> torch.Tensor:
        """y = (y if accumulate else 0) + A x, in place."""
        _f64(x, "x"), _f64(y, "y")
        if x.numel() != self.ncols or y.numel() != self.nrows:
            raise ValueError("spmv: x/y length mismatch")
        check(self._lib.lapis_b200_spmv_f64(self._h, _ptr(x), _ptr(y), c_int(1 if accumulate else 0), _stream()))
        return y

    def spmm(self, B: torch.Tensor, C: torch.Tensor, accumulate: bool = True) -> torch.Tensor:
        """C = (C if accumulate else 0) + A B, in place; B [ncols, k], C [nrows, k] row-major."""
        _f64(B, "B"), _f64(C, "C")
        if B.shape[0] != self.ncols or C.shape[0] != self.nrows or B.shape[1] != C.shape[1]:
            raise ValueError("spmm: B/C shape mismatch")
        check(self._lib.lapis_b200_spmm_f64(self._h, int(B.shape[1]), _ptr(B), _ptr(C), c_int(1 if accumulate else 0),
                                            _stream()))
        return C

    def pcg(self, b: torch.Tensor, dinv: torch.Tensor, tol: float, maxiter: int):
        """Returns (x, iters, relres); blocks until the solve has finished."""
        _f64(b, "b"), _f64(dinv, "dinv")
        x = torch.empty_like(b)
        iters, relres = c_u64(0), c_dbl(0.0)
        check(self._lib.lapis_b200_pcg_f64(self._h, _ptr(b), _ptr(dinv), c_dbl(tol), c_u64(maxiter), _ptr(x),
                                           ctypes.byref(iters), ctypes.byref(relres), _stream()))
        return x, int(iters.value), float(relres.value)

    def mht(self, mask: torch.Tensor, d: torch.Tensor, alpha: float, tol: float, maxiter: int, info: bool = False):
        """First two hitting-time moments (examples/hitting_times.py:151-194 in the LAPIS project): two PCG
        solves with mask*(d - alpha*A)*mask.  Returns (mom1, mom2), plus ((iters1, iters2), (relres1, relres2))
        with ``info``; blocks until finished.  The matrix values are not modified."""
        _f64(mask, "mask"), _f64(d, "d")
        if mask.numel() != self.nrows or d.numel() != self.nrows:
            raise ValueError("mht: mask/d length mismatch")
        m1, m2 = torch.empty_like(d), torch.empty_like(d)
        iters, relres = (c_u64 * 2)(), (c_dbl * 2)()
        check(self._lib.lapis_b200_mht_f64(self._h, _ptr(mask), _ptr(d), c_dbl(alpha), c_dbl(tol), c_u64(maxiter),
                                           _ptr(m1), _ptr(m2), iters, relres, _stream()))
        if info:
            return m1, m2, (int(iters[0]), int(iters[1])), (float(relres[0]), float(relres[1]))
        return m1, m2


def bspmm_csrv(pos: torch.Tensor, crd: torch.Tensor, val: torch.Tensor, B: torch.Tensor, n2: int, C=None) -> torch.Tensor:
    """Batched SpMM over a CSRV tensor (examples/bspmm.py:14-52 in the LAPIS project), fp32:
    C[n1, dh, nh] (+)= sum_j val[j, nh] * B[crd[j], dh, nh] over the stored entries j of row n1.  ``val`` holds
    nh values per stored entry.  With ``C`` given the product is added to it in place; otherwise a new
    zero-initialised result is returned."""
    if pos.dtype != crd.dtype or pos.dtype not in (torch.int32, torch.int64):
        raise TypeError("pos/crd must both be int32 or both int64")
    for t in (val, B):
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
            raise TypeError("val/B must be contiguous float32 CUDA tensors")
    if B.dim() != 3 or B.shape[0] != n2:
        raise ValueError("bspmm: B must be [n2, dh, nh]")
    n1, dh, nh = pos.numel() - 1, int(B.shape[1]), int(B.shape[2])
    if val.numel() != crd.numel() * nh:
        raise ValueError("bspmm: val must hold nh values per stored entry")
    accumulate = C is not None
    if C is None:
        C = torch.empty((n1, dh, nh), dtype=torch.float32, device=B.device)
    elif tuple(C.shape) != (n1, dh, nh) or C.dtype != torch.float32 or not C.is_contiguous():
        raise ValueError("bspmm: C must be a contiguous float32 [n1, dh, nh] tensor")
    check(load().lapis_b200_bspmm_csrv_f32(c_int(pos.element_size()), n1, n2, nh, dh, _ptr(pos), _ptr(crd), _ptr(val),
                                           _ptr(B), _ptr(C), c_int(1 if accumulate else 0), _stream()))
    return C


def spmm_dcsr(i1: torch.Tensor, p2: torch.Tensor, i2: torch.Tensor, val: torch.Tensor, B: torch.Tensor, C: torch.Tensor,
              ncols: int) -> torch.Tensor:
    """C[i1[r], :] += sum_j val[j] * B[i2[j], :] for the stored rows r of a DCSR matrix
    (examples/spmm_dcsr_opdsl.py:59-101 in the LAPIS project), in place; ``i1`` must ascend (a row number may repeat)."""
    if not (i1.dtype == p2.dtype == i2.dtype) or p2.dtype not in (torch.int32, torch.int64):
        raise TypeError("i1/p2/i2 must all be int32 or all int64")
    _f64(val, "val"), _f64(B, "B"), _f64(C, "C")
    if B.dim() != 2 or C.dim() != 2 or B.shape[0] != ncols or B.shape[1] != C.shape[1] or p2.numel() != i1.numel() + 1:
        raise ValueError("spmm_dcsr: shape mismatch")
    check(load().lapis_b200_spmm_dcsr_f64(c_int(p2.element_size()), int(C.shape[0]), ncols, i1.numel(), int(B.shape[1]),
                                          _ptr(i1), _ptr(p2), _ptr(i2), _ptr(val), _ptr(B), _ptr(C), _stream()))
    return C


def normalize_mom2(mom1: torch.Tensor, mom2: torch.Tensor) -> torch.Tensor:
    """sqrt(mom2 - mom1^2) elementwise (examples/hitting_times.py:196-218 in the LAPIS project)."""
    _f64(mom1, "mom1"), _f64(mom2, "mom2")
    if mom1.numel() != mom2.numel():
        raise ValueError("normalize_mom2: lengths differ")
    out = torch.empty_like(mom1)
    check(load().lapis_b200_normalize_mom2_f64(mom1.numel(), _ptr(mom1), _ptr(mom2), _ptr(out), _stream()))
    return out


def bgemm(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> torch.Tensor:
    """C = C + A @ B in place; fp32, [M,K]x[K,N] or batched [b,M,K]x[b,K,N]."""
    for t in (A, B, C):
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
            raise TypeError("bgemm operands must be contiguous float32 CUDA tensors")
    if A.dim() == 2:
        batch, (M, K), (K2, N) = 1, A.shape, B.shape
    else:
        batch, M, K = A.shape
        b2, K2, N = B.shape
        if b2 != batch:
            raise ValueError("mismatching contracting dimension")
    if K != K2:
        raise ValueError("mismatching contracting dimension")
    if tuple(C.shape) != (tuple(A.shape[:-1]) + (N,)):
        raise ValueError("bgemm: output shape mismatch")
    check(load().lapis_b200_bgemm_f32(batch, M, N, K, _ptr(A), _ptr(B), _ptr(C), _stream()))
    return C


def bgemm_status() -> None:
    """Synchronises and raises if the tensor-core matmul kernel reported a failed wait."""
    check(load().lapis_b200_bgemm_status(_stream()))


def dot(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    _f64(x, "x"), _f64(y, "y")
    out = torch.empty(1, dtype=torch.float64, device=x.device)
    check(load().lapis_b200_dot_f64(x.numel(), _ptr(x), _ptr(y), _ptr(out), _stream()))
    return out


def axpby(a: float, x: torch.Tensor, b: float, y: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    _f64(x, "x"), _f64(y, "y"), _f64(dst, "dst")
    check(load().lapis_b200_axpby_f64(x.numel(), c_dbl(a), _ptr(x), c_dbl(b), _ptr(y), _ptr(dst), _stream()))
    return dst


def mult(x: torch.Tensor, y: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    _f64(x, "x"), _f64(y, "y"), _f64(dst, "dst")
    check(load().lapis_b200_mult_f64(x.numel(), _ptr(x), _ptr(y), _ptr(dst), _stream()))
    return dst
