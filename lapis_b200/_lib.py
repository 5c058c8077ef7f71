"""Loads ``liblapis_b200.so`` and declares the C ABI of include/lapis_b200.h."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblapis_b200.so")

c_i64 = ctypes.c_int64
c_u64 = ctypes.c_uint64
c_int = ctypes.c_int
c_dbl = ctypes.c_double
c_vp = ctypes.c_void_p
c_sz = ctypes.c_size_t

STATUS_NAMES = {0: "LAPIS_OK", 1: "LAPIS_EBADSHAPE", 2: "LAPIS_ELAYOUT", 3: "LAPIS_ECUDA", 4: "LAPIS_EBADARG",
                5: "LAPIS_ENOTINIT", 6: "LAPIS_ETOOBIG"}


class LapisError(RuntimeError):
    """A call into liblapis_b200.so reported a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


# Layer-2 prototypes: name -> (restype, argtypes).  Layer-1 (py_*) functions take
# pointers only and return void.
_PROTOS = {
    "lapis_last_error": (c_int, []),
    "lapis_last_error_message": (ctypes.c_char_p, []),
    "lapis_initialize": (None, []),
    "lapis_finalize": (None, []),
    "lapis_b200_csr_create": (c_int, [ctypes.POINTER(c_vp), c_int, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "lapis_b200_csr_destroy": (c_int, [c_vp]),
    "lapis_b200_csr_nnz": (c_i64, [c_vp]),
    "lapis_b200_spmv_f64": (c_int, [c_vp, c_vp, c_vp, c_int, c_vp]),
    "lapis_b200_csr_tune": (c_int, [c_vp, c_vp]),
    "lapis_b200_csr_tune_relaxed": (c_int, [c_vp, c_vp]),
    "lapis_b200_csr_tuned_kernel": (c_int, [c_vp, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "lapis_b200_spmv_select_kernel": (c_int, [c_int, c_int, c_int]),
    "lapis_b200_spmv_status": (c_int, [c_vp]),
    "lapis_b200_spmv_f64_noalloc": (c_int, [c_int, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_vp]),
    "lapis_b200_spmm_f64": (c_int, [c_vp, c_i64, c_vp, c_vp, c_int, c_vp]),
    "lapis_b200_bgemm_f32": (c_int, [c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "lapis_b200_bgemm_status": (c_int, [c_vp]),
    "lapis_b200_dot_f64": (c_int, [c_i64, c_vp, c_vp, c_vp, c_vp]),
    "lapis_b200_axpby_f64": (c_int, [c_i64, c_dbl, c_vp, c_dbl, c_vp, c_vp, c_vp]),
    "lapis_b200_mult_f64": (c_int, [c_i64, c_vp, c_vp, c_vp, c_vp]),
    "lapis_b200_pcg_f64": (c_int, [c_vp, c_vp, c_vp, c_dbl, c_u64, c_vp, ctypes.POINTER(c_u64),
                                   ctypes.POINTER(c_dbl), c_vp]),
    "lapis_b200_pcg_workspace_bytes": (c_i64, [c_i64, c_i64]),
    "lapis_b200_pcg_init": (c_int, [c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_int, c_vp]),
    "lapis_b200_pcg_derive": (c_int, [c_vp, c_int, c_dbl, c_u64, c_vp]),
    "lapis_b200_pcg_workspace_layout": (c_int, [c_i64, c_i64, c_vp]),
    "lapis_b200_pcg_step_spmv": (c_int, [c_vp, c_vp, c_i64, c_i64, c_int, c_vp]),
    "lapis_b200_pcg_step_update": (c_int, [c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_int, c_dbl, c_u64, c_vp]),
    "lapis_b200_pcg_step_direction": (c_int, [c_vp, c_i64, c_i64, c_i64, c_vp]),
    "lapis_b200_bspmm_csrv_f32": (c_int, [c_int, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_vp]),
    "lapis_b200_spmm_dcsr_f64": (c_int, [c_int, c_i64, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "lapis_b200_mht_f64": (c_int, [c_vp, c_vp, c_vp, c_dbl, c_dbl, c_u64, c_vp, c_vp, ctypes.POINTER(c_u64),
                                   ctypes.POINTER(c_dbl), c_vp]),
    "lapis_b200_normalize_mom2_f64": (c_int, [c_i64, c_vp, c_vp, c_vp, c_vp]),
    "lapis_b200_pcg_p2p_mailbox_bytes": (c_i64, []),
    "lapis_b200_pcg_p2p_mailbox_layout": (None, [ctypes.POINTER(c_i64), ctypes.POINTER(c_i64)]),
    "lapis_b200_peer_alloc": (c_int, [c_i64, ctypes.POINTER(c_vp), ctypes.c_char_p]),
    "lapis_b200_peer_open": (c_int, [ctypes.c_char_p, ctypes.POINTER(c_vp)]),
    "lapis_b200_peer_close": (c_int, [c_vp]),
    "lapis_b200_peer_free": (c_int, [c_vp]),
    "lapis_b200_pcg_p2p_push_scalars": (c_int, [c_vp, c_int, c_int, c_int, c_vp, c_vp]),
    "lapis_b200_pcg_p2p_wait_reduce": (c_int, [c_vp, c_vp, c_int, c_int, c_int, c_dbl, c_u64, c_vp]),
    "lapis_b200_pcg_p2p_halo_push": (c_int, [c_vp, c_i64, c_i64, c_vp, c_int, c_vp]),
    "lapis_b200_pcg_p2p_halo_wait": (c_int, [c_vp, c_vp, c_vp, c_int, c_vp]),
    "lapis_b200_pcg_fused_spmv": (c_int, [c_vp, c_vp, c_i64, c_i64, c_dbl, c_u64, c_vp, c_vp]),
    "lapis_b200_pcg_fused_update": (c_int, [c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_dbl, c_u64, c_vp, c_vp]),
    "lapis_b200_pcg_fused_direction": (c_int, [c_vp, c_i64, c_i64, c_i64, c_dbl, c_u64, c_vp, c_vp]),
    "lapis_b200_pcg_folds_direction": (c_int, [c_vp]),
    "lapis_b200_pcg_fused_spmv_direction": (c_int, [c_vp, c_vp, c_i64, c_i64, c_dbl, c_u64, c_vp, c_vp]),
    "lapis_b200_pcg_p2p_set_wait_limit": (c_int, [ctypes.c_uint32]),
    "lapis_b200_pcg_status": (c_int, [c_vp, ctypes.POINTER(c_int), ctypes.POINTER(c_u64), ctypes.POINTER(c_dbl), c_vp]),
    "lapis_b200_read_matrix_market": (c_int, [ctypes.c_char_p, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64),
                                              ctypes.POINTER(c_i64), ctypes.POINTER(c_vp), ctypes.POINTER(c_vp),
                                              ctypes.POINTER(c_vp)]),
    "lapis_b200_mm_free": (None, [c_vp]),
    "lapis_b200_partition_rows": (c_int, [c_int, c_i64, c_vp, c_int, c_vp]),
    "lapis_b200_validate_csr_host": (c_int, [c_int, c_i64, c_i64, c_i64, c_vp, c_vp]),
}



class PcgExchange(ctypes.Structure):
    """``lapis_b200_pcg_exchange`` of include/lapis_b200.h."""
    _fields_ = [("me", c_int), ("world", c_int), ("d_mbox", c_vp), ("d_peer_mbox", c_vp), ("d_halo_srcs", c_vp),
                ("nsrc", c_int), ("d_z_pieces", c_vp), ("nzpieces", c_int), ("d_halo_ranges", c_vp), ("nranges", c_int)]


_LIB = None


def load() -> ctypes.CDLL:
    """Returns the library; raises if it has not been built (there is no fallback)."""
    global _LIB
    if _LIB is None:
        if not os.path.isfile(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m lapis_b200._build` "
                "(nvcc, sm_100a). lapis_b200 has no CPU or pure-PyTorch path.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = lib
    return _LIB


def check(status: int) -> None:
    if status != 0:
        raise LapisError(status, (load().lapis_last_error_message() or b"").decode())


def check_last() -> None:
    """For the void layer-1 entry points: raise if the call recorded an error."""
    lib = load()
    status = lib.lapis_last_error()
    if status != 0:
        raise LapisError(status, (lib.lapis_last_error_message() or b"").decode())
