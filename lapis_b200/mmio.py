"""MatrixMarket files as CSR arrays, read by the C library (``lapis_b200_read_matrix_market``)."""
from __future__ import annotations

import ctypes
import os

import numpy as np

from ._lib import c_i64, c_vp, check, load


def read_matrix_market(path, idx_dtype=np.int32):
    """Returns (pos, crd, val, (nrows, ncols)): ascending columns per row, duplicates summed,
    symmetric storage expanded -- what ``csr_matrix(mmread(path))`` with sorted indices gives."""
    idx_dtype = np.dtype(idx_dtype)
    if idx_dtype not in (np.dtype(np.int32), np.dtype(np.int64)):
        raise TypeError("idx_dtype must be int32 or int64")
    lib = load()
    m, n, nnz = c_i64(), c_i64(), c_i64()
    pos, crd, val = c_vp(), c_vp(), c_vp()
    check(lib.lapis_b200_read_matrix_market(os.fsencode(path), idx_dtype.itemsize, ctypes.byref(m), ctypes.byref(n),
                                            ctypes.byref(nnz), ctypes.byref(pos), ctypes.byref(crd), ctypes.byref(val)))
    try:
        def take(ptr, count, dtype):
            if count == 0:
                return np.empty(0, dtype=dtype)
            buf = (ctypes.c_char * (count * np.dtype(dtype).itemsize)).from_address(ptr.value)
            return np.frombuffer(buf, dtype=dtype).copy()
        return (take(pos, m.value + 1, idx_dtype), take(crd, nnz.value, idx_dtype), take(val, nnz.value, np.float64),
                (int(m.value), int(n.value)))
    finally:
        for p in (pos, crd, val):
            lib.lapis_b200_mm_free(p)
