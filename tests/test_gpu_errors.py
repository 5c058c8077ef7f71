"""Error behaviour of the emitted-module ABI on a GPU box.  The emitted code aborts the process
(Kokkos::abort from stridedMemrefToView, cf.assert); here the same conditions are reported as a status
that the Python surface raises, and the caller's output buffers are left untouched."""
import ctypes

import numpy as np
import pytest
import torch

from lapis_b200 import KokkosBackend as KB
from lapis_b200 import _memref
from lapis_b200._lib import LapisError, load
from tests import mlir_modules as mm

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def module():
    assert torch.cuda.is_available(), "needs a CUDA device"
    return KB.KokkosBackend(decompose_tensors=True).compile(mm.spmv(mm.CSR32))


def _csr():
    pos = np.array([0, 2, 3], dtype=np.int32)
    crd = np.array([0, 1, 1], dtype=np.int32)
    val = np.array([1.0, 2.0, 3.0])
    return pos, crd, val


def test_shape_mismatches_are_reported(module):
    pos, crd, val = _csr()
    y = np.full(2, 7.0)
    with pytest.raises(LapisError) as e:       # x has the wrong length
        module.spmv(pos, crd, val, ((2, 2), (3, 3, 3)), np.ones(3), y)
    assert e.value.status == 1 and np.all(y == 7.0)
    with pytest.raises(LapisError) as e:       # specifier disagrees with pos
        module.spmv(pos, crd, val, ((5, 2), (3, 3, 3)), np.ones(2), y)
    assert e.value.status == 1
    with pytest.raises(LapisError) as e:       # specifier claims more entries than crd/val hold
        module.spmv(pos, crd, val, ((2, 2), (3, 9, 9)), np.ones(2), y)
    assert e.value.status == 1 and np.all(y == 7.0)


def test_malformed_offsets_are_reported(module):
    _, crd, val = _csr()
    y = np.zeros(2)
    for bad in ([0, 3, 2], [1, 2, 3], [0, 1, 2]):   # decreasing; not starting at 0; not ending at nnz
        with pytest.raises(LapisError) as e:
            module.spmv(np.array(bad, dtype=np.int32), crd, val, ((2, 2), (3, 3, 3)), np.ones(2), y)
        assert e.value.status == 1
    assert np.all(y == 0.0)


def test_non_contiguous_descriptor_is_reported():
    """LAPISSupport.hpp:80-89 aborts on a descriptor that is not contiguous row-major."""
    assert torch.cuda.is_available()
    lib = load()
    lib.lapis_initialize()
    try:
        pos, crd, val = _csr()
        x = np.ones(4)[::2]                      # stride 2
        y = np.zeros(2)
        d = lambda a: ctypes.pointer(_memref.get_ranked_memref_descriptor(a))
        spec = np.array([2, 2, 3, 3, 3], dtype=np.int64)
        ret = ctypes.pointer(ctypes.pointer(_memref.make_nd_memref_descriptor(1)()))
        lib.py_spmv_f64_i32(ret, d(pos), d(crd), d(val), spec.ctypes.data_as(ctypes.c_void_p), d(x), d(y))
        assert lib.lapis_last_error() == 2       # LAPIS_ELAYOUT
        assert b"contiguous" in lib.lapis_last_error_message()
        assert np.all(y == 0.0)
        # the same call with a contiguous x succeeds and clears the status
        xc = np.ones(2)
        lib.py_spmv_f64_i32(ret, d(pos), d(crd), d(val), spec.ctypes.data_as(ctypes.c_void_p), d(xc), d(y))
        assert lib.lapis_last_error() == 0 and np.array_equal(y, [3.0, 3.0])
    finally:
        lib.lapis_finalize()


def test_empty_operands(module):
    """Zero rows / zero stored entries are valid inputs (empty and ragged cases of the reference's loops)."""
    y = np.zeros(0)
    out = module.spmv(np.zeros(1, dtype=np.int32), np.zeros(0, dtype=np.int32), np.zeros(0), ((0, 4), (1, 0, 0)),
                      np.ones(4), y)
    assert out.shape == (0,)
    y = np.arange(3.0)
    module.spmv(np.zeros(4, dtype=np.int32), np.zeros(0, dtype=np.int32), np.zeros(0), ((3, 4), (4, 0, 0)),
                np.ones(4), y)
    assert np.array_equal(y, np.arange(3.0))     # y_in + 0


def test_results_of_pcg_stay_valid_until_finalize():
    """A returned memref aliases module-owned memory until lapis_finalize (LAPISSupport.hpp:93-120)."""
    assert torch.cuda.is_available()
    from lapis_b200 import workloads as w
    m = KB.KokkosBackend(decompose_tensors=True).compile(mm.pcg(mm.CSR32))
    d = w.pcg_laplacian(16)
    n = 256
    spec = ((n, n), (n + 1, len(d["crd"]), len(d["val"])))
    x1, it1, _ = m.pcg(d["pos"], d["crd"], d["val"], spec, d["b"], d["dinv"], 0.0, 5)
    keep = x1.copy()
    x2, it2, _ = m.pcg(d["pos"], d["crd"], d["val"], spec, d["b"], d["dinv"], 0.0, 9)
    assert it1 == 5 and it2 == 9
    assert np.array_equal(x1, keep) and not np.array_equal(x1, x2)   # the first result was not overwritten
