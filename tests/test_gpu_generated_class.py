"""A module class in the form the LAPIS emitter generates binds to the library that ``compile()`` returns,
without an edit (needs a B200).

The emitter prints, per module, a Python class whose constructor loads the module's shared library and
calls ``lapis_initialize`` and whose methods marshal numpy arrays into memref descriptors and call
``self.libHandle.py_<func>`` (mlir/lib/Target/KokkosCpp/TranslateToKokkosCpp.cpp:4393-4411, :2757-2977).
``GeneratedModule`` below is such a class written out by hand from those rules (its ``rt`` helpers are the
ctypes restatement of ``mlir.runtime`` in lapis_b200/_memref.py).  It is pointed at
``module.libPath`` -- the per-module library with the emitter's export names -- and must give the oracle's y.
"""
import ctypes

import numpy
import numpy as np
import pytest
import torch

from lapis_b200 import KokkosBackend as KB
from lapis_b200 import _memref as rt
from lapis_b200 import modules as mm
from oracle import oracle

pytestmark = pytest.mark.gpu


class GeneratedModule:
    def __init__(self, libPath):
        self.libHandle = ctypes.CDLL(libPath)
        self.libHandle.lapis_initialize()

    def __del__(self):
        self.libHandle.lapis_finalize()

    def spmv(self, param0, param1, param2, param3, param4, param5):
        param0 = numpy.require(param0, dtype=numpy.int32, requirements=['C'])
        param1 = numpy.require(param1, dtype=numpy.int32, requirements=['C'])
        param2 = numpy.require(param2, dtype=numpy.double, requirements=['C'])
        param_flat3 = numpy.zeros(5, dtype=numpy.int64)
        for i in range(2):
            param_flat3[0 + i] = param3[0][i]
        for i in range(3):
            param_flat3[2 + i] = param3[1][i]
        param3 = param_flat3
        param4 = numpy.require(param4, dtype=numpy.double, requirements=['C'])
        param5 = numpy.require(param5, dtype=numpy.double, requirements=['C'])
        ret0 = ctypes.pointer(ctypes.pointer(rt.make_nd_memref_descriptor(1, ctypes.c_double)()))
        self.libHandle.py_spmv(ret0, ctypes.pointer(rt.get_ranked_memref_descriptor(param0)),
                               ctypes.pointer(rt.get_ranked_memref_descriptor(param1)),
                               ctypes.pointer(rt.get_ranked_memref_descriptor(param2)),
                               param3.ctypes.data_as(ctypes.c_void_p),
                               ctypes.pointer(rt.get_ranked_memref_descriptor(param4)),
                               ctypes.pointer(rt.get_ranked_memref_descriptor(param5)))
        return (rt.ranked_memref_to_numpy(ret0[0]))


def test_generated_class_binds_to_the_compiled_module_library(golden_dir):
    assert torch.cuda.is_available(), "needs a CUDA device"
    import os
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmv(mm.CSR32))
    assert os.path.isfile(module.libPath)
    gen = GeneratedModule(module.libPath)
    # examples/spmv_noalloc.py:16-37 in the LAPIS project
    g = np.load(os.path.join(golden_dir, "spmv_noalloc.npz"))
    y = np.zeros(5)
    out = gen.spmv(g["rowptrs"], g["colinds"], g["values"], ((5, 5), (6, 8, 8)), np.ones(5), y)
    assert gen.libHandle.lapis_last_error() == 0
    assert np.array_equal(out, oracle.spmv(g["rowptrs"], g["colinds"], g["values"], np.ones(5), np.zeros(5)))
    assert np.allclose(y, g["ycorrect"])
    # a larger random case through the same unchanged class
    rng = np.random.default_rng(4)
    n = 3000
    lens = rng.integers(0, 40, n)
    pos = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    crd = rng.integers(0, n, int(pos[-1])).astype(np.int32)
    val = rng.uniform(-1, 1, int(pos[-1]))
    x, y0 = rng.uniform(-1, 1, n), rng.uniform(-1, 1, n)
    y = y0.copy()
    gen.spmv(pos, crd, val, ((n, n), (n + 1, len(crd), len(val))), x, y)
    ref = oracle.spmv(pos, crd, val, x, y0)
    scale = oracle.spmv(pos, crd, np.abs(val) * np.abs(x[crd]), np.ones(n), np.abs(y0))
    assert np.all(np.abs(y - ref) <= 1e-12 * np.maximum(scale, 1e-300))
    # a bad column index is refused on the host, before any kernel sees it; the generated class reads the status
    bad = crd.copy()
    bad[17] = n
    gen.spmv(pos, bad, val, ((n, n), (n + 1, len(crd), len(val))), x, y)
    assert gen.libHandle.lapis_last_error() == 1  # LAPIS_EBADSHAPE
    del gen
