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


@pytest.mark.parametrize("fused", [True, False], ids=["fused", "separate_kernels"])
def test_a_wait_on_a_peer_that_never_delivers_runs_out(fused):
    """Failure detection of the row-partitioned solver, made on purpose without faulting anything: one rank
    with the peer-to-peer transport switched on (it is its own only peer) is told to expect a halo piece from
    a source that nobody provides.  The wait in front of the SpMV pass is bounded; with the bound lowered to
    about a thousand polls it runs out at once, the kernel writes its mark into the mailbox, sets the solver's
    done flag and returns, every later kernel of the iteration returns at its entry, and ``solve`` raises.
    The CUDA context stays usable.  (The emitted code would abort the process: LAPISSupport.hpp:76-89.)"""
    assert torch.cuda.is_available(), "needs a CUDA device"
    from lapis_b200 import workloads as w
    from lapis_b200._lib import check
    from lapis_b200.dist import DistPcg
    dev = torch.device("cuda:0")
    p = w.pcg_laplacian(48)
    m = p["shape"][0]
    lib = load()
    check(lib.lapis_b200_pcg_p2p_set_wait_limit(1 << 10))
    try:
        solver = DistPcg(p["pos"], p["crd"], p["val"], (m, m), p["b"], p["dinv"], dev, use_graph=False, comm="p2p",
                         transport_on_one_rank=True, fused=fused)
        assert solver.comm == "p2p" and solver._nsrc == 0
        # sanity: with nothing to wait for, the same solver runs
        _, iters, _ = solver.solve(0.0, 5, check_every=5)
        assert iters == 5 and solver.comm_error() == 0.0
        # now expect a halo piece from rank 0 (itself) that no pass ever stores
        solver._srcs = torch.tensor([0], dtype=torch.int32, device=dev)
        if fused:
            solver._nsrc_fused = 1   # the wait at the head of the fused SpMV pass
        else:
            solver._nsrc = 1         # the wait kernel in front of the SpMV pass
        solver._exchange_struct = None
        with pytest.raises(RuntimeError, match="did not deliver in time"):
            solver.solve(0.0, 5, check_every=5)
        assert solver.comm_error() == 9.0          # the halo wait's mark
        assert int(solver.flags[0].item()) == 1    # the done flag stopped the iteration
        assert int(solver.flags[1].item()) == 0    # no iteration completed
    finally:
        check(lib.lapis_b200_pcg_p2p_set_wait_limit(0))
    # the context is intact: an ordinary solve on the same device still works
    from lapis_b200.device import CsrMatrix
    A = CsrMatrix.from_host(p["pos"], p["crd"], p["val"], (m, m), dev)
    x, iters, relres = A.pcg(torch.as_tensor(p["b"]).to(dev), torch.as_tensor(p["dinv"]).to(dev), 0.0, 10)
    assert iters == 10 and np.isfinite(relres)
