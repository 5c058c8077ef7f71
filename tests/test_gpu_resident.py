"""Resident operands (DualView arguments) through the compiled module: same results as the per-call
upload path, and no bytes moved for operands whose host side did not change."""
import numpy as np
import pytest
import torch

from lapis_b200 import KokkosBackend as KB
from lapis_b200 import workloads as w
from lapis_b200.dualview import DualView
from oracle import oracle
from tests import mlir_modules as mm

pytestmark = pytest.mark.gpu


def _spec(d):
    n, m = d["shape"]
    return ((n, m), (n + 1, len(d["crd"]), len(d["val"])))


def test_spmv_resident_matches_upload_path_and_skips_copies():
    d = w.spmv_power_law(1 << 14)
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmv(mm.CSR64))
    n = d["shape"][0]
    pos, crd, val, x = (DualView(a) for a in (d["pos"], d["crd"], d["val"], d["x"]))
    y = DualView(np.zeros(n))
    out = module.spmv(pos, crd, val, _spec(d), x, y)
    assert out is y and y.modifiedDevice()
    out = module.spmv(pos, crd, val, _spec(d), x, y)          # y += A x once more, nothing re-uploaded
    assert [v.uploads for v in (pos, crd, val, x, y)] == [1, 1, 1, 1, 1] and y.downloads == 0
    assert len(module._plans) == 1
    y_host = np.zeros(n)
    for _ in range(2):
        module.spmv(d["pos"], d["crd"], d["val"], _spec(d), d["x"], y_host)
    assert np.array_equal(y.numpy(), y_host) and y.downloads == 1      # same kernels: same bits
    # a host-side change is seen only after modifyHost()
    x.host_view()[:] *= 2.0
    x.modifyHost()
    y2 = DualView(np.zeros(n))
    module.spmv(pos, crd, val, _spec(d), x, y2)
    assert x.uploads == 2 and pos.uploads == 1
    ref = oracle.spmv(d["pos"], d["crd"], d["val"], x.host_view(), np.zeros(n))
    scale = oracle.spmv(d["pos"], d["crd"], np.abs(d["val"]), np.abs(x.host_view()), np.zeros(n))
    assert np.all(np.abs(y2.numpy() - ref) <= 1e-12 * np.maximum(scale, 1e-300))
    # sync_host=True: the result arrives on the host with the call, block by block behind the kernel
    y4 = DualView(np.ones(n))
    out = module.spmv(pos, crd, val, _spec(d), x, y4, sync_host=True)
    assert out is y4 and not y4.modifiedDevice() and not y4.modifiedHost() and y4.downloads == 1
    ref4 = oracle.spmv(d["pos"], d["crd"], d["val"], x.host_view(), np.ones(n))
    assert np.all(np.abs(y4.host_view() - ref4) <= 1e-12 * np.maximum(scale + 1.0, 1e-300))
    assert torch.equal(y4.device_view().cpu(), torch.from_numpy(y4.host_view())) and y4.uploads == 1
    module.spmv(pos, crd, val, _spec(d), x, y4, sync_host=True)          # accumulates on the resident copy
    assert np.all(np.abs(y4.host_view() - (2 * ref4 - 1.0)) <= 4e-12 * np.maximum(scale + 1.0, 1e-300))
    # changing the matrix values rebuilds the plan
    val.host_view()[:] *= -1.0
    val.modifyHost()
    y3 = DualView(np.zeros(n))
    module.spmv(pos, crd, val, _spec(d), x, y3)
    assert np.array_equal(y3.numpy(), -y2.numpy()) and val.uploads == 2


def test_spmv_pipelined_upload_matches_oracle():
    """x large enough for the two-piece upload: the left column half of the matrix runs while the second
    piece of x is still being copied; result on the host with the call, correct to rounding, repeatable."""
    n = 1 << 21                                          # x is 16 MiB: above the pipelining threshold
    d = w.spmv_power_law(n, mean=4.0)
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmv(mm.CSR64))
    assert d["x"].nbytes >= module.PIPELINE_MIN_X_BYTES
    pos, crd, val, x = (DualView(a) for a in (d["pos"], d["crd"], d["val"], d["x"]))
    y_in = np.random.default_rng(3).uniform(-1, 1, n)
    y = DualView(y_in.copy())
    out = module.spmv(pos, crd, val, _spec(d), x, y, sync_host=True)
    assert out is y and not y.modifiedDevice() and not x.modifiedHost() and x.uploads == 1 and y.downloads == 1
    ref = oracle.spmv(d["pos"], d["crd"], d["val"], d["x"], y_in)
    scale = oracle.spmv(d["pos"], d["crd"], np.abs(d["val"]), np.abs(d["x"]), np.abs(y_in))
    assert np.all(np.abs(y.host_view() - ref) <= 2e-12 * np.maximum(scale, 1e-300))
    assert torch.equal(y.device_view().cpu(), torch.from_numpy(y.host_view()))
    first = y.host_view().copy()
    # a new x: the same pipeline again, on top of the resident y
    x.host_view()[:] = -x.host_view()
    x.modifyHost()
    module.spmv(pos, crd, val, _spec(d), x, y, sync_host=True)
    assert x.uploads == 2 and pos.uploads == 1
    assert np.all(np.abs(y.host_view() - y_in) <= 4e-12 * np.maximum(scale, 1e-300))   # +Ax then -Ax
    # unchanged x: no upload, the plain overlapped-download path
    module.spmv(pos, crd, val, _spec(d), x, y, sync_host=True)
    assert x.uploads == 2
    y2 = DualView(y_in.copy())
    x.host_view()[:] = -x.host_view()
    x.modifyHost()
    module.spmv(pos, crd, val, _spec(d), x, y2, sync_host=True)
    assert np.array_equal(y2.host_view(), first)                                        # repeatable bit for bit


def test_mixed_arguments_and_bad_specifier():
    d = w.spmv_power_law(1 << 10, idx_dtype=np.int32)
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmv(mm.CSR32))
    n = d["shape"][0]
    y = module.spmv(d["pos"], d["crd"], DualView(d["val"]), _spec(d), d["x"], np.zeros(n))   # one DualView is enough
    assert isinstance(y, DualView)
    ref = oracle.spmv(d["pos"], d["crd"], d["val"], d["x"], np.zeros(n))
    assert np.allclose(y.numpy(), ref, rtol=1e-12, atol=1e-12)
    from lapis_b200._lib import LapisError
    with pytest.raises(LapisError):
        module.spmv(d["pos"], d["crd"], DualView(d["val"]), ((n, n), (n, len(d["crd"]), len(d["val"]))), d["x"], np.zeros(n))
    with pytest.raises(TypeError):
        module.spmv(d["pos"], d["crd"], DualView(d["val"].astype(np.float32)), _spec(d), d["x"], np.zeros(n))


def test_spmm_matmul_and_pcg_resident():
    d = w.spmv_power_law(1 << 12)
    n = d["shape"][0]
    rng = np.random.default_rng(5)
    B = rng.standard_normal((n, 64))
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmm(mm.CSR64))
    C = module.spmm(DualView(d["pos"]), DualView(d["crd"]), DualView(d["val"]), _spec(d), DualView(B), DualView(np.zeros((n, 64))))
    assert np.array_equal(C.numpy(), oracle.spmm(d["pos"], d["crd"], d["val"], B, np.zeros((n, 64))))
    C2 = module.spmm(DualView(d["pos"]), DualView(d["crd"]), DualView(d["val"]), _spec(d), DualView(B), DualView(np.zeros((n, 64))),
                     sync_host=True)
    assert not C2.modifiedDevice() and np.array_equal(C2.host_view(), C.numpy())      # SpMM rows are independent: same bits

    a = rng.standard_normal((4, 48, 40)).astype(np.float32)
    b = rng.standard_normal((4, 40, 56)).astype(np.float32)
    module = KB.KokkosBackend().compile(mm.BATCH_MATMUL)
    c = module.forward(DualView(a), DualView(b), DualView(np.zeros((4, 48, 56), dtype=np.float32)))
    assert np.array_equal(c.numpy(), oracle.bgemm(a, b, np.zeros((4, 48, 56), dtype=np.float32)))

    p = w.pcg_laplacian(64)
    m = p["shape"][0]
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.pcg(mm.CSR32))
    spec = ((m, m), (m + 1, len(p["crd"]), len(p["val"])))
    ops = [DualView(p[k]) for k in ("pos", "crd", "val", "b", "dinv")]
    x, iters, relres = module.pcg(ops[0], ops[1], ops[2], spec, ops[3], ops[4], 1e-10, 1000)
    xh, ih, rh = module.pcg(p["pos"], p["crd"], p["val"], spec, p["b"], p["dinv"], 1e-10, 1000)
    assert isinstance(x, DualView) and relres <= 1e-10 and abs(iters - ih) <= 2
    assert np.max(np.abs(x.numpy() - xh)) <= 1e-8 * np.max(np.abs(xh))
    x2, it2, _ = module.pcg(ops[0], ops[1], ops[2], spec, ops[3], ops[4], 1e-10, 1000)
    assert [o.uploads for o in ops] == [1] * 5 and it2 == iters and np.array_equal(x2.numpy(), x.numpy())
