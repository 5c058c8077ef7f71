"""Host-side logic of the DualView pair (modify flags, lazy copies), with a CPU tensor standing in for
the device copy; the flag rules follow mlir/lib/Target/KokkosCpp/LAPISSupport.hpp:245-282."""
import numpy as np
import pytest

from lapis_b200.dualview import DualView


def test_first_sync_uploads_and_later_syncs_do_not():
    a = np.arange(6, dtype=np.float64)
    dv = DualView(a, device="cpu")
    assert dv.modifiedHost() and not dv.modifiedDevice()
    d = dv.device_view()
    assert dv.uploads == 1 and not dv.modifiedHost()
    assert np.array_equal(d.numpy(), a) and d.data_ptr() != a.ctypes.data
    dv.device_view()
    dv.syncDevice()
    assert dv.uploads == 1
    assert dv.host_view() is a and dv.extent(0) == 6


def test_modify_host_reuploads_and_bumps_version():
    a = np.zeros(4, dtype=np.float32)
    dv = DualView(a, device="cpu")
    dv.syncDevice()
    v = dv.version
    a[:] = 3.0
    assert float(dv.device_view()[0]) == 0.0          # not told about the change: no copy
    dv.modifyHost()
    assert dv.version == v + 1
    assert float(dv.device_view()[0]) == 3.0 and dv.uploads == 2


def test_device_side_changes_come_back_on_sync_host():
    a = np.zeros(3, dtype=np.int64)
    dv = DualView(a, device="cpu")
    dv.device_view().add_(7)
    dv.modifyDevice()
    assert dv.modifiedDevice() and np.all(a == 0)
    assert np.all(dv.numpy() == 7) and dv.downloads == 1 and not dv.modifiedDevice()
    dv.syncHost()
    assert dv.downloads == 1
    assert np.all(np.asarray(dv) == 7)


def test_conflicting_modifications_are_refused():
    dv = DualView(np.zeros(2), device="cpu")
    dv.device_view()
    dv.modifyDevice()
    with pytest.raises(RuntimeError):
        dv.modifyHost()
    dv.syncHost()
    dv.modifyHost()
    with pytest.raises(RuntimeError):
        dv.modifyDevice()


def test_from_device_and_layout_checks():
    import torch
    t = torch.arange(5, dtype=torch.float64)
    dv = DualView.from_device(t)
    assert dv.modifiedDevice() and np.array_equal(dv.numpy(), np.arange(5.0))
    with pytest.raises(ValueError):
        DualView(np.zeros((4, 4))[:, ::2], device="cpu")
    e = DualView(np.zeros(0), device="cpu")
    assert e.device_view().numel() == 0
