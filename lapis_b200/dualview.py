"""Host/device pair with modify flags: operands that stay on the GPU between module calls.

The emitted C++ keeps every memref in a ``LAPIS::DualView`` whose host and device copies are
reconciled lazily through two flags (mlir/lib/Target/KokkosCpp/LAPISSupport.hpp:122-134, 245-282 in
the LAPIS project): ``syncDevice`` copies host -> device only if the host side was modified,
``syncHost`` the other way round.  The emitted ``py_*`` wrappers build a fresh DualView around the
numpy buffers on every call, so a Python caller pays the upload every time.  This class gives the
Python caller the same object: wrap the numpy arrays once, pass the wrappers to the module's
functions, and repeated calls on unchanged operands move no bytes.

* ``DualView(array)`` borrows the numpy array as its host view; the host side starts *modified* (as
  the reference's constructor from a host pointer does), so the first ``syncDevice`` uploads.
* After writing into ``host_view()`` call ``modifyHost()``; kernels that write the device side call
  ``modifyDevice()``; ``syncHost()`` brings results back (``numpy()`` does it for you).
* ``version`` increases on every modify: users that derive device-side state from the contents (the
  CSR streaming plan) key their caches on it.
"""
from __future__ import annotations

import numpy as np
import torch


class DualView:
    __slots__ = ("_host", "_device", "_dev", "_mod_host", "_mod_device", "version", "uploads", "downloads", "__weakref__")

    def __init__(self, array, device="cuda"):
        a = np.asarray(array)
        if not a.flags["C_CONTIGUOUS"]:
            raise ValueError("DualView: the host array must be C-contiguous (it is borrowed, not copied)")
        if not a.flags["WRITEABLE"] and a.size:
            a = a.copy()  # torch cannot alias read-only memory
        self._host = a
        self._dev = torch.device(device)
        self._device = None
        self._mod_host, self._mod_device = True, False
        self.version = 0
        self.uploads = self.downloads = 0  # transfer counters (bytes moved are uploads * nbytes)

    @classmethod
    def from_device(cls, tensor: torch.Tensor) -> "DualView":
        """Wraps a result that was produced on the device; the host array is filled on the first syncHost."""
        t = tensor.contiguous()
        dv = cls(np.empty(tuple(t.shape), dtype=_numpy_dtype(t.dtype)), device=t.device)
        dv._device = t
        dv._mod_host, dv._mod_device = False, True
        return dv

    # -- the reference's interface ------------------------------------------------------
    def modifyHost(self):
        if self._mod_device:
            raise RuntimeError("DualView: host modified while the device copy holds unsynchronised changes")
        self._mod_host = True
        self.version += 1

    def modifyDevice(self):
        if self._mod_host and self._device is not None:
            raise RuntimeError("DualView: device modified while the host copy holds unsynchronised changes")
        self._mod_device = True
        self._mod_host = False
        self.version += 1

    def modifiedHost(self) -> bool:
        return self._mod_host

    def modifiedDevice(self) -> bool:
        return self._mod_device

    def syncDevice(self):
        if self._device is None:
            self._device = torch.empty(self._host.shape, dtype=_torch_dtype(self._host.dtype), device=self._dev)
            self._mod_host = True
        if self._mod_host:
            if self._host.size:
                self._device.copy_(torch.from_numpy(self._host))
            self._mod_host = False
            self.uploads += 1
        return self

    def syncHost(self):
        if self._mod_device:
            if self._host.size:
                torch.from_numpy(self._host).copy_(self._device)  # synchronises with the producing stream
            self._mod_device = False
            self.downloads += 1
        return self

    def host_view(self) -> np.ndarray:
        return self._host

    def device_view(self) -> torch.Tensor:
        """The device copy, current (uploads first if the host side was modified)."""
        self.syncDevice()
        return self._device

    def extent(self, dim: int) -> int:
        return int(self._host.shape[dim])

    # -- conveniences ---------------------------------------------------------------------
    def numpy(self) -> np.ndarray:
        """The host array with the device's results brought back if there are any."""
        self.syncHost()
        return self._host

    @property
    def shape(self):
        return self._host.shape

    @property
    def dtype(self):
        return self._host.dtype

    def __array__(self, dtype=None, copy=None):
        a = self.numpy()
        return a if dtype is None else a.astype(dtype)


def _torch_dtype(dt) -> torch.dtype:
    return {np.dtype(np.float64): torch.float64, np.dtype(np.float32): torch.float32, np.dtype(np.int32): torch.int32,
            np.dtype(np.int64): torch.int64}[np.dtype(dt)]


def _numpy_dtype(dt):
    return {torch.float64: np.float64, torch.float32: np.float32, torch.int32: np.int32, torch.int64: np.int64}[dt]
