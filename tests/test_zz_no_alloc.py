"""The allocation-free SpMV entry point against the handle-based one (needs a B200).

`lapis_b200_spmv_f64_noalloc` exists for callers that may not allocate device memory
while they call in (they run inside a memory pool that already spans the GPU, or in a
steady-state loop where cudaMalloc could stall or fail).  It keeps its streaming plan in
a fixed array inside the library, shared by all calls, so the checks here are: the same
bits as the handle-based entry point and agreement with the CPU oracle, on two calls in a
row with different matrices (the second must not see anything of the first in the shared
array), a row block addressed in place (pos[0] != 0), and a clear refusal above the size
limit.  This file sorts last so that a failure here cannot hide others.
"""
import ctypes

import numpy as np
import pytest
import torch

from lapis_b200 import workloads as w
from lapis_b200._lib import LapisError, check, load
from lapis_b200.device import CsrMatrix
from oracle import oracle

pytestmark = pytest.mark.gpu

TOL_F64 = 1e-12  # of |y_in| + sum_j |a_ij x_j| per row, the bar of the other SpMV tests


def _noalloc_spmv(pos_d, crd_d, val_d, shape, x_d, y_d, accumulate):
    lib = load()
    vp = lambda t: ctypes.c_void_p(t.data_ptr() if t.numel() else 0)
    check(lib.lapis_b200_spmv_f64_noalloc(pos_d.element_size(), shape[0], shape[1], vp(pos_d), vp(crd_d), vp(val_d),
                                          vp(x_d), vp(y_d), 1 if accumulate else 0,
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))


def test_noalloc_matches_handle_path_twice_in_a_row():
    assert torch.cuda.is_available(), "needs a CUDA device"
    dev = torch.device("cuda:0")
    # first a larger matrix (many plan entries), then a smaller one with other index width
    cases = [w.spmv_power_law(1 << 17, idx_dtype=np.int64), w.spmv_power_law(1 << 13, idx_dtype=np.int32, seed=99)]
    first_call = {8: True, 4: True}
    for d in cases:
        n = d["shape"][0]
        pos_d, crd_d, val_d, x_d = (torch.as_tensor(d[k]).to(dev) for k in ("pos", "crd", "val", "x"))
        y0 = torch.as_tensor(np.random.default_rng(3).uniform(-1, 1, n)).to(dev)
        A = CsrMatrix(pos_d, crd_d, val_d, (n, n))
        for accumulate in (False, True):
            want = y0.clone()
            A.spmv(x_d, want, accumulate=accumulate)
            got = y0.clone()
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info(dev)[0]
            _noalloc_spmv(pos_d, crd_d, val_d, (n, n), x_d, got, accumulate)
            torch.cuda.synchronize()
            # same kernel, same plan: identical bits (well inside the 1e-12 bound of the other tests)
            assert torch.equal(got, want)
            # and against the CPU oracle, which shares no code with either entry point
            y_in = y0.cpu().numpy() if accumulate else np.zeros(n)
            ref = oracle.spmv(d["pos"], d["crd"], d["val"], d["x"], y_in)
            scale = oracle.spmv(d["pos"], d["crd"], np.abs(d["val"]) * np.abs(d["x"][d["crd"]]), np.ones(n), np.abs(y_in))
            assert np.all(np.abs(got.cpu().numpy() - ref) <= TOL_F64 * np.maximum(scale, np.finfo(np.float64).tiny))
            # After the first call per kernel variant (when the driver may still load device code and the
            # entry point looks its array up), the driver's count of free device memory must not drop.
            if not first_call[pos_d.element_size()]:
                assert torch.cuda.mem_get_info(dev)[0] >= free_before
            first_call[pos_d.element_size()] = False


def test_noalloc_row_block_in_place_matches_oracle():
    """pos[0] != 0: rows [r0, r1) of a larger matrix addressed through the full crd / val arrays."""
    assert torch.cuda.is_available(), "needs a CUDA device"
    dev = torch.device("cuda:0")
    d = w.spmv_power_law(1 << 14, idx_dtype=np.int64)
    pos, crd, val, x = d["pos"], d["crd"], d["val"], d["x"]
    n = len(pos) - 1
    r0, r1 = 3001, 11_111
    assert pos[r0] % 4 != 0 or pos[r0 + 1] % 4 != 0  # an offset that is not a multiple of the chunk alignment
    if pos[r0] % 4 == 0:
        r0 += 1
    pos_d, crd_d, val_d, x_d = (torch.as_tensor(a).to(dev) for a in (pos, crd, val, x))
    y = torch.zeros(r1 - r0, dtype=torch.float64, device=dev)
    _noalloc_spmv(pos_d[r0:r1 + 1], crd_d, val_d, (r1 - r0, n), x_d, y, False)
    ref = oracle.spmv(pos, crd, val, x, np.zeros(n))[r0:r1]
    scale = oracle.spmv(pos, crd, np.abs(val) * np.abs(x[crd]), np.ones(n), np.zeros(n))[r0:r1]
    assert np.all(np.abs(y.cpu().numpy() - ref) <= TOL_F64 * np.maximum(scale, np.finfo(np.float64).tiny))


def test_noalloc_refuses_sizes_beyond_its_plan_buffer():
    assert torch.cuda.is_available(), "needs a CUDA device"
    dev = torch.device("cuda:0")
    pos_d = torch.tensor([0, (1 << 29) + 1], dtype=torch.int64, device=dev)  # one row claiming 2^29 + 1 entries
    dummy = torch.zeros(2, dtype=torch.float64, device=dev)
    crd_d = torch.zeros(2, dtype=torch.int64, device=dev)
    with pytest.raises(LapisError, match="the fixed plan buffer holds") as e:
        _noalloc_spmv(pos_d, crd_d, dummy, (1, 2), dummy, dummy[:1], False)
    assert e.value.status == 6  # LAPIS_ETOOBIG
    assert float(dummy.sum().item()) == 0.0  # nothing ran
