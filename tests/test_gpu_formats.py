"""Batched SpMM over CSRV tensors and SpMM over DCSR matrices on the GPU: bit-exact against the oracle's
sequential loop nests, and the reference examples' own checks (examples/bspmm.py:80-111,
examples/spmm_dcsr_opdsl.py:137-172 in the LAPIS project)."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

from lapis_b200 import KokkosBackend as KB
from lapis_b200 import device as D
from lapis_b200.dualview import DualView
from oracle import oracle
from tests import mlir_modules as mm

pytestmark = pytest.mark.gpu


def _csr(m, n, density, seed, dtype):
    A = sp.random(m, n, density=density, random_state=seed, format="csr")
    A.sort_indices()
    return A.indptr.astype(dtype), A.indices.astype(dtype), A


def test_bspmm_example_through_backend():
    # the example's pattern and sizes (examples/bspmm.py:63-76), values seeded here
    m, n, b, k, nnz = 5, 6, 8, 3, 8
    rowptrs = np.array([0, 1, 5, 6, 8, 8], dtype=np.int32)
    colinds = np.array([1, 0, 2, 3, 4, 5, 0, 1], dtype=np.int32)
    rng = np.random.default_rng(0)
    values = rng.uniform(1.0, 2.0, nnz * b).astype(np.float32)
    B = rng.uniform(1.0, 2.0, (n, k, b)).astype(np.float32)
    gold = np.zeros((m, k, b), dtype=np.float32)
    for i in range(b):
        gold[:, :, i] = sp.csr_matrix((values[i::b], colinds, rowptrs), (m, n)) @ B[:, :, i]
    module = KB.KokkosBackend(decompose_tensors=True, parallel_strategy="dense-outer-loop").compile(mm.bspmm(mm.CSRV32))
    C = module.bspmm(rowptrs, colinds, values, ((m, n, b), (m + 1, nnz, nnz * b)), B)
    assert C.shape == (m, k, b) and C.dtype == np.float32
    assert np.allclose(gold, C)                                                   # the example's check
    assert np.array_equal(C, oracle.bspmm(rowptrs, colinds, values, B))
    Cr = module.bspmm(DualView(rowptrs), DualView(colinds), DualView(values), ((m, n, b), (m + 1, nnz, nnz * b)), DualView(B))
    assert np.array_equal(Cr.numpy(), C)
    from lapis_b200._lib import LapisError
    with pytest.raises(LapisError):
        module.bspmm(rowptrs, colinds, values, ((m, n, b), (m + 1, nnz, nnz * b + 1)), B)
    with pytest.raises(LapisError):
        module.bspmm(rowptrs, np.where(colinds == 5, 6, colinds).astype(np.int32), values, ((m, n, b), (m + 1, nnz, nnz * b)), B)


@pytest.mark.parametrize("idx", [np.int32, np.int64])
@pytest.mark.parametrize("m,n,dh,nh,density", [(300, 200, 3, 8, 0.05), (257, 129, 64, 8, 0.04), (100, 90, 13, 10, 0.1),
                                                 (64, 64, 1, 1, 0.2), (50, 40, 150, 7, 0.1), (20000, 20000, 16, 8, 0.0008)])
def test_bspmm_bit_exact(idx, m, n, dh, nh, density):
    pos, crd, A = _csr(m, n, density, m + dh, idx)
    rng = np.random.default_rng(m * 7 + nh)
    val = rng.standard_normal(A.nnz * nh).astype(np.float32)
    B = rng.standard_normal((n, dh, nh)).astype(np.float32)
    dev = torch.device("cuda:0")
    t = lambda a: torch.as_tensor(a).to(dev)
    C = D.bspmm_csrv(t(pos), t(crd), t(val), t(B), n)
    ref = oracle.bspmm(pos, crd, val, B)
    assert np.array_equal(C.cpu().numpy(), ref)
    # in place on top of an existing result: every element continues from its old value
    C0 = rng.standard_normal((m, dh, nh)).astype(np.float32)
    C2 = D.bspmm_csrv(t(pos), t(crd), t(val), t(B), n, t(C0))
    assert np.array_equal(C2.cpu().numpy(), oracle.bspmm(pos, crd, val, B, C_in=C0))


def test_spmm_dcsr_example_through_backend():
    p1 = np.array([0, 3], dtype=np.int64)
    i1 = np.array([0, 1, 1], dtype=np.int64)
    p2 = np.array([0, 1, 3, 3], dtype=np.int64)
    i2 = np.array([0, 1, 2], dtype=np.int64)
    values = np.array([1.1, 2.2, 3.3])
    b = np.array([[1.0, 2.0], [4.0, 3.0], [5.0, 6.0], [8.0, 7.0]])
    c = np.zeros((3, 2))
    a = np.array([[1.1, 0.0, 0.0, 0.0], [0.0, 2.2, 3.3, 0.0], [0.0, 0.0, 0.0, 0.0]])
    module = KB.KokkosBackend(decompose_tensors=True, parallel_strategy="any-storage-outer-loop").compile(mm.spmm_dcsr(mm.DCSR64))
    out = module.spMxM(p1, i1, p2, i2, values, ((3, 4), (2, 3, 4, 3, 3)), b, c)
    assert out is c and np.allclose(c, np.matmul(a, b))                            # the example's check
    assert np.array_equal(c, oracle.spmm_dcsr(i1, p2, i2, values, b, np.zeros((3, 2))))
    from lapis_b200._lib import LapisError
    with pytest.raises(LapisError):
        module.spMxM(p1, np.array([1, 0, 1]), p2, i2, values, ((3, 4), (2, 3, 4, 3, 3)), b, c)


@pytest.mark.parametrize("idx", [np.int32, np.int64])
@pytest.mark.parametrize("m,n,k,density", [(40, 30, 17, 0.05), (5000, 4000, 64, 0.002), (300, 300, 200, 0.02), (100, 100, 1, 0.1)])
def test_spmm_dcsr_bit_exact(idx, m, n, k, density):
    _, _, A = _csr(m, n, density, m + k, idx)
    stored = np.flatnonzero(np.diff(A.indptr)).astype(idx)
    p2 = np.concatenate([[0], np.cumsum(np.diff(A.indptr)[stored])]).astype(idx)
    i2 = A.indices.astype(idx)
    rng = np.random.default_rng(k)
    B = rng.standard_normal((n, k))
    C0 = rng.standard_normal((m, k))
    ref = oracle.spmm_dcsr(stored, p2, i2, A.data, B, C0)
    dev = torch.device("cuda:0")
    t = lambda a: torch.as_tensor(np.ascontiguousarray(a)).to(dev)
    C = D.spmm_dcsr(t(stored), t(p2), t(i2), t(A.data), t(B), t(C0), n)
    assert np.array_equal(C.cpu().numpy(), ref)
    assert np.allclose(ref, C0 + A @ B)
    # through the module with resident operands
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.spmm_dcsr(mm.DCSR32 if idx == np.int32 else mm.DCSR64))
    p1 = np.array([0, len(stored)], dtype=idx)
    Cd = DualView(C0.copy())
    module.spMxM(p1, DualView(stored), DualView(p2), DualView(i2), DualView(A.data.copy()),
                 ((m, n), (2, len(stored), len(p2), len(i2), len(i2))), DualView(B), Cd)
    assert np.array_equal(Cd.numpy(), ref)
