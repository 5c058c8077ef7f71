"""Hitting-time moments on the GPU (masked-Laplacian PCG): against the reference's 17-digit golden vectors
(examples/hitting_times.py:219-222 in the LAPIS project), and against the oracle on a generated graph."""
import os

import numpy as np
import pytest
import torch

from lapis_b200 import KokkosBackend as KB
from lapis_b200.dualview import DualView
from oracle import oracle
from tests import mlir_modules as mm

pytestmark = pytest.mark.gpu


def _random_graph(n, deg, seed):
    """Symmetric weighted adjacency (no self loops) as int32 CSR, and its degree vector."""
    import scipy.sparse as sp
    rng = np.random.default_rng(seed)
    rows = np.repeat(np.arange(n), deg)
    cols = rng.integers(0, n, size=n * deg)
    keep = rows != cols
    w = rng.uniform(0.5, 1.5, size=keep.sum())
    A = sp.coo_matrix((w, (rows[keep], cols[keep])), shape=(n, n)).tocsr()
    A = (A + A.T).tocsr()
    A.sum_duplicates()
    A.sort_indices()
    d = np.asarray(A.sum(axis=1)).ravel() + 1e-3
    return A.indptr.astype(np.int32), A.indices.astype(np.int32), A.data.astype(np.float64), d


def test_mht_golden_vectors_through_backend(golden_dir):
    g = dict(np.load(os.path.join(golden_dir, "mht.npz")))
    n = len(g["D"])
    nnz = len(g["data"])
    module = KB.KokkosBackend(decompose_tensors=True).compile(mm.hitting_times(mm.CSR32))
    data_before = g["data"].copy()
    mom1, mom2 = module.mht(g["indptr"], g["indices"], g["data"], ((n, n), (n + 1, nnz, nnz)), g["mask"], g["D"],
                            float(g["alpha"]), float(g["tol"]), int(g["maxiter"]))
    mom2_norm = module.normalize_mom2(mom1, mom2)
    assert np.allclose(mom1, g["mom1_gold"]) and np.allclose(mom2_norm, g["mom2_gold"])      # the reference's own check
    assert np.allclose(mom1, g["mom1_gold"], rtol=1e-9, atol=1e-9)
    assert np.allclose(mom2_norm, g["mom2_gold"], rtol=1e-9, atol=1e-9)
    assert np.array_equal(g["data"], data_before)
    # 64-bit indices and resident operands give the same vectors
    module64 = KB.KokkosBackend(decompose_tensors=True).compile(mm.hitting_times(mm.CSR64))
    r1, r2 = module64.mht(DualView(g["indptr"].astype(np.int64)), DualView(g["indices"].astype(np.int64)), DualView(g["data"]),
                          ((n, n), (n + 1, nnz, nnz)), DualView(g["mask"]), DualView(g["D"]), float(g["alpha"]),
                          float(g["tol"]), int(g["maxiter"]))
    assert np.allclose(r1.numpy(), mom1, rtol=1e-12, atol=1e-12) and np.allclose(r2.numpy(), mom2, rtol=1e-12, atol=1e-12)
    assert np.allclose(module64.normalize_mom2(r1, r2).numpy(), mom2_norm, rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("n,deg,maxiter", [(3000, 4, 60), (200_000, 6, 80)])
def test_mht_matches_oracle_on_a_generated_graph(n, deg, maxiter):
    from lapis_b200.device import CsrMatrix, normalize_mom2
    pos, crd, val, d = _random_graph(n, deg, seed=n)
    mask = np.ones(n)
    mask[np.random.default_rng(1).choice(n, size=max(1, n // 100), replace=False)] = 0.0
    alpha, tol = 0.95, 1e-10
    o1, o2n = oracle.mht(pos, crd, val, mask, d, alpha, tol, maxiter)
    dev = torch.device("cuda:0")
    A = CsrMatrix.from_host(pos, crd, val, (n, n), dev)
    m1, m2, iters, relres = A.mht(torch.as_tensor(mask).to(dev), torch.as_tensor(d).to(dev), alpha, tol, maxiter, info=True)
    m2n = normalize_mom2(m1, m2)
    assert all(1 <= it <= maxiter for it in iters) and all(r <= tol or it == maxiter for r, it in zip(relres, iters))
    assert np.allclose(m1.cpu().numpy(), o1, rtol=1e-8, atol=1e-8 * np.max(np.abs(o1)))
    assert np.allclose(m2n.cpu().numpy(), o2n, rtol=1e-7, atol=1e-7 * np.max(np.abs(o2n)), equal_nan=True)
    assert np.all(m1.cpu().numpy()[mask == 0.0] == 0.0)
    assert torch.equal(A.val, torch.as_tensor(val).to(dev))          # values untouched
