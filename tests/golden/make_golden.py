"""Regenerates the golden fixtures in this folder from a LAPIS checkout.

    python tests/golden/make_golden.py /path/to/LAPIS

The fixtures hold the inputs and the known answers of the reference's own
example tests for the hot path, so that the oracle (and through it the CUDA
kernels) can be checked where the checkout is not available:

  spmv_noalloc.npz   examples/spmv_noalloc.py:16-32  (arrays and `ycorrect`
                     parsed from the script text)
  pcg_nos4.npz       examples/pcg_solve.py:106-133   (data/nos4.mtx as CSR,
                     b, dinv, and scipy's cg answer computed exactly as the
                     example computes its expected value)
  mht.npz            examples/hitting_times.py:196-222 (data/mht_A.mtx,
                     data/mht_D.mtx, mask, and the two 17-digit golden moment
                     vectors parsed from the script text)
  gemm.npz           examples/gemm_no_alloc.py:28-46 shapes (8x7x9) with seeded
                     inputs; expected = torch.matmul as in the example
  batched_gemm.npz   examples/batched_gemm_no_alloc.py:33-52 inputs (ones+eye,
                     ones-eye, batch 64 of 5x5); expected = torch.bmm

Nothing is run from the checkout: the example scripts are read as text and
the MatrixMarket files with scipy.
"""
import ast
import os
import re
import sys

import numpy as np
from scipy.io import mmread
from scipy.sparse import csr_matrix
from scipy.sparse.linalg import cg

HERE = os.path.dirname(os.path.abspath(__file__))


def _assigned_list(text, name):
    m = re.search(r"^\s*" + re.escape(name) + r"\s*=\s*(?:np\.array\()?(\[[^\]]*\])", text, re.M)
    if not m:
        raise RuntimeError(f"{name} not found")
    return ast.literal_eval(m.group(1))


def main(root):
    ex = os.path.join(root, "examples")

    # --- SpMV known answer -------------------------------------------------
    t = open(os.path.join(ex, "spmv_noalloc.py")).read()
    np.savez(os.path.join(HERE, "spmv_noalloc.npz"),
             rowptrs=np.array(_assigned_list(t, "rowptrs"), dtype=np.int32),
             colinds=np.array(_assigned_list(t, "colinds"), dtype=np.int32),
             values=np.array(_assigned_list(t, "values"), dtype=np.float64),
             ycorrect=np.array(_assigned_list(t, "ycorrect"), dtype=np.float64))

    # --- PCG on nos4 ---------------------------------------------------------
    A = csr_matrix(mmread(os.path.join(ex, "data", "nos4.mtx")))
    n = A.shape[0]
    xgold = np.ones(n)
    b = A @ xgold
    dinv = 1.0 / A.diagonal()
    reltol, maxiter = 1e-10, 40
    x_scipy, _info = cg(A, b, np.zeros(n), rtol=reltol, maxiter=maxiter, M=np.diag(dinv))
    np.savez(os.path.join(HERE, "pcg_nos4.npz"),
             indptr=A.indptr.astype(np.int32), indices=A.indices.astype(np.int32),
             data=A.data.astype(np.float64), b=b, dinv=dinv, reltol=reltol, maxiter=maxiter,
             x_scipy=x_scipy)

    # --- hitting-time moments ------------------------------------------------
    t = open(os.path.join(ex, "hitting_times.py")).read()
    A = csr_matrix(mmread(os.path.join(ex, "data", "mht_A.mtx")))
    D = csr_matrix(mmread(os.path.join(ex, "data", "mht_D.mtx"))).data
    mask = np.ones(A.shape[0])
    for s in _assigned_list(t, "seedset"):
        mask[s] = 0
    np.savez(os.path.join(HERE, "mht.npz"),
             indptr=A.indptr.astype(np.int32), indices=A.indices.astype(np.int32),
             data=A.data.astype(np.float64), D=D.astype(np.float64), mask=mask,
             alpha=0.99, tol=1e-10, maxiter=20,
             mom1_gold=np.array(_assigned_list(t, "mom1_gold"), dtype=np.float64),
             mom2_gold=np.array(_assigned_list(t, "mom2_gold"), dtype=np.float64))

    # --- GEMM examples (expected value computed the way the examples do) -----
    import torch
    g = torch.Generator().manual_seed(2024)
    a = torch.rand(8, 7, generator=g)
    bm = torch.rand(7, 9, generator=g)
    np.savez(os.path.join(HERE, "gemm.npz"), a=a.numpy(), b=bm.numpy(),
             c=torch.matmul(a, bm).numpy())
    a = (torch.ones((5, 5)) + torch.eye(5)).expand(64, 5, 5).contiguous()
    bm = (torch.ones((5, 5)) - torch.eye(5)).expand(64, 5, 5).contiguous()
    np.savez(os.path.join(HERE, "batched_gemm.npz"), a=a.numpy(), b=bm.numpy(),
             c=torch.bmm(a, bm).numpy())
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
