"""The MatrixMarket reader against scipy on files written for the test (general, symmetric,
skew-symmetric, pattern, integer; duplicates; empty rows) and on the shapes of the reference's
example matrices (tests/golden holds their CSR form)."""
import os

import numpy as np
import pytest
from scipy.io import mmread, mmwrite
from scipy.sparse import coo_matrix, csr_matrix

from lapis_b200._lib import LapisError
from lapis_b200.mmio import read_matrix_market


def _check(path, idx):
    pos, crd, val, shape = read_matrix_market(path, idx)
    ref = csr_matrix(mmread(path))
    ref.sum_duplicates()
    ref.sort_indices()
    assert shape == ref.shape and pos.dtype == idx and crd.dtype == idx
    assert np.array_equal(pos, ref.indptr) and np.array_equal(crd, ref.indices)
    assert np.array_equal(val, ref.data.astype(np.float64))


@pytest.mark.parametrize("idx", [np.int32, np.int64])
def test_general_and_symmetric(tmp_path, idx):
    rng = np.random.default_rng(0)
    A = coo_matrix((rng.uniform(-1, 1, 300), (rng.integers(0, 40, 300), rng.integers(0, 55, 300))), shape=(40, 55))
    p = str(tmp_path / "general.mtx")
    mmwrite(p, A)                      # contains duplicate coordinates and empty rows
    _check(p, idx)
    S = rng.uniform(-1, 1, (30, 30))
    S = np.where(np.abs(S) > 0.7, S, 0.0)
    S = S + S.T
    p = str(tmp_path / "symmetric.mtx")
    mmwrite(p, coo_matrix(S), symmetry="symmetric")
    _check(p, idx)
    K = np.triu(np.where(np.abs(rng.uniform(-1, 1, (20, 20))) > 0.6, 1.0, 0.0), 1)
    K = K - K.T
    p = str(tmp_path / "skew.mtx")
    mmwrite(p, coo_matrix(K), symmetry="skew-symmetric")
    _check(p, idx)
    p = str(tmp_path / "pattern.mtx")
    mmwrite(p, coo_matrix(np.abs(K)), field="pattern", symmetry="symmetric")
    _check(p, idx)
    p = str(tmp_path / "integer.mtx")
    mmwrite(p, coo_matrix((np.arange(1, 7), ([0, 1, 2, 3, 3, 5], [5, 4, 3, 2, 1, 0])), shape=(6, 6)), field="integer")
    _check(p, idx)


def test_reference_example_matrix_roundtrip(tmp_path, golden_dir):
    # the 100 x 100 SPD matrix of examples/pcg_solve.py, from its CSR fixture, through a symmetric .mtx file
    g = np.load(os.path.join(golden_dir, "pcg_nos4.npz"))
    A = csr_matrix((g["data"], g["indices"], g["indptr"]), shape=(100, 100))
    p = str(tmp_path / "nos4_like.mtx")
    mmwrite(p, A, symmetry="symmetric")
    pos, crd, val, shape = read_matrix_market(p, np.int32)
    A.sort_indices()
    assert shape == (100, 100) and np.array_equal(pos, A.indptr) and np.array_equal(crd, A.indices)
    assert np.allclose(val, A.data, rtol=1e-15)


def test_bad_files(tmp_path):
    with pytest.raises(LapisError):
        read_matrix_market(str(tmp_path / "missing.mtx"))
    p = tmp_path / "bad.mtx"
    p.write_text("%%MatrixMarket matrix array real general\n2 2\n1\n2\n3\n4\n")
    with pytest.raises(LapisError, match="unsupported"):
        read_matrix_market(str(p))
    p.write_text("%%MatrixMarket matrix coordinate real general\n2 2 1\n3 1 1.0\n")
    with pytest.raises(LapisError, match="bad entry"):
        read_matrix_market(str(p))
