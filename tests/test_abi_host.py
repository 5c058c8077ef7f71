"""CPU-side checks of the boundary: the library loads and exports what the header declares,
fails loudly without a device, and its host-side integer logic matches the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from lapis_b200 import KokkosBackend as KB
from lapis_b200 import _lib, _memref, partition
from lapis_b200 import workloads as w
from oracle import oracle
from tests import mlir_modules as mm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HAS_GPU = torch.cuda.is_available()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "lapis_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:lapis|py)_\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/lapis_b200.h but not exported"


def test_descriptor_layout_matches_strided_memref():
    # {T* basePtr; T* data; int64 offset; int64 sizes[N]; int64 strides[N]} (LAPISSupport.hpp:7-14)
    for rank in (1, 2, 3):
        D = _memref.make_nd_memref_descriptor(rank)
        assert ctypes.sizeof(D) == 8 * (3 + 2 * rank)
    a = np.arange(24, dtype=np.float64).reshape(2, 3, 4)
    d = _memref.get_ranked_memref_descriptor(a)
    assert list(d.shape) == [2, 3, 4] and list(d.strides) == [12, 4, 1] and d.offset == 0
    back = _memref.ranked_memref_to_numpy(ctypes.pointer(d), np.float64)
    assert np.array_equal(back, a) and back.ctypes.data == a.ctypes.data


@pytest.mark.skipif(HAS_GPU, reason="checks the no-device behaviour")
def test_no_device_fails_loudly():
    lib = _lib.load()
    lib.lapis_initialize()
    assert lib.lapis_last_error() == 3  # LAPIS_ECUDA
    assert b"no CPU path" in lib.lapis_last_error_message()
    with pytest.raises(_lib.LapisError):
        KB.KokkosBackend(decompose_tensors=True).compile(mm.spmv())


def test_csr_validator_refuses_bad_offsets_and_columns():
    """The check the py_* wrappers run on a CSR operand before any kernel sees it (host only, no CUDA call):
    a column index outside [0, ncols) or a broken pos is LAPIS_EBADSHAPE."""
    lib = _lib.load()
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    for idx in (np.int32, np.int64):
        pos = np.array([0, 2, 2, 5], dtype=idx)
        crd = np.array([0, 3, 1, 2, 3], dtype=idx)
        nb = np.dtype(idx).itemsize
        assert lib.lapis_b200_validate_csr_host(nb, 3, 4, 5, vp(pos), vp(crd)) == 0
        bad = crd.copy(); bad[3] = 4            # == ncols
        assert lib.lapis_b200_validate_csr_host(nb, 3, 4, 5, vp(pos), vp(bad)) == 1
        assert b"column index out of range" in lib.lapis_last_error_message()
        bad = crd.copy(); bad[0] = -1
        assert lib.lapis_b200_validate_csr_host(nb, 3, 4, 5, vp(pos), vp(bad)) == 1
        badpos = np.array([0, 3, 2, 5], dtype=idx)   # decreasing
        assert lib.lapis_b200_validate_csr_host(nb, 3, 4, 5, vp(badpos), vp(crd)) == 1
        assert lib.lapis_b200_validate_csr_host(nb, 3, 4, 4, vp(pos), vp(crd)) == 1   # pos[rows] != nnz
    # the threaded path (more than 2^20 entries): one bad index in the middle of the last slice
    n = (1 << 20) + 12345
    crd = (np.arange(n, dtype=np.int64) * 7) % 1000
    pos = np.array([0, n], dtype=np.int64)
    assert lib.lapis_b200_validate_csr_host(8, 1, 1000, n, vp(pos), vp(crd)) == 0
    crd[n - 77] = 1000
    assert lib.lapis_b200_validate_csr_host(8, 1, 1000, n, vp(pos), vp(crd)) == 1


def test_module_library_exports_the_emitted_names(tmp_path):
    """The per-module library that compile() builds exports py_<func> under the emitter's names
    (TranslateToKokkosCpp.cpp:2541: `extern "C" void py_<funcName>(`; `main` becomes `lapis_main`, :2351-2355)
    and resolves the lifecycle symbols through liblapis_b200.so.  No compute call."""
    from lapis_b200 import _shim
    bindings = {"spmv": ("spmv", "i64", np.int64), "pcg": ("pcg", "i32", np.int32), "main": ("batch_matmul", "", None),
                "show": ("print", "densexcompressed", None)}
    so = _shim.build(bindings, str(tmp_path), "lapis_package")
    assert os.path.isfile(so) and _shim.build(bindings, str(tmp_path), "lapis_package") == so  # reused
    h = ctypes.CDLL(so)
    for name in ("py_spmv", "py_pcg", "py_lapis_main", "lapis_initialize", "lapis_finalize", "lapis_last_error"):
        assert hasattr(h, name), name
    assert not hasattr(h, "py_show") and not hasattr(h, "py_main")
    text = _shim.source(bindings)
    assert "py_spmv_f64_i64(ret0, pos, crd, val, spec, x, y)" in text and "py_pcg_f64_i32(" in text


def test_compute_before_initialize_is_refused():
    lib = _lib.load()
    pos = np.array([0, 1], dtype=np.int32)
    crd = np.array([0], dtype=np.int32)
    val = np.array([2.0])
    x = np.array([3.0])
    y = np.zeros(1)
    spec = np.array([1, 1, 2, 1, 1], dtype=np.int64)
    d = lambda a: ctypes.pointer(_memref.get_ranked_memref_descriptor(a))
    ret = ctypes.pointer(ctypes.pointer(_memref.make_nd_memref_descriptor(1)()))
    # make sure no module is alive in this process
    while lib.lapis_last_error() != 5:
        lib.lapis_finalize()
        lib.py_spmv_f64_i32(ret, d(pos), d(crd), d(val), spec.ctypes.data_as(ctypes.c_void_p), d(x), d(y))
        if lib.lapis_last_error() == 0:
            continue
        break
    assert lib.lapis_last_error() in (5, 3)
    assert y[0] == 0.0


def test_backend_classifies_on_path_modules():
    enc = KB._parse_encodings(mm.pcg())
    funcs = KB._parse_functions(mm.pcg(), enc)
    by = {f["name"]: f for f in funcs}
    assert set(by) == {"spmv", "dot", "axpby", "mult", "pcg"}
    assert by["spmv"]["private"] and not by["pcg"]["private"]
    assert KB._classify(by["pcg"], by, mm.pcg())[:2] == ("pcg", "i32")
    for text, want in ((mm.spmv(mm.CSR32), ("spmv", "i32")), (mm.spmv(mm.CSR64), ("spmv", "i64")),
                       (mm.spmv(mm.CSRIDX), ("spmv", "i64")), (mm.spmm(), ("spmm", "i64")),
                       (mm.MATMUL, ("matmul", "")), (mm.BATCH_MATMUL, ("batch_matmul", ""))):
        enc = KB._parse_encodings(text)
        funcs = KB._parse_functions(text, enc)
        public = [f for f in funcs if not f["private"]]
        assert len(public) == 1
        assert KB._classify(public[0], {f["name"]: f for f in funcs}, text)[:2] == want


def _classify_text(text):
    funcs = KB._parse_functions(text, KB._parse_encodings(text))
    by = {f["name"]: f for f in funcs}
    return [KB._classify(f, by, text)[:2] for f in funcs if not f["private"]]


def test_backend_refuses_functions_that_only_resemble_a_known_one():
    """A function is bound to a kernel only if it IS the operation: near-misses would silently compute
    something else than what was written."""
    # a matvec followed by a scale of the result
    scaled = mm.spmv().replace(
        "return %r : tensor<?xf64>",
        "%two = arith.constant 2.0 : f64\n    %s = linalg.generic {indexing_maps = [affine_map<(i) -> (i)>], "
        "iterator_types = [\"parallel\"]} outs(%r : tensor<?xf64>) {\n    ^bb0(%o: f64):\n      %t = arith.mulf %o, %two : f64\n"
        "      linalg.yield %t : f64\n    } -> tensor<?xf64>\n    return %s : tensor<?xf64>")
    assert scaled != mm.spmv()
    # operands wired differently: A^T-like use of y as the input vector
    swapped = mm.spmv().replace("ins(%A, %x :", "ins(%A, %y :").replace("outs(%y :", "outs(%x :")
    # two products in one function
    twice = mm.MATMUL.replace(
        "return %r : tensor<?x?xf32>",
        "%r2 = linalg.matmul ins(%a, %b : tensor<?x?xf32>, tensor<?x?xf32>) outs(%r : tensor<?x?xf32>) -> tensor<?x?xf32>\n"
        "    return %r2 : tensor<?x?xf32>")
    # PCG with another stop test, another iteration start, another update
    pcg = mm.pcg()
    variants = [scaled, swapped, twice,
                pcg.replace("arith.cmpf ogt, %rel, %tol", "arith.cmpf oge, %rel, %tol"),
                pcg.replace("%i = %c1)", "%i = %c0)"),
                pcg.replace("%alpha = arith.divf %rz, %pAp", "%alpha = arith.divf %pAp, %rz"),
                pcg.replace("%x0 = tensor.splat %f0[%n]", "%x0 = tensor.splat %f1[%n]"),
                mm.hitting_times().replace("math.sqrt", "math.absf")]
    for text in variants:
        with pytest.raises(Exception, match="not on the accelerated path"):
            _classify_text(text)
    # what is accepted stays accepted: renamed values, other alias names, extra dead bookkeeping
    renamed = mm.pcg().replace("%alpha", "%step").replace("#id", "#identity")
    assert _classify_text(renamed) == [("pcg", "i32")]
    padded = mm.spmv().replace("%r = linalg.matvec", "%c7 = arith.constant 7 : index\n    %r = linalg.matvec")
    assert _classify_text(padded) == [("spmv", "i32")]


# a checkout of the LAPIS project: LAPIS_SOURCE_DIR, else a directory `reference` beside this repository
_LAPIS_SRC = os.environ.get("LAPIS_SOURCE_DIR") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


@pytest.mark.skipif(not os.path.isdir(os.path.join(_LAPIS_SRC, "examples")), reason="needs a checkout of the LAPIS project")
def test_backend_accepts_the_reference_examples_as_written():
    """The module texts of the LAPIS examples, read from the checkout, bind without an edit."""
    want = {"pcg_solve.py": [("pcg", "i32")], "hitting_times.py": [("mht", "i32"), ("normalize_mom2", "")],
            "spmv_noalloc.py": [("spmv", "i32")], "gemm_no_alloc.py": [("matmul", "")],
            "batched_gemm_no_alloc.py": [("batch_matmul", "")]}
    for fname, kinds in want.items():
        text = open(os.path.join(_LAPIS_SRC, "examples", fname)).read()
        module = re.search(r'=\s*"""(.*?)"""', text, re.S).group(1)
        assert _classify_text(module) == kinds, fname


def test_backend_classifies_the_hitting_times_module():
    for enc_text, sfx in ((mm.CSR32, "i32"), (mm.CSR64, "i64")):
        text = mm.hitting_times(enc_text)
        funcs = KB._parse_functions(text, KB._parse_encodings(text))
        by = {f["name"]: f for f in funcs}
        public = sorted(f["name"] for f in funcs if not f["private"])
        assert public == ["mht", "normalize_mom2"]
        assert KB._classify(by["mht"], by, text)[:2] == ("mht", sfx)
        assert KB._classify(by["normalize_mom2"], by, text)[:2] == ("normalize_mom2", "")
    # the plain solver's module is not mistaken for it, and a module without the masked operator is refused
    text = mm.hitting_times().replace("@plpt", "@other")
    funcs = KB._parse_functions(text, KB._parse_encodings(text))
    by = {f["name"]: f for f in funcs}
    with pytest.raises(Exception, match="not on the accelerated path"):
        KB._classify(by["mht"], by, text)


def test_backend_classifies_neighbouring_formats():
    for text, want in ((mm.bspmm(mm.CSRV32), ("bspmm", "i32")), (mm.bspmm(mm.CSRV64), ("bspmm", "i64")),
                       (mm.spmm_dcsr(mm.DCSR64), ("spmm_dcsr", "i64")), (mm.spmm_dcsr(mm.DCSR32), ("spmm_dcsr", "i32"))):
        funcs = KB._parse_functions(text, KB._parse_encodings(text))
        by = {f["name"]: f for f in funcs}
        public = [f for f in funcs if not f["private"]]
        assert len(public) == 1 and KB._classify(public[0], by, text)[:2] == want
    # a CSRV contraction over another index pair is not the batched SpMM
    text = mm.bspmm().replace("-> (n2, dh, nh)", "-> (n2, nh, dh)")
    funcs = KB._parse_functions(text, KB._parse_encodings(text))
    with pytest.raises(Exception, match="not on the accelerated path"):
        KB._classify(funcs[0], {f["name"]: f for f in funcs}, text)
    # a print-only function is bound to host code
    text = mm.CSRV32 + """
module {
  func.func @show(%A: tensor<?x?x?xf32, #CSRV>) {
    sparse_tensor.print %A : tensor<?x?x?xf32, #CSRV>
    return
  }
}"""
    funcs = KB._parse_functions(text, KB._parse_encodings(text))
    assert KB._classify(funcs[0], {}, text)[:2] == ("print", "densexcompressedxdense")


def test_oracle_bspmm_and_dcsr_against_scipy():
    """The two restatements against scipy's own products (the check examples/bspmm.py:80-90 and
    examples/spmm_dcsr_opdsl.py:163-172 make), and each other's index widths."""
    import scipy.sparse as sp
    rng = np.random.default_rng(3)
    m, n, b, k = 50, 60, 8, 3
    A = sp.random(m, n, density=0.1, random_state=7, format="csr")
    A.sort_indices()
    nnz = A.nnz
    vals = rng.uniform(1.0, 2.0, nnz * b).astype(np.float32)
    B = rng.uniform(1.0, 2.0, (n, k, b)).astype(np.float32)
    C = oracle.bspmm(A.indptr.astype(np.int32), A.indices.astype(np.int32), vals, B)
    gold = np.zeros((m, k, b), dtype=np.float32)
    for i in range(b):
        gold[:, :, i] = sp.csr_matrix((vals[i::b], A.indices, A.indptr), (m, n)) @ B[:, :, i]
    assert np.allclose(C, gold)
    assert np.array_equal(C, oracle.bspmm(A.indptr.astype(np.int64), A.indices.astype(np.int64), vals, B))
    assert np.array_equal(oracle.bspmm(A.indptr.astype(np.int32), A.indices.astype(np.int32), vals, B, C_in=C),
                          oracle.bspmm(A.indptr.astype(np.int64), A.indices.astype(np.int64), vals, B, C_in=C))
    # DCSR: the example's 3x4 matrix, then a generated one with empty rows
    p2, i1, i2 = np.array([0, 1, 3, 3]), np.array([0, 1, 1]), np.array([0, 1, 2])
    vals = np.array([1.1, 2.2, 3.3])
    Bd = np.array([[1.0, 2.0], [4.0, 3.0], [5.0, 6.0], [8.0, 7.0]])
    dense = np.array([[1.1, 0, 0, 0], [0, 2.2, 3.3, 0], [0, 0, 0, 0]])
    # the example's buffers list row 1 twice in i1, the second time with an empty segment
    C = oracle.spmm_dcsr(i1, p2, i2, vals, Bd, np.zeros((3, 2)))
    assert np.allclose(C, dense @ Bd)
    A = sp.random(40, 30, density=0.05, random_state=11, format="csr")
    A.sort_indices()
    stored = np.flatnonzero(np.diff(A.indptr))
    p2 = np.concatenate([[0], np.cumsum(np.diff(A.indptr)[stored])])
    Bd = rng.standard_normal((30, 17))
    C0 = rng.standard_normal((40, 17))
    C = oracle.spmm_dcsr(stored, p2, A.indices, A.data, Bd, C0)
    assert np.allclose(C, C0 + A @ Bd)
    untouched = np.setdiff1d(np.arange(40), stored)
    assert np.array_equal(C[untouched], C0[untouched])


def test_backend_rejects_off_path_modules():
    with pytest.raises(Exception, match="not on the accelerated path"):
        KB.KokkosBackend().compile(mm.UNSUPPORTED)
    with pytest.raises(Exception, match="decompose_tensors"):
        KB.KokkosBackend(decompose_tensors=False).compile(mm.spmv())
    with pytest.raises(Exception, match="parallelization strategy"):
        KB.KokkosBackend(parallel_strategy="bogus")


@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_partition_rows_matches_oracle(G):
    rng = np.random.default_rng(G)
    lens = rng.integers(0, 30, 5000)
    lens[100:400] = 0
    lens[2500] = 4096
    for dt in (np.int32, np.int64):
        pos = np.zeros(5001, dtype=dt)
        pos[1:] = np.cumsum(lens)
        got = partition.partition_rows(pos, G)
        assert np.array_equal(got, oracle.partition_rows(pos, G))
        assert np.array_equal(got, oracle.partition_rows_numpy(pos, G))
        # a slice with a non-zero base partitions like the rebased slice
        sub = pos[1000:3001]
        assert np.array_equal(partition.partition_rows(np.ascontiguousarray(sub), G),
                              oracle.partition_rows_numpy(sub - sub[0], G))


def test_exchange_plan_and_windows():
    from lapis_b200 import workloads as w
    pos, crd, val = w.laplacian_2d(16)
    bounds = partition.partition_rows(pos, 4)
    from lapis_b200.dist import all_windows
    wins = all_windows(pos, crd, bounds)
    recv, send = partition.exchange_plan(bounds, wins)
    for g in range(4):
        r0, r1 = bounds[g], bounds[g + 1]
        c0, c1 = wins[g]
        assert c0 == max(0, r0 - 16) and c1 == min(256, r1 + 16)
        covered = sum(e - s for _, s, e in recv[g]) + (r1 - r0)
        assert covered == c1 - c0
        for (o, s, e) in recv[g]:
            assert bounds[o] <= s < e <= bounds[o + 1]
            assert (g, s, e) in send[o]
    lpos, lcrd, lval = partition.row_block(pos, crd, val, int(bounds[1]), int(bounds[2]))
    assert lpos[0] == 0 and lpos[-1] == len(lcrd) == len(lval)


@pytest.mark.parametrize("world", [2, 3, 5])
def test_push_pieces_cover_every_halo_exactly(world):
    """The records of the peer-memory halo push, decoded back: every rank's non-owned window entries are
    written exactly once, by their owner, from the owner's own entries; flags land in the right slots."""
    from lapis_b200 import partition as part
    from lapis_b200.dist import all_windows
    d = w.pcg_laplacian(24)
    pos, crd = d["pos"], d["crd"]
    bounds = part.partition_rows(pos, world)
    windows = all_windows(pos, crd, bounds)
    recv, send = part.exchange_plan(bounds, windows)
    lens = [c1 - c0 for c0, c1 in windows]
    p_index = [100 + 7 * g for g in range(world)]
    work = [1 << 40 | g << 32 for g in range(world)]        # disjoint fake address ranges
    mbox = [1 << 44 | g << 32 for g in range(world)]
    HALO = 256
    written = [np.zeros(n, dtype=np.int64) for n in lens]
    for r in range(world):
        rec = part.push_pieces(send[r], windows, r, lens, p_index, work, mbox, HALO)
        assert len(rec) == 4 * len(send[r])
        for (consumer, s, e), k in zip(send[r], range(0, len(rec), 4)):
            dst, src_off, length, flag = rec[k:k + 4]
            assert flag == mbox[consumer] + 8 * (HALO + r)
            dst_index = (dst - work[consumer]) // 8 - p_index[consumer]
            assert (dst - work[consumer]) % 8 == 0 and 0 <= dst_index and dst_index + length <= lens[consumer]
            # source entries are owned by r; destination entries are the same global indices
            g0 = windows[r][0] + src_off
            assert bounds[r] <= g0 and g0 + length <= bounds[r + 1]
            assert windows[consumer][0] + dst_index == g0 == s and length == e - s
            written[consumer][dst_index:dst_index + length] += 1
    for g in range(world):
        own = np.zeros(lens[g], dtype=bool)
        own[int(bounds[g]) - windows[g][0]:int(bounds[g + 1]) - windows[g][0]] = True
        assert np.all(written[g][~own] == 1) and np.all(written[g][own] == 0)
    with pytest.raises(RuntimeError):
        part.push_pieces([(1, windows[1][0] - 5, windows[1][0] + 1)], windows, 0, lens, p_index, work, mbox, HALO)
