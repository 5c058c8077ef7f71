"""Compile-and-call surface of ``lapis.KokkosBackend`` bound to prebuilt sm_100a kernels.

The reference class (python/lapis/KokkosBackend.py:10-121 in the LAPIS project)
shells out to ``lapis-opt`` and ``lapis-translate``, builds the emitted Kokkos C++
with CMake and returns a generated ``LAPISModule`` whose methods call the
``py_<func>`` symbols of the built library
(mlir/lib/Target/KokkosCpp/TranslateToKokkosCpp.cpp:2757-2977, :4393-4411).

Here no kernel is compiled at call time.  ``compile()`` reads the MLIR text, finds
the public functions, and binds each one that lies on the accelerated path --
CSR ``linalg.matvec`` (SpMV), CSR x dense ``linalg.matmul`` (SpMM), dense
``linalg.matmul`` / ``linalg.batch_matmul`` in f32, and the ``@pcg`` solve loop of
examples/pcg_solve.py -- to the matching entry point of ``liblapis_b200.so``.  A
module with any other public function is rejected: there is no general MLIR
lowering and no CPU fallback in this package.

Calling convention of the returned object, as in the generated class: memref
arguments are numpy arrays (or CPU torch tensors), forced C-contiguous with
``numpy.require``; a decomposed sparse tensor is the four arguments
``pos, crd, val, ((rows, cols), (len(pos), len(crd), len(val)))``; results come
back as numpy arrays / python scalars, several results as a tuple.
"""
from __future__ import annotations

import ctypes
import os
import re

import numpy as np

from . import _forms
from . import _memref as rt
from . import _shim
from ._lib import LapisError, check_last, load

_PAR_STRATEGIES = ("none", "dense-outer-loop", "any-storage-outer-loop", "dense-any-loop", "any-storage-any-loop")


# ---------------------------------------------------------------------------
# MLIR text inspection
# ---------------------------------------------------------------------------
def _split_top(s: str):
    out, depth, cur = [], 0, []
    for ch in s:
        if ch in "<([":
            depth += 1
        elif ch in ">)]":
            depth -= 1
        if ch == "," and depth == 0:
            out.append("".join(cur).strip())
            cur = []
        else:
            cur.append(ch)
    tail = "".join(cur).strip()
    if tail:
        out.append(tail)
    return out


class _Type:
    def __init__(self, text: str, encodings: dict):
        self.text = text.strip()
        self.rank = None
        self.elem = None
        self.sparse = None  # encoding dict when the tensor has a sparse encoding
        m = re.match(r"(?:tensor|memref)<(.*)>$", self.text, re.S)
        if m:
            parts = _split_top(m.group(1))
            dims = parts[0].split("x")
            self.elem = dims[-1].strip()
            self.rank = len(dims) - 1
            if len(parts) > 1 and parts[1].startswith("#"):
                self.sparse = encodings.get(parts[1].strip())
                if self.sparse is None:
                    raise Exception(f"unknown tensor encoding {parts[1]}")
        else:
            self.elem = self.text
            self.rank = 0 if self.text in ("f64", "f32", "index", "i32", "i64") else None


def _parse_encodings(text: str) -> dict:
    enc = {}
    for m in re.finditer(r"(#\w+)\s*=\s*#sparse_tensor\.encoding<\{(.*?)\}>", text, re.S):
        body = m.group(2)
        lvl = re.search(r"map\s*=\s*\([^)]*\)\s*->\s*\(([^)]*)\)", body)
        levels = re.findall(r"\w+\s*:\s*(\w+)", lvl.group(1)) if lvl else []
        pw = re.search(r"posWidth\s*=\s*(\d+)", body)
        cw = re.search(r"crdWidth\s*=\s*(\d+)", body)
        enc[m.group(1)] = {"levels": levels, "posWidth": int(pw.group(1)) if pw else 0,
                           "crdWidth": int(cw.group(1)) if cw else 0}
    return enc


def _parse_functions(text: str, encodings: dict):
    funcs = []
    for m in re.finditer(r"func\.func\s+(private\s+)?@(\w+)\s*\(", text):
        # argument list: balance parentheses from m.end()
        i, depth = m.end(), 1
        while depth:
            depth += {"(": 1, ")": -1}.get(text[i], 0)
            i += 1
        args_text = text[m.end():i - 1]
        j = text.index("{", i)
        res_text = text[i:j].strip()
        if "attributes" in res_text:
            res_text = res_text.split("attributes")[0].strip()
        res_text = res_text[2:].strip() if res_text.startswith("->") else ""
        if res_text.startswith("("):
            res_text = res_text[1:res_text.rindex(")")]
        k, depth = j + 1, 1
        while depth:
            depth += {"{": 1, "}": -1}.get(text[k], 0)
            k += 1
        args = []
        for a in _split_top(args_text):
            args.append(_Type(a.split(":", 1)[1], encodings))
        results = [_Type(r, encodings) for r in _split_top(res_text)] if res_text else []
        funcs.append({"name": m.group(2), "private": bool(m.group(1)), "args": args, "results": results,
                      "body": text[j:k]})
    return funcs


def _is_csr(t: _Type) -> bool:
    return t.sparse is not None and t.rank == 2 and t.sparse["levels"] == ["dense", "compressed"]


def _index_dtype(enc: dict):
    widths = {enc["posWidth"], enc["crdWidth"]}
    if widths == {32}:
        return np.int32, "i32"
    if widths <= {0, 64} and len(widths) == 1:
        # width 0 means `index`, emitted as size_t (TranslateToKokkosCpp.cpp:4440-4441): 64-bit here
        return np.int64, "i64"
    raise Exception("posWidth and crdWidth must both be 32 or both be 64/index on the accelerated path")


def _dense(t: _Type, rank: int, elem: str) -> bool:
    return t.sparse is None and t.rank == rank and t.elem == elem


def _is_csrv(t: _Type) -> bool:
    return t.sparse is not None and t.rank == 3 and t.sparse["levels"] == ["dense", "compressed", "dense"]


def _is_dcsr(t: _Type) -> bool:
    return t.sparse is not None and t.rank == 2 and t.sparse["levels"] == ["compressed", "compressed"]


def _indexing_maps(text: str):
    """Every `indexing_maps = [...]` list of the text as tuples of dimension positions."""
    out = []
    for m in re.finditer(r"indexing_maps\s*=\s*\[(.*?)\]", text, re.S):
        maps = []
        for mm_ in re.finditer(r"affine_map<\(([^)]*)\)\s*->\s*\(([^)]*)\)>", m.group(1)):
            dims = [d.strip() for d in mm_.group(1).split(",")]
            try:
                maps.append(tuple(dims.index(d.strip()) for d in mm_.group(2).split(",")))
            except ValueError:
                maps.append(None)
        out.append(maps)
    return out


def _off_path(fn: dict, why: str = ""):
    return Exception(
        f"function @{fn['name']} is not on the accelerated path (CSR matvec/matmul in f64, dense matmul / "
        "batch_matmul in f32, the Jacobi PCG loop, the hitting-time moments, CSRV batched SpMM, DCSR SpMM)"
        + (f": {why}" if why else "") + "; lapis_b200 has no general MLIR lowering and no fallback")


def _classify(fn: dict, all_funcs: dict, module_text: str = ""):
    """Returns (kind, index suffix, index dtype) or raises for an off-path function.

    The argument and result types select a candidate kind; the body must then BE that operation
    (lapis_b200/_forms.py): exactly one named linalg operation for the single-operation kinds, a canonical
    form with an accepted digest for the loops.  A function that only resembles a known one -- a matvec
    followed by a scale, a PCG loop with another stop test -- is refused, as it would compute something the
    bound kernel does not."""
    a, r, body = fn["args"], fn["results"], fn["body"]
    text = _forms.function_texts(module_text).get(fn["name"], "") if module_text else ""

    def one_op(op):
        if not _forms.single_named_op(text, op):
            raise _off_path(fn, f"its body is not a single linalg.{op} on its arguments")

    def known_form():
        if _forms.closure_digest(fn["name"], module_text) not in _forms.accepted_digests():
            raise _off_path(fn, "it differs from every accepted form of that operation")

    # a function that only prints its sparse argument (examples/bspmm.py:54-58, spmm_dcsr_opdsl.py:66-68): host work
    if len(a) == 1 and a[0].sparse is not None and len(r) == 0 and "sparse_tensor.print" in body and "linalg." not in body:
        return "print", "x".join(a[0].sparse["levels"]), None
    # batched SpMM over a CSRV tensor (examples/bspmm.py:14-52): out(n1,dh,nh) = sum_n2 A(n1,n2,nh) * B(n2,dh,nh)
    if len(a) == 2 and _is_csrv(a[0]) and a[0].elem == "f32" and _dense(a[1], 3, "f32") and len(r) == 1:
        known_form()
        dt, sfx = _index_dtype(a[0].sparse)
        return "bspmm", sfx, dt
    if len(a) == 3 and _is_dcsr(a[0]) and a[0].elem == "f64" and _dense(a[1], 2, "f64") and _dense(a[2], 2, "f64") and len(r) == 1:
        one_op("matmul")
        dt, sfx = _index_dtype(a[0].sparse)
        return "spmm_dcsr", sfx, dt
    if len(a) == 3 and _is_csr(a[0]) and a[0].elem == "f64" and _dense(a[1], 1, "f64") and _dense(a[2], 1, "f64") and len(r) == 1:
        one_op("matvec")
        dt, sfx = _index_dtype(a[0].sparse)
        return "spmv", sfx, dt
    if len(a) == 3 and _is_csr(a[0]) and a[0].elem == "f64" and _dense(a[1], 2, "f64") and _dense(a[2], 2, "f64") and len(r) == 1:
        one_op("matmul")
        dt, sfx = _index_dtype(a[0].sparse)
        return "spmm", sfx, dt
    if len(a) == 3 and all(_dense(t, 2, "f32") for t in a) and len(r) == 1:
        one_op("matmul")
        return "matmul", "", None
    if len(a) == 3 and all(_dense(t, 3, "f32") for t in a) and len(r) == 1:
        one_op("batch_matmul")
        return "batch_matmul", "", None
    if (len(a) == 5 and _is_csr(a[0]) and a[0].elem == "f64" and _dense(a[1], 1, "f64") and _dense(a[2], 1, "f64")
            and a[3].elem == "f64" and a[4].elem == "index" and len(r) == 3):
        known_form()  # examples/pcg_solve.py:52-101
        dt, sfx = _index_dtype(a[0].sparse)
        return "pcg", sfx, dt
    # hitting-time moments (examples/hitting_times.py:151-194): scale, two masked-Laplacian PCG solves
    if (len(a) == 6 and _is_csr(a[0]) and a[0].elem == "f64" and _dense(a[1], 1, "f64") and _dense(a[2], 1, "f64")
            and a[3].elem == "f64" and a[4].elem == "f64" and a[5].elem == "index" and len(r) == 2):
        known_form()
        dt, sfx = _index_dtype(a[0].sparse)
        return "mht", sfx, dt
    if len(a) == 2 and _dense(a[0], 1, "f64") and _dense(a[1], 1, "f64") and len(r) == 1:
        known_form()  # examples/hitting_times.py:196-218
        return "normalize_mom2", "", None
    raise _off_path(fn)


# ---------------------------------------------------------------------------
# The module object returned by compile()
# ---------------------------------------------------------------------------
def _desc(arr):
    return ctypes.pointer(rt.get_ranked_memref_descriptor(arr))


def _ret_slot(rank):
    return ctypes.pointer(ctypes.pointer(rt.make_nd_memref_descriptor(rank)()))


def _flatten_spec(spec):
    flat = np.zeros(5, dtype=np.int64)
    for i in range(2):
        flat[i] = spec[0][i]
    for i in range(3):
        flat[2 + i] = spec[1][i]
    return flat


def _resident(*args) -> bool:
    from .dualview import DualView
    return any(isinstance(a, DualView) for a in args)


class LAPISModule:
    """Same lifecycle as the generated class: initialize on construction, finalize on deletion.

    Every function takes numpy arrays as the generated module does (operands are uploaded, results
    downloaded, on every call).  If any array argument is a ``lapis_b200.dualview.DualView`` the call takes
    the resident path instead: operands are uploaded only when their host side was modified, the CSR
    streaming plan is kept per (pos, crd, val) triple, results stay on the device until ``syncHost()`` /
    ``numpy()``, and the in/out argument is returned as a DualView.
    """

    def __init__(self, libPath: str, bindings: dict):
        # libPath: the module's own library (lapis_b200/_shim.py), exporting py_<func> under the names the
        # emitter uses; it depends on liblapis_b200.so, loaded first so that a missing build fails loudly
        load()
        self.libPath = libPath
        self.libHandle = ctypes.CDLL(libPath)
        self.libHandle.lapis_last_error.restype = ctypes.c_int
        self.libHandle.lapis_initialize()
        check_last()
        self._live = True
        self._plans = {}  # (id(pos), id(crd), id(val)) -> (weakrefs, versions, shape, CsrMatrix)
        for name, (kind, sfx, idx_dtype) in bindings.items():
            setattr(self, name, self._bind(name, kind, sfx, idx_dtype))

    def __del__(self):
        if getattr(self, "_live", False):
            self._live = False
            self.libHandle.lapis_finalize()

    # -- resident path ---------------------------------------------------------------------
    @staticmethod
    def _dv(a, dtype):
        from .dualview import DualView
        if isinstance(a, DualView):
            if a.dtype != np.dtype(dtype):
                raise TypeError(f"DualView of {a.dtype} where {np.dtype(dtype)} is expected")
            return a
        return DualView(np.require(a, dtype=dtype, requirements=["C"]))

    def _plan(self, pos, crd, val, spec, idx_dtype):
        """The device CSR with its streaming plan, rebuilt only if one of the three arrays changed."""
        import weakref
        from .device import CsrMatrix
        pos, crd, val = self._dv(pos, idx_dtype), self._dv(crd, idx_dtype), self._dv(val, np.float64)
        flat = _flatten_spec(spec)
        shape = (int(flat[0]), int(flat[1]))
        if pos.extent(0) != flat[2] or crd.extent(0) != flat[3] or val.extent(0) != flat[4] or flat[2] != flat[0] + 1:
            raise LapisError(1, "storage specifier does not match the pos/crd/val arrays")
        key = (id(pos), id(crd), id(val))
        versions = (pos.version, crd.version, val.version)
        hit = self._plans.get(key)
        if hit is not None and all(r() is o for r, o in zip(hit[0], (pos, crd, val))) and hit[1] == versions and hit[2] == shape:
            return hit[3]
        A = CsrMatrix(pos.device_view(), crd.device_view(), val.device_view(), shape, tune=True)
        if len(self._plans) >= 16:
            self._plans.pop(next(iter(self._plans)))
        self._plans[key] = (tuple(weakref.ref(o) for o in (pos, crd, val)), versions, shape, A)
        return A

    def _row_blocks(self, A, pos_dv, nblocks: int = 0):
        """Handles over nnz-balanced row blocks of a planned matrix (they share its device arrays; a handle
        may start at any row because the plan is built from pos[r0:r1+1]), kept with the plan."""
        from . import partition as part
        from .device import CsrMatrix
        blocks = getattr(A, "_row_blocks", None)
        if blocks is None:
            nblocks = nblocks or self.PIPELINE_ROW_BLOCKS
            bounds = part.partition_rows(pos_dv.host_view(), nblocks)
            blocks = []
            for g in range(nblocks):
                r0, r1 = int(bounds[g]), int(bounds[g + 1])
                if r1 > r0:
                    blocks.append((r0, r1, CsrMatrix(A.pos[r0:r1 + 1], A.crd, A.val, (r1 - r0, A.ncols), tune=True)))
            A._row_blocks = blocks
        return blocks

    def _run_and_download(self, A, pos_dv, out_dv, run_block):
        """Runs ``run_block(handle, r0, r1)`` row block by row block and copies each finished block of the
        result to the host on a second stream while the next block computes; returns with the host side of
        ``out_dv`` current.  With a page-locked host array the copies are asynchronous and overlap."""
        import torch
        dev_out, host = out_dv.device_view(), torch.from_numpy(out_dv.host_view())
        main = torch.cuda.current_stream()
        copy = getattr(self, "_copy_stream", None)
        if copy is None:
            copy = self._copy_stream = torch.cuda.Stream()
        for r0, r1, Ab in self._row_blocks(A, pos_dv):
            run_block(Ab, r0, r1)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(copy):
                copy.wait_event(done)
                host[r0:r1].copy_(dev_out[r0:r1], non_blocking=True)
        copy.synchronize()
        out_dv.modifyDevice()       # version bump: the contents changed ...
        out_dv._mod_device = False  # ... and both sides already agree
        out_dv.downloads += 1

    # An SpMV whose x arrives from the host every call cannot start before x is on the device -- unless the
    # matrix is also kept as two column halves: the half that only reads x[:mid] runs while x[mid:] is still
    # on its way.  Used by spmv(..., sync_host=True) for large x whose host side was modified.
    PIPELINE_MIN_X_BYTES = 8 << 20
    PIPELINE_ROW_BLOCKS = 4  # row blocks whose results go back to the host one behind the other

    def _column_halves(self, A, pos_dv, crd_dv, val_dv, nblocks: int = 0):
        """(mid, handle over columns [0, mid), row-block handles over columns [mid, ncols)), kept with the plan."""
        import torch
        from . import partition as part
        from .device import CsrMatrix
        halves = getattr(A, "_col_halves", None)
        if halves is None:
            nblocks = nblocks or self.PIPELINE_ROW_BLOCKS
            pos, crd, val = pos_dv.host_view(), crd_dv.host_view(), val_dv.host_view()
            mid = A.ncols // 2
            left = crd < mid
            before = np.zeros(len(crd) + 1, dtype=np.int64)
            np.cumsum(left, out=before[1:])
            pos1 = before[pos].astype(pos.dtype)          # entries of each row that fall into the left half
            pos2 = (pos - pos1).astype(pos.dtype)
            del before
            dev = A.pos.device
            A1 = CsrMatrix.from_host(pos1, crd[left], val[left], (A.nrows, A.ncols), dev, tune=True)
            right = ~left
            del left
            dpos2 = torch.as_tensor(pos2).to(dev)
            dcrd2 = torch.as_tensor(np.ascontiguousarray(crd[right])).to(dev)
            dval2 = torch.as_tensor(np.ascontiguousarray(val[right])).to(dev)
            bounds = part.partition_rows(pos2, nblocks)  # bounds[0] = 0, bounds[-1] = nrows: the blocks cover every row
            blocks = []
            for g in range(nblocks):
                r0, r1 = int(bounds[g]), int(bounds[g + 1])
                if r1 > r0:
                    blocks.append((r0, r1, CsrMatrix(dpos2[r0:r1 + 1], dcrd2, dval2, (r1 - r0, A.ncols), tune=True)))
            halves = A._col_halves = (mid, A1, blocks)
        return halves

    def _spmv_pipelined(self, A, pos_dv, crd_dv, val_dv, x, y):
        """y += A x with x uploaded in two pieces: the left column half of A runs on x[:mid] while x[mid:] is
        uploaded; the right half runs row block by row block and each finished block of y goes back to the
        host while the next computes.  Returns with both sides of x and y in agreement.  A row's sum is formed as
        (y_in + left part) + right part: it agrees with the unsplit call to rounding, not bit for bit."""
        import torch
        mid, A1, blocks = self._column_halves(A, pos_dv, crd_dv, val_dv)
        yd, yh = y.device_view(), torch.from_numpy(y.host_view())
        if x._device is None:
            x._device = torch.empty(x.shape, dtype=torch.float64, device=A.pos.device)
        xd, xh = x._device, torch.from_numpy(x.host_view())
        main = torch.cuda.current_stream()
        for name in ("_copy_stream", "_upload_stream"):
            if getattr(self, name, None) is None:
                setattr(self, name, torch.cuda.Stream())
        copy, up = self._copy_stream, self._upload_stream
        up.wait_stream(main)  # earlier kernels may still read x
        with torch.cuda.stream(up):
            xd[:mid].copy_(xh[:mid], non_blocking=True)
            first = torch.cuda.Event()
            first.record(up)
            xd[mid:].copy_(xh[mid:], non_blocking=True)
            second = torch.cuda.Event()
            second.record(up)
        main.wait_event(first)
        A1.spmv(xd, yd, accumulate=True)
        main.wait_event(second)
        for r0, r1, Ab in blocks:
            Ab.spmv(xd, yd[r0:r1], accumulate=True)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(copy):
                copy.wait_event(done)
                yh[r0:r1].copy_(yd[r0:r1], non_blocking=True)
        copy.synchronize()
        up.synchronize()
        x._mod_host = False
        x.uploads += 1
        y.modifyDevice()
        y._mod_device = False
        y.downloads += 1

    def _bind(self, name, kind, sfx, idx_dtype):
        lib = self.libHandle
        symbol = "py_" + _shim.export_name(name)  # the emitter's export name, from the module's own library

        def csr_args(pos, crd, val, spec):
            pos = np.require(pos, dtype=idx_dtype, requirements=["C"])
            crd = np.require(crd, dtype=idx_dtype, requirements=["C"])
            val = np.require(val, dtype=np.float64, requirements=["C"])
            flat = _flatten_spec(spec)
            return (pos, crd, val, flat), (_desc(pos), _desc(crd), _desc(val), flat.ctypes.data_as(ctypes.c_void_p))

        if kind == "spmv":
            fn = getattr(lib, symbol)

            def spmv(pos, crd, val, spec, x, y, sync_host=False):
                """``sync_host=True`` (resident path only): return with y already on the host; the matrix is
                processed in row blocks and each finished block of y is downloaded while the next computes."""
                if _resident(pos, crd, val, x, y):
                    A = self._plan(pos, crd, val, spec, idx_dtype)
                    x, y = self._dv(x, np.float64), self._dv(y, np.float64)
                    if sync_host and A.nrows > 0:
                        if x.modifiedHost() and x.host_view().nbytes >= self.PIPELINE_MIN_X_BYTES:
                            self._spmv_pipelined(A, self._dv(pos, idx_dtype), self._dv(crd, idx_dtype),
                                                 self._dv(val, np.float64), x, y)
                            return y
                        xd, yd = x.device_view(), y.device_view()
                        self._run_and_download(A, self._dv(pos, idx_dtype), y,
                                               lambda Ab, r0, r1: Ab.spmv(xd, yd[r0:r1], accumulate=True))
                        return y
                    A.spmv(x.device_view(), y.device_view(), accumulate=True)
                    y.modifyDevice()
                    return y
                keep, cargs = csr_args(pos, crd, val, spec)
                x = np.require(x, dtype=np.float64, requirements=["C"])
                y = np.require(y, dtype=np.float64, requirements=["C"])
                ret0 = _ret_slot(1)
                fn(ret0, *cargs, _desc(x), _desc(y))
                check_last()
                del keep
                return y  # the function returns its outs argument

            return spmv
        if kind == "spmm":
            fn = getattr(lib, symbol)

            def spmm(pos, crd, val, spec, B, C, sync_host=False):
                """``sync_host=True`` (resident path only): as for spmv, C comes back block by block."""
                if _resident(pos, crd, val, B, C):
                    A = self._plan(pos, crd, val, spec, idx_dtype)
                    B, C = self._dv(B, np.float64), self._dv(C, np.float64)
                    if sync_host and A.nrows > 0:
                        Bd, Cd = B.device_view(), C.device_view()
                        self._run_and_download(A, self._dv(pos, idx_dtype), C,
                                               lambda Ab, r0, r1: Ab.spmm(Bd, Cd[r0:r1], accumulate=True))
                        return C
                    A.spmm(B.device_view(), C.device_view(), accumulate=True)
                    C.modifyDevice()
                    return C
                keep, cargs = csr_args(pos, crd, val, spec)
                B = np.require(B, dtype=np.float64, requirements=["C"])
                C = np.require(C, dtype=np.float64, requirements=["C"])
                ret0 = _ret_slot(2)
                fn(ret0, *cargs, _desc(B), _desc(C))
                check_last()
                del keep
                return C

            return spmm
        if kind in ("matmul", "batch_matmul"):
            fn = getattr(lib, symbol)
            rank = 2 if kind == "matmul" else 3

            def forward(A, B, C):
                if _resident(A, B, C):
                    from . import device as D
                    A, B, C = (self._dv(t, np.float32) for t in (A, B, C))
                    D.bgemm(A.device_view(), B.device_view(), C.device_view())
                    C.modifyDevice()
                    return C
                A = np.require(A, dtype=np.float32, requirements=["C"])
                B = np.require(B, dtype=np.float32, requirements=["C"])
                C = np.require(C, dtype=np.float32, requirements=["C"])
                ret0 = _ret_slot(rank)
                fn(ret0, _desc(A), _desc(B), _desc(C))
                check_last()
                return C

            return forward
        if kind == "pcg":
            fn = getattr(lib, symbol)

            def pcg(pos, crd, val, spec, b, dinv, tol, maxiter):
                if _resident(pos, crd, val, b, dinv):
                    from .dualview import DualView
                    A = self._plan(pos, crd, val, spec, idx_dtype)
                    b, dinv = self._dv(b, np.float64), self._dv(dinv, np.float64)
                    x, iters, relres = A.pcg(b.device_view(), dinv.device_view(), float(tol), int(maxiter))
                    return DualView.from_device(x), iters, relres
                keep, cargs = csr_args(pos, crd, val, spec)
                b = np.require(b, dtype=np.float64, requirements=["C"])
                dinv = np.require(dinv, dtype=np.float64, requirements=["C"])
                ret0 = _ret_slot(1)
                ret1 = ctypes.c_size_t(0)
                ret2 = ctypes.c_double(0.0)
                fn(ret0, ctypes.byref(ret1), ctypes.byref(ret2), *cargs, _desc(b), _desc(dinv),
                   ctypes.c_double(tol), ctypes.c_size_t(maxiter))
                check_last()
                del keep
                # unmanaged alias of module-owned memory, valid until lapis_finalize
                return (rt.ranked_memref_to_numpy(ret0[0], np.float64), int(ret1.value), float(ret2.value))

            return pcg
        if kind == "print":
            nbuf = 2 * sfx.split("x").count("compressed") + 1  # pos and crd per compressed level, then the values

            def print_tensor(*args):
                """Prints the decomposed sparse tensor (buffers..., specifier) on the host in the layout of
                ``sparse_tensor.print``: stored-entry count, dimensions, then each level's buffers."""
                if len(args) != nbuf + 1:
                    raise TypeError(f"expected {nbuf} buffers and the storage specifier")
                bufs = [np.asarray(getattr(b, "numpy", lambda: b)()) for b in args[:nbuf]]
                dims = tuple(int(x) for x in args[-1][0])
                print("---- Sparse Tensor ----")
                print(f"nse = {len(bufs[-1])}")
                print("dim = ( " + ", ".join(str(x) for x in dims) + " )")
                lvl = 0
                it = iter(bufs[:-1])
                for kind_ in sfx.split("x"):
                    if kind_ == "compressed":
                        for name in ("pos", "crd"):
                            print(f"{name}[{lvl}] : ( " + ", ".join(str(int(x)) for x in next(it)) + " )")
                    lvl += 1
                print("values : ( " + ", ".join(repr(float(x)) for x in bufs[-1]) + " )")
                print("----")

            return print_tensor
        if kind == "bspmm":
            fn = getattr(lib, symbol)

            def bspmm(pos, crd, val, spec, B):
                flat = np.array(list(spec[0]) + list(spec[1]), dtype=np.int64)
                if flat.shape != (6,):
                    raise LapisError(1, "the CSRV specifier is ((n1, n2, nh), (len pos, len crd, len val))")
                if _resident(pos, crd, val, B):
                    from . import device as D
                    from .dualview import DualView
                    pos, crd = self._dv(pos, idx_dtype), self._dv(crd, idx_dtype)
                    val, B = self._dv(val, np.float32), self._dv(B, np.float32)
                    if (pos.extent(0), crd.extent(0), val.extent(0)) != tuple(flat[3:]) or flat[3] != flat[0] + 1:
                        raise LapisError(1, "storage specifier does not match the pos/crd/val arrays")
                    C = D.bspmm_csrv(pos.device_view(), crd.device_view(), val.device_view(), B.device_view(),
                                     int(flat[1]), None)
                    return DualView.from_device(C)
                pos = np.require(pos, dtype=idx_dtype, requirements=["C"])
                crd = np.require(crd, dtype=idx_dtype, requirements=["C"])
                val = np.require(val, dtype=np.float32, requirements=["C"])
                B = np.require(B, dtype=np.float32, requirements=["C"])
                ret0 = _ret_slot(3)
                fn(ret0, _desc(pos), _desc(crd), _desc(val), flat.ctypes.data_as(ctypes.c_void_p), _desc(B))
                check_last()
                return rt.ranked_memref_to_numpy(ret0[0], np.float32)

            return bspmm
        if kind == "spmm_dcsr":
            fn = getattr(lib, symbol)

            def spmm_dcsr(p1, i1, p2, i2, val, spec, B, C):
                flat = np.array(list(spec[0]) + list(spec[1]), dtype=np.int64)
                if flat.shape != (7,):
                    raise LapisError(1, "the DCSR specifier is ((rows, cols), (len p1, len i1, len p2, len i2, len val))")
                if _resident(p1, i1, p2, i2, val, B, C):
                    from . import device as D
                    i1, p2, i2 = (self._dv(t, idx_dtype) for t in (i1, p2, i2))
                    val, B, C = (self._dv(t, np.float64) for t in (val, B, C))
                    if (i1.extent(0), p2.extent(0), i2.extent(0), val.extent(0)) != tuple(flat[3:]) or flat[4] != flat[3] + 1:
                        raise LapisError(1, "storage specifier does not match the DCSR arrays")
                    D.spmm_dcsr(i1.device_view(), p2.device_view(), i2.device_view(), val.device_view(),
                                B.device_view(), C.device_view(), int(flat[1]))
                    C.modifyDevice()
                    return C
                arrs = [np.require(t, dtype=idx_dtype, requirements=["C"]) for t in (p1, i1, p2, i2)]
                val = np.require(val, dtype=np.float64, requirements=["C"])
                B = np.require(B, dtype=np.float64, requirements=["C"])
                C = np.require(C, dtype=np.float64, requirements=["C"])
                ret0 = _ret_slot(2)
                fn(ret0, *[_desc(t) for t in arrs], _desc(val), flat.ctypes.data_as(ctypes.c_void_p), _desc(B), _desc(C))
                check_last()
                return C

            return spmm_dcsr
        if kind == "mht":
            fn = getattr(lib, symbol)

            def mht(pos, crd, val, spec, mask, d, alpha, tol, maxiter):
                if _resident(pos, crd, val, mask, d):
                    from .dualview import DualView
                    A = self._plan(pos, crd, val, spec, idx_dtype)
                    mask, d = self._dv(mask, np.float64), self._dv(d, np.float64)
                    m1, m2 = A.mht(mask.device_view(), d.device_view(), float(alpha), float(tol), int(maxiter))
                    return DualView.from_device(m1), DualView.from_device(m2)
                keep, cargs = csr_args(pos, crd, val, spec)
                mask = np.require(mask, dtype=np.float64, requirements=["C"])
                d = np.require(d, dtype=np.float64, requirements=["C"])
                ret0, ret1 = _ret_slot(1), _ret_slot(1)
                fn(ret0, ret1, *cargs, _desc(mask), _desc(d), ctypes.c_double(alpha), ctypes.c_double(tol),
                   ctypes.c_size_t(maxiter))
                check_last()
                del keep
                return (rt.ranked_memref_to_numpy(ret0[0], np.float64), rt.ranked_memref_to_numpy(ret1[0], np.float64))

            return mht
        if kind == "normalize_mom2":
            fn = getattr(lib, symbol)

            def normalize_mom2(mom1, mom2):
                if _resident(mom1, mom2):
                    from . import device as D
                    from .dualview import DualView
                    mom1, mom2 = self._dv(mom1, np.float64), self._dv(mom2, np.float64)
                    return DualView.from_device(D.normalize_mom2(mom1.device_view(), mom2.device_view()))
                mom1 = np.require(mom1, dtype=np.float64, requirements=["C"])
                mom2 = np.require(mom2, dtype=np.float64, requirements=["C"])
                ret0 = _ret_slot(1)
                fn(ret0, _desc(mom1), _desc(mom2))
                check_last()
                return rt.ranked_memref_to_numpy(ret0[0], np.float64)

            return normalize_mom2
        raise AssertionError(kind)


class KokkosBackend:
    """Main entry point, same constructor as the reference class (python/lapis/KokkosBackend.py:13)."""

    def __init__(self, decompose_tensors=False, parallel_strategy="any-storage-any-loop", dump_mlir=False,
                 index_instance=0, num_instances=0, ws=os.getcwd()):
        super().__init__()
        if parallel_strategy not in _PAR_STRATEGIES:
            raise Exception(f"unknown parallelization strategy {parallel_strategy!r}")
        self.dump_mlir = dump_mlir
        self.ws = ws
        self.index_instance = index_instance
        self.num_instances = num_instances
        self.decompose_tensors = decompose_tensors
        self.parallel_strategy = parallel_strategy
        self.package_name = "lapis_package" if index_instance == 0 else "lapis_package_" + str(index_instance)

    def compile(self, module):
        moduleText = str(module)
        if self.dump_mlir:
            print("== High-Level ==")
            print(moduleText)
        encodings = _parse_encodings(moduleText)
        funcs = _parse_functions(moduleText, encodings)
        by_name = {f["name"]: f for f in funcs}
        public = [f for f in funcs if not f["private"]]
        if not public:
            raise Exception("module has no public function")
        bindings = {}
        for fn in public:
            kind, sfx, dt = _classify(fn, by_name, moduleText)
            if sfx and kind != "print" and not self.decompose_tensors:
                raise Exception("sparse tensor arguments need decompose_tensors=True (pos, crd, val, specifier "
                                "arguments); the opaque sparse-runtime handle form is not supported")
            bindings[fn["name"]] = (kind, sfx, dt)
        if self.dump_mlir:
            print("== Bound ==")
            for name, (kind, sfx, _) in bindings.items():
                print(f"@{name} -> {kind}{'_' + sfx if sfx else ''}")
        # the module's own library: py_<func> under the emitter's names, forwarding to the typed entry points
        return LAPISModule(_shim.build(bindings, self.ws, self.package_name), bindings)
