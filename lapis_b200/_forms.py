"""Canonical forms of the MLIR functions that ``KokkosBackend.compile`` binds to prebuilt kernels.

The compile step has no MLIR lowering: a function is bound to a kernel only if it IS one of the known
operations, not if it merely resembles one.  Two checks, both on the text:

* single-operation functions (CSR matvec / matmul, dense matmul / batch_matmul): the body may contain one
  named linalg operation, wired from the function's first two arguments into its third and returned, plus
  shape bookkeeping without effect on the result (constants, ``tensor.dim``, index casts, comparisons,
  ``cf.assert``).  Anything else in the body -- a scale after the product, a second operation -- is refused.
* multi-operation functions (the PCG loop, the hitting-time moments, the CSRV batched SpMM, ...): the
  function together with every function it calls is brought into a canonical form (comments and dead
  bookkeeping removed, affine-map and trait aliases expanded, SSA values / blocks / aliases renamed in order
  of appearance, dimension names of affine maps normalised, whitespace dropped) and its SHA-256 must be one
  of the accepted digests: those of this package's own module texts (lapis_b200/modules.py) and those of the
  LAPIS project's example scripts (lapis_b200/_accepted_forms.py, generated from the examples read as text
  by tests/golden/make_accepted_forms.py).  A loop with another stop test or another initial guess has
  another digest and is refused.
"""
from __future__ import annotations

import hashlib
import re

_DEAD_OK = ("arith.constant", "tensor.dim", "tensor.empty", "arith.index_cast", "arith.cmpi")
_ID = r"%[\w.$-]+"


def strip_comments(text: str) -> str:
    return re.sub(r"//[^\n]*", "", text)


def function_texts(module_text: str) -> dict:
    """name -> text of every ``func.func`` (signature and body)."""
    out = {}
    text = strip_comments(module_text)
    for m in re.finditer(r"func\.func\s+(?:private\s+)?@(\w+)\s*\(", text):
        i, depth = m.end(), 1
        while depth:
            depth += {"(": 1, ")": -1}.get(text[i], 0)
            i += 1
        j = text.index("{", i)
        k, depth = j + 1, 1
        while depth:
            depth += {"{": 1, "}": -1}.get(text[k], 0)
            k += 1
        out[m.group(1)] = text[m.start():k]
    return out


def aliases(module_text: str) -> dict:
    """Top-level ``#name = value`` definitions other than sparse-tensor encodings, value text balanced."""
    text = strip_comments(module_text)
    out = {}
    for m in re.finditer(r"^\s*(#\w+)\s*=\s*", text, re.M):
        i = m.end()
        if text.startswith("#sparse_tensor", i):
            continue
        depth, j = 0, i
        while j < len(text):
            ch = text[j]
            if ch in "<{[(":
                depth += 1
            elif ch in ">}])":
                # '->' inside affine maps is not a closing bracket
                if not (ch == ">" and text[j - 1] == "-"):
                    depth -= 1
            elif ch == "\n" and depth == 0:
                break
            j += 1
        out[m.group(1)] = text[i:j].strip()
    return out


def _normalise_affine_dims(text: str) -> str:
    def fix(m):
        dims = [d.strip() for d in m.group(1).split(",")]
        body = m.group(2)
        for n, d in enumerate(dims):
            body = re.sub(r"\b" + re.escape(d) + r"\b", f"d{n}", body)
        return "affine_map<(" + ",".join(f"d{n}" for n in range(len(dims))) + ")->(" + body + ")>"
    return re.sub(r"affine_map<\(([^)]*)\)\s*->\s*\(([^)]*)\)>", fix, text)


def canonical(name: str, fn_text: str, module_text: str) -> str:
    t = strip_comments(fn_text)
    for alias, value in aliases(module_text).items():
        t = re.sub(re.escape(alias) + r"(?![\w])", lambda _m, v=value: v, t)
    t = _normalise_affine_dims(t)
    t = re.sub(r"func\.func\s+private\s+", "func.func ", t)
    t = re.sub(r"@" + re.escape(name) + r"(?=\s*\()", "@__F__", t, count=1)
    lines = [ln.strip() for ln in t.split("\n") if ln.strip()]
    changed = True
    while changed:  # bookkeeping whose single result nobody reads
        changed = False
        for i, ln in enumerate(lines):
            m = re.match(r"(" + _ID + r")\s*=\s*([\w.]+)", ln)
            if m and m.group(2) in _DEAD_OK:
                pat = re.compile(re.escape(m.group(1)) + r"(?![\w.$-])")
                if not any(pat.search(x) for j, x in enumerate(lines) if j != i):
                    del lines[i]
                    changed = True
                    break
    t = "\n".join(lines)
    ids, blocks, als = {}, {}, {}
    t = re.sub(_ID, lambda m: ids.setdefault(m.group(0), f"%{len(ids)}"), t)
    t = re.sub(r"\^\w+", lambda m: blocks.setdefault(m.group(0), f"^b{len(blocks)}"), t)
    t = re.sub(r"#(?!sparse_tensor)\w+", lambda m: als.setdefault(m.group(0), f"#a{len(als)}"), t)
    t = re.sub(r"\s+", "", t)
    t = re.sub(r"(\d)\.0+e\+00", r"\1.0", t)  # 0.000000e+00 and 0.0 are the same constant
    return t


def closure_digest(name: str, module_text: str) -> str:
    """SHA-256 over the canonical forms of @name and of every function it calls, directly or not."""
    fns = function_texts(module_text)
    if name not in fns:
        raise KeyError(name)
    seen, todo = [], [name]
    while todo:
        f = todo.pop()
        if f in seen:
            continue
        seen.append(f)
        for callee in re.findall(r"@(\w+)", fns[f]):
            if callee in fns and callee not in seen:
                todo.append(callee)
    parts = [canonical(name, fns[name], module_text)]
    parts += [f + ":" + canonical(f, fns[f], module_text) for f in sorted(seen) if f != name]
    return hashlib.sha256("\n".join(parts).encode()).hexdigest()


def single_named_op(fn_text: str, op: str) -> bool:
    """True iff the function body is ``%r = linalg.<op> ins(%arg0, %arg1 ...) outs(%arg2 ...)`` returned as
    is, plus bookkeeping that cannot change the result."""
    t = strip_comments(fn_text)
    sig = re.match(r"func\.func\s+(?:private\s+)?@\w+\s*\((.*?)\)\s*->", t, re.S)
    if not sig:
        return False
    args = re.findall(r"(" + _ID + r")\s*:", sig.group(1))
    if len(args) != 3:
        return False
    body = t[t.index("{", sig.end()) + 1:t.rindex("}")]
    stmts = [s.strip() for s in body.split("\n") if s.strip()]
    result = None
    for s in stmts:
        m = re.match(r"(" + _ID + r")\s*=\s*linalg\.(\w+)\s+ins\(\s*(" + _ID + r")\s*,\s*(" + _ID + r")\s*:[^)]*\)\s*outs\(\s*("
                     + _ID + r")\s*:[^)]*\)\s*->", s)
        if m:
            if result is not None or m.group(2) != op or [m.group(3), m.group(4), m.group(5)] != args:
                return False
            result = m.group(1)
            continue
        if re.match(r"(?:func\.)?return\s+(" + _ID + r")\s*:", s):
            if result is None or re.match(r"(?:func\.)?return\s+(" + _ID + r")", s).group(1) != result:
                return False
            continue
        if re.match(_ID + r"\s*=\s*(arith\.constant|tensor\.dim|arith\.index_cast|arith\.cmpi)\b", s) or re.match(r"cf\.assert\b", s):
            continue
        return False
    return result is not None


_OWN = None


def accepted_digests() -> set:
    """Digests of this package's own module texts and of the LAPIS examples'."""
    global _OWN
    if _OWN is None:
        from . import modules as mm
        own = set()
        for text, names in ((mm.pcg(mm.CSR32), ["pcg"]), (mm.hitting_times(mm.CSR32), ["mht", "normalize_mom2"]),
                            (mm.bspmm(mm.CSRV32), ["bspmm"])):
            for n in names:
                own.add(closure_digest(n, text))
        try:
            from ._accepted_forms import REFERENCE_EXAMPLE_DIGESTS
            own |= set(REFERENCE_EXAMPLE_DIGESTS.values())
        except ImportError:
            pass
        _OWN = own
    return _OWN
