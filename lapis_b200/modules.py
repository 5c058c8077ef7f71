"""MLIR inputs of the accelerated path: the same operations a LAPIS user hands to
``KokkosBackend.compile``, written out for this package (its tests, its benchmark, and as the forms the
compile step recognises)."""

CSR32 = "#CSR = #sparse_tensor.encoding<{ map = (i, j) -> (i : dense, j : compressed), posWidth = 32, crdWidth = 32 }>"
CSR64 = "#CSR = #sparse_tensor.encoding<{ map = (i, j) -> (i : dense, j : compressed), posWidth = 64, crdWidth = 64 }>"
CSRIDX = "#CSR = #sparse_tensor.encoding<{ map = (i, j) -> (i : dense, j : compressed) }>"


def spmv(enc=CSR32):
    return enc + """
module {
  func.func @spmv(%A: tensor<?x?xf64, #CSR>, %x: tensor<?xf64>, %y: tensor<?xf64>) -> tensor<?xf64> {
    %r = linalg.matvec ins(%A, %x : tensor<?x?xf64, #CSR>, tensor<?xf64>) outs(%y : tensor<?xf64>) -> tensor<?xf64>
    return %r : tensor<?xf64>
  }
}"""


def spmm(enc=CSR64):
    return enc + """
module {
  func.func @spmm(%A: tensor<?x?xf64, #CSR>, %B: tensor<?x?xf64>, %C: tensor<?x?xf64>) -> tensor<?x?xf64> {
    %r = linalg.matmul ins(%A, %B : tensor<?x?xf64, #CSR>, tensor<?x?xf64>) outs(%C : tensor<?x?xf64>) -> tensor<?x?xf64>
    return %r : tensor<?x?xf64>
  }
}"""


MATMUL = """
module {
  func.func @forward(%a: tensor<?x?xf32>, %b: tensor<?x?xf32>, %c: tensor<?x?xf32>) -> tensor<?x?xf32> {
    %i1 = arith.constant 1 : index
    %i0 = arith.constant 0 : index
    %ka = tensor.dim %a, %i1 : tensor<?x?xf32>
    %kb = tensor.dim %b, %i0 : tensor<?x?xf32>
    %same = arith.cmpi eq, %ka, %kb : index
    cf.assert %same, "mismatching contracting dimension for torch.aten.mm"
    %r = linalg.matmul ins(%a, %b : tensor<?x?xf32>, tensor<?x?xf32>) outs(%c : tensor<?x?xf32>) -> tensor<?x?xf32>
    return %r : tensor<?x?xf32>
  }
}"""

BATCH_MATMUL = """
module {
  func.func @forward(%a: tensor<?x?x?xf32>, %b: tensor<?x?x?xf32>, %c: tensor<?x?x?xf32>) -> tensor<?x?x?xf32> {
    %r = linalg.batch_matmul ins(%a, %b : tensor<?x?x?xf32>, tensor<?x?x?xf32>) outs(%c : tensor<?x?x?xf32>) -> tensor<?x?x?xf32>
    return %r : tensor<?x?x?xf32>
  }
}"""


def pcg(enc=CSR32):
    return enc + """
#id = affine_map<(i) -> (i)>
module {
  func.func private @spmv(%A: tensor<?x?xf64, #CSR>, %x: tensor<?xf64>, %y: tensor<?xf64>) -> tensor<?xf64> {
    %z = arith.constant 0.0 : f64
    %y0 = linalg.fill ins(%z : f64) outs(%y : tensor<?xf64>) -> tensor<?xf64>
    %r = linalg.matvec ins(%A, %x : tensor<?x?xf64, #CSR>, tensor<?xf64>) outs(%y0 : tensor<?xf64>) -> tensor<?xf64>
    return %r : tensor<?xf64>
  }
  func.func private @dot(%x: tensor<?xf64>, %y: tensor<?xf64>) -> f64 {
    %z = arith.constant 0.0 : f64
    %acc = tensor.splat %z[] : tensor<f64>
    %d = linalg.dot ins(%x, %y : tensor<?xf64>, tensor<?xf64>) outs(%acc : tensor<f64>) -> tensor<f64>
    %s = tensor.extract %d[] : tensor<f64>
    return %s : f64
  }
  func.func private @axpby(%a: f64, %x: tensor<?xf64>, %b: f64, %y: tensor<?xf64>, %dst: tensor<?xf64>) -> tensor<?xf64> {
    %r = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel"]}
        ins(%x, %y : tensor<?xf64>, tensor<?xf64>) outs(%dst : tensor<?xf64>) {
    ^bb0(%xv: f64, %yv: f64, %o: f64):
      %t0 = arith.mulf %xv, %a : f64
      %t1 = arith.mulf %yv, %b : f64
      %t2 = arith.addf %t0, %t1 : f64
      linalg.yield %t2 : f64
    } -> tensor<?xf64>
    return %r : tensor<?xf64>
  }
  func.func private @mult(%x: tensor<?xf64>, %y: tensor<?xf64>, %dst: tensor<?xf64>) -> tensor<?xf64> {
    %r = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel"]}
        ins(%x, %y : tensor<?xf64>, tensor<?xf64>) outs(%dst : tensor<?xf64>) {
    ^bb0(%xv: f64, %yv: f64, %o: f64):
      %t = arith.mulf %xv, %yv : f64
      linalg.yield %t : f64
    } -> tensor<?xf64>
    return %r : tensor<?xf64>
  }
  func.func @pcg(%A: tensor<?x?xf64, #CSR>, %b: tensor<?xf64>, %dinv: tensor<?xf64>, %tol: f64, %maxiter: index) -> (tensor<?xf64>, index, f64) {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %n = tensor.dim %b, %c0 : tensor<?xf64>
    %f0 = arith.constant 0.0 : f64
    %f1 = arith.constant 1.0 : f64
    %e0 = tensor.empty(%n) : tensor<?xf64>
    %e1 = tensor.empty(%n) : tensor<?xf64>
    %e2 = tensor.empty(%n) : tensor<?xf64>
    %e3 = tensor.empty(%n) : tensor<?xf64>
    %r0 = linalg.copy ins(%b : tensor<?xf64>) outs(%e0 : tensor<?xf64>) -> tensor<?xf64>
    %z0 = func.call @mult(%r0, %dinv, %e1) : (tensor<?xf64>, tensor<?xf64>, tensor<?xf64>) -> tensor<?xf64>
    %p0 = linalg.copy ins(%z0 : tensor<?xf64>) outs(%e2 : tensor<?xf64>) -> tensor<?xf64>
    %x0 = tensor.splat %f0[%n] : tensor<?xf64>
    %rr0 = func.call @dot(%r0, %r0) : (tensor<?xf64>, tensor<?xf64>) -> f64
    %res0 = math.sqrt %rr0 : f64
    %x, %p, %z, %r, %relres, %rzout, %iters = scf.while (%xi = %x0, %pi = %p0, %zi = %z0, %ri = %r0, %rzi = %f0, %i = %c1)
        : (tensor<?xf64>, tensor<?xf64>, tensor<?xf64>, tensor<?xf64>, f64, index)
        -> (tensor<?xf64>, tensor<?xf64>, tensor<?xf64>, tensor<?xf64>, f64, f64, index) {
      %Ap = func.call @spmv(%A, %pi, %e3) : (tensor<?x?xf64, #CSR>, tensor<?xf64>, tensor<?xf64>) -> tensor<?xf64>
      %pAp = func.call @dot(%pi, %Ap) : (tensor<?xf64>, tensor<?xf64>) -> f64
      %rz = func.call @dot(%ri, %zi) : (tensor<?xf64>, tensor<?xf64>) -> f64
      %alpha = arith.divf %rz, %pAp : f64
      %nalpha = arith.negf %alpha : f64
      %xn = func.call @axpby(%f1, %xi, %alpha, %pi, %xi) : (f64, tensor<?xf64>, f64, tensor<?xf64>, tensor<?xf64>) -> tensor<?xf64>
      %rn = func.call @axpby(%f1, %ri, %nalpha, %Ap, %ri) : (f64, tensor<?xf64>, f64, tensor<?xf64>, tensor<?xf64>) -> tensor<?xf64>
      %rr = func.call @dot(%rn, %rn) : (tensor<?xf64>, tensor<?xf64>) -> f64
      %nrm = math.sqrt %rr : f64
      %rel = arith.divf %nrm, %res0 : f64
      %open = arith.cmpf ogt, %rel, %tol : f64
      %more = arith.cmpi ne, %i, %maxiter : index
      %go = arith.andi %open, %more : i1
      scf.condition(%go) %xn, %pi, %zi, %rn, %rel, %rz, %i : tensor<?xf64>, tensor<?xf64>, tensor<?xf64>, tensor<?xf64>, f64, f64, index
    } do {
    ^bb0(%xi: tensor<?xf64>, %pi: tensor<?xf64>, %zi: tensor<?xf64>, %ri: tensor<?xf64>, %unused: f64, %rzi: f64, %i: index):
      %zn = func.call @mult(%ri, %dinv, %zi) : (tensor<?xf64>, tensor<?xf64>, tensor<?xf64>) -> tensor<?xf64>
      %rzn = func.call @dot(%ri, %zn) : (tensor<?xf64>, tensor<?xf64>) -> f64
      %beta = arith.divf %rzn, %rzi : f64
      %pn = func.call @axpby(%f1, %zn, %beta, %pi, %pi) : (f64, tensor<?xf64>, f64, tensor<?xf64>, tensor<?xf64>) -> tensor<?xf64>
      %in = arith.addi %i, %c1 : index
      scf.yield %xi, %pn, %zn, %ri, %rzn, %in : tensor<?xf64>, tensor<?xf64>, tensor<?xf64>, tensor<?xf64>, f64, index
    }
    return %x, %iters, %relres : tensor<?xf64>, index, f64
  }
}"""

def hitting_times(enc=CSR32):
    """The hitting-time moments program (the operations of examples/hitting_times.py in the LAPIS project: a
    masked-Laplacian operator, a PCG loop that divides by the diagonal, the two-moment driver and the
    normalisation), written out for these tests."""
    vec = "tensor<?xf64>"
    mat = "tensor<?x?xf64, #CSR>"
    ew = '{indexing_maps = [#id, #id, #id], iterator_types = ["parallel"]}'
    ew5 = '{indexing_maps = [#id, #id, #id, #id, #id], iterator_types = ["parallel"]}'
    return enc + f"""
#id = affine_map<(i) -> (i)>
module {{
  func.func private @spmv(%A: {mat}, %x: {vec}, %y: {vec}) -> {vec} {{
    %z = arith.constant 0.0 : f64
    %y0 = linalg.fill ins(%z : f64) outs(%y : {vec}) -> {vec}
    %r = linalg.matvec ins(%A, %x : {mat}, {vec}) outs(%y0 : {vec}) -> {vec}
    return %r : {vec}
  }}
  func.func private @dot(%x: {vec}, %y: {vec}) -> f64 {{
    %z = arith.constant 0.0 : f64
    %acc = tensor.splat %z[] : tensor<f64>
    %d = linalg.dot ins(%x, %y : {vec}, {vec}) outs(%acc : tensor<f64>) -> tensor<f64>
    %s = tensor.extract %d[] : tensor<f64>
    return %s : f64
  }}
  func.func private @axpby(%a: f64, %x: {vec}, %b: f64, %y: {vec}, %dst: {vec}) -> {vec} {{
    %r = linalg.generic {ew} ins(%x, %y : {vec}, {vec}) outs(%dst : {vec}) {{
    ^bb0(%xv: f64, %yv: f64, %o: f64):
      %t0 = arith.mulf %xv, %a : f64
      %t1 = arith.mulf %yv, %b : f64
      %t2 = arith.addf %t0, %t1 : f64
      linalg.yield %t2 : f64
    }} -> {vec}
    return %r : {vec}
  }}
  func.func private @mult(%x: {vec}, %y: {vec}, %dst: {vec}) -> {vec} {{
    %r = linalg.generic {ew} ins(%x, %y : {vec}, {vec}) outs(%dst : {vec}) {{
    ^bb0(%xv: f64, %yv: f64, %o: f64):
      %t = arith.mulf %xv, %yv : f64
      linalg.yield %t : f64
    }} -> {vec}
    return %r : {vec}
  }}
  func.func private @scale_csr(%A: {mat}, %alpha: f64) -> {mat} {{
    %r = linalg.generic {{indexing_maps = [affine_map<(i, j) -> (i, j)>], iterator_types = ["parallel", "parallel"]}}
        outs(%A : {mat}) {{
    ^bb0(%a: f64):
      %s = sparse_tensor.unary %a : f64 to f64
        present = {{
        ^bb1(%v: f64):
          %t = arith.mulf %v, %alpha : f64
          sparse_tensor.yield %t : f64
        }}
        absent = {{}}
      linalg.yield %s : f64
    }} -> {mat}
    return %r : {mat}
  }}
  func.func private @plpt(%A: {mat}, %x: {vec}, %d: {vec}, %mask: {vec}, %tmp: {vec}, %dst: {vec}) -> {vec} {{
    %mx = func.call @mult(%x, %mask, %tmp) : ({vec}, {vec}, {vec}) -> {vec}
    %amx = func.call @spmv(%A, %mx, %dst) : ({mat}, {vec}, {vec}) -> {vec}
    %r = linalg.generic {ew5} ins(%amx, %mx, %mask, %d : {vec}, {vec}, {vec}, {vec}) outs(%dst : {vec}) {{
    ^bb0(%av: f64, %xv: f64, %mv: f64, %dv: f64, %o: f64):
      %t0 = arith.mulf %dv, %xv : f64
      %t1 = arith.subf %t0, %av : f64
      %t2 = arith.mulf %t1, %mv : f64
      linalg.yield %t2 : f64
    }} -> {vec}
    return %r : {vec}
  }}
  func.func private @pcg(%A: {mat}, %b: {vec}, %mask: {vec}, %d: {vec}, %tol: f64, %maxiter: index) -> ({vec}, index, f64) {{
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %n = tensor.dim %b, %c0 : {vec}
    %f0 = arith.constant 0.0 : f64
    %f1 = arith.constant 1.0 : f64
    %e0 = tensor.empty(%n) : {vec}
    %e1 = tensor.empty(%n) : {vec}
    %e2 = tensor.empty(%n) : {vec}
    %e3 = tensor.empty(%n) : {vec}
    %e4 = tensor.empty(%n) : {vec}
    %r0 = linalg.copy ins(%b : {vec}) outs(%e0 : {vec}) -> {vec}
    %z0 = linalg.div ins(%r0, %d : {vec}, {vec}) outs(%e1 : {vec}) -> {vec}
    %p0 = linalg.copy ins(%z0 : {vec}) outs(%e2 : {vec}) -> {vec}
    %x0 = tensor.splat %f0[%n] : {vec}
    %rr0 = func.call @dot(%r0, %r0) : ({vec}, {vec}) -> f64
    %res0 = math.sqrt %rr0 : f64
    %x, %p, %z, %r, %relres, %rzout, %iters = scf.while (%xi = %x0, %pi = %p0, %zi = %z0, %ri = %r0, %rzi = %f0, %i = %c1)
        : ({vec}, {vec}, {vec}, {vec}, f64, index) -> ({vec}, {vec}, {vec}, {vec}, f64, f64, index) {{
      %Ap = func.call @plpt(%A, %pi, %d, %mask, %e3, %e4) : ({mat}, {vec}, {vec}, {vec}, {vec}, {vec}) -> {vec}
      %pAp = func.call @dot(%pi, %Ap) : ({vec}, {vec}) -> f64
      %rz = func.call @dot(%ri, %zi) : ({vec}, {vec}) -> f64
      %alpha = arith.divf %rz, %pAp : f64
      %nalpha = arith.negf %alpha : f64
      %xn = func.call @axpby(%f1, %xi, %alpha, %pi, %xi) : (f64, {vec}, f64, {vec}, {vec}) -> {vec}
      %rn = func.call @axpby(%f1, %ri, %nalpha, %Ap, %ri) : (f64, {vec}, f64, {vec}, {vec}) -> {vec}
      %rr = func.call @dot(%rn, %rn) : ({vec}, {vec}) -> f64
      %nrm = math.sqrt %rr : f64
      %rel = arith.divf %nrm, %res0 : f64
      %open = arith.cmpf ogt, %rel, %tol : f64
      %more = arith.cmpi ne, %i, %maxiter : index
      %go = arith.andi %open, %more : i1
      scf.condition(%go) %xn, %pi, %zi, %rn, %rel, %rz, %i : {vec}, {vec}, {vec}, {vec}, f64, f64, index
    }} do {{
    ^bb0(%xi: {vec}, %pi: {vec}, %zi: {vec}, %ri: {vec}, %unused: f64, %rzi: f64, %i: index):
      %zn = linalg.div ins(%ri, %d : {vec}, {vec}) outs(%zi : {vec}) -> {vec}
      %rzn = func.call @dot(%ri, %zn) : ({vec}, {vec}) -> f64
      %beta = arith.divf %rzn, %rzi : f64
      %pn = func.call @axpby(%f1, %zn, %beta, %pi, %pi) : (f64, {vec}, f64, {vec}, {vec}) -> {vec}
      %in = arith.addi %i, %c1 : index
      scf.yield %xi, %pn, %zn, %ri, %rzn, %in : {vec}, {vec}, {vec}, {vec}, f64, index
    }}
    return %x, %iters, %relres : {vec}, index, f64
  }}
  func.func @mht(%A: {mat}, %mask: {vec}, %d: {vec}, %alpha: f64, %tol: f64, %maxiter: index) -> ({vec}, {vec}) {{
    %c0 = arith.constant 0 : index
    %As = func.call @scale_csr(%A, %alpha) : ({mat}, f64) -> {mat}
    %n = tensor.dim %d, %c0 : {vec}
    %e0 = tensor.empty(%n) : {vec}
    %b1 = func.call @mult(%d, %mask, %e0) : ({vec}, {vec}, {vec}) -> {vec}
    %m1, %i1, %r1 = func.call @pcg(%As, %b1, %mask, %d, %tol, %maxiter) : ({mat}, {vec}, {vec}, {vec}, f64, index) -> ({vec}, index, f64)
    %am1 = func.call @spmv(%As, %m1, %e0) : ({mat}, {vec}, {vec}) -> {vec}
    %b2 = linalg.generic {ew5} ins(%am1, %mask, %m1, %d : {vec}, {vec}, {vec}, {vec}) outs(%e0 : {vec}) {{
    ^bb0(%av: f64, %mv: f64, %xv: f64, %dv: f64, %o: f64):
      %t0 = arith.mulf %dv, %xv : f64
      %t1 = arith.addf %t0, %av : f64
      %t2 = arith.mulf %t1, %mv : f64
      linalg.yield %t2 : f64
    }} -> {vec}
    %m2, %i2, %r2 = func.call @pcg(%As, %b2, %mask, %d, %tol, %maxiter) : ({mat}, {vec}, {vec}, {vec}, f64, index) -> ({vec}, index, f64)
    return %m1, %m2 : {vec}, {vec}
  }}
  func.func @normalize_mom2(%m1: {vec}, %m2: {vec}) -> {vec} {{
    %c0 = arith.constant 0 : index
    %n = tensor.dim %m1, %c0 : {vec}
    %e0 = tensor.empty(%n) : {vec}
    %r = linalg.generic {ew} ins(%m1, %m2 : {vec}, {vec}) outs(%e0 : {vec}) {{
    ^bb0(%a: f64, %b: f64, %o: f64):
      %sq = arith.mulf %a, %a : f64
      %var = arith.subf %b, %sq : f64
      %sd = math.sqrt %var : f64
      linalg.yield %sd : f64
    }} -> {vec}
    return %r : {vec}
  }}
}}"""


CSRV32 = ("#CSRV = #sparse_tensor.encoding<{ map = (i, j, h) -> (i : dense, j : compressed, h : dense), "
          "posWidth = 32, crdWidth = 32 }>")
CSRV64 = "#CSRV = #sparse_tensor.encoding<{ map = (i, j, h) -> (i : dense, j : compressed, h : dense) }>"


def bspmm(enc=CSRV32):
    """Batched SpMM over a CSRV tensor: out(n1, dh, nh) = sum over n2 of A(n1, n2, nh) * B(n2, dh, nh), the
    operation of examples/bspmm.py in the LAPIS project, written out for these tests."""
    return enc + """
#trait = {
  indexing_maps = [affine_map<(n1, n2, dh, nh) -> (n1, n2, nh)>,
                   affine_map<(n1, n2, dh, nh) -> (n2, dh, nh)>,
                   affine_map<(n1, n2, dh, nh) -> (n1, dh, nh)>],
  iterator_types = ["parallel", "reduction", "parallel", "parallel"]
}
module {
  func.func @bspmm(%A: tensor<?x?x?xf32, #CSRV>, %B: tensor<?x?x?xf32>) -> tensor<?x?x?xf32> {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %c2 = arith.constant 2 : index
    %z = arith.constant 0.0 : f32
    %n1 = tensor.dim %A, %c0 : tensor<?x?x?xf32, #CSRV>
    %nh = tensor.dim %A, %c2 : tensor<?x?x?xf32, #CSRV>
    %dh = tensor.dim %B, %c1 : tensor<?x?x?xf32>
    %e = tensor.empty(%n1, %dh, %nh) : tensor<?x?x?xf32>
    %init = linalg.fill ins(%z : f32) outs(%e : tensor<?x?x?xf32>) -> tensor<?x?x?xf32>
    %r = linalg.generic #trait ins(%A, %B : tensor<?x?x?xf32, #CSRV>, tensor<?x?x?xf32>) outs(%init : tensor<?x?x?xf32>) {
    ^bb0(%a: f32, %b: f32, %o: f32):
      %p = arith.mulf %a, %b : f32
      %s = arith.addf %p, %o : f32
      linalg.yield %s : f32
    } -> tensor<?x?x?xf32>
    return %r : tensor<?x?x?xf32>
  }
}"""


DCSR64 = "#DCSR = #sparse_tensor.encoding<{ map = (i, j) -> (i : compressed, j : compressed) }>"
DCSR32 = "#DCSR = #sparse_tensor.encoding<{ map = (i, j) -> (i : compressed, j : compressed), posWidth = 32, crdWidth = 32 }>"


def spmm_dcsr(enc=DCSR64):
    """C += A B with A compressed in both levels (the operation of examples/spmm_dcsr_opdsl.py)."""
    return enc + """
module {
  func.func @spMxM(%A: tensor<?x?xf64, #DCSR>, %B: tensor<?x?xf64>, %C: tensor<?x?xf64>) -> tensor<?x?xf64> {
    %r = linalg.matmul ins(%A, %B : tensor<?x?xf64, #DCSR>, tensor<?x?xf64>) outs(%C : tensor<?x?xf64>) -> tensor<?x?xf64>
    return %r : tensor<?x?xf64>
  }
}"""


UNSUPPORTED = """
module {
  func.func @relu(%x: tensor<?xf32>) -> tensor<?xf32> {
    %z = arith.constant 0.0 : f32
    %r = linalg.generic {indexing_maps = [affine_map<(i) -> (i)>, affine_map<(i) -> (i)>], iterator_types = ["parallel"]}
        ins(%x : tensor<?xf32>) outs(%x : tensor<?xf32>) {
    ^bb0(%v: f32, %o: f32):
      %m = arith.maximumf %v, %z : f32
      linalg.yield %m : f32
    } -> tensor<?xf32>
    return %r : tensor<?xf32>
  }
}"""
