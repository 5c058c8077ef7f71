/*
 * CPU oracle for the LAPIS data-parallel hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the loops that LAPIS's Kokkos emitter produces
 * for CSR SpMV / SpMM, dense and batched matmul, the vector kernels and the PCG
 * solve loop, in the evaluation order of a Kokkos Serial / OpenMP build.  It is
 * the checker the CUDA kernels are compared with and the timed CPU baseline;
 * nothing in the product path may call, link or load it.
 *
 * Parity status: the reference's own executable (lapis-opt, lapis-translate,
 * Kokkos) cannot be built where this file was written, so the restatement is
 * pinned against the known answers the reference's example tests hold:
 *   examples/spmv_noalloc.py:16-37   (5x5 CSR SpMV, expected y)
 *   examples/pcg_solve.py:106-141    (PCG on data/nos4.mtx vs scipy cg)
 *   examples/hitting_times.py:196-228 (two 17-digit golden vectors of a PCG
 *                                      based solve on data/mht_A.mtx, mht_D.mtx)
 *   examples/gemm_no_alloc.py:28-52, examples/batched_gemm_no_alloc.py:33-59
 * Below np.allclose precision (rtol 1e-5) the reference pins nothing except
 * the hitting-times vectors, which are printed to 17 digits.
 *
 * Every function cites the reference lines (paths within the LAPIS project)
 * whose loop it follows.  `nthreads <= 1` gives the Kokkos-Serial order
 * (deterministic; this is what tests compare with).  `nthreads > 1` runs rows /
 * elements under OpenMP the way a Kokkos-OpenMP build would and is used only
 * for the timed CPU baseline.
 *
 * Build with -ffp-contract=off: the emitted code has separate arith.mulf and
 * arith.addf operations and a Debug-built Kokkos module does not fuse them.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

static int clamp_threads(int nthreads) {
#ifdef _OPENMP
  if (nthreads <= 0) return 1;
  return nthreads;
#else
  (void)nthreads;
  return 1;
#endif
}

ORACLE_API int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------
 * CSR SpMV.  tests/Dialect/Kokkos/loop_mapping_2.mlir.gold:12-37: per row,
 * init = y[row]; lo = pos[row]; hi = pos[row+1]; the inner range_parallel
 * reduces val[j]*x[crd[j]] over j in [lo,hi).  The emitter starts the inner
 * reduction from the identity and joins the init afterwards
 * (mlir/lib/Target/KokkosCpp/TranslateToKokkosCpp.cpp:1671-1690, :1821-1841),
 * so the result is (((0 + p_lo) + p_lo+1) + ...) + y_in.
 * ---------------------------------------------------------------------- */
#define DEFINE_SPMV(SUFFIX, IDX)                                                      \
  ORACLE_API void oracle_spmv_f64_##SUFFIX(int64_t nrows, const IDX *pos,             \
                                           const IDX *crd, const double *val,         \
                                           const double *x, double *y, int nthreads) { \
    int nt = clamp_threads(nthreads);                                                 \
    (void)nt;                                                                         \
    _Pragma("omp parallel for schedule(static) num_threads(nt) if (nt > 1)")          \
    for (int64_t row = 0; row < nrows; row++) {                                       \
      double init = y[row];                                                           \
      int64_t lo = (int64_t)pos[row], hi = (int64_t)pos[row + 1];                     \
      double acc = 0.0;                                                               \
      for (int64_t j = lo; j < hi; j++) {                                             \
        double prod = val[j] * x[(int64_t)crd[j]];                                    \
        acc = acc + prod;                                                             \
      }                                                                               \
      y[row] = acc + init;                                                            \
    }                                                                                 \
  }
DEFINE_SPMV(i32, int32_t)
DEFINE_SPMV(i64, int64_t)

/* ------------------------------------------------------------------------
 * CSR SpMM, sparse A (nrows x ncols) times dense row-major B (ncols x k) into
 * dense row-major C (nrows x k): C[i,c] = C_in[i,c] + sum_j val[j]*B[crd[j],c].
 * Generic sparse-times-dense form of examples/bspmm.py:15-23,43-50 and
 * examples/spmm_dcsr_opdsl.py:40-101; only the outer row loop is parallel
 * (spmm_dcsr_opdsl.py:132-135), j ascends sequentially inside a row, and the
 * reduction init is joined last as in SpMV.
 * ---------------------------------------------------------------------- */
#define DEFINE_SPMM(SUFFIX, IDX)                                                      \
  ORACLE_API void oracle_spmm_f64_##SUFFIX(int64_t nrows, int64_t k, const IDX *pos,  \
                                           const IDX *crd, const double *val,         \
                                           const double *B, double *C, int nthreads) { \
    int nt = clamp_threads(nthreads);                                                 \
    (void)nt;                                                                         \
    _Pragma("omp parallel for schedule(static) num_threads(nt) if (nt > 1)")          \
    for (int64_t row = 0; row < nrows; row++) {                                       \
      int64_t lo = (int64_t)pos[row], hi = (int64_t)pos[row + 1];                     \
      double *crow = C + row * k;                                                     \
      for (int64_t c0 = 0; c0 < k; c0 += 64) {                                        \
        int64_t cw = k - c0 < 64 ? k - c0 : 64;                                       \
        double acc[64];                                                               \
        for (int64_t c = 0; c < cw; c++) acc[c] = 0.0;                                \
        for (int64_t j = lo; j < hi; j++) {                                           \
          double a = val[j];                                                          \
          const double *brow = B + (int64_t)crd[j] * k + c0;                          \
          for (int64_t c = 0; c < cw; c++) acc[c] = acc[c] + a * brow[c];             \
        }                                                                             \
        for (int64_t c = 0; c < cw; c++) crow[c0 + c] = acc[c] + crow[c0 + c];        \
      }                                                                               \
    }                                                                                 \
  }
DEFINE_SPMM(i32, int32_t)
DEFINE_SPMM(i64, int64_t)

/* ------------------------------------------------------------------------
 * Dense and batched matmul, fp32.  tests/Dialect/Kokkos/linalg_to_loops_3
 * .mlir.gold:6-20 (from mlir/lib/Dialect/Kokkos/Transforms/
 * DenseLinalgToParallelLoops.cpp:309-348): one output element per outer
 * iteration, c0 = C[i,j]; the k loop reduces A[i,k]*B[k,j] from the identity in
 * ascending k with separate multiply and add; C[i,j] = sum + c0.  The batched
 * form (benchmarks/batched_gemm/batched_gemm.mlir:21) iterates (b,i,j) with j
 * fastest (mlir/lib/Dialect/Kokkos/Transforms/KokkosLoopMapping.cpp:608-635).
 * ---------------------------------------------------------------------- */
ORACLE_API void oracle_bgemm_f32(int64_t batch, int64_t M, int64_t N, int64_t K,
                                 const float *A, const float *B, float *C, int nthreads) {
  int nt = clamp_threads(nthreads);
  (void)nt;
  int64_t total = batch * M;
#pragma omp parallel for schedule(static) num_threads(nt) if (nt > 1)
  for (int64_t bi = 0; bi < total; bi++) {
    int64_t b = bi / M, i = bi % M;
    const float *a = A + (b * M + i) * K;
    const float *bm = B + b * K * N;
    float *c = C + (b * M + i) * N;
    for (int64_t j = 0; j < N; j++) {
      float c0 = c[j];
      float acc = 0.0f;
      for (int64_t k = 0; k < K; k++) {
        float prod = a[k] * bm[k * N + j];
        acc = acc + prod;
      }
      c[j] = acc + c0;
    }
  }
}

ORACLE_API void oracle_gemm_f32(int64_t M, int64_t N, int64_t K, const float *A,
                                const float *B, float *C, int nthreads) {
  oracle_bgemm_f32(1, M, N, K, A, B, C, nthreads);
}

/* Accuracy yardstick (not a reference restatement): the same product with a
 * double accumulator, used to measure how far either fp32 result is from the
 * exact one.  Cache-blocked over k so that large sizes finish. */
ORACLE_API void oracle_bgemm_f32_acc64(int64_t batch, int64_t M, int64_t N, int64_t K,
                                       const float *A, const float *B, const float *Cin,
                                       double *Cout, int nthreads) {
  int nt = clamp_threads(nthreads);
  (void)nt;
  int64_t total = batch * M;
#pragma omp parallel for schedule(static) num_threads(nt) if (nt > 1)
  for (int64_t bi = 0; bi < total; bi++) {
    int64_t b = bi / M, i = bi % M;
    const float *a = A + (b * M + i) * K;
    const float *bm = B + b * K * N;
    double *c = Cout + (b * M + i) * N;
    const float *cin = Cin + (b * M + i) * N;
    for (int64_t j = 0; j < N; j++) c[j] = 0.0;
    for (int64_t k = 0; k < K; k++) {
      double av = (double)a[k];
      const float *brow = bm + k * N;
      for (int64_t j = 0; j < N; j++) c[j] += av * (double)brow[j];
    }
    for (int64_t j = 0; j < N; j++) c[j] += (double)cin[j];
  }
}

/* ------------------------------------------------------------------------
 * Vector kernels used inside PCG.
 *   dot   examples/pcg_solve.py:22-28; lowered form tests/Dialect/Kokkos/
 *         linalg_to_loops_0.mlir.gold:7-18 (result = sum + init, init = 0).
 *   axpby examples/pcg_solve.py:30-39: (x*a) + (y*b), two roundings then add.
 *   mult  examples/pcg_solve.py:41-48.
 *   div   linalg.div, examples/hitting_times.py:119,143.
 * With nthreads > 1 the dot is an OpenMP reduction whose summation order
 * depends on the thread count, as a Kokkos-OpenMP parallel_reduce does.
 * ---------------------------------------------------------------------- */
ORACLE_API double oracle_dot_f64(int64_t n, const double *x, const double *y, int nthreads) {
  int nt = clamp_threads(nthreads);
  double acc = 0.0;
  if (nt > 1) {
#pragma omp parallel for schedule(static) num_threads(nt) reduction(+ : acc)
    for (int64_t i = 0; i < n; i++) acc += x[i] * y[i];
  } else {
    for (int64_t i = 0; i < n; i++) {
      double prod = x[i] * y[i];
      acc = acc + prod;
    }
  }
  return acc + 0.0;
}

ORACLE_API void oracle_axpby_f64(int64_t n, double a, const double *x, double b,
                                 const double *y, double *dst, int nthreads) {
  int nt = clamp_threads(nthreads);
  (void)nt;
#pragma omp parallel for schedule(static) num_threads(nt) if (nt > 1)
  for (int64_t i = 0; i < n; i++) {
    double t0 = x[i] * a;
    double t1 = y[i] * b;
    dst[i] = t0 + t1;
  }
}

ORACLE_API void oracle_mult_f64(int64_t n, const double *x, const double *y, double *dst,
                                int nthreads) {
  int nt = clamp_threads(nthreads);
  (void)nt;
#pragma omp parallel for schedule(static) num_threads(nt) if (nt > 1)
  for (int64_t i = 0; i < n; i++) dst[i] = x[i] * y[i];
}

ORACLE_API void oracle_div_f64(int64_t n, const double *x, const double *y, double *dst,
                               int nthreads) {
  int nt = clamp_threads(nthreads);
  (void)nt;
#pragma omp parallel for schedule(static) num_threads(nt) if (nt > 1)
  for (int64_t i = 0; i < n; i++) dst[i] = x[i] / y[i];
}

ORACLE_API void oracle_fill_f64(int64_t n, double v, double *dst, int nthreads) {
  int nt = clamp_threads(nthreads);
  (void)nt;
#pragma omp parallel for schedule(static) num_threads(nt) if (nt > 1)
  for (int64_t i = 0; i < n; i++) dst[i] = v;
}

/* ------------------------------------------------------------------------
 * PCG driver, statement for statement from examples/pcg_solve.py:52-101
 * (and the structurally identical solver of examples/hitting_times.py:97-149).
 * The operator and the preconditioner are parameters so that both examples run
 * through the same loop:
 *   op == OP_SPMV : Ap = 0; Ap += A p                (pcg_solve.py:13-20,75)
 *   op == OP_PLPT : Ap = mask*(d*(mask*p) - A(mask*p)) (hitting_times.py:73-92)
 *   precond == PC_MULT_DINV : z = r * dinv           (pcg_solve.py:66,93)
 *   precond == PC_DIV_D     : z = r / d              (hitting_times.py:119,143)
 * Optional trace arrays (length maxiter each, may be NULL) receive alpha, beta
 * and relres per iteration for step-wise comparisons.
 * ---------------------------------------------------------------------- */
enum { OP_SPMV = 0, OP_PLPT = 1 };
enum { PC_MULT_DINV = 0, PC_DIV_D = 1 };

typedef struct {
  int64_t n;
  int idx_bytes;
  const void *pos, *crd;
  const double *val;
  int op;
  const double *d, *mask; /* OP_PLPT only */
  double *tmp;            /* OP_PLPT only: mask*p */
  int nthreads;
} oracle_operator;

static void csr_matvec_acc(const oracle_operator *A, const double *x, double *y) {
  if (A->idx_bytes == 4)
    oracle_spmv_f64_i32(A->n, (const int32_t *)A->pos, (const int32_t *)A->crd, A->val, x, y,
                        A->nthreads);
  else
    oracle_spmv_f64_i64(A->n, (const int64_t *)A->pos, (const int64_t *)A->crd, A->val, x, y,
                        A->nthreads);
}

static void apply_operator(const oracle_operator *A, const double *p, double *Ap) {
  int nt = A->nthreads;
  if (A->op == OP_SPMV) {
    oracle_fill_f64(A->n, 0.0, Ap, nt);
    csr_matvec_acc(A, p, Ap);
    return;
  }
  /* hitting_times.py:73-92 */
  oracle_mult_f64(A->n, p, A->mask, A->tmp, nt);
  oracle_fill_f64(A->n, 0.0, Ap, nt);
  csr_matvec_acc(A, A->tmp, Ap);
  for (int64_t i = 0; i < A->n; i++) {
    double t1 = A->d[i] * A->tmp[i];
    double t2 = t1 - Ap[i];
    Ap[i] = t2 * A->mask[i];
  }
}

static void precondition(int precond, int64_t n, const double *r, const double *dvec, double *z,
                         int nt) {
  if (precond == PC_MULT_DINV)
    oracle_mult_f64(n, r, dvec, z, nt);
  else
    oracle_div_f64(n, r, dvec, z, nt);
}

/* work: 4*n doubles (r, z, p, Ap).  Returns the iteration count. */
static uint64_t pcg_loop(const oracle_operator *A, int precond, const double *b,
                         const double *dvec, double tol, uint64_t maxiter, double *x,
                         double *relres_out, double *work, double *trace_alpha,
                         double *trace_beta, double *trace_relres) {
  int64_t n = A->n;
  int nt = A->nthreads;
  double *r = work, *z = work + n, *p = work + 2 * n, *Ap = work + 3 * n;
  memcpy(r, b, (size_t)n * sizeof(double));    /* pcg_solve.py:65 */
  precondition(precond, n, r, dvec, z, nt);    /* :66 */
  memcpy(p, z, (size_t)n * sizeof(double));    /* :67 */
  oracle_fill_f64(n, 0.0, x, nt);              /* :68 */
  double rr0 = oracle_dot_f64(n, r, r, nt);    /* :70 */
  double initres = sqrt(rr0);                  /* :71 */
  double rziter = 0.0;
  uint64_t i = 1;                              /* :72 */
  double relres;
  for (;;) {
    apply_operator(A, p, Ap);                  /* :75 */
    double pAp = oracle_dot_f64(n, p, Ap, nt); /* :76 */
    double rz = oracle_dot_f64(n, r, z, nt);   /* :77 */
    double alpha = rz / pAp;                   /* :78 */
    double malpha = -alpha;                    /* :79 */
    oracle_axpby_f64(n, 1.0, x, alpha, p, x, nt);   /* :81 */
    oracle_axpby_f64(n, 1.0, r, malpha, Ap, r, nt); /* :82 */
    double rr = oracle_dot_f64(n, r, r, nt);   /* :84 */
    double rnorm = sqrt(rr);                   /* :85 */
    relres = rnorm / initres;                  /* :86 */
    if (trace_alpha) trace_alpha[i - 1] = alpha;
    if (trace_relres) trace_relres[i - 1] = relres;
    int not_converged = relres > tol;          /* :87, ordered greater-than */
    int below_maxiter = i != maxiter;          /* :89 */
    rziter = rz;
    if (!(not_converged && below_maxiter)) break; /* :90-91 */
    precondition(precond, n, r, dvec, z, nt);  /* :94 */
    double rznext = oracle_dot_f64(n, r, z, nt); /* :95 */
    double beta = rznext / rziter;             /* :96 */
    if (trace_beta) trace_beta[i - 1] = beta;
    oracle_axpby_f64(n, 1.0, z, beta, p, p, nt); /* :97 */
    i = i + 1;                                 /* :98 */
  }
  *relres_out = relres;
  return i;
}

#define DEFINE_PCG(SUFFIX, IDX, IDXB)                                                       \
  ORACLE_API uint64_t oracle_pcg_f64_##SUFFIX(                                              \
      int64_t n, const IDX *pos, const IDX *crd, const double *val, const double *b,        \
      const double *dinv, double tol, uint64_t maxiter, double *x, double *relres_out,      \
      double *work, double *trace_alpha, double *trace_beta, double *trace_relres,          \
      int nthreads) {                                                                       \
    oracle_operator A = {n, IDXB, pos, crd, val, OP_SPMV, NULL, NULL, NULL,                 \
                         clamp_threads(nthreads)};                                          \
    return pcg_loop(&A, PC_MULT_DINV, b, dinv, tol, maxiter, x, relres_out, work,           \
                    trace_alpha, trace_beta, trace_relres);                                 \
  }
DEFINE_PCG(i32, int32_t, 4)
DEFINE_PCG(i64, int64_t, 8)

/* ------------------------------------------------------------------------
 * Hitting-time moments, examples/hitting_times.py:151-194 (@mht) followed by
 * :196-218 (@normalize_mom2).  Present only to pin pcg_loop against the
 * 17-digit golden vectors at examples/hitting_times.py:221-222.
 * val is scaled in place by alpha (scale_csr, :50-70).  work: 7*n doubles.
 * ---------------------------------------------------------------------- */
ORACLE_API void oracle_mht_f64_i32(int64_t n, const int32_t *pos, const int32_t *crd, double *val,
                                   const double *mask, const double *d, double alpha, double tol,
                                   uint64_t maxiter, double *mom1, double *mom2_norm,
                                   double *work) {
  int64_t nnz = pos[n];
  for (int64_t j = 0; j < nnz; j++) val[j] = val[j] * alpha; /* :50-70 */
  double *bbuf = work, *tmp = work + n, *mom2 = work + 2 * n, *pcgwork = work + 3 * n;
  oracle_operator A = {n, 4, pos, crd, val, OP_PLPT, d, mask, tmp, 1};
  oracle_mult_f64(n, d, mask, bbuf, 1); /* :158 */
  double relres;
  pcg_loop(&A, PC_DIV_D, bbuf, d, tol, maxiter, mom1, &relres, pcgwork, NULL, NULL, NULL); /* :160 */
  /* :163-176: b2 = mask * (d*mom1 + Aalpha*mom1) */
  oracle_fill_f64(n, 0.0, bbuf, 1);
  oracle_spmv_f64_i32(n, pos, crd, val, mom1, bbuf, 1);
  for (int64_t i = 0; i < n; i++) {
    double t1 = d[i] * mom1[i];
    double t2 = t1 + bbuf[i];
    bbuf[i] = t2 * mask[i];
  }
  pcg_loop(&A, PC_DIV_D, bbuf, d, tol, maxiter, mom2, &relres, pcgwork, NULL, NULL, NULL); /* :177 */
  for (int64_t i = 0; i < n; i++) { /* :196-218 */
    double sq = mom1[i] * mom1[i];
    double var = mom2[i] - sq;
    mom2_norm[i] = sqrt(var);
  }
}

/* ------------------------------------------------------------------------
 * Batched SpMM over a CSRV tensor, examples/bspmm.py:14-52: loop nest rows -> stored
 * entries -> dh -> nh, out[n1,dh,nh] = a*b + out[n1,dh,nh] in place (:47-49), fp32.
 * val holds nh values per stored entry; B is [n2, dh, nh]; C is [n1, dh, nh].
 * ---------------------------------------------------------------------- */
#define DEFINE_BSPMM(SUFFIX, IDX)                                                          \
  ORACLE_API void oracle_bspmm_f32_##SUFFIX(int64_t n1, int64_t nh, int64_t dh,             \
                                            const IDX *pos, const IDX *crd, const float *val, \
                                            const float *B, float *C) {                     \
    for (int64_t i = 0; i < n1; i++)                                                        \
      for (int64_t j = (int64_t)pos[i]; j < (int64_t)pos[i + 1]; j++) {                     \
        const float *brow = B + (int64_t)crd[j] * dh * nh;                                  \
        for (int64_t d = 0; d < dh; d++)                                                    \
          for (int64_t h = 0; h < nh; h++) {                                                \
            float prod = val[j * nh + h] * brow[d * nh + h];                                \
            C[(i * dh + d) * nh + h] = prod + C[(i * dh + d) * nh + h];                     \
          }                                                                                 \
      }                                                                                     \
  }
DEFINE_BSPMM(i32, int32_t)
DEFINE_BSPMM(i64, int64_t)

/* ------------------------------------------------------------------------
 * SpMM with A in DCSR, examples/spmm_dcsr_opdsl.py:59-101: stored rows -> stored
 * entries -> k, C[row,k] = C[row,k] + a*b in place, fp64.
 * ---------------------------------------------------------------------- */
#define DEFINE_SPMM_DCSR(SUFFIX, IDX)                                                      \
  ORACLE_API void oracle_spmm_dcsr_f64_##SUFFIX(int64_t nstored, int64_t k, const IDX *i1,  \
                                                const IDX *p2, const IDX *i2,               \
                                                const double *val, const double *B,         \
                                                double *C) {                                \
    for (int64_t r = 0; r < nstored; r++) {                                                 \
      double *crow = C + (int64_t)i1[r] * k;                                                \
      for (int64_t j = (int64_t)p2[r]; j < (int64_t)p2[r + 1]; j++) {                       \
        const double *brow = B + (int64_t)i2[j] * k;                                        \
        for (int64_t c = 0; c < k; c++) {                                                   \
          double prod = val[j] * brow[c];                                                   \
          crow[c] = crow[c] + prod;                                                         \
        }                                                                                   \
      }                                                                                     \
    }                                                                                       \
  }
DEFINE_SPMM_DCSR(i32, int32_t)
DEFINE_SPMM_DCSR(i64, int64_t)

/* ------------------------------------------------------------------------
 * Integer host logic that must be bit-exact.
 * nnz-balanced row partition: boundary g is the first row whose start offset
 * is >= g*nnz/G (lower bound on pos), g = 0..G, with boundary G = nrows.
 * The reference has no multi-device path; this is the partition rule of this
 * library, restated here so the CUDA/host implementation can be checked.
 * ---------------------------------------------------------------------- */
#define DEFINE_PARTITION(SUFFIX, IDX)                                                  \
  ORACLE_API void oracle_partition_rows_##SUFFIX(int64_t nrows, const IDX *pos, int G, \
                                                 int64_t *bounds) {                    \
    int64_t base = (int64_t)pos[0];                                                    \
    int64_t nnz = (int64_t)pos[nrows] - base;                                          \
    for (int g = 0; g <= G; g++) {                                                     \
      if (g == G) {                                                                    \
        bounds[g] = nrows;                                                             \
        continue;                                                                      \
      }                                                                                \
      int64_t target = base + (int64_t)(((__int128)nnz * g) / G);                      \
      int64_t lo = 0, hi = nrows;                                                      \
      while (lo < hi) {                                                                \
        int64_t mid = lo + (hi - lo) / 2;                                              \
        if ((int64_t)pos[mid] < target)                                                \
          lo = mid + 1;                                                                \
        else                                                                           \
          hi = mid;                                                                    \
      }                                                                                \
      bounds[g] = lo;                                                                  \
    }                                                                                  \
  }
DEFINE_PARTITION(i32, int32_t)
DEFINE_PARTITION(i64, int64_t)
