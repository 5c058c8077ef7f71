/*
 * lapis_b200 -- C ABI of the B200-native replacement for the kernels that the
 * LAPIS Kokkos emitter produces for CSR SpMV / SpMM, dense and batched matmul,
 * and the PCG solve loop.
 *
 * Two layers, both plain C (pointers and sizes only):
 *
 *  1. The emitted-module ABI (host buffers in, host-visible results out).  These
 *     are the symbols a LAPIS-generated module exports and its generated Python
 *     class binds: lapis_initialize / lapis_finalize and one py_<func> per public
 *     function, taking StridedMemRefType descriptors.  One LAPIS module is
 *     compiled for one index width, and C has no overloading, so the entry point
 *     names carry the element / index types as a suffix; the Python
 *     `KokkosBackend.compile()` binds the un-suffixed method name (`spmv`, `pcg`,
 *     `forward`) to the right one.
 *
 *  2. The device-resident layer (lapis_b200_*): what a C++ caller that keeps
 *     LAPIS::DualViews on the device does (benchmarks/spmv/main.cpp:52-62).
 *     All pointers are device pointers on the current CUDA device; `stream` is a
 *     cudaStream_t passed as void* (NULL = default stream).  Calls are
 *     asynchronous on that stream unless stated otherwise.
 *
 * Error behaviour: the emitted code aborts the process (Kokkos::abort).  Here no
 * entry point aborts: layer-2 functions return a status, layer-1 functions keep
 * the emitted `void` signature and record the status, which the caller reads
 * with lapis_last_error() (the Python binding raises).  There is no CPU
 * fallback: without a usable CUDA device every compute entry point fails with
 * LAPIS_ECUDA.
 *
 * Threading: like the emitted modules (LAPISSupport.hpp:114 keeps a plain static
 * vector), one caller thread per process at a time.
 *
 * Citations are paths within the LAPIS project.
 */
#ifndef LAPIS_B200_H
#define LAPIS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes --------------------------------------------------------- */
enum {
  LAPIS_OK = 0,
  LAPIS_EBADSHAPE = 1,   /* inconsistent sizes, mismatching contraction dimension */
  LAPIS_ELAYOUT = 2,     /* descriptor is not C-contiguous (LAPISSupport.hpp:80-89 aborts) */
  LAPIS_ECUDA = 3,       /* CUDA runtime error, or no device */
  LAPIS_EBADARG = 4,     /* null pointer, bad handle, misaligned device pointer */
  LAPIS_ENOTINIT = 5,    /* compute call before lapis_initialize */
  LAPIS_ETOOBIG = 6      /* size beyond a stated limit of the entry point */
};

/* Last status recorded by this thread's most recent call and its message. */
int lapis_last_error(void);
const char *lapis_last_error_message(void);

/* ---- descriptors ---------------------------------------------------------- */
/* Layout-identical to StridedMemRefType<T,N> (LAPISSupport.hpp:7-14):
 * {T* basePtr; T* data; int64 offset; int64 sizes[N]; int64 strides[N]}.
 * The element pointer is data + offset; all memrefs must be C-contiguous. */
typedef struct { void *basePtr; void *data; int64_t offset; int64_t sizes[1]; int64_t strides[1]; } lapis_memref1;
typedef struct { void *basePtr; void *data; int64_t offset; int64_t sizes[2]; int64_t strides[2]; } lapis_memref2;
typedef struct { void *basePtr; void *data; int64_t offset; int64_t sizes[3]; int64_t strides[3]; } lapis_memref3;

/* Sparse storage specifier as the emitter flattens it for a 2-D CSR tensor
 * (TranslateToKokkosCpp.cpp:4495-4546; benchmarks/spmv/main.cpp:48-51):
 * {rows, cols, len(pos), len(crd), len(val)} as five contiguous int64. */
typedef struct { int64_t dims[2]; int64_t mem_sizes[3]; } lapis_csr_spec;
/* The same for a 3-D CSRV tensor (dense, compressed, dense), examples/bspmm.py:103:
 * {n1, n2, nh, len(pos), len(crd), len(val) = stored entries * nh}. */
typedef struct { int64_t dims[3]; int64_t mem_sizes[3]; } lapis_csrv_spec;
/* And for a 2-D DCSR matrix (compressed, compressed), buffers in the order of
 * examples/spmm_dcsr_opdsl.py:137-143, 156: {rows, cols, len(p1), len(i1), len(p2), len(i2), len(val)}. */
typedef struct { int64_t dims[2]; int64_t mem_sizes[5]; } lapis_dcsr_spec;

/* ---- layer 1: emitted-module ABI ------------------------------------------ */

/* TranslateToKokkosCpp.cpp:4281-4378.  initialize is idempotent; finalize frees
 * every result buffer handed out since initialize (LAPISSupport.hpp:93-120). */
void lapis_initialize(void);
void lapis_finalize(void);

/* y = y_in + A x on CSR A; returns (aliases) the caller's y buffer.
 * Replaces the module function `spmv` of benchmarks/spmv/spmv.mlir:1-7 and
 * examples/spmv_noalloc.py:7-13,29 (wrapper shape: TranslateToKokkosCpp.cpp:2541-2684). */
void py_spmv_f64_i32(lapis_memref1 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                     const lapis_csr_spec *spec, lapis_memref1 *x, lapis_memref1 *y);
void py_spmv_f64_i64(lapis_memref1 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                     const lapis_csr_spec *spec, lapis_memref1 *x, lapis_memref1 *y);

/* C = C_in + A B, CSR A times dense row-major B; returns the caller's C.
 * Same convention as py_spmv for a `linalg.matmul` with a CSR first operand
 * (semantics: examples/spmm_dcsr_opdsl.py:40-101, examples/bspmm.py:15-52). */
void py_spmm_f64_i32(lapis_memref2 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                     const lapis_csr_spec *spec, lapis_memref2 *B, lapis_memref2 *C);
void py_spmm_f64_i64(lapis_memref2 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                     const lapis_csr_spec *spec, lapis_memref2 *B, lapis_memref2 *C);

/* C = C_in + A B, fp32, row-major; returns the caller's C.  Replaces `forward`
 * of examples/gemm_no_alloc.py:8-24,38 / benchmarks/gemm/gemm.mlir:1-15.
 * A contraction-dimension mismatch (cf.assert, gemm.mlir:10-11) gives LAPIS_EBADSHAPE. */
void py_matmul_f32(lapis_memref2 **ret0, lapis_memref2 *A, lapis_memref2 *B, lapis_memref2 *C);

/* C[b] = C_in[b] + A[b] B[b], fp32.  Replaces `forward` of
 * examples/batched_gemm_no_alloc.py:8-31,45 / benchmarks/batched_gemm/batched_gemm.mlir:1-24. */
void py_batch_matmul_f32(lapis_memref3 **ret0, lapis_memref3 *A, lapis_memref3 *B, lapis_memref3 *C);

/* Jacobi-preconditioned CG, examples/pcg_solve.py:52-101,129: returns x (module-owned,
 * valid until lapis_finalize), the iteration count and the final relative residual. */
void py_pcg_f64_i32(lapis_memref1 **ret0, size_t *ret1, double *ret2, lapis_memref1 *pos, lapis_memref1 *crd,
                    lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *b, lapis_memref1 *dinv,
                    double tol, size_t maxiter);
void py_pcg_f64_i64(lapis_memref1 **ret0, size_t *ret1, double *ret2, lapis_memref1 *pos, lapis_memref1 *crd,
                    lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *b, lapis_memref1 *dinv,
                    double tol, size_t maxiter);

/* Hitting-time moments of a graph, examples/hitting_times.py:151-194 (`mht`, called at :216): two
 * Jacobi-PCG solves with the masked Laplacian mask*(d - alpha*A)*mask (`plpt`, :73-92) and z = r / d.
 * Returns the two moment vectors (module-owned, valid until lapis_finalize).  The caller's values array is
 * not modified (the emitted code scales it in place on the device; the host copy never sees that). */
void py_mht_f64_i32(lapis_memref1 **ret0, lapis_memref1 **ret1, lapis_memref1 *pos, lapis_memref1 *crd,
                    lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *mask, lapis_memref1 *d,
                    double alpha, double tol, size_t maxiter);
void py_mht_f64_i64(lapis_memref1 **ret0, lapis_memref1 **ret1, lapis_memref1 *pos, lapis_memref1 *crd,
                    lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *mask, lapis_memref1 *d,
                    double alpha, double tol, size_t maxiter);
/* sqrt(mom2 - mom1^2), examples/hitting_times.py:196-218 (`normalize_mom2`, called at :218). */
void py_normalize_mom2_f64(lapis_memref1 **ret0, lapis_memref1 *mom1, lapis_memref1 *mom2);

/* Batched SpMM over a CSRV tensor, fp32: out[n1, dh, nh] = sum_n2 A[n1, n2, nh] * B[n2, dh, nh].  Replaces
 * `pte_local_bspmm` of examples/bspmm.py:26-52 (called at :103): the result is a new zero-initialised tensor
 * (module-owned, valid until lapis_finalize). */
void py_bspmm_f32_i32(lapis_memref3 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                      const lapis_csrv_spec *spec, lapis_memref3 *B);
void py_bspmm_f32_i64(lapis_memref3 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                      const lapis_csrv_spec *spec, lapis_memref3 *B);

/* C += A B with A in DCSR, fp64.  The operation of `spMxM` in examples/spmm_dcsr_opdsl.py:59-101 (called at
 * :160) in the decomposed-argument form (the example itself passes an opaque sparse-runtime handle, which
 * this library does not take).  Returns its in/out argument C. */
void py_spmm_dcsr_f64_i32(lapis_memref2 **ret0, lapis_memref1 *p1, lapis_memref1 *i1, lapis_memref1 *p2,
                          lapis_memref1 *i2, lapis_memref1 *val, const lapis_dcsr_spec *spec, lapis_memref2 *B,
                          lapis_memref2 *C);
void py_spmm_dcsr_f64_i64(lapis_memref2 **ret0, lapis_memref1 *p1, lapis_memref1 *i1, lapis_memref1 *p2,
                          lapis_memref1 *i2, lapis_memref1 *val, const lapis_dcsr_spec *spec, lapis_memref2 *B,
                          lapis_memref2 *C);

/* ---- layer 2: device-resident entry points -------------------------------- */

/* A CSR matrix resident on the device plus this library's streaming plan for it
 * (row ranges per thread block, in device scratch owned by the handle).
 * Counterpart of the DualViews a C++ caller keeps alive across calls
 * (benchmarks/spmv/main.cpp:42-51).  pos/crd/val stay owned by the caller and
 * must outlive the handle; val and crd must be 16-byte aligned.  pos[0] may be
 * non-zero (a row block of a larger matrix addressed in place). */
typedef struct lapis_b200_csr *lapis_b200_csr_t;

/* idx_bytes: 4 (int32 pos/crd) or 8 (int64).  Synchronises `stream` once. */
int lapis_b200_csr_create(lapis_b200_csr_t *out, int idx_bytes, int64_t nrows, int64_t ncols,
                          const void *d_pos, const void *d_crd, const double *d_val, void *stream);
int lapis_b200_csr_destroy(lapis_b200_csr_t h);
int64_t lapis_b200_csr_nnz(lapis_b200_csr_t h);

/* y = (accumulate ? y : 0) + A x.  The emitted kernel always accumulates
 * (loop_mapping_2.mlir.gold:12-37); accumulate = 0 fuses the linalg.fill that
 * callers put in front of it (examples/pcg_solve.py:13-20). */
int lapis_b200_spmv_f64(lapis_b200_csr_t h, const double *d_x, double *d_y, int accumulate, void *stream);

/* Two SpMV kernels exist: one chunk of 2048 stored entries per thread block (threads, blocks
 * per SM in {(256,4), (256,6), (512,3)}), and a persistent kernel that stages chunks with bulk
 * asynchronous copies (threads = -256 or -512, blocks_per_sm resident blocks per SM).  Which is
 * faster depends on the matrix: the persistent one when x is served from cache (banded
 * matrices), the other when the gathers of x dominate.  lapis_b200_csr_tune times the
 * candidates on the matrix (a few SpMV launches into scratch buffers it allocates and frees;
 * synchronises `stream`) and stores the winner in the handle; untuned handles use (256,4).
 * lapis_b200_spmv_select_kernel forces one variant process-wide (threads = 0 returns to the
 * handles' own choice); the environment variable LAPIS_B200_SPMV="threads,blocks,l2_hint" does
 * the same from outside.  l2_hint marks x evict-last in L2.
 * A third kind, threads = 1 and blocks_per_sm = 0, gives every row to one thread; the tuner considers it
 * (and the launch honours it) only for matrices whose longest row has at most 32 entries -- up to there it
 * returns the same bits as the others -- and such matrices (stencils, bounded-degree graphs) are where it
 * wins.  On other matrices, and on handles that were never tuned, a request for it runs (256,4).
 * A fourth kind, threads = 2 (256 threads, blocks_per_sm in {4, 5}) or threads = 3 (512 threads,
 * blocks_per_sm in {2, 3, 4}), is the chunk kernel with the row sums done by a
 * segmented scan in registers instead of one lane per row over shared memory (less shared-memory traffic
 * when the gathers of x already saturate L1).  It adds a row's products in scan order, so y agrees with the
 * other kernels to 1e-12 of the row's magnitude but not bit for bit; lapis_b200_csr_tune therefore leaves it
 * out, and lapis_b200_csr_tune_relaxed is the same tuner with it among the candidates, for callers who want
 * the fastest kernel within the tolerance rather than one set of bits whichever kernel runs. */
int lapis_b200_csr_tune(lapis_b200_csr_t h, void *stream);
int lapis_b200_csr_tune_relaxed(lapis_b200_csr_t h, void *stream);
int lapis_b200_csr_tuned_kernel(lapis_b200_csr_t h, int *threads, int *blocks_per_sm);
int lapis_b200_spmv_select_kernel(int threads, int blocks_per_sm, int l2_hint);
/* The persistent kernel bounds its waits on the bulk copies; this synchronises `stream` and
 * returns LAPIS_ECUDA if a block gave up (then y of that launch is invalid), clearing the flag. */
int lapis_b200_spmv_status(void *stream);

/* The same SpMV for callers that must not allocate device memory in the call -- code
 * running inside a pool that already owns the whole GPU, or a steady-state loop where
 * a cudaMalloc could stall the device or fail.  No counterpart in the reference (its
 * emitted kernels need no plan).  Takes the raw CSR arrays instead of a handle and
 * keeps the streaming plan and the carries in a fixed 4 MiB array inside the library's device image,
 * so it calls neither cudaMalloc nor cudaFree.
 *   - Limit: 2^18 chunks of 2048 stored entries counted from pos[0] rounded down to a multiple of 4: 2^29
 *     (536,870,912) entries when pos[0] is a multiple of 4, up to 3 fewer otherwise; larger matrices get
 *     LAPIS_ETOOBIG.
 *   - The first call on a device looks the array's address up (cudaGetSymbolAddress); make that first call
 *     outside any stream capture.  Every call, not only the first, copies pos[0] and pos[nrows] back to the
 *     host and synchronises `stream`, so no call to this entry point can sit inside a stream capture.
 *   - All calls on a device share the one array: calls that can overlap on the GPU
 *     (different streams, no ordering between them) race.  Calls on one stream are safe.
 *   - Like the rest of the library: one caller thread per process at a time (the per-device address cache
 *     is a plain static).
 *   - The device arrays are trusted (see lapis_b200_validate_csr_host).
 * Arguments as lapis_b200_csr_create followed by lapis_b200_spmv_f64. */
int lapis_b200_spmv_f64_noalloc(int idx_bytes, int64_t nrows, int64_t ncols, const void *d_pos, const void *d_crd,
                                const double *d_val, const double *d_x, double *d_y, int accumulate, void *stream);

/* C = (accumulate ? C : 0) + A B with dense row-major B (ncols x k), C (nrows x k). */
int lapis_b200_spmm_f64(lapis_b200_csr_t h, int64_t k, const double *d_B, double *d_C, int accumulate,
                        void *stream);

/* C[b] = C[b] + A[b] B[b], fp32 row-major, batch >= 1 (batch = 1: dense matmul). */
int lapis_b200_bgemm_f32(int64_t batch, int64_t M, int64_t N, int64_t K, const float *d_A, const float *d_B,
                         float *d_C, void *stream);

/* Tile-aligned problems (M, N multiples of 128, K of 32) run on the tensor cores, whose kernel
 * bounds every internal wait and records a flag instead of hanging.  This reads and clears
 * that flag after synchronising `stream`: LAPIS_OK, or LAPIS_ECUDA when the last launches on
 * this device did not complete normally (their output is then invalid). */
int lapis_b200_bgemm_status(void *stream);

/* Vector kernels of examples/pcg_solve.py:22-48.  dot writes its result to *d_out. */
int lapis_b200_dot_f64(int64_t n, const double *d_x, const double *d_y, double *d_out, void *stream);
int lapis_b200_axpby_f64(int64_t n, double a, const double *d_x, double b, const double *d_y, double *d_dst,
                         void *stream);
int lapis_b200_mult_f64(int64_t n, const double *d_x, const double *d_y, double *d_dst, void *stream);

/* PCG with all state on the device (examples/pcg_solve.py:52-101).  d_x receives
 * the solution; *iters and *relres are host outputs.  Blocks until finished. */
int lapis_b200_pcg_f64(lapis_b200_csr_t h, const double *d_b, const double *d_dinv, double tol, uint64_t maxiter,
                       double *d_x, uint64_t *iters, double *relres, void *stream);

/* Batched SpMM over a CSRV tensor on the device (examples/bspmm.py:14-52): d_val holds nh values per stored
 * entry, d_B is [n2, dh, nh], d_C is [n1, dh, nh], all row-major fp32.  Every output element is updated in
 * ascending entry order starting from its old value (accumulate != 0) or from zero: bit-identical to the
 * sequential loop nest. */
int lapis_b200_bspmm_csrv_f32(int idx_bytes, int64_t n1, int64_t n2, int64_t nh, int64_t dh, const void *d_pos,
                              const void *d_crd, const float *d_val, const float *d_B, float *d_C, int accumulate,
                              void *stream);
/* C[i1[r], :] += sum_j val[j] * B[i2[j], :] over the nstored stored rows of a DCSR matrix
 * (examples/spmm_dcsr_opdsl.py:59-101); rows that are not stored keep their values; d_i1 ascends (a row
 * number may repeat).  Bit-identical to the sequential loop nest. */
int lapis_b200_spmm_dcsr_f64(int idx_bytes, int64_t nrows, int64_t ncols, int64_t nstored, int64_t k, const void *d_i1,
                             const void *d_p2, const void *d_i2, const double *d_val, const double *d_B, double *d_C,
                             void *stream);

/* Hitting-time moments with all operands on the device (examples/hitting_times.py:151-194): d_mom1 and d_mom2
 * receive the first two moments; iters2 / relres2 (host, two entries each, may be null) the iteration counts
 * and final relative residuals of the two solves.  The matrix values are read through a scaled copy; the
 * caller's array is not modified.  Blocks until finished. */
int lapis_b200_mht_f64(lapis_b200_csr_t h, const double *d_mask, const double *d_d, double alpha, double tol,
                       uint64_t maxiter, double *d_mom1, double *d_mom2, uint64_t *iters2, double *relres2, void *stream);
/* d_out[i] = sqrt(d_mom2[i] - d_mom1[i]^2)  (examples/hitting_times.py:196-218). */
int lapis_b200_normalize_mom2_f64(int64_t n, const double *d_mom1, const double *d_mom2, double *d_out, void *stream);

/* Step-level PCG entry points: the three passes of one iteration, for callers that
 * put an exchange between them (row-block partitioned solves put a halo copy of p in
 * front of pass A and an allreduce of the scalar block behind passes A and B).
 * lapis_b200_pcg_f64 above is exactly these steps in a loop.
 *
 * d_work is caller-allocated device memory of lapis_b200_pcg_workspace_bytes(n, n_p)
 * bytes, 16-byte aligned.  Layout in doubles: [0] p.Ap, [1] r.r, [2] r.z (new),
 * [3] r.z (carried), [4] initial residual norm, [5] relres, [6] alpha, [7] beta,
 * [8] done flag and [9] count of completed iterations as int64, then scratch and the vectors
 * r, z, p, Ap and a z halo buffer as long as p.  n = local rows; n_p >= n = length of the p buffer the matrix's
 * column indices address; the local part of p starts at p_offset in it.
 * `derive` != 0 lets the pass also run the scalar recurrence that consumes its
 * sums (single-device use); with derive == 0 the caller reduces slots [0] or
 * [1..2] across devices and then calls lapis_b200_pcg_derive.
 * kind: 1 = after init, 2 = alpha after pass A, 3 = stop test and beta after pass B. */
int64_t lapis_b200_pcg_workspace_bytes(int64_t n, int64_t n_p);
/* Offsets (in doubles from d_work) of the vectors r, z, p, Ap. */
int lapis_b200_pcg_workspace_layout(int64_t n, int64_t n_p, int64_t *offsets4);
int lapis_b200_pcg_init(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, const double *d_b,
                        const double *d_dinv, double *d_x, int derive, void *stream);
int lapis_b200_pcg_derive(void *d_work, int kind, double tol, uint64_t maxiter, void *stream);
int lapis_b200_pcg_step_spmv(void *d_work, lapis_b200_csr_t h, int64_t n_p, int64_t p_offset, int derive,
                             void *stream);
int lapis_b200_pcg_step_update(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, const double *d_dinv,
                               double *d_x, int derive, double tol, uint64_t maxiter, void *stream);
int lapis_b200_pcg_step_direction(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, void *stream);
/* The same exchanges without library collectives (one process per GPU on one node): a rank maps every
 * peer's mailbox and workspace with CUDA IPC and the exchanges are stores into peer memory over NVLink
 * plus sequence-numbered flags; the waits are bounded and stop the solve with an error mark in the
 * mailbox if a peer never delivers.  No counterpart in the reference (it has no multi-device path).
 *   peer_alloc / peer_open / peer_close / peer_free: device memory exported as a 64-byte IPC handle and
 *     mapped by the peers (open with the consuming device current).
 *   mailbox: lapis_b200_pcg_p2p_mailbox_bytes() bytes per rank, zero-initialised, from peer_alloc.
 *   The caller stores epoch * 2^32 (a different epoch per solve) in workspace slot [10] after
 *   lapis_b200_pcg_init.  phase: 0 = p.Ap, 1 = r.r / r.z, 2 = their initial values.
 *   push_scalars: this rank's local sums (workspace slots [0] or [1..2]) to every rank's mailbox
 *     (d_peer_mbox: device array of `world` mailbox addresses, own included).
 *   wait_reduce: waits for all ranks' values of the phase, adds them in rank order (identical on every
 *     rank) and runs the scalar recurrence `derive` (1, 2 or 3 as for lapis_b200_pcg_derive).
 *   halo_push: copies pieces of this rank's p window into the peers' windows (d_pieces: device array of
 *     {uint64 destination address, int64 source offset in the window, int64 length, uint64 flag address}).
 *   halo_wait: waits until the ranks in d_srcs (device int array) have delivered this iteration's pieces. */
int64_t lapis_b200_pcg_p2p_mailbox_bytes(void);
/* Index, in doubles, of the first halo flag (one per source rank) and of the error mark in a mailbox. */
void lapis_b200_pcg_p2p_mailbox_layout(int64_t *halo_index, int64_t *error_index);
int lapis_b200_peer_alloc(int64_t bytes, void **ptr, unsigned char *handle64);
int lapis_b200_peer_open(const unsigned char *handle64, void **ptr);
int lapis_b200_peer_close(void *ptr);
int lapis_b200_peer_free(void *ptr);
int lapis_b200_pcg_p2p_push_scalars(void *d_work, int phase, int me, int world, const void *d_peer_mbox, void *stream);
int lapis_b200_pcg_p2p_wait_reduce(void *d_work, void *d_mbox, int phase, int world, int derive, double tol,
                                   uint64_t maxiter, void *stream);
int lapis_b200_pcg_p2p_halo_push(void *d_work, int64_t n, int64_t n_p, const void *d_pieces, int npieces, void *stream);
int lapis_b200_pcg_p2p_halo_wait(void *d_work, void *d_mbox, const void *d_srcs, int nsrc, void *stream);
/* One iteration in three launches.  The passes above leave the sums to a single-block kernel (or to the
 * caller's collective) between them; these variants add the per-block partial sums inside the pass, in the
 * block that finishes last, and -- with an exchange description -- do the row-partitioned solver's exchanges
 * inside the passes too: pass A ends by storing this rank's p.Ap into every rank's mailbox; pass B starts by
 * waiting for every rank's p.Ap (each block adds them in rank order and derives alpha itself), also stores the
 * rows of z behind its neighbours' halo of p into their z halo buffers, and ends by storing r.r and r.z; pass C
 * starts by waiting for those, repeats the stop test, and updates p on the own rows and on the halo entries of
 * the window (p_halo = z_halo + beta * p_halo, the owner's operation on the owner's operands), so the halo of p
 * needs no exchange of its own: two points per iteration at which ranks wait for each other.  Plain peer stores
 * and local polling only; every wait is bounded (lapis_b200_pcg_p2p_set_wait_limit polls, 0 = the default of
 * 2^22, about a second) and a wait that runs out marks the mailbox and sets the done flag instead of hanging.
 * exchange == NULL (or d_mbox == NULL): one device, scalars derived locally -- lapis_b200_pcg_f64 is these
 * three calls in a loop.  The initial exchange still uses push_scalars / wait_reduce / halo_push / halo_wait
 * above (the halo of the first p travels as p); nsrc > 0 makes pass A wait for halo flags like halo_wait does.
 * The z halo buffer of a workspace has n_p doubles and follows Ap: offsets4[3] + n of
 * lapis_b200_pcg_workspace_layout.
 * Replaces the loop body of examples/pcg_solve.py:74-98 (host loop TranslateToKokkosCpp.cpp:1512-1593). */
typedef struct {
  int me, world;             /* this rank and the number of ranks (at most 16) */
  void *d_mbox;              /* this rank's mailbox (NULL: no exchange) */
  const void *d_peer_mbox;   /* device array of `world` mailbox addresses, own included */
  const void *d_halo_srcs;   /* device int array: ranks whose halo flags pass A waits for (normally none) */
  int nsrc;
  const void *d_z_pieces;    /* device array of {dst address in the peer's z halo buffer, source offset in this
                                rank's window, length, unused}: the rows of z the neighbours need */
  int nzpieces;              /* at most 32 */
  const void *d_halo_ranges; /* device int64 array of {start, length} pairs: halo parts of this rank's window */
  int nranges;
} lapis_b200_pcg_exchange;
int lapis_b200_pcg_fused_spmv(void *d_work, lapis_b200_csr_t h, int64_t n_p, int64_t p_offset, double tol, uint64_t maxiter,
                              const lapis_b200_pcg_exchange *exchange, void *stream);
int lapis_b200_pcg_fused_update(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, const double *d_dinv, double *d_x,
                                double tol, uint64_t maxiter, const lapis_b200_pcg_exchange *exchange, void *stream);
int lapis_b200_pcg_fused_direction(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, double tol, uint64_t maxiter,
                                   const lapis_b200_pcg_exchange *exchange, void *stream);
/* Two launches per iteration where the matrix allows it (lapis_b200_pcg_folds_direction(h) != 0: rows short enough
 * for the one-thread-per-row SpMV kernel): lapis_b200_pcg_fused_spmv_direction is pass A with the direction update
 * of the iteration before folded in (its SpMV reads z + beta * p_old wherever it gathers and stores the new p into
 * the second p buffer of the workspace), followed by lapis_b200_pcg_fused_update; lapis_b200_pcg_fused_direction
 * is not called.  Same bits as the three-launch form.  With an exchange, the stop test of an iteration runs at
 * the head of the next lapis_b200_pcg_fused_spmv_direction: call it once more after the last update before
 * reading lapis_b200_pcg_status.  One solve uses one form throughout. */
int lapis_b200_pcg_folds_direction(lapis_b200_csr_t h);
int lapis_b200_pcg_fused_spmv_direction(void *d_work, lapis_b200_csr_t h, int64_t n_p, int64_t p_offset, double tol,
                                        uint64_t maxiter, const lapis_b200_pcg_exchange *exchange, void *stream);
int lapis_b200_pcg_p2p_set_wait_limit(uint32_t polls);
/* Copies {done, iters, relres} to the host; synchronises `stream`. */
int lapis_b200_pcg_status(void *d_work, int *done, uint64_t *iters, double *relres, void *stream);

/* MatrixMarket coordinate file -> CSR on the host (ascending columns per row, duplicates summed,
 * symmetric / skew-symmetric storage expanded, pattern entries = 1): the format step in front of the
 * SpMV path, done in the reference's benchmark by the KokkosSparse reader vendored beside
 * benchmarks/spmv/main.cpp (:36-38).  The three arrays are allocated here; release each with
 * lapis_b200_mm_free. */
int lapis_b200_read_matrix_market(const char *path, int idx_bytes, int64_t *nrows, int64_t *ncols, int64_t *nnz,
                                  void **pos, void **crd, double **val);
void lapis_b200_mm_free(void *p);

/* Host-side validation the py_* wrappers run on a CSR operand before any kernel sees it (host arrays, no CUDA
 * call): pos[0] == 0, pos non-decreasing, pos[nrows] == nnz, and 0 <= crd[j] < ncols for every stored entry;
 * LAPIS_EBADSHAPE otherwise.  The emitted code aborts on bad descriptors (LAPISSupport.hpp:76-89) and indexes
 * with crd unchecked.  The layer-2 entry points that take device pointers (lapis_b200_csr_create, ..._noalloc)
 * cannot look at the arrays and trust them: callers holding host copies validate with this first. */
int lapis_b200_validate_csr_host(int idx_bytes, int64_t nrows, int64_t ncols, int64_t nnz, const void *pos,
                                 const void *crd);

/* nnz-balanced contiguous row partition of a CSR matrix over G devices (host
 * arrays): bounds[g] = first row whose start offset is >= pos[0] + g*nnz/G,
 * bounds[G] = nrows.  The reference has no multi-device path; this is the
 * partition rule of this library. */
int lapis_b200_partition_rows(int idx_bytes, int64_t nrows, const void *pos, int G, int64_t *bounds);

#ifdef __cplusplus
}
#endif
#endif /* LAPIS_B200_H */
