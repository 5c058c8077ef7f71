// Vector kernels and the PCG solve loop for sm_100a.
//
// The emitted PCG (examples/pcg_solve.py:52-101, host `while` loop printed by
// mlir/lib/Target/KokkosCpp/TranslateToKokkosCpp.cpp:1512-1593) launches ten
// Kokkos kernels per iteration (fill, SpMV, 4 dots, 3 axpby, mult) and reads four
// scalars back to the host.  Here one iteration is three streaming passes whose
// scalars never leave the device:
//
//   pass A  Ap = A p, fused with the partial sums of p.Ap          (spmv.cu)
//   pass B  x += alpha p ; r -= alpha Ap ; z = r*dinv ; partial r.r and r.z
//   pass C  p = z + beta p
//
// r.z at the top of an iteration equals the r.z' computed at the end of the
// previous one (same operands), so it is carried instead of recomputed.
// The per-block partial sums of a pass are added in a fixed order (results are run-to-run
// identical) by the block of that pass that finishes last, which also derives alpha / relres /
// beta and the stop flag -- or, in a row-partitioned solve, hands the sums to the other ranks
// (pcg_fuse.h): three launches per iteration.  (The step-level entry points further down keep
// the older form with a single-block summing kernel between the passes, for callers that put
// their own collectives there.)  Every kernel returns at once when the stop flag is set, so the
// host can enqueue iterations ahead and only look at the flag now and then.
//
// Arithmetic follows the emitted element-wise bodies: axpby is (x*a) + (y*b) with
// separate roundings (examples/pcg_solve.py:30-39), mult is x*y (:41-48).
#include <cmath>

#include "common.h"
#include "pcg_fuse.h"

namespace lapis_b200 {

int spmv_launch(const lapis_b200_csr *h, const double *x, double *y, int accumulate, const double *dotvec,
                double *blk_partial, const int *skip_flag, cudaStream_t st);
bool spmv_fuses_pcg_pass(const lapis_b200_csr *h);
int spmv_launch_pcg_pass(const lapis_b200_csr *h, const double *x, double *y, const double *dotvec, double *blk_partial,
                         const int *skip_flag, cudaStream_t st, const PcgExchange &ex);
int spmv_launch_pcg_direction_pass(const lapis_b200_csr *h, int64_t p_off, double *pw0, double *pw1, double *Ap,
                                   double *blk_partial, cudaStream_t st, const PcgExchange &ex);

constexpr int VEC_THREADS = 256;
constexpr int SUM_THREADS = 1024;

__device__ __forceinline__ double block_sum_vec(double v, double *s_red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = __dadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) s_red[warp] = v;
  __syncthreads();
  double t = 0.0;
  if (warp == 0) {
    t = lane < (int)(blockDim.x >> 5) ? s_red[lane] : 0.0;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t = __dadd_rn(t, __shfl_xor_sync(0xffffffffu, t, off));
  }
  return t;  // valid in thread 0
}

// out[c] = sum_b partials[c*nb + b] for c < count (count <= 2), fixed order; then
// optionally the scalar step that consumes the sums.
__global__ void __launch_bounds__(SUM_THREADS)
sum_partials_kernel(const double *__restrict__ partials, int64_t nb, int count, double *out0, double *out1,
                    int derive, double *sc, long long *fl, double tol, unsigned long long maxiter,
                    const long long *skip) {
  __shared__ double s_red[SUM_THREADS / 32];
  if (skip != nullptr && skip[FL_DONE] != 0) return;
  for (int c = 0; c < count; ++c) {
    double acc = 0.0;
    const double *p = partials + (int64_t)c * nb;
    for (int64_t i = threadIdx.x; i < nb; i += SUM_THREADS) acc = __dadd_rn(acc, p[i]);
    const double t = block_sum_vec(acc, s_red);
    if (threadIdx.x == 0) *(c == 0 ? out0 : out1) = t;
  }
  if (derive != DERIVE_NONE && threadIdx.x == 0) pcg_derive(derive, sc, fl, tol, maxiter);
}

__global__ void pcg_derive_kernel(int kind, double *sc, long long *fl, double tol, unsigned long long maxiter) {
  if (kind != DERIVE_INIT && fl[FL_DONE] != 0) return;
  pcg_derive(kind, sc, fl, tol, maxiter);
}

// ---- plain vector kernels (examples/pcg_solve.py:22-48) ------------------------
__global__ void __launch_bounds__(VEC_THREADS)
dot_partial_kernel(int64_t n, const double *__restrict__ x, const double *__restrict__ y,
                   double *__restrict__ partials) {
  __shared__ double s_red[VEC_THREADS / 32];
  double acc = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS)
    acc = __dadd_rn(acc, __dmul_rn(x[i], y[i]));
  const double t = block_sum_vec(acc, s_red);
  if (threadIdx.x == 0) partials[blockIdx.x] = t;
}

__global__ void __launch_bounds__(VEC_THREADS)
axpby_kernel(int64_t n, double a, const double *__restrict__ x, double b, const double *__restrict__ y,
             double *__restrict__ dst) {
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS)
    dst[i] = __dadd_rn(__dmul_rn(x[i], a), __dmul_rn(y[i], b));
}

__global__ void __launch_bounds__(VEC_THREADS)
mult_kernel(int64_t n, const double *__restrict__ x, const double *__restrict__ y, double *__restrict__ dst) {
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS)
    dst[i] = __dmul_rn(x[i], y[i]);
}

// ---- PCG passes --------------------------------------------------------------------
// r = b; z = r*dinv; p = z; x = 0; partials of r.r and r.z  (examples/pcg_solve.py:65-70)
__global__ void __launch_bounds__(VEC_THREADS)
pcg_init_kernel(int64_t n, const double *__restrict__ b, const double *__restrict__ dinv, double *__restrict__ r,
                double *__restrict__ z, double *__restrict__ p, double *__restrict__ x,
                double *__restrict__ partials) {
  __shared__ double s_red[VEC_THREADS / 32];
  double rr = 0.0, rz = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS) {
    const double ri = b[i];
    const double zi = __dmul_rn(ri, dinv[i]);
    r[i] = ri;
    z[i] = zi;
    p[i] = zi;
    x[i] = 0.0;
    rr = __dadd_rn(rr, __dmul_rn(ri, ri));
    rz = __dadd_rn(rz, __dmul_rn(ri, zi));
  }
  const double t0 = block_sum_vec(rr, s_red);
  const double t1 = block_sum_vec(rz, s_red);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = t0;
    partials[gridDim.x + blockIdx.x] = t1;
  }
}

// x = x*1 + p*alpha ; r = r*1 + Ap*(-alpha) ; z = r*dinv ; partials of r.r and r.z
// (examples/pcg_solve.py:79-84, 94-95)
__global__ void __launch_bounds__(VEC_THREADS)
pcg_update_kernel(int64_t n, const double *__restrict__ sc, const long long *__restrict__ fl,
                  const double *__restrict__ p, const double *__restrict__ Ap, const double *__restrict__ dinv,
                  double *__restrict__ x, double *__restrict__ r, double *__restrict__ z,
                  double *__restrict__ partials) {
  __shared__ double s_red[VEC_THREADS / 32];
  if (fl[FL_DONE] != 0) return;
  const double alpha = sc[SC_ALPHA];
  const double malpha = -alpha;
  double rr = 0.0, rz = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS) {
    const double xi = __dadd_rn(__dmul_rn(x[i], 1.0), __dmul_rn(p[i], alpha));
    const double ri = __dadd_rn(__dmul_rn(r[i], 1.0), __dmul_rn(Ap[i], malpha));
    const double zi = __dmul_rn(ri, dinv[i]);
    x[i] = xi;
    r[i] = ri;
    z[i] = zi;
    rr = __dadd_rn(rr, __dmul_rn(ri, ri));
    rz = __dadd_rn(rz, __dmul_rn(ri, zi));
  }
  const double t0 = block_sum_vec(rr, s_red);
  const double t1 = block_sum_vec(rz, s_red);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = t0;
    partials[gridDim.x + blockIdx.x] = t1;
  }
}

// p = z*1 + p*beta  (examples/pcg_solve.py:97)
__global__ void __launch_bounds__(VEC_THREADS)
pcg_direction_kernel(int64_t n, const double *__restrict__ sc, const long long *__restrict__ fl,
                     const double *__restrict__ z, double *__restrict__ p) {
  if (fl[FL_DONE] != 0) return;
  const double beta = sc[SC_BETA];
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS)
    p[i] = __dadd_rn(__dmul_rn(z[i], 1.0), __dmul_rn(p[i], beta));
}

static inline unsigned vec_grid(int64_t n) {
  const int64_t want = (n + VEC_THREADS - 1) / VEC_THREADS;
  const int64_t cap = (int64_t)sm_count() * 8;
  int64_t g = want < cap ? want : cap;
  return (unsigned)(g < 1 ? 1 : g);
}

// Workspace layout (doubles): [scalars 8][flags 2 (as int64)][pad to 16][partials 2*G][r n][z n][p n_p][Ap n][zh n_p][p1 n_p]
// where G = 8 * SM count, n_p >= n is the length of the (halo-extended) p buffer, zh is the window-indexed
// buffer of z (the fused passes keep the own rows of z there too; neighbours store the rows behind this rank's
// halo of p into it) and p1 is the second p buffer of the two-pass form.
struct PcgWork {
  double *sc;
  long long *fl;
  double *partials;
  double *r, *z, *p, *Ap, *zh, *p1;
  unsigned grid;
};

static inline int64_t pcg_partials_len() { return 2 * (int64_t)sm_count() * 8; }

static PcgWork carve(void *d_work, int64_t n, int64_t n_p) {
  PcgWork w;
  double *base = static_cast<double *>(d_work);
  w.sc = base;
  w.fl = reinterpret_cast<long long *>(base + SC_COUNT);
  w.partials = base + 16;
  double *vecs = w.partials + pcg_partials_len();
  w.r = vecs;
  w.z = vecs + n;
  w.p = vecs + 2 * n;
  w.Ap = vecs + 2 * n + n_p;
  w.zh = vecs + 3 * n + n_p;
  w.p1 = vecs + 3 * n + 2 * n_p;
  w.grid = vec_grid(n);
  return w;
}


// ---- fused passes: heads that wait for the other ranks' sums, tails in the last block (pcg_fuse.h) --------
static unsigned g_p2p_spin_limit = P2P_SPIN_LIMIT;  // polls per bounded wait; lapis_b200_pcg_p2p_set_wait_limit

// Pass B.  alpha comes from the scalar block (no exchange) or from every rank's p.Ap (exchange).  With an
// exchange the rows of z that neighbours need (they stand behind the neighbours' halo of p) are also stored into
// the neighbours' z halo buffers, and the tail's sequence number covers them.
constexpr int PCG_MAX_FUSED_PIECES = 32;
__global__ void __launch_bounds__(VEC_THREADS)
pcg_update_fused_kernel(int64_t n, int64_t p_off, PcgExchange ex, const double *p_first, const double *p_second,
                        const double *__restrict__ Ap, const double *__restrict__ dinv, double *__restrict__ x,
                        double *__restrict__ r, double *__restrict__ z, double *__restrict__ partials) {
  __shared__ double s_red[VEC_THREADS / 32];
  __shared__ double s_vals[3];
  __shared__ int s_flag;
  __shared__ HaloPiece s_pieces[PCG_MAX_FUSED_PIECES];
  if (ex.fl[FL_DONE] != 0) return;
  // the own rows of the current p: the two-pass form alternates between two buffers
  const double *__restrict__ p = reinterpret_cast<const long long *>(ex.sc)[SC_PCUR] != 0 ? p_second : p_first;
  double alpha;
  const int npieces = ex.mbox != nullptr ? ex.npieces : 0;
  if (ex.mbox != nullptr) {
    for (int q = threadIdx.x; q < npieces; q += VEC_THREADS) s_pieces[q] = ex.pieces[q];
    double pap, unused;
    if (!pcg_wait_sums(ex, PH_A, s_vals, pap, unused)) return;  // its barrier also publishes s_pieces
    alpha = ex.sc[SC_RZ] / pap;
  } else {
    alpha = ex.sc[SC_ALPHA];
  }
  const double malpha = -alpha;
  double rr = 0.0, rz = 0.0;
  bool stored_to_peer = false;
  // four elements per round, all loads first: the stores into the neighbours' buffers may alias anything as far
  // as the compiler knows, so it would not overlap the loads of successive elements by itself
  const int64_t stride = (int64_t)gridDim.x * VEC_THREADS;
  for (int64_t i0 = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i0 < n; i0 += 4 * stride) {
    double xv[4], pv[4], rv[4], av[4], dv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t i = i0 + k * stride;
      const bool in = i < n;
      xv[k] = in ? x[i] : 0.0;
      pv[k] = in ? p[i] : 0.0;
      rv[k] = in ? r[i] : 0.0;
      av[k] = in ? Ap[i] : 0.0;
      dv[k] = in ? dinv[i] : 0.0;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t i = i0 + k * stride;
      if (i >= n) break;
      const double xi = __dadd_rn(__dmul_rn(xv[k], 1.0), __dmul_rn(pv[k], alpha));
      const double ri = __dadd_rn(__dmul_rn(rv[k], 1.0), __dmul_rn(av[k], malpha));
      const double zi = __dmul_rn(ri, dv[k]);
      x[i] = xi;
      r[i] = ri;
      z[i] = zi;
      rr = __dadd_rn(rr, __dmul_rn(ri, ri));
      rz = __dadd_rn(rz, __dmul_rn(ri, zi));
      const int64_t wi = p_off + i;  // position in this rank's window
      for (int q = 0; q < npieces; ++q) {
        const int64_t d = wi - s_pieces[q].src_off;
        if (d >= 0 && d < s_pieces[q].len) {
          reinterpret_cast<double *>(s_pieces[q].dst_addr)[d] = zi;
          stored_to_peer = true;
        }
      }
    }
  }
  if (stored_to_peer) __threadfence_system();  // this thread's stores into a neighbour's buffer, before the block's ticket
  const double t0 = block_sum_vec(rr, s_red);
  const double t1 = block_sum_vec(rz, s_red);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = t0;
    partials[gridDim.x + blockIdx.x] = t1;
  }
  if (!pcg_last_block(pcg_tickets(ex.sc) + 1, gridDim.x, &s_flag)) return;
  const double srr = pcg_block_total(partials, gridDim.x, s_red);
  const double srz = pcg_block_total(partials + gridDim.x, gridDim.x, s_red);
  if (threadIdx.x == 0) {
    s_vals[0] = srr;
    s_vals[1] = srz;
    ex.sc[SC_RR] = srr;  // this rank's parts when the sums are exchanged
    ex.sc[SC_RZNEW] = srz;
    if (ex.mbox == nullptr) pcg_derive(DERIVE_DECIDE, ex.sc, ex.fl, ex.tol, ex.maxiter);
    else ex.sc[SC_ALPHA] = alpha;
  }
  __syncthreads();
  // every block's stores into the neighbours' buffers were fenced before its ticket; the fence inside the push
  // orders them before the sequence number that the neighbours wait for
  if (ex.mbox != nullptr) pcg_push_sums(ex, PH_B, s_vals[0], s_vals[1], pcg_seq(ex));
}

// Pass C with an exchange (without one the stop test ran in pass B's tail and the plain pass is used): every block
// repeats the stop test on every rank's r.r and r.z, updates its part of the own rows of p, and the halo entries of
// the window are updated too -- from the rows of z that the neighbours stored in pass B and the halo's old values
// of p, the operation the owner performs on the same operands.  The block that finishes last advances the
// iteration.
__global__ void __launch_bounds__(VEC_THREADS)
pcg_direction_fused_kernel(int64_t n, int64_t p_off, PcgExchange ex, const double *__restrict__ z, double *__restrict__ pw) {
  __shared__ double s_vals[3];
  __shared__ int s_flag;
  if (ex.fl[FL_DONE] != 0) return;
  double *__restrict__ p = pw + p_off;
  double rr, rznew;
  if (!pcg_wait_sums(ex, PH_B, s_vals, rr, rznew)) return;
  const double relres = sqrt(rr) / ex.sc[SC_INITRES];
  const unsigned long long iter = (unsigned long long)ex.fl[FL_ITERS] + 1;  // i starts at 1
  const bool go = (relres > ex.tol) && (iter != ex.maxiter);                // ordered compare: NaN stops the loop
  const double rz_old = ex.sc[SC_RZ];
  const double beta = rznew / rz_old;
  if (go) {
    for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS)
      p[i] = __dadd_rn(__dmul_rn(z[i], 1.0), __dmul_rn(p[i], beta));
    // halo entries of the window: the blocks share each range
    for (int q = 0; q < ex.nranges; ++q) {
      const long long start = ex.halo_ranges[2 * q], len = ex.halo_ranges[2 * q + 1];
      for (long long j = (long long)blockIdx.x * VEC_THREADS + threadIdx.x; j < len; j += (long long)gridDim.x * VEC_THREADS)
        pw[start + j] = __dadd_rn(__dmul_rn(ex.zhalo[start + j], 1.0), __dmul_rn(pw[start + j], beta));
    }
  }
  if (!pcg_last_block(pcg_tickets(ex.sc) + 2, gridDim.x, &s_flag)) return;
  if (threadIdx.x == 0) {
    ex.sc[SC_RR] = rr;
    ex.sc[SC_RZNEW] = rznew;
    ex.sc[SC_RELRES] = relres;
    if (go) {
      ex.sc[SC_BETA] = beta;
      ex.sc[SC_RZ] = rznew;
    } else {
      ex.fl[FL_DONE] = 1;
    }
    __threadfence();
    ex.fl[FL_ITERS] = (long long)iter;
  }
}

// Pass A's head and tail as kernels of their own, around SpMV kernels that do not carry them.
__global__ void pcg_halo_wait_kernel(PcgExchange ex) {
  __shared__ int s_flag;
  if (ex.fl[FL_DONE] != 0) return;
  pcg_wait_halo(ex, &s_flag);
}
__global__ void __launch_bounds__(SUM_THREADS)
pcg_pass_a_tail_kernel(PcgExchange ex, const double *__restrict__ blk_partial, int64_t nb) {
  __shared__ double s_red[SUM_THREADS / 32];
  if (ex.fl[FL_DONE] != 0) return;
  pcg_tail_pass_a(ex, blk_partial, nb, s_red);
}

static PcgExchange make_exchange(const PcgWork &w, const lapis_b200_pcg_exchange *e, double tol, uint64_t maxiter) {
  PcgExchange ex = {};
  ex.sc = w.sc;
  ex.fl = w.fl;
  ex.world = 1;
  ex.spin_limit = g_p2p_spin_limit;
  ex.tol = tol;
  ex.maxiter = maxiter;
  ex.zhalo = w.zh;  // the window-indexed z buffer (own rows and halo)
  if (e != nullptr && e->d_mbox != nullptr) {
    ex.mbox = static_cast<double *>(e->d_mbox);
    ex.peer_mbox = static_cast<const unsigned long long *>(e->d_peer_mbox);
    ex.halo_srcs = static_cast<const int *>(e->d_halo_srcs);
    ex.pieces = static_cast<const HaloPiece *>(e->d_z_pieces);
    ex.halo_ranges = static_cast<const long long *>(e->d_halo_ranges);
    ex.me = e->me;
    ex.world = e->world;
    ex.nsrc = e->nsrc;
    ex.npieces = e->nzpieces;
    ex.nranges = e->nranges;
  }
  return ex;
}

static int check_exchange(const lapis_b200_pcg_exchange *e, const char *what) {
  if (e == nullptr || e->d_mbox == nullptr) return LAPIS_OK;
  if (e->world < 1 || e->world > P2P_MAXW || e->me < 0 || e->me >= e->world || e->d_peer_mbox == nullptr || e->nsrc < 0 ||
      e->nsrc > 32 || e->nzpieces < 0 || e->nzpieces > PCG_MAX_FUSED_PIECES || e->nranges < 0 ||
      (e->nsrc > 0 && e->d_halo_srcs == nullptr) || (e->nzpieces > 0 && e->d_z_pieces == nullptr) ||
      (e->nranges > 0 && e->d_halo_ranges == nullptr))
    return fail(LAPIS_EBADARG, "%s: bad exchange description (up to %d ranks, 32 halo sources, %d halo pieces)", what,
                P2P_MAXW, PCG_MAX_FUSED_PIECES);
  return LAPIS_OK;
}

}  // namespace lapis_b200

using namespace lapis_b200;

extern "C" int lapis_b200_dot_f64(int64_t n, const double *d_x, const double *d_y, double *d_out, void *stream) {
  clear_error();
  if (n < 0) return fail(LAPIS_EBADSHAPE, "dot: negative length");
  if (d_out == nullptr || (n > 0 && (d_x == nullptr || d_y == nullptr))) return fail(LAPIS_EBADARG, "dot: null operand");
  cudaStream_t st = as_stream(stream);
  const unsigned g = vec_grid(n);
  double *partials = nullptr;
  LAPIS_CUDA_TRY(cudaMallocAsync(&partials, g * sizeof(double), st));
  dot_partial_kernel<<<g, VEC_THREADS, 0, st>>>(n, d_x, d_y, partials);
  sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(partials, g, 1, d_out, nullptr, DERIVE_NONE, nullptr, nullptr, 0.0, 0,
                                                 nullptr);
  LAPIS_CUDA_TRY(cudaGetLastError());
  LAPIS_CUDA_TRY(cudaFreeAsync(partials, st));
  return LAPIS_OK;
}

extern "C" int lapis_b200_axpby_f64(int64_t n, double a, const double *d_x, double b, const double *d_y,
                                    double *d_dst, void *stream) {
  clear_error();
  if (n < 0) return fail(LAPIS_EBADSHAPE, "axpby: negative length");
  if (n == 0) return LAPIS_OK;
  if (d_x == nullptr || d_y == nullptr || d_dst == nullptr) return fail(LAPIS_EBADARG, "axpby: null operand");
  axpby_kernel<<<vec_grid(n), VEC_THREADS, 0, as_stream(stream)>>>(n, a, d_x, b, d_y, d_dst);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

extern "C" int lapis_b200_mult_f64(int64_t n, const double *d_x, const double *d_y, double *d_dst, void *stream) {
  clear_error();
  if (n < 0) return fail(LAPIS_EBADSHAPE, "mult: negative length");
  if (n == 0) return LAPIS_OK;
  if (d_x == nullptr || d_y == nullptr || d_dst == nullptr) return fail(LAPIS_EBADARG, "mult: null operand");
  mult_kernel<<<vec_grid(n), VEC_THREADS, 0, as_stream(stream)>>>(n, d_x, d_y, d_dst);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

// ---- step-level PCG entry points (shared by the single-device driver below and by
// ---- multi-device callers that put a halo exchange / allreduce between the steps) ---
extern "C" int64_t lapis_b200_pcg_workspace_bytes(int64_t n, int64_t n_p) {
  if (n < 0 || n_p < n) return -1;
  return (int64_t)sizeof(double) * (16 + pcg_partials_len() + 3 * n + 3 * n_p);
}

extern "C" int lapis_b200_pcg_workspace_layout(int64_t n, int64_t n_p, int64_t *offsets4) {
  clear_error();
  if (n < 0 || n_p < n || offsets4 == nullptr) return fail(LAPIS_EBADARG, "pcg_workspace_layout: bad arguments");
  const int64_t vecs = 16 + pcg_partials_len();
  offsets4[0] = vecs;               // r
  offsets4[1] = vecs + n;           // z
  offsets4[2] = vecs + 2 * n;       // p (length n_p)
  offsets4[3] = vecs + 2 * n + n_p; // Ap
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_init(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, const double *d_b,
                                   const double *d_dinv, double *d_x, int derive, void *stream) {
  clear_error();
  if (d_work == nullptr || n < 0 || n_p < n || p_offset < 0 || p_offset + n > n_p)
    return fail(LAPIS_EBADARG, "pcg_init: bad workspace arguments");
  PcgWork w = carve(d_work, n, n_p);
  cudaStream_t st = as_stream(stream);
  LAPIS_CUDA_TRY(cudaMemsetAsync(w.sc, 0, 16 * sizeof(double), st));
  if (n_p > n) LAPIS_CUDA_TRY(cudaMemsetAsync(w.p, 0, (size_t)n_p * sizeof(double), st));
  LAPIS_CUDA_TRY(cudaMemsetAsync(w.p1, 0, (size_t)n_p * sizeof(double), st));
  LAPIS_CUDA_TRY(cudaMemsetAsync(w.partials, 0, (size_t)pcg_partials_len() * sizeof(double), st));
  pcg_init_kernel<<<w.grid, VEC_THREADS, 0, st>>>(n, d_b, d_dinv, w.r, w.z, w.p + p_offset, d_x, w.partials);
  sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(w.partials, w.grid, 2, w.sc + SC_RR, w.sc + SC_RZNEW,
                                                 derive ? DERIVE_INIT : DERIVE_NONE, w.sc, w.fl, 0.0, 0, nullptr);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_derive(void *d_work, int kind, double tol, uint64_t maxiter, void *stream) {
  clear_error();
  if (d_work == nullptr || kind < DERIVE_INIT || kind > DERIVE_DECIDE) return fail(LAPIS_EBADARG, "pcg_derive: bad arguments");
  double *base = static_cast<double *>(d_work);
  pcg_derive_kernel<<<1, 1, 0, as_stream(stream)>>>(kind, base, reinterpret_cast<long long *>(base + SC_COUNT), tol, maxiter);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

// Pass A: Ap = A p_ext (p_ext = the workspace's p buffer of length n_p, columns of A
// index into it), partial sums of p.Ap reduced into the scalar block.
extern "C" int lapis_b200_pcg_step_spmv(void *d_work, lapis_b200_csr_t h, int64_t n_p, int64_t p_offset, int derive,
                                        void *stream) {
  clear_error();
  if (d_work == nullptr || h == nullptr) return fail(LAPIS_EBADARG, "pcg_step_spmv: null argument");
  const int64_t n = h->nrows;
  PcgWork w = carve(d_work, n, n_p);
  cudaStream_t st = as_stream(stream);
  const int *skip = reinterpret_cast<const int *>(w.fl);  // low word of the little-endian int64 flag
  LAPIS_TRY(spmv_launch(h, w.p, w.Ap, 0, w.p + p_offset, h->blk_partial, skip, st));
  sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(h->blk_partial, h->nblk, 1, w.sc + SC_PAP, nullptr,
                                                 derive ? DERIVE_ALPHA : DERIVE_NONE, w.sc, w.fl, 0.0, 0, w.fl);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

// Pass B: x, r, z updates and the partial sums of r.r and r.z.
extern "C" int lapis_b200_pcg_step_update(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, const double *d_dinv,
                                          double *d_x, int derive, double tol, uint64_t maxiter, void *stream) {
  clear_error();
  if (d_work == nullptr) return fail(LAPIS_EBADARG, "pcg_step_update: null workspace");
  PcgWork w = carve(d_work, n, n_p);
  cudaStream_t st = as_stream(stream);
  pcg_update_kernel<<<w.grid, VEC_THREADS, 0, st>>>(n, w.sc, w.fl, w.p + p_offset, w.Ap, d_dinv, d_x, w.r, w.z,
                                                    w.partials);
  sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(w.partials, w.grid, 2, w.sc + SC_RR, w.sc + SC_RZNEW,
                                                 derive ? DERIVE_DECIDE : DERIVE_NONE, w.sc, w.fl, tol, maxiter, w.fl);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

// Pass C: p = z + beta p.
extern "C" int lapis_b200_pcg_step_direction(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, void *stream) {
  clear_error();
  if (d_work == nullptr) return fail(LAPIS_EBADARG, "pcg_step_direction: null workspace");
  PcgWork w = carve(d_work, n, n_p);
  pcg_direction_kernel<<<w.grid, VEC_THREADS, 0, as_stream(stream)>>>(n, w.sc, w.fl, w.z, w.p + p_offset);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

// ---- fused step entry points ------------------------------------------------------------------------------
extern "C" int lapis_b200_pcg_p2p_set_wait_limit(uint32_t polls) {
  clear_error();
  g_p2p_spin_limit = polls == 0 ? P2P_SPIN_LIMIT : polls;
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_fused_spmv(void *d_work, lapis_b200_csr_t h, int64_t n_p, int64_t p_offset, double tol,
                                         uint64_t maxiter, const lapis_b200_pcg_exchange *exchange, void *stream) {
  clear_error();
  if (d_work == nullptr || h == nullptr) return fail(LAPIS_EBADARG, "pcg_fused_spmv: null argument");
  LAPIS_TRY(check_exchange(exchange, "pcg_fused_spmv"));
  const int64_t n = h->nrows;
  PcgWork w = carve(d_work, n, n_p);
  cudaStream_t st = as_stream(stream);
  const PcgExchange ex = make_exchange(w, exchange, tol, maxiter);
  const int *skip = reinterpret_cast<const int *>(w.fl);  // low word of the little-endian int64 flag
  if (spmv_fuses_pcg_pass(h)) return spmv_launch_pcg_pass(h, w.p, w.Ap, w.p + p_offset, h->blk_partial, skip, st, ex);
  if (ex.mbox != nullptr && ex.nsrc > 0) pcg_halo_wait_kernel<<<1, 32, 0, st>>>(ex);
  LAPIS_TRY(spmv_launch(h, w.p, w.Ap, 0, w.p + p_offset, h->blk_partial, skip, st));
  pcg_pass_a_tail_kernel<<<1, SUM_THREADS, 0, st>>>(ex, h->blk_partial, h->nblk);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_fused_update(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, const double *d_dinv,
                                           double *d_x, double tol, uint64_t maxiter,
                                           const lapis_b200_pcg_exchange *exchange, void *stream) {
  clear_error();
  if (d_work == nullptr) return fail(LAPIS_EBADARG, "pcg_fused_update: null workspace");
  LAPIS_TRY(check_exchange(exchange, "pcg_fused_update"));
  PcgWork w = carve(d_work, n, n_p);
  const PcgExchange ex = make_exchange(w, exchange, tol, maxiter);
  // z goes into the window-indexed buffer (own rows at the window's own offset)
  pcg_update_fused_kernel<<<w.grid, VEC_THREADS, 0, as_stream(stream)>>>(n, p_offset, ex, w.p + p_offset, w.p1 + p_offset, w.Ap,
                                                                         d_dinv, d_x, w.r, w.zh + p_offset, w.partials);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_fused_direction(void *d_work, int64_t n, int64_t n_p, int64_t p_offset, double tol,
                                              uint64_t maxiter, const lapis_b200_pcg_exchange *exchange, void *stream) {
  clear_error();
  if (d_work == nullptr) return fail(LAPIS_EBADARG, "pcg_fused_direction: null workspace");
  LAPIS_TRY(check_exchange(exchange, "pcg_fused_direction"));
  PcgWork w = carve(d_work, n, n_p);
  const PcgExchange ex = make_exchange(w, exchange, tol, maxiter);
  if (ex.mbox == nullptr)  // the stop test and beta are in the scalar block already: the plain pass
    pcg_direction_kernel<<<w.grid, VEC_THREADS, 0, as_stream(stream)>>>(n, w.sc, w.fl, w.zh + p_offset, w.p + p_offset);
  else
    pcg_direction_fused_kernel<<<w.grid, VEC_THREADS, 0, as_stream(stream)>>>(n, p_offset, ex, w.zh + p_offset, w.p);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

// Whether the matrix is served by the kernel that folds the direction update into the SpMV pass (two launches
// per iteration: lapis_b200_pcg_fused_spmv_direction, lapis_b200_pcg_fused_update).
extern "C" int lapis_b200_pcg_folds_direction(lapis_b200_csr_t h) { return h != nullptr && spmv_fuses_pcg_pass(h) ? 1 : 0; }

extern "C" int lapis_b200_pcg_fused_spmv_direction(void *d_work, lapis_b200_csr_t h, int64_t n_p, int64_t p_offset, double tol,
                                                   uint64_t maxiter, const lapis_b200_pcg_exchange *exchange, void *stream) {
  clear_error();
  if (d_work == nullptr || h == nullptr) return fail(LAPIS_EBADARG, "pcg_fused_spmv_direction: null argument");
  if (h->ncols != n_p || p_offset < 0 || p_offset + h->nrows > n_p)
    return fail(LAPIS_EBADSHAPE, "pcg_fused_spmv_direction: matrix columns must index the p window");
  LAPIS_TRY(check_exchange(exchange, "pcg_fused_spmv_direction"));
  PcgWork w = carve(d_work, h->nrows, n_p);
  const PcgExchange ex = make_exchange(w, exchange, tol, maxiter);
  return spmv_launch_pcg_direction_pass(h, p_offset, w.p, w.p1, w.Ap, h->blk_partial, as_stream(stream), ex);
}

// Reads {done, iters} and relres back (synchronises the stream).
extern "C" int lapis_b200_pcg_status(void *d_work, int *done, uint64_t *iters, double *relres, void *stream) {
  clear_error();
  if (d_work == nullptr) return fail(LAPIS_EBADARG, "pcg_status: null workspace");
  double host[16];
  cudaStream_t st = as_stream(stream);
  LAPIS_CUDA_TRY(cudaMemcpyAsync(host, d_work, sizeof(host), cudaMemcpyDeviceToHost, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  const long long *fl = reinterpret_cast<const long long *>(host + SC_COUNT);
  if (done) *done = (int)fl[FL_DONE];
  if (iters) *iters = (uint64_t)fl[FL_ITERS];
  if (relres) *relres = host[SC_RELRES];
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_f64(lapis_b200_csr_t h, const double *d_b, const double *d_dinv, double tol,
                                  uint64_t maxiter, double *d_x, uint64_t *iters, double *relres, void *stream) {
  clear_error();
  if (h == nullptr) return fail(LAPIS_EBADARG, "pcg: null matrix handle");
  if (h->nrows != h->ncols) return fail(LAPIS_EBADSHAPE, "pcg: matrix is not square");
  const int64_t n = h->nrows;
  if (n > 0 && (d_b == nullptr || d_dinv == nullptr || d_x == nullptr)) return fail(LAPIS_EBADARG, "pcg: null operand");
  cudaStream_t st = as_stream(stream);
  if (n == 0) {  // 0/0 residual: the ordered compare fails and the loop stops after one pass
    if (iters) *iters = 1;
    if (relres) *relres = NAN;
    return LAPIS_OK;
  }
  // a solve runs the SpMV pass many times: pick the kernel variant for this matrix first
  if (h->tuned_threads == 0 && (maxiter == 0 || maxiter >= 16)) LAPIS_TRY(lapis_b200_csr_tune(h, st));
  void *work = nullptr;
  LAPIS_CUDA_TRY(cudaMalloc(&work, (size_t)lapis_b200_pcg_workspace_bytes(n, n)));
  int status = lapis_b200_pcg_init(work, n, n, 0, d_b, d_dinv, d_x, 1, st);
  int done = 0;
  uint64_t it = 0;
  double rel = 0.0;
  // The emitted loop stops when relres <= tol or i == maxiter with i starting at 1
  // (examples/pcg_solve.py:72,86-90); maxiter == 0 therefore never stops on the count.
  // The same holds here, up to a bound of 2^31 iterations.
  const uint64_t limit = maxiter == 0 ? (1ull << 31) : maxiter;
  const uint64_t check_every = 16;
  const bool two_pass = lapis_b200_pcg_folds_direction(h) != 0;  // the direction update inside the next SpMV pass
  for (uint64_t i = 1; status == LAPIS_OK && !done && i <= limit; ++i) {
    if (two_pass) {
      status = lapis_b200_pcg_fused_spmv_direction(work, h, n, 0, tol, maxiter, nullptr, st);
      if (status == LAPIS_OK) status = lapis_b200_pcg_fused_update(work, n, n, 0, d_dinv, d_x, tol, maxiter, nullptr, st);
    } else {
      status = lapis_b200_pcg_fused_spmv(work, h, n, 0, tol, maxiter, nullptr, st);
      if (status == LAPIS_OK) status = lapis_b200_pcg_fused_update(work, n, n, 0, d_dinv, d_x, tol, maxiter, nullptr, st);
      if (status == LAPIS_OK) status = lapis_b200_pcg_fused_direction(work, n, n, 0, tol, maxiter, nullptr, st);
    }
    if (status == LAPIS_OK && (i % check_every == 0 || i == limit))
      status = lapis_b200_pcg_status(work, &done, &it, &rel, st);
  }
  if (status == LAPIS_OK && !done) status = lapis_b200_pcg_status(work, &done, &it, &rel, st);
  // a persistent SpMV block whose bounded wait gave up leaves Ap incomplete: the solve is not valid then
  if (status == LAPIS_OK) status = lapis_b200_spmv_status(st);
  cudaFree(work);
  if (status != LAPIS_OK) return status;
  if (iters) *iters = it;
  if (relres) *relres = rel;
  return LAPIS_OK;
}

// ---------------------------------------------------------------------------------------------
// Row-partitioned PCG without library collectives: the three exchanges of an iteration (p.Ap; r.r and
// r.z; the halo of p) are stores into the peers' memory over NVLink plus sequence-numbered flags, and
// the consumers are small kernels that wait for the flags with a bound.  One process per GPU; a rank
// maps every peer's mailbox and workspace with CUDA IPC (lapis_b200_peer_*).  The reference has no
// multi-device path; this is this library's own.
//
// Mailbox of a rank (doubles): slot (phase, src) at (phase*16 + src)*4 = {v0, v1, seq, -}; halo flag of
// src at 256 + src; error flag at 272.  Phases: 0 = p.Ap, 1 = r.r / r.z, 2 and 3 = the initial r.r / r.z
// of even and odd epochs.  seq = epoch * 2^32 + iteration; the caller stores epoch * 2^32 in workspace
// slot 10 after lapis_b200_pcg_init and raises the epoch by one per initialisation, so values left by an
// earlier solve never match (a device-resident value keeps a captured CUDA graph of one iteration valid
// across solves).  A slot is rewritten only after its reader has consumed it: a rank pushes phase 0 of
// iteration k+1 after its phase-1 wait of iteration k, which needs every peer's phase-1 push, which each
// peer does after its own phase-0 read of iteration k (and symmetrically for phase 1 and for the halo).
// Two initialisations may follow one another with no iteration between them, hence the two initial
// slots: the push of epoch e+2 comes after the wait of epoch e+1, which needs every peer's push of e+1,
// which each peer issues after its own read of epoch e.
// Every rank adds the same values in rank order, so all ranks derive bit-identical scalars.
// ---------------------------------------------------------------------------------------------
namespace lapis_b200 {

// Slot row of a phase: the initial exchange alternates between two rows by the parity of the epoch.
__device__ __forceinline__ int p2p_slot_row(int phase, double base_seq) {
  return phase == PH_INIT ? PH_INIT + (int)((long long)(base_seq * (1.0 / 4294967296.0)) & 1) : phase;
}

__global__ void p2p_push_scalars_kernel(const double *__restrict__ sc, const long long *__restrict__ fl, int phase, int me,
                                        int world, const unsigned long long *__restrict__ peer_mbox) {
  const int j = threadIdx.x;
  if (j >= world) return;
  const double base_seq = sc[SC_EPOCH];
  if (phase != PH_INIT && fl[FL_DONE] != 0) return;
  const double seq = base_seq + (phase == PH_INIT ? 0.0 : (double)(fl[FL_ITERS] + 1));
  const double v0 = phase == PH_A ? sc[SC_PAP] : sc[SC_RR];
  const double v1 = phase == PH_A ? 0.0 : sc[SC_RZNEW];
  volatile double *slot = reinterpret_cast<volatile double *>(peer_mbox[j]) + (p2p_slot_row(phase, base_seq) * P2P_MAXW + me) * 4;
  slot[0] = v0;
  slot[1] = v1;
  __threadfence_system();  // values before the sequence number, system-wide
  slot[2] = seq;
}

__global__ void p2p_wait_reduce_kernel(double *sc, long long *fl, double *mbox, int phase, int world, int derive,
                                       double tol, unsigned long long maxiter, unsigned spin_limit) {
  const int j = threadIdx.x;  // one warp
  const double base_seq = sc[SC_EPOCH];
  if (phase != PH_INIT && fl[FL_DONE] != 0) return;
  const double expected = base_seq + (phase == PH_INIT ? 0.0 : (double)(fl[FL_ITERS] + 1));
  const int row = p2p_slot_row(phase, base_seq);
  bool ok = true;
  if (j < world) ok = p2p_wait_equal(mbox + (row * P2P_MAXW + j) * 4 + 2, expected, spin_limit);
  const bool all_ok = __all_sync(0xffffffffu, ok);
  if (j != 0) return;
  if (!all_ok) {  // a peer never delivered: stop the solve and let the host see why
    mbox[P2P_ERR] = 1.0 + phase;
    fl[FL_DONE] = 1;
    return;
  }
  __threadfence_system();
  double v0 = 0.0, v1 = 0.0;
  for (int r = 0; r < world; ++r) {  // rank order on every rank
    const volatile double *slot = mbox + (row * P2P_MAXW + r) * 4;
    v0 = __dadd_rn(v0, slot[0]);
    v1 = __dadd_rn(v1, slot[1]);
  }
  if (phase == PH_A) {
    sc[SC_PAP] = v0;
  } else {
    sc[SC_RR] = v0;
    sc[SC_RZNEW] = v1;
  }
  pcg_derive(derive, sc, fl, tol, maxiter);
}

__global__ void __launch_bounds__(256)
p2p_halo_push_kernel(const double *__restrict__ p_window, const double *__restrict__ sc, const long long *__restrict__ fl,
                     const HaloPiece *__restrict__ pieces) {
  if (fl[FL_DONE] != 0) return;
  const double base_seq = sc[SC_EPOCH];
  const HaloPiece pc = pieces[blockIdx.x];
  double *dst = reinterpret_cast<double *>(pc.dst_addr);
  for (long long i = threadIdx.x; i < pc.len; i += blockDim.x) dst[i] = p_window[pc.src_off + i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile double *>(pc.flag_addr) = base_seq + (double)(fl[FL_ITERS] + 1);
}

__global__ void p2p_halo_wait_kernel(const double *sc, long long *fl, double *mbox, const int *__restrict__ srcs, int nsrc,
                                     unsigned spin_limit) {
  const int j = threadIdx.x;  // one warp
  if (fl[FL_DONE] != 0) return;
  const double base_seq = sc[SC_EPOCH];
  const double expected = base_seq + (double)(fl[FL_ITERS] + 1);
  bool ok = true;
  if (j < nsrc) ok = p2p_wait_equal(mbox + P2P_HALO + srcs[j], expected, spin_limit);
  const bool all_ok = __all_sync(0xffffffffu, ok);
  if (j == 0 && !all_ok) {
    mbox[P2P_ERR] = 9.0;
    fl[FL_DONE] = 1;
  }
}

}  // namespace lapis_b200

extern "C" int64_t lapis_b200_pcg_p2p_mailbox_bytes(void) { return (int64_t)P2P_MBOX_DOUBLES * 8; }

// Index (in doubles) of the first halo flag and of the error mark inside a mailbox.
extern "C" void lapis_b200_pcg_p2p_mailbox_layout(int64_t *halo_index, int64_t *error_index) {
  if (halo_index) *halo_index = P2P_HALO;
  if (error_index) *error_index = P2P_ERR;
}

// Device memory that peers can map: allocated here (zeroed), exported as a CUDA IPC handle (64 bytes).
extern "C" int lapis_b200_peer_alloc(int64_t bytes, void **ptr, unsigned char *handle64) {
  clear_error();
  if (bytes <= 0 || ptr == nullptr || handle64 == nullptr) return fail(LAPIS_EBADARG, "peer_alloc: bad arguments");
  void *p = nullptr;
  LAPIS_CUDA_TRY(cudaMalloc(&p, (size_t)bytes));
  cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(LAPIS_ECUDA, "peer_alloc: %s", cudaGetErrorString(e));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return LAPIS_OK;
}

// Maps a peer's allocation into this process for the current device (peer access is enabled by the
// open itself); the pointer may be dereferenced by kernels running on the current device.
extern "C" int lapis_b200_peer_open(const unsigned char *handle64, void **ptr) {
  clear_error();
  if (handle64 == nullptr || ptr == nullptr) return fail(LAPIS_EBADARG, "peer_open: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void *p = nullptr;
  LAPIS_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return LAPIS_OK;
}
extern "C" int lapis_b200_peer_close(void *ptr) {
  clear_error();
  if (ptr != nullptr) LAPIS_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return LAPIS_OK;
}
extern "C" int lapis_b200_peer_free(void *ptr) {
  clear_error();
  if (ptr != nullptr) LAPIS_CUDA_TRY(cudaFree(ptr));
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_p2p_push_scalars(void *d_work, int phase, int me, int world, const void *d_peer_mbox,
                                               void *stream) {
  clear_error();
  if (d_work == nullptr || d_peer_mbox == nullptr || world < 1 || world > P2P_MAXW || me < 0 || me >= world || phase < 0 ||
      phase > 2)
    return fail(LAPIS_EBADARG, "pcg_p2p_push_scalars: bad arguments");
  double *base = static_cast<double *>(d_work);
  p2p_push_scalars_kernel<<<1, 32, 0, as_stream(stream)>>>(base, reinterpret_cast<long long *>(base + SC_COUNT), phase, me,
                                                           world, static_cast<const unsigned long long *>(d_peer_mbox));
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_p2p_wait_reduce(void *d_work, void *d_mbox, int phase, int world, int derive, double tol,
                                              uint64_t maxiter, void *stream) {
  clear_error();
  if (d_work == nullptr || d_mbox == nullptr || world < 1 || world > P2P_MAXW || phase < 0 || phase > 2 || derive < 1 ||
      derive > 3)
    return fail(LAPIS_EBADARG, "pcg_p2p_wait_reduce: bad arguments");
  double *base = static_cast<double *>(d_work);
  p2p_wait_reduce_kernel<<<1, 32, 0, as_stream(stream)>>>(base, reinterpret_cast<long long *>(base + SC_COUNT),
                                                          static_cast<double *>(d_mbox), phase, world, derive, tol, maxiter,
                                                          g_p2p_spin_limit);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

// pieces: device array of npieces records {dst address, source offset in the p window, length, flag address}.
extern "C" int lapis_b200_pcg_p2p_halo_push(void *d_work, int64_t n, int64_t n_p, const void *d_pieces, int npieces,
                                            void *stream) {
  clear_error();
  if (npieces == 0) return LAPIS_OK;
  if (d_work == nullptr || d_pieces == nullptr || npieces < 0) return fail(LAPIS_EBADARG, "pcg_p2p_halo_push: bad arguments");
  PcgWork w = carve(d_work, n, n_p);
  p2p_halo_push_kernel<<<npieces, 256, 0, as_stream(stream)>>>(w.p, w.sc, w.fl, static_cast<const HaloPiece *>(d_pieces));
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

extern "C" int lapis_b200_pcg_p2p_halo_wait(void *d_work, void *d_mbox, const void *d_srcs, int nsrc, void *stream) {
  clear_error();
  if (nsrc == 0) return LAPIS_OK;
  if (d_work == nullptr || d_mbox == nullptr || d_srcs == nullptr || nsrc < 0 || nsrc > 32)
    return fail(LAPIS_EBADARG, "pcg_p2p_halo_wait: bad arguments");
  double *base = static_cast<double *>(d_work);
  p2p_halo_wait_kernel<<<1, 32, 0, as_stream(stream)>>>(base, reinterpret_cast<long long *>(base + SC_COUNT),
                                                        static_cast<double *>(d_mbox), static_cast<const int *>(d_srcs), nsrc,
                                                        g_p2p_spin_limit);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

// ---------------------------------------------------------------------------------------------
// Hitting-time moments (examples/hitting_times.py:151-194 in the LAPIS project): two Jacobi-PCG solves
// with the masked graph Laplacian y = M (D - alpha A) M x as the operator (@plpt, :73-92) and z = r / d
// as the preconditioner (:113, :140).  Same three passes per iteration as the plain solver:
//   A  t = (alpha A) mp with the fused partial sums of mp.t        (mp = mask * p, kept beside p)
//   B  Ap = (d*mp - t)*mask on the fly; x, r, z updates; partial sums of r.r and r.z
//   C  p = z + beta p; mp = mask*p; partial sums of d*mp*mp
// so p.Ap = sum d mp^2 - mp.t needs no pass of its own.
// ---------------------------------------------------------------------------------------------
namespace lapis_b200 {

__global__ void __launch_bounds__(VEC_THREADS)
scale_copy_kernel(int64_t n, const double *__restrict__ src, double a, double *__restrict__ dst) {
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS)
    dst[i] = __dmul_rn(src[i], a);  // hitting_times.py:50-70
}

// r = b; z = r/d; p = z; mp = mask*p; x = 0; partial sums of r.r, r.z and d*mp*mp  (hitting_times.py:111-117)
__global__ void __launch_bounds__(VEC_THREADS)
mht_init_kernel(int64_t n, const double *__restrict__ b, const double *__restrict__ d, const double *__restrict__ mask,
                double *__restrict__ r, double *__restrict__ z, double *__restrict__ p, double *__restrict__ mp,
                double *__restrict__ x, double *__restrict__ partials) {
  __shared__ double s_red[VEC_THREADS / 32];
  double rr = 0.0, rz = 0.0, dm = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS) {
    const double ri = b[i], di = d[i];
    const double zi = __ddiv_rn(ri, di);
    const double mpi = __dmul_rn(zi, mask[i]);
    r[i] = ri;
    z[i] = zi;
    p[i] = zi;
    mp[i] = mpi;
    x[i] = 0.0;
    rr = __dadd_rn(rr, __dmul_rn(ri, ri));
    rz = __dadd_rn(rz, __dmul_rn(ri, zi));
    dm = __dadd_rn(dm, __dmul_rn(__dmul_rn(di, mpi), mpi));
  }
  const double t0 = block_sum_vec(rr, s_red);
  const double t1 = block_sum_vec(rz, s_red);
  const double t2 = block_sum_vec(dm, s_red);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = t0;
    partials[gridDim.x + blockIdx.x] = t1;
    partials[2 * gridDim.x + blockIdx.x] = t2;
  }
}

// Ap = (d*mp - t)*mask (hitting_times.py:84-88); x += alpha p; r -= alpha Ap; z = r/d; partial sums of r.r, r.z
__global__ void __launch_bounds__(VEC_THREADS)
mht_update_kernel(int64_t n, const double *__restrict__ sc, const long long *__restrict__ fl,
                  const double *__restrict__ p, const double *__restrict__ mp, const double *__restrict__ t,
                  const double *__restrict__ d, const double *__restrict__ mask, double *__restrict__ x,
                  double *__restrict__ r, double *__restrict__ z, double *__restrict__ partials) {
  __shared__ double s_red[VEC_THREADS / 32];
  if (fl[FL_DONE] != 0) return;
  const double alpha = sc[SC_ALPHA];
  const double malpha = -alpha;
  double rr = 0.0, rz = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS) {
    const double di = d[i];
    const double api = __dmul_rn(__dsub_rn(__dmul_rn(di, mp[i]), t[i]), mask[i]);
    const double xi = __dadd_rn(__dmul_rn(x[i], 1.0), __dmul_rn(p[i], alpha));
    const double ri = __dadd_rn(__dmul_rn(r[i], 1.0), __dmul_rn(api, malpha));
    const double zi = __ddiv_rn(ri, di);
    x[i] = xi;
    r[i] = ri;
    z[i] = zi;
    rr = __dadd_rn(rr, __dmul_rn(ri, ri));
    rz = __dadd_rn(rz, __dmul_rn(ri, zi));
  }
  const double t0 = block_sum_vec(rr, s_red);
  const double t1 = block_sum_vec(rz, s_red);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = t0;
    partials[gridDim.x + blockIdx.x] = t1;
  }
}

// p = z + beta p (hitting_times.py:143); mp = mask*p; partial sums of d*mp*mp
__global__ void __launch_bounds__(VEC_THREADS)
mht_direction_kernel(int64_t n, const double *__restrict__ sc, const long long *__restrict__ fl,
                     const double *__restrict__ z, const double *__restrict__ d, const double *__restrict__ mask,
                     double *__restrict__ p, double *__restrict__ mp, double *__restrict__ partials) {
  __shared__ double s_red[VEC_THREADS / 32];
  if (fl[FL_DONE] != 0) return;
  const double beta = sc[SC_BETA];
  double dm = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS) {
    const double pi = __dadd_rn(__dmul_rn(z[i], 1.0), __dmul_rn(p[i], beta));
    const double mpi = __dmul_rn(pi, mask[i]);
    p[i] = pi;
    mp[i] = mpi;
    dm = __dadd_rn(dm, __dmul_rn(__dmul_rn(d[i], mpi), mpi));
  }
  const double t0 = block_sum_vec(dm, s_red);
  if (threadIdx.x == 0) partials[2 * gridDim.x + blockIdx.x] = t0;
}

// b2 = mask * (d*mom1 + t) with t = (alpha A) mom1  (hitting_times.py:163-176)
__global__ void __launch_bounds__(VEC_THREADS)
mht_rhs2_kernel(int64_t n, const double *__restrict__ t, const double *__restrict__ mask, const double *__restrict__ mom1,
                const double *__restrict__ d, double *__restrict__ b2) {
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS)
    b2[i] = __dmul_rn(__dadd_rn(__dmul_rn(d[i], mom1[i]), t[i]), mask[i]);
}

// sqrt(mom2 - mom1^2)  (hitting_times.py:196-218)
__global__ void __launch_bounds__(VEC_THREADS)
normalize_mom2_kernel(int64_t n, const double *__restrict__ mom1, const double *__restrict__ mom2, double *__restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * VEC_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * VEC_THREADS)
    out[i] = sqrt(__dsub_rn(mom2[i], __dmul_rn(mom1[i], mom1[i])));
}

// One masked solve.  work: [16 header][3*G partials][r][z][p][mp][t], G = vec_grid(n).
static int mht_solve(const lapis_b200_csr *A, const double *d_b, const double *d_d, const double *d_mask, double tol,
                     uint64_t maxiter, double *d_x, double *work, uint64_t *iters, double *relres, cudaStream_t st) {
  const int64_t n = A->nrows;
  const unsigned G = vec_grid(n);
  double *sc = work;
  long long *fl = reinterpret_cast<long long *>(work + SC_COUNT);
  double *partials = work + 16;
  double *r = partials + 3 * (int64_t)G, *z = r + n, *p = z + n, *mp = p + n, *t = mp + n;
  const int *skip = reinterpret_cast<const int *>(fl);
  LAPIS_CUDA_TRY(cudaMemsetAsync(work, 0, 16 * sizeof(double), st));
  mht_init_kernel<<<G, VEC_THREADS, 0, st>>>(n, d_b, d_d, d_mask, r, z, p, mp, d_x, partials);
  sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(partials + 2 * (int64_t)G, G, 1, sc + SC_DMP2, nullptr, DERIVE_NONE, sc, fl,
                                                 0.0, 0, nullptr);
  sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(partials, G, 2, sc + SC_RR, sc + SC_RZNEW, DERIVE_INIT, sc, fl, 0.0, 0,
                                                 nullptr);
  LAPIS_CUDA_TRY(cudaGetLastError());
  const uint64_t limit = maxiter == 0 ? (1ull << 31) : maxiter;
  const uint64_t check_every = 16;
  int done = 0;
  double host[16];
  for (uint64_t i = 1; !done && i <= limit; ++i) {
    LAPIS_TRY(spmv_launch(A, mp, t, 0, mp, A->blk_partial, skip, st));
    sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(A->blk_partial, A->nblk, 1, sc + SC_PAP, nullptr, DERIVE_ALPHA_MASKED, sc,
                                                   fl, 0.0, 0, fl);
    mht_update_kernel<<<G, VEC_THREADS, 0, st>>>(n, sc, fl, p, mp, t, d_d, d_mask, d_x, r, z, partials);
    sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(partials, G, 2, sc + SC_RR, sc + SC_RZNEW, DERIVE_DECIDE, sc, fl, tol,
                                                   maxiter, fl);
    mht_direction_kernel<<<G, VEC_THREADS, 0, st>>>(n, sc, fl, z, d_d, d_mask, p, mp, partials);
    sum_partials_kernel<<<1, SUM_THREADS, 0, st>>>(partials + 2 * (int64_t)G, G, 1, sc + SC_DMP2, nullptr, DERIVE_NONE, sc,
                                                   fl, 0.0, 0, fl);
    LAPIS_CUDA_TRY(cudaGetLastError());
    if (i % check_every == 0 || i == limit) {
      LAPIS_CUDA_TRY(cudaMemcpyAsync(host, work, sizeof(host), cudaMemcpyDeviceToHost, st));
      LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
      done = (int)reinterpret_cast<const long long *>(host + SC_COUNT)[FL_DONE];
    }
  }
  LAPIS_CUDA_TRY(cudaMemcpyAsync(host, work, sizeof(host), cudaMemcpyDeviceToHost, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  if (iters) *iters = (uint64_t) reinterpret_cast<const long long *>(host + SC_COUNT)[FL_ITERS];
  if (relres) *relres = host[SC_RELRES];
  return LAPIS_OK;
}

}  // namespace lapis_b200

extern "C" int lapis_b200_mht_f64(lapis_b200_csr_t h, const double *d_mask, const double *d_d, double alpha, double tol,
                                  uint64_t maxiter, double *d_mom1, double *d_mom2, uint64_t *iters2, double *relres2,
                                  void *stream) {
  clear_error();
  if (h == nullptr) return fail(LAPIS_EBADARG, "mht: null matrix handle");
  if (h->nrows != h->ncols) return fail(LAPIS_EBADSHAPE, "mht: matrix is not square");
  const int64_t n = h->nrows;
  if (n == 0) return LAPIS_OK;
  if (d_mask == nullptr || d_d == nullptr || d_mom1 == nullptr || d_mom2 == nullptr)
    return fail(LAPIS_EBADARG, "mht: null operand");
  cudaStream_t st = as_stream(stream);
  // two solves run the SpMV pass many times: pick the kernel variant for this matrix first
  if (h->tuned_threads == 0 && (maxiter == 0 || maxiter >= 16)) LAPIS_TRY(lapis_b200_csr_tune(h, st));
  const unsigned G = vec_grid(n);
  const size_t work_doubles = 16 + 3 * (size_t)G + 5 * (size_t)n;
  // [work][b][pad][scaled values][pad]: the SpMV kernels stream the values with 16-byte accesses starting at
  // entry (base & ~3) of the array the handle points to, so "scaled copy - base" must be 16-byte aligned
  // like the caller's array is, and the few entries in front of the copy must be readable (they are
  // masked out, not used).
  size_t sval_index = work_doubles + (size_t)n + 4;
  if (((int64_t)sval_index - h->base) & 1) sval_index += 1;
  double *buf = nullptr;
  LAPIS_CUDA_TRY(cudaMalloc(&buf, (sval_index + (size_t)h->nnz + 8) * sizeof(double)));
  double *work = buf, *bbuf = buf + work_doubles, *sval = buf + sval_index;
  // the emitted code scales the matrix values in place; here the caller's array stays as it is and the
  // solves read a scaled copy through a shallow copy of the handle (same streaming plan)
  lapis_b200_csr scaled = *h;
  const double *val0 = h->val + h->base;  // the handle's arrays are indexed by absolute offsets
  if (h->nnz > 0) scale_copy_kernel<<<vec_grid(h->nnz), VEC_THREADS, 0, st>>>(h->nnz, val0, alpha, sval);
  scaled.val = sval - h->base;
  uint64_t it[2] = {0, 0};
  double rel[2] = {0.0, 0.0};
  mult_kernel<<<G, VEC_THREADS, 0, st>>>(n, d_d, d_mask, bbuf);  // hitting_times.py:158
  int status = mht_solve(&scaled, bbuf, d_d, d_mask, tol, maxiter, d_mom1, work, &it[0], &rel[0], st);
  if (status == LAPIS_OK) status = spmv_launch(&scaled, d_mom1, work + 16, 0, nullptr, nullptr, nullptr, st);
  if (status == LAPIS_OK) {
    mht_rhs2_kernel<<<G, VEC_THREADS, 0, st>>>(n, work + 16, d_mask, d_mom1, d_d, bbuf);
    status = mht_solve(&scaled, bbuf, d_d, d_mask, tol, maxiter, d_mom2, work, &it[1], &rel[1], st);
  }
  cudaError_t e = cudaStreamSynchronize(st);
  cudaFree(buf);
  if (status != LAPIS_OK) return status;
  if (e != cudaSuccess) return fail(LAPIS_ECUDA, "mht: %s", cudaGetErrorString(e));
  LAPIS_TRY(lapis_b200_spmv_status(st));  // a persistent SpMV block that gave up leaves its output incomplete
  if (iters2) iters2[0] = it[0], iters2[1] = it[1];
  if (relres2) relres2[0] = rel[0], relres2[1] = rel[1];
  return LAPIS_OK;
}

extern "C" int lapis_b200_normalize_mom2_f64(int64_t n, const double *d_mom1, const double *d_mom2, double *d_out,
                                             void *stream) {
  clear_error();
  if (n < 0) return fail(LAPIS_EBADSHAPE, "normalize_mom2: negative length");
  if (n == 0) return LAPIS_OK;
  if (d_mom1 == nullptr || d_mom2 == nullptr || d_out == nullptr) return fail(LAPIS_EBADARG, "normalize_mom2: null operand");
  normalize_mom2_kernel<<<vec_grid(n), VEC_THREADS, 0, as_stream(stream)>>>(n, d_mom1, d_mom2, d_out);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}
