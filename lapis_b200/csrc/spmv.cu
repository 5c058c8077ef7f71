// CSR SpMV and SpMM for sm_100a.
//
// Replaces the loop the LAPIS emitter prints for `linalg.matvec` on a CSR operand
// (tests/Dialect/Kokkos/loop_mapping_2.mlir.gold:12-37; emitted by
// mlir/lib/Target/KokkosCpp/TranslateToKokkosCpp.cpp:1966-2064 and :1692-1845):
// one row per Kokkos thread with a vector length taken from the *average* row
// length.  That shape streams val/crd uncoalesced for short rows and serialises
// long ones.  Here the stored entries are the unit of work instead:
//
//   * The entry range is cut into chunks of a fixed size T (2048 by default); thread
//     block b processes exactly chunk b, so every block streams T consecutive
//     (val, crd) pairs with aligned 16-byte loads that are fully coalesced whatever
//     the row lengths are, gathers x through the read-only path, and parks the
//     products in shared memory.  All in-chunk indexing is 32-bit.
//   * A per-matrix plan (8 bytes per chunk, one binary search each) gives the first
//     row that ends inside each chunk.  Rows that end in the chunk are reduced out
//     of shared memory: rows of up to 32 in-chunk entries by one lane each, in the
//     sequential CPU order (measured: more lanes per short row only add instructions),
//     longer rows by a whole warp in a second pass, so one long row among short ones
//     does not serialise a thread.
//     A variant (spmv_scan_kernel) keeps the products in registers and sums the rows by a
//     warp-level segmented scan instead; it is offered by the relaxed tuner only, because it
//     adds a row's products in scan order.
//   * A row that runs past the end of its chunk leaves its partial sum in carry[b];
//     a tiny second kernel adds the carries to the row's y in chunk order.  No
//     atomics on the data path: results are run-to-run identical.
//
// Arithmetic: products and sums use explicit round-to-nearest multiplies and adds
// (no FMA contraction), as the emitted code has separate arith.mulf / arith.addf.
// A row of up to 32 entries that lies inside one chunk is summed exactly like the
// sequential CPU loop (identical bits).  Rows handled by a warp, and rows cut by a chunk
// boundary, are summed in another fixed order (documented tolerance 1e-12 of the row's
// magnitude).
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "common.h"
#include "pcg_fuse.h"

namespace lapis_b200 {

#ifndef LAPIS_SPMV_TILE
#define LAPIS_SPMV_TILE 2048
#endif
constexpr int SPMV_TILE = LAPIS_SPMV_TILE;       // stored entries per chunk == per thread block (part of the plan's meaning)
constexpr int SPMV_POS_CACHE = 1024;  // row offsets staged per block; further rows read global memory
constexpr int SPMV_LONG_ROW = 32;     // rows with more in-chunk entries than this are reduced by a whole warp

// ---------------------------------------------------------------------------
// Plan: plan[b] = first row r with pos[r+1] > abase + b*TILE (the row holding the
// chunk's first entry), plan[0] = 0, plan[nblk] = nrows; abase = pos[0] & ~3.
// ---------------------------------------------------------------------------
template <typename I>
__global__ void spmv_plan_kernel(const I *__restrict__ pos, int64_t nrows, int64_t nblk,
                                 int64_t *__restrict__ plan, int tile = SPMV_TILE) {
  int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b > nblk) return;
  if (b == nblk) {
    plan[b] = nrows;
    return;
  }
  if (b == 0) {
    plan[0] = 0;
    return;
  }
  const int64_t c0 = ((int64_t)pos[0] & ~(int64_t)3) + b * (int64_t)tile;
  int64_t lo = 0, hi = nrows;
  while (lo < hi) {
    int64_t mid = lo + ((hi - lo) >> 1);
    if ((int64_t)pos[mid + 1] > c0)
      hi = mid;
    else
      lo = mid + 1;
  }
  plan[b] = lo;
}

template <typename I>
struct IndexPair;
template <>
struct IndexPair<int32_t> {
  using type = int2;
};
template <>
struct IndexPair<int64_t> {
  using type = longlong2;
};

__device__ __forceinline__ double block_sum(double v, double *s_red) {
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

// x is re-read by every block: ask L2 to keep it (evict_last) while the streamed
// val/crd entries, read once, are marked evict_first by ld.global.cs.
__device__ __forceinline__ double load_x(const double *p, uint64_t policy, bool hint) {
  if (!hint) return __ldg(p);
  double v;
  asm volatile("ld.global.nc.L2::cache_hint.f64 %0, [%1], %2;" : "=d"(v) : "l"(p), "l"(policy));
  return v;
}

struct ChunkCtx {
  int64_t row0;      // first row looked at by this block
  int nr;            // rows looked at (the last one may only leave a carry)
  int len;           // entries in the chunk
  int ncached;       // entries of s_rel that are valid
  bool has_tail;     // row row0 + nr - 1 runs past the chunk (or starts beyond it)
  int64_t c0;
};

// Chunk-relative start offset of local row i, clamped to [0, len].
template <typename I>
__device__ __forceinline__ int rel_at(const ChunkCtx &c, const int *s_rel, const I *__restrict__ pos, int i) {
  if (i < c.ncached) return s_rel[i];
  int64_t d = (int64_t)pos[c.row0 + i] - c.c0;
  d = d < 0 ? 0 : d;
  return (int)(d > c.len ? c.len : d);
}

// Stores one finished in-chunk row sum: y for rows ending here, carry for the tail row.
template <bool FUSE_DOT>
__device__ __forceinline__ void finish_row(const ChunkCtx &c, int i, int s, double acc, double yin, double dv,
                                           double *__restrict__ y, double *__restrict__ carry,
                                           double &dot_local, int chunk) {
  const int64_t r = c.row0 + i;
  if (c.has_tail && i == c.nr - 1) {
    if (s >= c.len) return;  // the row starts beyond this chunk: not ours
    carry[chunk] = acc;
  } else {
    y[r] = __dadd_rn(acc, yin);
  }
  if (FUSE_DOT) dot_local = __dadd_rn(dot_local, __dmul_rn(acc, dv));
}

template <typename I, int THREADS, int L, bool FUSE_DOT>
__device__ __forceinline__ void reduce_short_rows(const ChunkCtx &c, const int *s_rel, const I *__restrict__ pos,
                                                  const double *s_prod, int *s_long, int *s_nlong,
                                                  double *__restrict__ y, int accumulate, double *__restrict__ carry,
                                                  const double *__restrict__ dotvec, double &dot_local, int chunk) {
  const int tid = threadIdx.x;
  const int grp = tid / L, lane = tid % L;
  constexpr int NGRP = THREADS / L;
  for (int ib = 0; ib < c.nr; ib += NGRP) {
    const int i = ib + grp;
    const bool valid = i < c.nr;
    double acc = 0.0, yin = 0.0, dv = 0.0;
    int s = 0, e = 0;
    bool is_long = false;
    if (valid) {
      s = rel_at<I>(c, s_rel, pos, i);
      e = rel_at<I>(c, s_rel, pos, i + 1);
      is_long = (e - s) > SPMV_LONG_ROW;
      if (accumulate && lane == 0 && !is_long && !(c.has_tail && i == c.nr - 1)) yin = y[c.row0 + i];
      if (FUSE_DOT && lane == 0 && !is_long) dv = dotvec[c.row0 + i];  // in flight while the row is summed
      if (!is_long)
        for (int j = s + lane; j < e; j += L) acc = __dadd_rn(acc, s_prod[j]);
    }
#pragma unroll
    for (int off = L / 2; off > 0; off >>= 1) acc = __dadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if (valid && lane == 0) {
      if (is_long)
        s_long[atomicAdd(s_nlong, 1)] = i;  // order of the list does not matter: rows are independent
      else
        finish_row<FUSE_DOT>(c, i, s, acc, yin, dv, y, carry, dot_local, chunk);
    }
  }
}

// y = (accumulate ? y : 0) + A x for the rows ending in chunk blockIdx.x; carry[b] for the row
// running past it.  With FUSE_DOT, blk_partial[b] = sum over this chunk of (row partial) * dotvec[row].
template <typename I, int THREADS, int MINB, bool FUSE_DOT, bool HINT>
__global__ void __launch_bounds__(THREADS, MINB)
spmv_chunk_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                  const int64_t *__restrict__ plan, int64_t abase, int64_t nnz_end, int64_t nrows,
                  const double *__restrict__ x, double *__restrict__ y, int accumulate,
                  double *__restrict__ carry, const double *__restrict__ dotvec,
                  double *__restrict__ blk_partial, const int *__restrict__ skip_flag) {
  constexpr int T = SPMV_TILE;
  constexpr int PAIRS = T / (2 * THREADS);
  __shared__ __align__(16) double s_prod[T];
  __shared__ int s_rel[SPMV_POS_CACHE + 2];
  __shared__ int s_long[T / SPMV_LONG_ROW];
  __shared__ int s_nlong;
  __shared__ double s_red[THREADS / 32];
  using Pair = typename IndexPair<I>::type;

  asm volatile("griddepcontrol.launch_dependents;");  // the fix-up kernel may start launching; it waits for our completion
  if (skip_flag != nullptr && *skip_flag != 0) return;

  const int tid = threadIdx.x;
  ChunkCtx c;
  c.c0 = abase + (int64_t)blockIdx.x * T;
  const int64_t left = nnz_end - c.c0;
  c.len = (int)(left < T ? (left < 0 ? 0 : left) : T);
  c.row0 = plan[blockIdx.x];
  const int64_t rn = plan[blockIdx.x + 1];
  c.has_tail = rn < nrows;
  const int64_t nr64 = rn - c.row0 + (c.has_tail ? 1 : 0);
  c.nr = (int)(nr64 > 0x7fffffff ? 0x7fffffff : nr64);
  c.ncached = (int)(nr64 + 1 < SPMV_POS_CACHE + 2 ? nr64 + 1 : SPMV_POS_CACHE + 2);

  uint64_t policy = 0;
  if (HINT) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));

  // ---- stream phase: aligned 16-byte loads, gather x, stage products ------------------
  const double *vb = val + c.c0;
  const I *cb = crd + c.c0;
  double2 v[PAIRS];
  Pair ci[PAIRS];
#pragma unroll
  for (int k = 0; k < PAIRS; ++k) {
    const int j = 2 * (tid + k * THREADS);
    v[k] = make_double2(0.0, 0.0);
    ci[k].x = 0;
    ci[k].y = 0;
    if (j + 1 < c.len) {
      v[k] = __ldcs(reinterpret_cast<const double2 *>(vb + j));
      ci[k] = __ldcs(reinterpret_cast<const Pair *>(cb + j));
    } else if (j < c.len) {  // odd tail of the last chunk
      v[k].x = __ldcs(vb + j);
      ci[k].x = __ldcs(cb + j);
    }
  }
  // row offsets of this block, chunk-relative and clamped, while the loads are in flight
  for (int i = tid; i < c.ncached; i += THREADS) {
    int64_t d = (int64_t)pos[c.row0 + i] - c.c0;
    d = d < 0 ? 0 : d;
    s_rel[i] = (int)(d > c.len ? c.len : d);
  }
  if (tid == 0) s_nlong = 0;
#pragma unroll
  for (int k = 0; k < PAIRS; ++k) {
    const int j = 2 * (tid + k * THREADS);
    if (j < c.len) {
      double2 p;
      p.x = __dmul_rn(v[k].x, load_x(x + ci[k].x, policy, HINT));
      p.y = (j + 1 < c.len) ? __dmul_rn(v[k].y, load_x(x + ci[k].y, policy, HINT)) : 0.0;
      *reinterpret_cast<double2 *>(s_prod + j) = p;
    }
  }
  __syncthreads();

  // ---- pass 1: rows of up to SPMV_LONG_ROW in-chunk entries, L lanes per row --------
  double dot_local = 0.0;
  reduce_short_rows<I, THREADS, 1, FUSE_DOT>(c, s_rel, pos, s_prod, s_long, &s_nlong, y, accumulate, carry, dotvec,
                                             dot_local, (int)blockIdx.x);
  __syncthreads();

  // ---- pass 2: long rows, one warp each -------------------------------------------------
  const int nlong = s_nlong;
  const int warp = tid >> 5, lane = tid & 31;
  for (int q = warp; q < nlong; q += THREADS / 32) {
    const int i = s_long[q];
    const int s = rel_at<I>(c, s_rel, pos, i), e = rel_at<I>(c, s_rel, pos, i + 1);
    double yin = 0.0, dv = 0.0;
    if (accumulate && lane == 0 && !(c.has_tail && i == c.nr - 1)) yin = y[c.row0 + i];
    if (FUSE_DOT && lane == 0) dv = dotvec[c.row0 + i];
    double acc = 0.0;
    for (int j = s + lane; j < e; j += 32) acc = __dadd_rn(acc, s_prod[j]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc = __dadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if (lane == 0) finish_row<FUSE_DOT>(c, i, s, acc, yin, dv, y, carry, dot_local, (int)blockIdx.x);
  }

  if (FUSE_DOT) {
    const double t = block_sum(dot_local, s_red);
    if (tid == 0) blk_partial[blockIdx.x] = t;
  }
}

// ---------------------------------------------------------------------------
// Segmented-scan variant of the chunk kernel.  The chunk kernel's row sums read the
// staged products with one lane per row; lanes of a warp walk different rows and collide
// on banks, and that traffic is a third of the kernel's L1 wavefronts.  Here the products
// never leave the registers before they are summed: row starts are marked in a bit mask
// (one shared atomic per row), every warp runs a segmented inclusive scan over each
// 64-entry group it holds (a pair per lane, five shuffle steps), and only the scanned
// values are stored -- one conflict-free 16-byte store per pair.  A row then costs one
// thread one read: the scanned value at its last entry, plus the closing values ("tails")
// of the earlier groups it spans.  With 512 threads a thread holds four entries and the
// kernel fits 32 registers, so four blocks fill an SM.
// Measured on a matrix with uniformly random columns (2^23 rows, 1.3e8 entries): 0.80 ms
// with 256 threads x 5 blocks or 512 x 4 against 0.83-0.86 ms for the chunk kernel -- a few
// per cent, so the row sums were not the limiter there; residency is what moved the time.
//
// Same plan, carry array and fix-up kernel as the chunk kernel.  A row is summed in scan
// order, not entry order: results are identical from run to run and within 1e-12 of the
// row's magnitude of the sequential sum, but not bit-identical to the other variants
// (rows of a single entry and empty rows are).
// ---------------------------------------------------------------------------
template <typename I, int THREADS, int MINB, bool FUSE_DOT, bool HINT>
__global__ void __launch_bounds__(THREADS, MINB)
spmv_scan_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                 const int64_t *__restrict__ plan, int64_t abase, int64_t nnz_end, int64_t nrows,
                 const double *__restrict__ x, double *__restrict__ y, int accumulate,
                 double *__restrict__ carry, const double *__restrict__ dotvec,
                 double *__restrict__ blk_partial, const int *__restrict__ skip_flag) {
  constexpr int T = SPMV_TILE;
  constexpr int PAIRS = T / (2 * THREADS);  // 256 threads: eight entries per thread; 512: four
  constexpr int NGROUPS = T / 64;  // group g = entries [64 g, 64 g + 64): the pairs one warp holds for one k
  static_assert(T % (2 * THREADS) == 0, "a chunk is a whole number of pairs per thread");
  __shared__ __align__(16) double s_scan[T];
  __shared__ int s_rel[SPMV_POS_CACHE + 2];
  __shared__ unsigned s_head[T / 32];
  __shared__ double s_tail[NGROUPS];
  __shared__ double s_red[THREADS / 32];
  using Pair = typename IndexPair<I>::type;

  asm volatile("griddepcontrol.launch_dependents;");
  if (skip_flag != nullptr && *skip_flag != 0) return;

  const int tid = threadIdx.x, lane = tid & 31;
  const int chunk = (int)blockIdx.x;
  ChunkCtx c;
  c.c0 = abase + (int64_t)blockIdx.x * T;
  const int64_t left = nnz_end - c.c0;
  c.len = (int)(left < T ? (left < 0 ? 0 : left) : T);
  c.row0 = plan[blockIdx.x];
  const int64_t rn = plan[blockIdx.x + 1];
  c.has_tail = rn < nrows;
  const int64_t nr64 = rn - c.row0 + (c.has_tail ? 1 : 0);
  c.nr = (int)(nr64 > 0x7fffffff ? 0x7fffffff : nr64);
  c.ncached = (int)(nr64 + 1 < SPMV_POS_CACHE + 2 ? nr64 + 1 : SPMV_POS_CACHE + 2);

  uint64_t policy = 0;
  if (HINT) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));

  // ---- stream phase: the chunk's (val, crd) pairs into registers ---------------------------
  const double *vb = val + c.c0;
  const I *cb = crd + c.c0;
  double2 v[PAIRS];
  Pair ci[PAIRS];
#pragma unroll
  for (int k = 0; k < PAIRS; ++k) {
    const int j = 2 * (tid + k * THREADS);
    v[k] = make_double2(0.0, 0.0);
    ci[k].x = 0;
    ci[k].y = 0;
    if (j + 1 < c.len) {
      v[k] = __ldcs(reinterpret_cast<const double2 *>(vb + j));
      ci[k] = __ldcs(reinterpret_cast<const Pair *>(cb + j));
    } else if (j < c.len) {  // odd tail of the last chunk
      v[k].x = __ldcs(vb + j);
      ci[k].x = __ldcs(cb + j);
    }
  }
  if (tid < T / 32) s_head[tid] = 0u;
  __syncthreads();
  // row offsets (chunk-relative, clamped) and the row-start marks, while the loads are in flight
  for (int i = tid; i < c.nr || i < c.ncached; i += THREADS) {
    int64_t d = (int64_t)pos[c.row0 + i] - c.c0;
    d = d < 0 ? 0 : d;
    const int rel = (int)(d > c.len ? c.len : d);
    if (i < c.ncached) s_rel[i] = rel;
    if (i < c.nr && rel < c.len) atomicOr(&s_head[rel >> 5], 1u << (rel & 31));
  }
  // gathers: entries past the chunk's end have val = 0 and crd = 0 (x[0] is a valid address when ncols > 0;
  // the product is computed only for entries inside the chunk)
  double2 xv[PAIRS];
#pragma unroll
  for (int k = 0; k < PAIRS; ++k) {
    const int j = 2 * (tid + k * THREADS);
    xv[k].x = (j < c.len) ? load_x(x + ci[k].x, policy, HINT) : 0.0;
    xv[k].y = (j + 1 < c.len) ? load_x(x + ci[k].y, policy, HINT) : 0.0;
  }
  __syncthreads();  // the marks are complete

  // ---- segmented inclusive scan of every 64-entry group, in registers ------------------------
#pragma unroll
  for (int k = 0; k < PAIRS; ++k) {
    const int j = 2 * (tid + k * THREADS);
    const double a = __dmul_rn(v[k].x, xv[k].x), b = __dmul_rn(v[k].y, xv[k].y);
    const unsigned hw = s_head[j >> 5] >> (j & 31);
    const bool h0 = hw & 1u, h1 = hw & 2u;
    // t: the sum of the still open row piece at the end of this pair
    double t = h1 ? b : __dadd_rn(a, b);
    const unsigned heads = __ballot_sync(0xffffffffu, h0 || h1);
    const unsigned below = heads & (0xffffffffu >> (31 - lane));
    const int first = below ? 31 - __clz(below) : 0;  // nearest lane at or below this one whose pair holds a row start
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const double u = __shfl_up_sync(0xffffffffu, t, off);
      if (lane - off >= first) t = __dadd_rn(t, u);
    }
    double before = __shfl_up_sync(0xffffffffu, t, 1);  // open piece at the end of the previous lane's pair
    if (lane == 0) before = 0.0;
    double2 s;
    s.x = h0 ? a : __dadd_rn(before, a);
    s.y = h1 ? b : __dadd_rn(s.x, b);
    *reinterpret_cast<double2 *>(s_scan + j) = s;
    if (lane == 31) s_tail[j >> 6] = s.y;
  }
  __syncthreads();

  // ---- one thread per row: value at the row's last entry + tails of the earlier groups it spans ----
  double dot_local = 0.0;
  for (int i = tid; i < c.nr; i += THREADS) {
    const int s = rel_at<I>(c, s_rel, pos, i), e = rel_at<I>(c, s_rel, pos, i + 1);
    const bool is_tail = c.has_tail && i == c.nr - 1;
    double yin = 0.0, dv = 0.0;
    if (accumulate && !is_tail) yin = y[c.row0 + i];
    if (FUSE_DOT) dv = dotvec[c.row0 + i];
    double acc = 0.0;
    if (e > s) {
      const int g = (e - 1) >> 6;
      for (int q = s >> 6; q < g; ++q) acc = __dadd_rn(acc, s_tail[q]);
      acc = __dadd_rn(acc, s_scan[e - 1]);
    }
    finish_row<FUSE_DOT>(c, i, s, acc, yin, dv, y, carry, dot_local, chunk);
  }

  if (FUSE_DOT) {
    const double t = block_sum(dot_local, s_red);
    if (tid == 0) blk_partial[blockIdx.x] = t;
  }
}

// ---------------------------------------------------------------------------
// Persistent variant: each block walks chunks b, b + grid, ... and keeps the next
// chunk's val/crd in flight with bulk asynchronous copies (cp.async.bulk, completion
// on an mbarrier) into a second shared-memory stage while it gathers and reduces the
// current one, so the streamed entries bypass the load/store unit and registers.
// Products overwrite val in place.  Every barrier wait is bounded; a block that gives
// up records g_spmv_error and leaves the loop.
// ---------------------------------------------------------------------------
__device__ int g_spmv_error;
constexpr uint32_t SPMV_WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool spmv_mbar_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t addr = smem_addr(bar);
  for (uint32_t i = 0; i < SPMV_WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// Streamed once: the copy carries an evict-first L2 policy so that it does not push x out of L2.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_addr(dst)),
      "l"(src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}

template <typename I, int THREADS, bool FUSE_DOT, bool HINT>
__global__ void __launch_bounds__(THREADS)
spmv_pipe_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                 const int64_t *__restrict__ plan, int64_t abase, int64_t nnz_end, int64_t nrows, int64_t nblk,
                 const double *__restrict__ x, double *__restrict__ y, int accumulate, double *__restrict__ carry,
                 const double *__restrict__ dotvec, double *__restrict__ blk_partial,
                 const int *__restrict__ skip_flag) {
  constexpr int T = SPMV_TILE;
  constexpr int PER = T / THREADS;
  extern __shared__ __align__(128) uint8_t pipe_smem[];
  double *s_val0 = reinterpret_cast<double *>(pipe_smem);      // two stages of T values
  I *s_crd0 = reinterpret_cast<I *>(pipe_smem + 2 * T * 8);    // two stages of T column indices
  uint8_t *tail = pipe_smem + 2 * T * 8 + 2 * T * sizeof(I);
  int *s_rel = reinterpret_cast<int *>(tail);
  int *s_long = s_rel + SPMV_POS_CACHE + 2;
  int *s_nlong = s_long + T / SPMV_LONG_ROW;
  double *s_red = reinterpret_cast<double *>(s_nlong + 2);
  uint64_t *full = reinterpret_cast<uint64_t *>(s_red + THREADS / 32);

  asm volatile("griddepcontrol.launch_dependents;");
  if (skip_flag != nullptr && *skip_flag != 0) return;
  const int tid = threadIdx.x;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&full[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&full[1])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  uint64_t policy = 0, stream_policy = 0;
  if (HINT) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(stream_policy));

  // entries of chunk b moved by the bulk copies: whole groups of 4 (16-byte multiples for both arrays)
  auto chunk_len = [&](int64_t b) {
    const int64_t left = nnz_end - (abase + b * T);
    return (int)(left < T ? (left < 0 ? 0 : left) : T);
  };
  auto issue = [&](int64_t b, int s) {
    const int len4 = chunk_len(b) & ~3;
    if (len4 > 0) {
      const int64_t c0 = abase + b * T;
      const uint32_t bytes = (uint32_t)len4 * (8u + (uint32_t)sizeof(I));
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&full[s])), "r"(bytes)
                   : "memory");
      bulk_load(s_val0 + s * T, val + c0, (uint32_t)len4 * 8u, &full[s], stream_policy);
      bulk_load(s_crd0 + s * T, crd + c0, (uint32_t)len4 * (uint32_t)sizeof(I), &full[s], stream_policy);
    } else {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&full[s])) : "memory");
    }
  };

  double dot_local = 0.0;
  int it = 0;
  if (tid == 0 && (int64_t)blockIdx.x < nblk) issue(blockIdx.x, 0);
  for (int64_t b = blockIdx.x; b < nblk; b += gridDim.x, ++it) {
    const int s = it & 1;
    const int64_t bn = b + gridDim.x;
    if (tid == 0 && bn < nblk) issue(bn, s ^ 1);  // stage s^1 was released by the barrier ending the last pass

    ChunkCtx c;
    c.c0 = abase + b * T;
    c.len = chunk_len(b);
    c.row0 = plan[b];
    const int64_t rn = plan[b + 1];
    c.has_tail = rn < nrows;
    const int64_t nr64 = rn - c.row0 + (c.has_tail ? 1 : 0);
    c.nr = (int)(nr64 > 0x7fffffff ? 0x7fffffff : nr64);
    c.ncached = (int)(nr64 + 1 < SPMV_POS_CACHE + 2 ? nr64 + 1 : SPMV_POS_CACHE + 2);
    for (int i = tid; i < c.ncached; i += THREADS) {
      int64_t d = (int64_t)pos[c.row0 + i] - c.c0;
      d = d < 0 ? 0 : d;
      s_rel[i] = (int)(d > c.len ? c.len : d);
    }
    if (tid == 0) *s_nlong = 0;

    const bool landed = spmv_mbar_wait(&full[s], (uint32_t)(it >> 1) & 1u);
    if (!__syncthreads_and(landed ? 1 : 0)) {  // also orders s_rel / s_nlong before their readers
      if (tid == 0) atomicExch(&g_spmv_error, 1);
      break;
    }

    // ---- gather x and turn val into products, in place ----------------------------------
    const int len4 = c.len & ~3;
    double *prod = s_val0 + s * T;
    const I *cs = s_crd0 + s * T;
    I ci[PER];
    double xv[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int j = tid + k * THREADS;
      ci[k] = 0;
      if (j < len4)
        ci[k] = cs[j];
      else if (j < c.len)
        ci[k] = crd[c.c0 + j];  // up to three entries at the very end of the arrays
    }
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int j = tid + k * THREADS;
      xv[k] = (j < c.len) ? load_x(x + ci[k], policy, HINT) : 0.0;
    }
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int j = tid + k * THREADS;
      if (j < len4)
        prod[j] = __dmul_rn(prod[j], xv[k]);
      else if (j < c.len)
        prod[j] = __dmul_rn(val[c.c0 + j], xv[k]);
    }
    __syncthreads();

    // ---- rows ending in this chunk (same two passes as the one-chunk-per-block kernel) ------
    reduce_short_rows<I, THREADS, 1, FUSE_DOT>(c, s_rel, pos, prod, s_long, s_nlong, y, accumulate, carry, dotvec,
                                               dot_local, (int)b);
    __syncthreads();
    const int nlong = *s_nlong;
    const int warp = tid >> 5, lane = tid & 31;
    for (int q = warp; q < nlong; q += THREADS / 32) {
      const int i = s_long[q];
      const int s0 = rel_at<I>(c, s_rel, pos, i), e0 = rel_at<I>(c, s_rel, pos, i + 1);
      double yin = 0.0, dv = 0.0;
      if (accumulate && lane == 0 && !(c.has_tail && i == c.nr - 1)) yin = y[c.row0 + i];
      if (FUSE_DOT && lane == 0) dv = dotvec[c.row0 + i];
      double acc = 0.0;
      for (int j = s0 + lane; j < e0; j += 32) acc = __dadd_rn(acc, prod[j]);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc = __dadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
      if (lane == 0) finish_row<FUSE_DOT>(c, i, s0, acc, yin, dv, y, carry, dot_local, (int)b);
    }
    // the next bulk copy into this stage must not overtake these shared-memory accesses
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
  }

  if (FUSE_DOT) {
    // one partial per block; the blocks past the grid size contribute nothing
    const double t = block_sum(dot_local, s_red);
    if (tid == 0) blk_partial[blockIdx.x] = t;
    for (int64_t e = gridDim.x + (int64_t)blockIdx.x * THREADS + tid; e < nblk; e += (int64_t)gridDim.x * THREADS)
      blk_partial[e] = 0.0;
  }
}

// ---------------------------------------------------------------------------
// Warp-walk variant: no shared memory, no block barrier.
//
// What bounds an SpMV whose columns are spread over a vector much larger than L1 is the load/store path of
// the SM, not HBM: every gathered x element is its own request from L1 to the crossbar (one per cycle per SM),
// and the number of such misses in flight is proportional to the L1 capacity, which every kilobyte of shared
// memory takes away.  A store-free dot product over the same arrays (the floor) runs 1.4x slower with 64 KB of
// shared memory per SM carved out and 4.5x slower with 192 KB.  So this kernel keeps everything in registers:
//
//   * One warp owns one chunk of the plan (2048 stored entries) and walks it in steps of 128 entries; a lane
//     holds four consecutive entries, fetched with one 32-byte load per array (marked evict-first in L1 and
//     L2), and the next step's entries are requested before the current step's gathers are consumed.
//   * The row ends inside a step come from pos: lane i looks at row r_cur + i, a ballot counts the rows that
//     end in the step, and four warp OR-reductions build the 128-bit mask of row-start offsets.
//   * Products are summed by a segmented scan: sequentially inside a lane, five shuffle levels across lanes.
//     The running sum of the row that is still open leaves the step on the scan's last shuffle (a rotation)
//     and enters the next step in lane 0's first product.
//   * A row is stored by the lane that holds its last entry; its row number is r_cur plus the number of row
//     ends before that entry (popcounts of the mask).  Steps that contain empty rows cannot rank rows that
//     way and fetch each row's sum with indexed shuffles instead.
//   * The piece of a row that runs past the chunk goes to carry[chunk]; spmv_fixup_kernel adds the carries.
//
// Rows are summed in scan order: run-to-run identical, within 1e-12 of the row's magnitude of the sequential
// sum, not the bits of the chunk kernels (relaxed tuner only).  val and crd must be 32-byte aligned.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void load_stream_256(const void *p, uint64_t &a, uint64_t &b, uint64_t &c, uint64_t &d) {
  asm volatile("ld.global.nc.L1::evict_first.L2::evict_first.v4.b64 {%0,%1,%2,%3}, [%4];"
               : "=l"(a), "=l"(b), "=l"(c), "=l"(d)
               : "l"(p));
}
__device__ __forceinline__ void load_entries4(const int64_t *crd, const double *val, int64_t j, int64_t c[4], double a[4]) {
  uint64_t q0, q1, q2, q3, v0, v1, v2, v3;
  load_stream_256(crd + j, q0, q1, q2, q3);
  load_stream_256(val + j, v0, v1, v2, v3);
  c[0] = (int64_t)q0; c[1] = (int64_t)q1; c[2] = (int64_t)q2; c[3] = (int64_t)q3;
  a[0] = __longlong_as_double((long long)v0); a[1] = __longlong_as_double((long long)v1);
  a[2] = __longlong_as_double((long long)v2); a[3] = __longlong_as_double((long long)v3);
}
__device__ __forceinline__ void load_entries4(const int32_t *crd, const double *val, int64_t j, int64_t c[4], double a[4]) {
  uint64_t v0, v1, v2, v3;
  const int4 q = __ldcs(reinterpret_cast<const int4 *>(crd + j));
  load_stream_256(val + j, v0, v1, v2, v3);
  c[0] = q.x; c[1] = q.y; c[2] = q.z; c[3] = q.w;
  a[0] = __longlong_as_double((long long)v0); a[1] = __longlong_as_double((long long)v1);
  a[2] = __longlong_as_double((long long)v2); a[3] = __longlong_as_double((long long)v3);
}
__device__ __forceinline__ double load_x_ordered(const double *p) {  // volatile: stays behind the loads issued before it
  double v;
  asm volatile("ld.global.nc.f64 %0, [%1];" : "=d"(v) : "l"(p));
  return v;
}

constexpr int SPMV_WALK_THREADS = 128;
constexpr int SPMV_WALK_FINE_TILE = 512;  // entries per warp on matrices too small to fill the SMs with 2048-entry ranges
constexpr int SPMV_WALK_STEP = 128;  // entries per step: four per lane

template <typename I, bool FUSE_DOT>
__global__ void __launch_bounds__(SPMV_WALK_THREADS, FUSE_DOT ? 6 : 8)
spmv_walk_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                 const int64_t *__restrict__ plan, int64_t abase, int64_t base, int64_t nnz_end, int64_t nrows,
                 int64_t nblk, int tile, const double *__restrict__ x, double *__restrict__ y, int accumulate,
                 double *__restrict__ carry, const double *__restrict__ dotvec, double *__restrict__ blk_partial,
                 const int *__restrict__ skip_flag) {
  constexpr unsigned FULL = 0xffffffffu;
  constexpr int S = SPMV_WALK_STEP;
  asm volatile("griddepcontrol.launch_dependents;");
  if (skip_flag != nullptr && *skip_flag != 0) return;
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (SPMV_WALK_THREADS / 32) + (threadIdx.x >> 5);
  if (w >= nblk) return;
  const int64_t c_begin = abase + w * tile;  // tile: entries per warp, the granularity of the plan this launch uses
  const int64_t c_end = (c_begin + tile < nnz_end) ? c_begin + tile : nnz_end;
  int64_t r_cur = plan[w];
  double open = 0.0;  // sum so far of the row that is still open; meaningful in lane 0
  double dot_local = 0.0;
  const int wsel = lane >> 3, shift = 4 * (lane & 7);

  auto fetch = [&](int64_t c, int64_t cc[4], double aa[4]) {
    const int64_t j0 = c + 4 * lane;
    if (j0 + 4 <= c_end) {
      load_entries4(crd, val, j0, cc, aa);
    } else {  // ragged end of the arrays
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        cc[k] = 0;
        aa[k] = 0.0;
        if (j0 + k < c_end) {
          cc[k] = (int64_t)crd[j0 + k];
          aa[k] = val[j0 + k];
        }
      }
    }
  };
  // row-end offset of row r relative to c, S + 1 for "beyond this step"
  auto end_offset = [&](int64_t r, int64_t c) {
    int e = S + 1;
    if (r < nrows) {
      const int64_t d = (int64_t)pos[r + 1] - c;
      e = d > S ? S + 1 : (d < 0 ? 0 : (int)d);
    }
    return e;
  };

  if (c_begin >= c_end) {  // a matrix without stored entries (one chunk, one warp): every row is empty
    if (!accumulate)
      for (int64_t r = lane; r < nrows; r += 32) y[r] = 0.0;
    if (lane == 0) {
      carry[w] = 0.0;
      if (FUSE_DOT) blk_partial[w] = 0.0;
    }
    return;
  }
  int64_t cn[4];
  double an[4];
  fetch(c_begin, cn, an);

  for (int64_t c = c_begin; c < c_end; c += S) {
    int64_t ci[4];
    double a[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      ci[k] = cn[k];
      a[k] = an[k];
    }
    const int e = end_offset(r_cur + lane, c);
    double xv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) xv[k] = load_x_ordered(x + ci[k]);
    if (c + S < c_end) fetch(c + S, cn, an);

    // ---- rows that end in this step; bit e of the mask for every end offset e < S ------------------
    int nfin = __popc(__ballot_sync(FULL, e <= S));
    unsigned any_full = __ballot_sync(FULL, e == S);
    unsigned hm0, hm1, hm2, hm3;
    {
      const unsigned bit = (e < S) ? (1u << (e & 31)) : 0u;
      const int q = e >> 5;
      hm0 = __reduce_or_sync(FULL, q == 0 ? bit : 0u);
      hm1 = __reduce_or_sync(FULL, q == 1 ? bit : 0u);
      hm2 = __reduce_or_sync(FULL, q == 2 ? bit : 0u);
      hm3 = __reduce_or_sync(FULL, q == 3 ? bit : 0u);
    }
    int total_fin = nfin;
    for (int64_t rbase = r_cur + 32; nfin == 32; rbase += 32) {  // more than 32 rows may end in one step
      const int e2 = end_offset(rbase + lane, c);
      nfin = __popc(__ballot_sync(FULL, e2 <= S));
      any_full |= __ballot_sync(FULL, e2 == S);
      total_fin += nfin;
      const unsigned bit = (e2 < S) ? (1u << (e2 & 31)) : 0u;
      const int q = e2 >> 5;
      hm0 |= __reduce_or_sync(FULL, q == 0 ? bit : 0u);
      hm1 |= __reduce_or_sync(FULL, q == 1 ? bit : 0u);
      hm2 |= __reduce_or_sync(FULL, q == 2 ? bit : 0u);
      hm3 |= __reduce_or_sync(FULL, q == 3 ? bit : 0u);
    }
    const unsigned hcur = wsel == 0 ? hm0 : (wsel == 1 ? hm1 : (wsel == 2 ? hm2 : hm3));
    const unsigned hnext = wsel == 0 ? hm1 : (wsel == 1 ? hm2 : (wsel == 2 ? hm3 : (any_full ? 1u : 0u)));
    const unsigned h5 = __funnelshift_r(hcur, hnext, shift) & 0x1fu;  // mask bits 4*lane .. 4*lane + 4
    const unsigned h = h5 & 0xfu;                                     // a row starts at this lane's entry k
    const int p0 = __popc(hm0), p1 = p0 + __popc(hm1), p2 = p1 + __popc(hm2);
    const int distinct = p2 + __popc(hm3) + (any_full ? 1 : 0);
    // every finished row has its own end offset and none ends at offset 0: no empty rows among them
    const bool simple = (distinct == total_fin) && !(hm0 & 1u);
    // rows that end at or before this lane's first entry
    const int below = (wsel == 0 ? 0 : (wsel == 1 ? p0 : (wsel == 2 ? p1 : p2))) + __popc(hcur & ((2u << shift) - 1u));

    double yin[4] = {0.0, 0.0, 0.0, 0.0}, dv[4] = {0.0, 0.0, 0.0, 0.0};
    if (simple) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (h5 & (2u << k)) {
          const int64_t row = r_cur + below + __popc(h & (((2u << k) - 1u) & ~1u));
          if (accumulate) yin[k] = y[row];
          if (FUSE_DOT) dv[k] = dotvec[row];
        }
    }

    // ---- segmented scan ----------------------------------------------------------------------------
    double p[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = __dmul_rn(a[k], xv[k]);
    if (c < base || c + S > c_end) {
      // the chunks start on a multiple of four entries, up to three in front of pos[0]; the last step may reach
      // past the arrays' end: neither kind of slot belongs to a row
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t j = c + 4 * lane + k;
        if (j < base || j >= c_end) p[k] = 0.0;
      }
    }
    if (lane == 0 && !(h & 1u)) p[0] = __dadd_rn(open, p[0]);
    double t = p[0];
    t = (h & 2u) ? p[1] : __dadd_rn(t, p[1]);
    t = (h & 4u) ? p[2] : __dadd_rn(t, p[2]);
    t = (h & 8u) ? p[3] : __dadd_rn(t, p[3]);
    const unsigned heads = __ballot_sync(FULL, h != 0u);
    const unsigned at_or_below = heads & (0xffffffffu >> (31 - lane));
    const int first = at_or_below ? 31 - __clz(at_or_below) : 0;  // nearest lane at or below this one with a row start
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const double u = __shfl_up_sync(FULL, t, off);
      if (lane - off >= first) t = __dadd_rn(t, u);
    }
    // lane l receives the open piece at the end of lane l - 1; lane 0 receives lane 31's: the step's open piece
    const double rot = __shfl_sync(FULL, t, (lane + 31) & 31);
    const double before = lane == 0 ? 0.0 : rot;
    double s[4];
    s[0] = (h & 1u) ? p[0] : __dadd_rn(before, p[0]);
    s[1] = (h & 2u) ? p[1] : __dadd_rn(s[0], p[1]);
    s[2] = (h & 4u) ? p[2] : __dadd_rn(s[1], p[2]);
    s[3] = (h & 8u) ? p[3] : __dadd_rn(s[2], p[3]);
    open = any_full ? 0.0 : rot;  // a row that ends with the step leaves nothing open

    if (simple) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (h5 & (2u << k)) {  // entry k is the last entry of its row
          const int64_t row = r_cur + below + __popc(h & (((2u << k) - 1u) & ~1u));
          y[row] = __dadd_rn(s[k], yin[k]);
          if (FUSE_DOT) dot_local = __dadd_rn(dot_local, __dmul_rn(s[k], dv[k]));
        }
    } else {
      int prev_e = 0;
      int64_t rbase = r_cur;
      for (int done = 0; done < total_fin; done += 32, rbase += 32) {
        const int re = done == 0 ? e : end_offset(rbase + lane, c);
        int st = __shfl_up_sync(FULL, re, 1);  // where this lane's row starts = where the previous row ends
        if (lane == 0) st = prev_e;
        const bool finished = re <= S;
        const int idx = finished && re > 0 ? re - 1 : 0;
        const int src = idx >> 2, kk = idx & 3;
        const double v0 = __shfl_sync(FULL, s[0], src), v1 = __shfl_sync(FULL, s[1], src);
        const double v2 = __shfl_sync(FULL, s[2], src), v3 = __shfl_sync(FULL, s[3], src);
        if (finished) {
          double sum = kk == 0 ? v0 : (kk == 1 ? v1 : (kk == 2 ? v2 : v3));
          if (re <= st) sum = 0.0;  // an empty row
          const int64_t row = rbase + lane;
          const double yi = accumulate ? y[row] : 0.0;
          y[row] = __dadd_rn(sum, yi);
          if (FUSE_DOT) dot_local = __dadd_rn(dot_local, __dmul_rn(sum, dotvec[row]));
        }
        prev_e = __shfl_sync(FULL, re, 31);
      }
    }
    r_cur += total_fin;
  }
  if (lane == 0) {
    const bool has_tail = r_cur < nrows && c_end < nnz_end;  // row r_cur runs past this chunk (or starts at its end: open == 0)
    carry[w] = has_tail ? open : 0.0;
    if (FUSE_DOT && has_tail) dot_local = __dadd_rn(dot_local, __dmul_rn(open, dotvec[r_cur]));
  }
  if (FUSE_DOT) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot_local = __dadd_rn(dot_local, __shfl_xor_sync(FULL, dot_local, off));
    if (lane == 0) blk_partial[w] = dot_local;
  }
}

template <typename I>
constexpr int spmv_pipe_smem_bytes(int threads) {
  return 2 * SPMV_TILE * 8 + 2 * SPMV_TILE * (int)sizeof(I) + (SPMV_POS_CACHE + 2) * 4 + (SPMV_TILE / SPMV_LONG_ROW) * 4 +
         8 + (threads / 32) * 8 + 16 + 64;
}

// Adds the carries to their rows.  Chunk b left a carry iff row q = plan[b+1] exists and starts
// before the chunk's end; consecutive chunks carrying into the same row form a run that the
// thread of its first chunk adds up in chunk order.
template <typename I>
__global__ void spmv_fixup_kernel(const I *__restrict__ pos, const int64_t *__restrict__ plan, int64_t abase,
                                  int64_t nblk, int64_t nrows, const double *__restrict__ carry,
                                  double *__restrict__ y, const int *__restrict__ skip_flag, int tile) {
  // Launched with programmatic stream serialization: the blocks may already be resident while the SpMV
  // kernel drains; nothing is read before that kernel has completed and its writes are visible.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (skip_flag != nullptr && *skip_flag != 0) return;
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblk - 1) return;
  const int64_t q = plan[b + 1];
  if (q >= nrows) return;
  const int64_t start = (int64_t)pos[q];
  const int64_t c0 = abase + b * (int64_t)tile;
  if (start >= c0 + tile) return;                   // row q starts in a later chunk: nothing carried
  if (b > 0 && plan[b] == q && start < c0) return;  // chunk b-1 carried into q too: not the head of the run
  double acc = carry[b];
  for (int64_t b2 = b + 1; b2 < nblk - 1 && plan[b2 + 1] == q; ++b2) acc = __dadd_rn(acc, carry[b2]);
  y[q] = __dadd_rn(y[q], acc);
}

// ---------------------------------------------------------------------------
// One thread per row, for matrices whose rows are all short (at most 32 entries; stencils, graphs of bounded
// degree).  A warp's 32 rows are adjacent in the arrays, so the lines it touches are used completely over the
// few iterations of the row loop and there is nothing to stage or to synchronise.  A row is summed in entry
// order; a row that crosses a chunk boundary of the plan is summed in the same two pieces, joined in the same
// order, as the chunk kernels plus the fix-up kernel do: y has the same bits whichever kernel ran.
// The grid has one block per chunk of the plan (blocks loop over 256-row tiles), so that blk_partial has the
// length its consumers expect.
// ---------------------------------------------------------------------------
template <typename I>
__device__ __forceinline__ double row_piece_sum(const I *__restrict__ crd, const double *__restrict__ val,
                                                const double *__restrict__ x, int64_t lo, int64_t hi) {
  double acc = 0.0;
  int64_t j = lo;
  for (; j + 3 < hi; j += 4) {
    double a[4], xv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      a[u] = __ldg(val + j + u);
      xv[u] = __ldg(x + (int64_t)__ldg(crd + j + u));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) acc = __dadd_rn(acc, __dmul_rn(a[u], xv[u]));
  }
  for (; j < hi; ++j) acc = __dadd_rn(acc, __dmul_rn(__ldg(val + j), __ldg(x + (int64_t)__ldg(crd + j))));
  return acc;
}

// PCG_FUSED: the kernel is pass A of a PCG iteration: its blocks first wait for the neighbours' halo pieces of x
// (row-partitioned solves), and the block that finishes last turns the per-block partial sums into p.Ap and
// derives alpha or hands the sum to the other ranks (pcg_fuse.h).
template <typename I, bool FUSE_DOT, bool PCG_FUSED>
__global__ void __launch_bounds__(256)
spmv_rowthread_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                      int64_t abase, int64_t nrows, int64_t ntiles, const double *__restrict__ x,
                      double *__restrict__ y, int accumulate, const double *__restrict__ dotvec,
                      double *__restrict__ blk_partial, const int *__restrict__ skip_flag, PcgExchange ex) {
  __shared__ double s_red[8];
  __shared__ int s_flag;
  if (skip_flag != nullptr && *skip_flag != 0) return;
  if (PCG_FUSED && ex.mbox != nullptr && !pcg_wait_halo(ex, &s_flag)) return;
  double dot_local = 0.0;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t row = tile * 256 + threadIdx.x;
    if (row >= nrows) continue;
    const int64_t lo = (int64_t)pos[row], hi = (int64_t)pos[row + 1];
    const double yin = accumulate ? y[row] : 0.0;
    double dv = 0.0;
    if (FUSE_DOT) dv = dotvec[row];
    const int64_t bnd = abase + ((lo - abase) / SPMV_TILE + 1) * (int64_t)SPMV_TILE;  // first chunk boundary after lo
    if (bnd >= hi) {
      const double s = row_piece_sum<I>(crd, val, x, lo, hi);
      y[row] = __dadd_rn(s, yin);
      if (FUSE_DOT) dot_local = __dadd_rn(dot_local, __dmul_rn(s, dv));
    } else {  // (piece in the later chunk + y_in) + carried piece; rows of at most 32 entries cross one boundary
      const double s_first = row_piece_sum<I>(crd, val, x, lo, bnd);
      double carried = s_first;
      int64_t b0 = bnd;
      while (b0 + SPMV_TILE < hi) {  // longer rows (not selected by the tuner): middle pieces, in chunk order
        carried = __dadd_rn(carried, row_piece_sum<I>(crd, val, x, b0, b0 + SPMV_TILE));
        b0 += SPMV_TILE;
      }
      const double s_last = row_piece_sum<I>(crd, val, x, b0, hi);
      y[row] = __dadd_rn(__dadd_rn(s_last, yin), carried);
      if (FUSE_DOT) dot_local = __dadd_rn(dot_local, __dmul_rn(__dadd_rn(carried, s_last), dv));
    }
  }
  if (FUSE_DOT) {
    const double t = block_sum(dot_local, s_red);
    if (threadIdx.x == 0) blk_partial[blockIdx.x] = t;
    if (PCG_FUSED && pcg_last_block(pcg_tickets(ex.sc) + 0, gridDim.x, &s_flag)) pcg_tail_pass_a(ex, blk_partial, gridDim.x, s_red);
  }
}

// ---------------------------------------------------------------------------
// Pass A of a PCG iteration with the direction update of the iteration before folded in (pcg_fuse.h, two-pass
// form): the operand of the SpMV at column c is z[c] + beta * p_old[c], which the kernel also stores for its own
// rows (and the halo entries of its window) as the new p.  Row sums are formed exactly as in
// spmv_rowthread_kernel, on operand values that have the bits pass C would have stored, so Ap, p and p.Ap are
// those of the three-pass form.
// ---------------------------------------------------------------------------
template <typename I, bool DIR>
__device__ __forceinline__ double row_piece_sum_pcg(const I *__restrict__ crd, const double *__restrict__ val,
                                                    const double *__restrict__ zw, const double *__restrict__ pw,
                                                    double beta, int64_t lo, int64_t hi) {
  auto operand = [&](int64_t c) {
    const double pv = __ldg(pw + c);
    if (!DIR) return pv;
    return __dadd_rn(__dmul_rn(__ldg(zw + c), 1.0), __dmul_rn(pv, beta));
  };
  double acc = 0.0;
  int64_t j = lo;
  for (; j + 3 < hi; j += 4) {
    double a[4], xv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      a[u] = __ldg(val + j + u);
      xv[u] = operand((int64_t)__ldg(crd + j + u));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) acc = __dadd_rn(acc, __dmul_rn(a[u], xv[u]));
  }
  for (; j < hi; ++j) acc = __dadd_rn(acc, __dmul_rn(__ldg(val + j), operand((int64_t)__ldg(crd + j))));
  return acc;
}

template <typename I, bool DIR>
__device__ __forceinline__ double pcg_spmv_rows(const I *__restrict__ pos, const I *__restrict__ crd,
                                                const double *__restrict__ val, int64_t abase, int64_t nrows,
                                                int64_t ntiles, int64_t p_off, const double *__restrict__ zw,
                                                const double *__restrict__ pold, double *__restrict__ pnew,
                                                double beta, double *__restrict__ Ap) {
  double dot_local = 0.0;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t row = tile * 256 + threadIdx.x;
    if (row >= nrows) continue;
    const int64_t lo = (int64_t)pos[row], hi = (int64_t)pos[row + 1];
    double dv = pold[p_off + row];
    if (DIR) {
      dv = __dadd_rn(__dmul_rn(zw[p_off + row], 1.0), __dmul_rn(dv, beta));
      pnew[p_off + row] = dv;
    }
    const int64_t bnd = abase + ((lo - abase) / SPMV_TILE + 1) * (int64_t)SPMV_TILE;  // first chunk boundary after lo
    if (bnd >= hi) {
      const double s = row_piece_sum_pcg<I, DIR>(crd, val, zw, pold, beta, lo, hi);
      Ap[row] = __dadd_rn(s, 0.0);
      dot_local = __dadd_rn(dot_local, __dmul_rn(s, dv));
    } else {  // the pieces and their order of spmv_rowthread_kernel
      double carried = row_piece_sum_pcg<I, DIR>(crd, val, zw, pold, beta, lo, bnd);
      int64_t b0 = bnd;
      while (b0 + SPMV_TILE < hi) {
        carried = __dadd_rn(carried, row_piece_sum_pcg<I, DIR>(crd, val, zw, pold, beta, b0, b0 + SPMV_TILE));
        b0 += SPMV_TILE;
      }
      const double s_last = row_piece_sum_pcg<I, DIR>(crd, val, zw, pold, beta, b0, hi);
      Ap[row] = __dadd_rn(__dadd_rn(s_last, 0.0), carried);
      dot_local = __dadd_rn(dot_local, __dmul_rn(__dadd_rn(carried, s_last), dv));
    }
  }
  return dot_local;
}

template <typename I>
__global__ void __launch_bounds__(256, 5)
pcg_spmv_direction_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                          int64_t abase, int64_t nrows, int64_t ntiles, int64_t p_off, double *pw0, double *pw1,
                          double *__restrict__ Ap, double *__restrict__ blk_partial, PcgExchange ex) {
  __shared__ double s_red[8];
  __shared__ double s_vals[3];
  __shared__ int s_flag;
  if (ex.fl[FL_DONE] != 0) return;
  long long *hdr = reinterpret_cast<long long *>(ex.sc);
  const long long stage = hdr[SC_STAGE], cur = hdr[SC_PCUR];
  double beta = 0.0, rr = 0.0, rznew = 0.0, relres = 0.0;
  unsigned long long iter = 0;
  bool go = true;
  if (stage == 0) {  // the first pass of a solve: p as initialised (its halo travelled as p)
    if (ex.mbox != nullptr && !pcg_wait_halo(ex, &s_flag)) return;
  } else if (ex.mbox != nullptr) {  // the head of pass C: every rank's r.r and r.z, stop test, beta
    if (!pcg_wait_sums(ex, PH_B, s_vals, rr, rznew)) return;
    relres = sqrt(rr) / ex.sc[SC_INITRES];
    iter = (unsigned long long)ex.fl[FL_ITERS] + 1;    // i starts at 1
    go = (relres > ex.tol) && (iter != ex.maxiter);    // ordered compare: NaN stops the loop
    beta = rznew / ex.sc[SC_RZ];
  } else {
    beta = ex.sc[SC_BETA];  // derived by pass B's tail, which also ran the stop test
  }
  const double *pold = cur != 0 ? pw1 : pw0;
  double *pnew = cur != 0 ? pw0 : pw1;
  const double *zw = ex.zhalo;
  double dot_local = 0.0;
  if (go) {
    if (stage == 0) {
      dot_local = pcg_spmv_rows<I, false>(pos, crd, val, abase, nrows, ntiles, p_off, zw, pold, pnew, 0.0, Ap);
    } else {
      // halo entries of the new p's window, from the neighbours' rows of z and the old halo: the blocks share each range
      for (int q = 0; q < ex.nranges; ++q) {
        const long long start = ex.halo_ranges[2 * q], len = ex.halo_ranges[2 * q + 1];
        for (long long j = (long long)blockIdx.x * 256 + threadIdx.x; j < len; j += (long long)gridDim.x * 256)
          pnew[start + j] = __dadd_rn(__dmul_rn(zw[start + j], 1.0), __dmul_rn(pold[start + j], beta));
      }
      dot_local = pcg_spmv_rows<I, true>(pos, crd, val, abase, nrows, ntiles, p_off, zw, pold, pnew, beta, Ap);
    }
  }
  const double t = block_sum(dot_local, s_red);
  if (threadIdx.x == 0) blk_partial[blockIdx.x] = t;
  if (!pcg_last_block(pcg_tickets(ex.sc) + 0, gridDim.x, &s_flag)) return;
  if (threadIdx.x == 0) {
    if (stage != 0 && ex.mbox != nullptr) {  // pass C's bookkeeping
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
    if (stage == 0) hdr[SC_STAGE] = 1;
    else if (go) hdr[SC_PCUR] = cur ^ 1;
    __threadfence();
  }
  __syncthreads();
  if (go) pcg_tail_pass_a(ex, blk_partial, gridDim.x, s_red);  // reads the iteration counter advanced above
}

template <typename I>
__global__ void max_row_len_kernel(const I *__restrict__ pos, int64_t nrows, unsigned long long *out) {
  unsigned long long m = 0;
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < nrows; r += (int64_t)gridDim.x * blockDim.x) {
    const unsigned long long len = (unsigned long long)((int64_t)pos[r + 1] - (int64_t)pos[r]);
    m = len > m ? len : m;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, m, off);
    m = o > m ? o : m;
  }
  if ((threadIdx.x & 31) == 0 && m > 0) atomicMax(out, m);
}

// ---------------------------------------------------------------------------
// SpMM: C[r, :] = (accumulate ? C[r, :] : 0) + sum_j val[j] * B[crd[j], :].
// One warp per row; lane l owns columns {2l, 2l+1} of a 64-column panel, so a B
// row is fetched as one coalesced 512-byte request and every output element is
// summed in ascending j by a single lane: bit-identical to the sequential row
// loop (examples/bspmm.py:15-23, spmm_dcsr_opdsl.py:132-135 outer-loop-only
// parallelism).  Four B rows are in flight per warp.
// ---------------------------------------------------------------------------
template <typename I, bool VEC2, int SPMM_WARPS, int SPMM_UNROLL>
__global__ void __launch_bounds__(SPMM_WARPS * 32)
spmm_row_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                int64_t nrows, int64_t k, const double *__restrict__ B, double *__restrict__ C,
                int accumulate) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * SPMM_WARPS + (threadIdx.x >> 5);
  if (row >= nrows) return;
  const int64_t lo = (int64_t)pos[row], hi = (int64_t)pos[row + 1];
  double *crow = C + row * k;
  for (int64_t c0 = 0; c0 < k; c0 += 64) {
    const int64_t col = c0 + 2 * lane;
    const bool in0 = col < k, in1 = col + 1 < k;
    double acc0 = 0.0, acc1 = 0.0;
    for (int64_t jb = lo; jb < hi; jb += 32) {
      // lanes fetch up to 32 (crd, val) pairs of the row at once, then broadcast them
      const int64_t jm = jb + lane;
      int64_t cj = 0;
      double aj = 0.0;
      if (jm < hi) {
        cj = (int64_t)__ldcs(crd + jm);
        aj = __ldcs(val + jm);
      }
      const int cnt = (int)((hi - jb) < 32 ? (hi - jb) : 32);
      for (int t0 = 0; t0 < cnt; t0 += SPMM_UNROLL) {
        double b0[SPMM_UNROLL], b1[SPMM_UNROLL], a[SPMM_UNROLL];
#pragma unroll
        for (int u = 0; u < SPMM_UNROLL; ++u) {
          const int t = t0 + u;
          const int src = t < cnt ? t : 0;
          const int64_t cc = __shfl_sync(0xffffffffu, cj, src);
          a[u] = __shfl_sync(0xffffffffu, aj, src);
          b0[u] = 0.0;
          b1[u] = 0.0;
          if (t < cnt) {
            const double *brow = B + cc * k;
            if (VEC2) {
              if (in0) {
                const double2 bb = __ldg(reinterpret_cast<const double2 *>(brow + col));
                b0[u] = bb.x;
                b1[u] = bb.y;
              }
            } else {
              if (in0) b0[u] = __ldg(brow + col);
              if (in1) b1[u] = __ldg(brow + col + 1);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < SPMM_UNROLL; ++u) {
          if (t0 + u < cnt) {
            acc0 = __dadd_rn(acc0, __dmul_rn(a[u], b0[u]));
            acc1 = __dadd_rn(acc1, __dmul_rn(a[u], b1[u]));
          }
        }
      }
    }
    if (VEC2) {
      if (in0) {
        double2 cin = make_double2(0.0, 0.0);
        if (accumulate) cin = *reinterpret_cast<const double2 *>(crow + col);
        double2 out;
        out.x = __dadd_rn(acc0, cin.x);
        out.y = __dadd_rn(acc1, cin.y);
        *reinterpret_cast<double2 *>(crow + col) = out;
      }
    } else {
      if (in0) crow[col] = __dadd_rn(acc0, accumulate ? crow[col] : 0.0);
      if (in1) crow[col + 1] = __dadd_rn(acc1, accumulate ? crow[col + 1] : 0.0);
    }
  }
}

// The same row mapping without the shuffle broadcast: every lane reads the row's (crd, val) pairs itself (one
// address per warp, served as a broadcast) and keeps UNROLL rows of B in flight as 16-byte loads.  k even, B and
// C 16-byte aligned.  Same sums in the same order as spmm_row_kernel.
template <typename I, int SPMM_WARPS, int SPMM_UNROLL>
__global__ void __launch_bounds__(SPMM_WARPS * 32)
spmm_row_direct_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                       int64_t nrows, int64_t k2, const double2 *__restrict__ B2, double2 *__restrict__ C2,
                       int accumulate) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * SPMM_WARPS + (threadIdx.x >> 5);
  if (row >= nrows) return;
  const int64_t lo = (int64_t)pos[row], hi = (int64_t)pos[row + 1];
  double2 *crow = C2 + row * k2;
  for (int64_t c = lane; c < k2; c += 32) {
    double2 acc = make_double2(0.0, 0.0);
    int64_t j = lo;
    for (; j + SPMM_UNROLL <= hi; j += SPMM_UNROLL) {
      double a[SPMM_UNROLL];
      double2 b[SPMM_UNROLL];
#pragma unroll
      for (int u = 0; u < SPMM_UNROLL; ++u) {
        a[u] = __ldg(val + j + u);
        b[u] = __ldg(B2 + (int64_t)crd[j + u] * k2 + c);
      }
#pragma unroll
      for (int u = 0; u < SPMM_UNROLL; ++u) {
        acc.x = __dadd_rn(acc.x, __dmul_rn(a[u], b[u].x));
        acc.y = __dadd_rn(acc.y, __dmul_rn(a[u], b[u].y));
      }
    }
    for (; j < hi; ++j) {
      const double a = __ldg(val + j);
      const double2 b = __ldg(B2 + (int64_t)crd[j] * k2 + c);
      acc.x = __dadd_rn(acc.x, __dmul_rn(a, b.x));
      acc.y = __dadd_rn(acc.y, __dmul_rn(a, b.y));
    }
    double2 cin = make_double2(0.0, 0.0);
    if (accumulate) cin = crow[c];
    crow[c] = make_double2(__dadd_rn(acc.x, cin.x), __dadd_rn(acc.y, cin.y));
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// Kernel variant: {threads, blocks per SM, L2 hint}.  threads >= 256: one chunk per block; threads == 2 / 3: the
// segmented-scan chunk kernel with 256 / 512 threads (minb blocks per SM); threads == 1: one thread per row;
// threads < 0: the persistent bulk-copy kernel with |threads| threads.  Which one is faster
// depends on the matrix (the persistent kernel wins when x is served from L1/L2, as for banded
// matrices; the one-chunk kernel when the gathers of x dominate), so lapis_b200_csr_tune times
// the candidates on the matrix itself and stores the winner in the handle.  A process-wide
// override (LAPIS_B200_SPMV="threads,blocks,hint" or lapis_b200_spmv_select_kernel) beats both.
struct SpmvVariant {
  int threads, minb, hint;
};
constexpr SpmvVariant SPMV_DEFAULT{256, 4, 1};
static SpmvVariant &spmv_override() {  // threads == 0: no override
  static SpmvVariant v = [] {
    SpmvVariant d{0, 0, 0};
    if (const char *e = std::getenv("LAPIS_B200_SPMV")) {
      int t = 0, m = 0, h = 0;
      if (sscanf(e, "%d,%d,%d", &t, &m, &h) == 3) d = SpmvVariant{t, m, h};
    }
    return d;
  }();
  return v;
}
constexpr int SPMV_ROWTHREAD_MAX_LEN = 32;
static bool spmv_variant_known(int threads, int minb) {
  if (threads == 1) return minb == 0;  // one thread per row
  if (threads == 4) return minb == 0;  // one warp per chunk, no shared memory
  if (threads == 2) return minb == 4 || minb == 5;  // segmented-scan chunk kernel, 256 threads, blocks per SM
  if (threads == 3) return minb >= 2 && minb <= 4 && SPMV_TILE >= 1024;  // the same with 512 threads
  if (threads == -256 || threads == -512) return minb >= 1 && minb <= 8;
  return (threads == 256 && (minb == 4 || minb == 6)) || (threads == 512 && minb == 3 && SPMV_TILE >= 1024);
}

template <typename I, int THREADS, int MINB, bool HINT>
static void launch_chunks(const lapis_b200_csr *h, const double *x, double *y, int accumulate, const double *dotvec,
                          double *blk_partial, const int *skip_flag, cudaStream_t st) {
  const I *pos = static_cast<const I *>(h->pos);
  const I *crd = static_cast<const I *>(h->crd);
  const int64_t abase = h->base & ~(int64_t)3, nnz_end = h->base + h->nnz;
  if (dotvec != nullptr)
    spmv_chunk_kernel<I, THREADS, MINB, true, HINT><<<(unsigned)h->nblk, THREADS, 0, st>>>(
        pos, crd, h->val, h->blk_row, abase, nnz_end, h->nrows, x, y, accumulate, h->carry, dotvec, blk_partial,
        skip_flag);
  else
    spmv_chunk_kernel<I, THREADS, MINB, false, HINT><<<(unsigned)h->nblk, THREADS, 0, st>>>(
        pos, crd, h->val, h->blk_row, abase, nnz_end, h->nrows, x, y, accumulate, h->carry, nullptr, nullptr,
        skip_flag);
}

template <typename I, int THREADS, int MINB, bool HINT>
static void launch_scan(const lapis_b200_csr *h, const double *x, double *y, int accumulate, const double *dotvec,
                        double *blk_partial, const int *skip_flag, cudaStream_t st) {
  const I *pos = static_cast<const I *>(h->pos);
  const I *crd = static_cast<const I *>(h->crd);
  const int64_t abase = h->base & ~(int64_t)3, nnz_end = h->base + h->nnz;
  if (dotvec != nullptr)
    spmv_scan_kernel<I, THREADS, MINB, true, HINT><<<(unsigned)h->nblk, THREADS, 0, st>>>(
        pos, crd, h->val, h->blk_row, abase, nnz_end, h->nrows, x, y, accumulate, h->carry, dotvec, blk_partial,
        skip_flag);
  else
    spmv_scan_kernel<I, THREADS, MINB, false, HINT><<<(unsigned)h->nblk, THREADS, 0, st>>>(
        pos, crd, h->val, h->blk_row, abase, nnz_end, h->nrows, x, y, accumulate, h->carry, nullptr, nullptr,
        skip_flag);
}

template <typename I, int THREADS, bool HINT>
static int launch_pipe(const lapis_b200_csr *h, int ctas_per_sm, const double *x, double *y, int accumulate,
                       const double *dotvec, double *blk_partial, const int *skip_flag, cudaStream_t st) {
  const I *pos = static_cast<const I *>(h->pos);
  const I *crd = static_cast<const I *>(h->crd);
  const int64_t abase = h->base & ~(int64_t)3, nnz_end = h->base + h->nnz;
  constexpr int smem = spmv_pipe_smem_bytes<I>(THREADS);
  static bool attr_done[64][2] = {};  // per device: the attribute belongs to the device's copy of the kernel
  int dev = 0;
  LAPIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(LAPIS_EBADARG, "spmv: device index %d not supported", dev);
  int64_t grid = (int64_t)sm_count() * ctas_per_sm;
  if (grid > h->nblk) grid = h->nblk;
  if (dotvec != nullptr) {
    auto k = spmv_pipe_kernel<I, THREADS, true, HINT>;
    if (!attr_done[dev][1]) {
      LAPIS_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      attr_done[dev][1] = true;
    }
    k<<<(unsigned)grid, THREADS, smem, st>>>(pos, crd, h->val, h->blk_row, abase, nnz_end, h->nrows, h->nblk, x, y,
                                             accumulate, h->carry, dotvec, blk_partial, skip_flag);
  } else {
    auto k = spmv_pipe_kernel<I, THREADS, false, HINT>;
    if (!attr_done[dev][0]) {
      LAPIS_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      attr_done[dev][0] = true;
    }
    k<<<(unsigned)grid, THREADS, smem, st>>>(pos, crd, h->val, h->blk_row, abase, nnz_end, h->nrows, h->nblk, x, y,
                                             accumulate, h->carry, nullptr, nullptr, skip_flag);
  }
  return LAPIS_OK;
}

// Adds the carries of a launch over `nblk` chunks of `tile` entries to their rows.
template <typename I>
static int launch_fixup(const lapis_b200_csr *h, const int64_t *plan, const double *carry, int64_t nblk, int tile, double *y,
                        const int *skip_flag, cudaStream_t st) {
  if (nblk <= 1) return LAPIS_OK;
  const I *pos = static_cast<const I *>(h->pos);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((nblk - 1 + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;  // lets the fix-up blocks become resident while the SpMV kernel drains
  LAPIS_CUDA_TRY(cudaLaunchKernelEx(&cfg, spmv_fixup_kernel<I>, pos, plan, (int64_t)(h->base & ~(int64_t)3), nblk,
                                    (int64_t)h->nrows, carry, y, skip_flag, tile));
  return LAPIS_OK;
}

// Whether spmv_launch will run the one-thread-per-row kernel for this handle (the variant that can carry the
// head and tail of a PCG iteration's first pass).
static bool uses_rowthread(const lapis_b200_csr *h) {
  SpmvVariant v = spmv_override();
  if (v.threads == 0) v = h->tuned_threads != 0 ? SpmvVariant{h->tuned_threads, h->tuned_minb, h->tuned_hint} : SPMV_DEFAULT;
  return v.threads == 1 && h->max_row_len >= 0 && h->max_row_len <= SPMV_ROWTHREAD_MAX_LEN;
}

// Grid of the SpMV pass of a PCG iteration in both of its forms (spmv_rowthread_kernel with head and tail,
// pcg_spmv_direction_kernel): the blocks that are resident at once for either kernel, looping over the row
// tiles.  One size for both, so that the per-block partial sums of p.Ap group the same way and the two forms
// return the same bits.
template <typename I>
static int pcg_pass_grid(const lapis_b200_csr *h, unsigned *grid) {
  static int per_sm[64] = {0};
  int dev = 0;
  LAPIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(LAPIS_EBADARG, "spmv: device index %d not supported", dev);
  if (per_sm[dev] == 0) {
    int na = 0, nb = 0;
    LAPIS_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&na, spmv_rowthread_kernel<I, true, true>, 256, 0));
    LAPIS_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, pcg_spmv_direction_kernel<I>, 256, 0));
    const int m = na < nb ? na : nb;
    per_sm[dev] = m > 0 ? m : 1;
  }
  const int64_t ntiles = (h->nrows + 255) / 256, resident = (int64_t)sm_count() * per_sm[dev];
  const int64_t g = std::min<int64_t>(std::min<int64_t>(h->nblk, ntiles), resident);
  *grid = (unsigned)(g < 1 ? 1 : g);
  return LAPIS_OK;
}

template <typename I>
static int launch_spmv(const lapis_b200_csr *h, const double *x, double *y, int accumulate,
                       const double *dotvec, double *blk_partial, const int *skip_flag,
                       cudaStream_t st, const PcgExchange *ex) {
  SpmvVariant v = spmv_override();
  if (v.threads == 0) v = h->tuned_threads != 0 ? SpmvVariant{h->tuned_threads, h->tuned_minb, h->tuned_hint} : SPMV_DEFAULT;
  if (v.threads == 1) {
    // one thread per row: only where it returns the chunk kernels' bits (rows of at most 32 entries, which the
    // tuner has checked); otherwise the default kernel runs
    if (h->max_row_len >= 0 && h->max_row_len <= SPMV_ROWTHREAD_MAX_LEN) {
      const I *pos = static_cast<const I *>(h->pos);
      const I *crd = static_cast<const I *>(h->crd);
      const int64_t abase = h->base & ~(int64_t)3, ntiles = (h->nrows + 255) / 256;
      const PcgExchange none = {};
      if (dotvec != nullptr && ex != nullptr) {
        // as pass A of a PCG iteration: a grid of exactly the blocks that are resident at once, looping over the
        // row tiles, so that the block that finishes last has about a thousand partial sums to add, not one per
        // chunk of the plan (a grid larger than what is resident would run its last blocks on a nearly empty GPU)
        unsigned grid = 1;
        LAPIS_TRY(pcg_pass_grid<I>(h, &grid));
        spmv_rowthread_kernel<I, true, true><<<grid, 256, 0, st>>>(pos, crd, h->val, abase, h->nrows, ntiles, x, y,
                                                                                  accumulate, dotvec, blk_partial, skip_flag, *ex);
      }
      else if (dotvec != nullptr)
        spmv_rowthread_kernel<I, true, false><<<(unsigned)h->nblk, 256, 0, st>>>(pos, crd, h->val, abase, h->nrows, ntiles, x, y,
                                                                                 accumulate, dotvec, blk_partial, skip_flag, none);
      else
        spmv_rowthread_kernel<I, false, false><<<(unsigned)h->nblk, 256, 0, st>>>(pos, crd, h->val, abase, h->nrows, ntiles, x, y,
                                                                                  accumulate, nullptr, nullptr, skip_flag, none);
      LAPIS_CUDA_TRY(cudaGetLastError());
      return LAPIS_OK;
    }
    v = SPMV_DEFAULT;
  }
  if (ex != nullptr) return fail(LAPIS_EBADARG, "spmv: the fused PCG pass needs the one-thread-per-row kernel");
  if (v.threads == 4) {
    // one warp per chunk: its 32-byte loads need val and crd 32-byte aligned; otherwise the default kernel runs
    if (((reinterpret_cast<uintptr_t>(h->val) | reinterpret_cast<uintptr_t>(h->crd)) & 31) != 0) v = SPMV_DEFAULT;
  }
  if (v.threads == 4) {
    const I *pos = static_cast<const I *>(h->pos);
    const I *crd = static_cast<const I *>(h->crd);
    const int64_t abase = h->base & ~(int64_t)3, nnz_end = h->base + h->nnz;
    constexpr int WPB = SPMV_WALK_THREADS / 32;
    if (dotvec != nullptr || h->walk_plan == nullptr) {
      // chunks of the shared plan (the consumers of the fused dot product expect one partial per chunk)
      const unsigned grid = (unsigned)((h->nblk + WPB - 1) / WPB);
      if (dotvec != nullptr)
        spmv_walk_kernel<I, true><<<grid, SPMV_WALK_THREADS, 0, st>>>(pos, crd, h->val, h->blk_row, abase, h->base, nnz_end,
                                                                      h->nrows, h->nblk, SPMV_TILE, x, y, accumulate, h->carry,
                                                                      dotvec, blk_partial, skip_flag);
      else
        spmv_walk_kernel<I, false><<<grid, SPMV_WALK_THREADS, 0, st>>>(pos, crd, h->val, h->blk_row, abase, h->base, nnz_end,
                                                                       h->nrows, h->nblk, SPMV_TILE, x, y, accumulate, h->carry,
                                                                       nullptr, nullptr, skip_flag);
    } else {
      // a small matrix: shorter ranges per warp (the handle's second plan), so that the warps fill the SMs evenly
      const unsigned grid = (unsigned)((h->walk_nblk + WPB - 1) / WPB);
      spmv_walk_kernel<I, false><<<grid, SPMV_WALK_THREADS, 0, st>>>(pos, crd, h->val, h->walk_plan, abase, h->base, nnz_end,
                                                                     h->nrows, h->walk_nblk, h->walk_tile, x, y, accumulate,
                                                                     h->walk_carry, nullptr, nullptr, skip_flag);
      LAPIS_CUDA_TRY(cudaGetLastError());
      return launch_fixup<I>(h, h->walk_plan, h->walk_carry, h->walk_nblk, h->walk_tile, y, skip_flag, st);
    }
  } else if (v.threads < 0) {  // persistent bulk-copy kernel: threads = -256 or -512, minb = blocks per SM
    int rc;
    if (v.threads == -256)
      rc = v.hint ? launch_pipe<I, 256, true>(h, v.minb, x, y, accumulate, dotvec, blk_partial, skip_flag, st)
                  : launch_pipe<I, 256, false>(h, v.minb, x, y, accumulate, dotvec, blk_partial, skip_flag, st);
    else if (v.threads == -512)
      rc = v.hint ? launch_pipe<I, 512, true>(h, v.minb, x, y, accumulate, dotvec, blk_partial, skip_flag, st)
                  : launch_pipe<I, 512, false>(h, v.minb, x, y, accumulate, dotvec, blk_partial, skip_flag, st);
    else
      return fail(LAPIS_EBADARG, "LAPIS_B200_SPMV names an unknown kernel variant");
    LAPIS_TRY(rc);
  } else if (v.threads == 2 || v.threads == 3) {  // segmented-scan chunk kernel with 256 / 512 threads
#define LAPIS_S(T, M)                                                                                     \
  if ((v.threads == 2 ? 256 : 512) == T && v.minb == M) {                                                 \
    if (v.hint)                                                                                           \
      launch_scan<I, T, M, true>(h, x, y, accumulate, dotvec, blk_partial, skip_flag, st);                \
    else                                                                                                  \
      launch_scan<I, T, M, false>(h, x, y, accumulate, dotvec, blk_partial, skip_flag, st);               \
  } else
    LAPIS_S(256, 4)
    LAPIS_S(256, 5)
#if LAPIS_SPMV_TILE >= 1024
    LAPIS_S(512, 2)
    LAPIS_S(512, 3)
    LAPIS_S(512, 4)
#endif
    { return fail(LAPIS_EBADARG, "LAPIS_B200_SPMV names an unknown kernel variant"); }
#undef LAPIS_S
  } else
#define LAPIS_V(T, M)                                                                                     \
  if (v.threads == T && v.minb == M) {                                                                    \
    if (v.hint)                                                                                           \
      launch_chunks<I, T, M, true>(h, x, y, accumulate, dotvec, blk_partial, skip_flag, st);              \
    else                                                                                                  \
      launch_chunks<I, T, M, false>(h, x, y, accumulate, dotvec, blk_partial, skip_flag, st);             \
  } else
  LAPIS_V(256, 6)
  LAPIS_V(256, 4)
#if LAPIS_SPMV_TILE >= 1024
  LAPIS_V(512, 3)
#endif

  { return fail(LAPIS_EBADARG, "LAPIS_B200_SPMV names an unknown kernel variant"); }
#undef LAPIS_V
  LAPIS_CUDA_TRY(cudaGetLastError());
  return launch_fixup<I>(h, h->blk_row, h->carry, h->nblk, SPMV_TILE, y, skip_flag, st);
}

int spmv_launch(const lapis_b200_csr *h, const double *x, double *y, int accumulate,
                const double *dotvec, double *blk_partial, const int *skip_flag, cudaStream_t st) {
  if (h->nrows == 0) return LAPIS_OK;
  if (h->idx_bytes == 4)
    return launch_spmv<int32_t>(h, x, y, accumulate, dotvec, blk_partial, skip_flag, st, nullptr);
  return launch_spmv<int64_t>(h, x, y, accumulate, dotvec, blk_partial, skip_flag, st, nullptr);
}

// Pass A of a PCG iteration with its head and tail inside the SpMV kernel; only for handles on which
// spmv_fuses_pcg_pass() is true.
bool spmv_fuses_pcg_pass(const lapis_b200_csr *h) { return h->nrows > 0 && uses_rowthread(h); }
int spmv_launch_pcg_pass(const lapis_b200_csr *h, const double *x, double *y, const double *dotvec, double *blk_partial,
                         const int *skip_flag, cudaStream_t st, const PcgExchange &ex) {
  if (h->idx_bytes == 4) return launch_spmv<int32_t>(h, x, y, 0, dotvec, blk_partial, skip_flag, st, &ex);
  return launch_spmv<int64_t>(h, x, y, 0, dotvec, blk_partial, skip_flag, st, &ex);
}

// Pass A with the direction update folded in (two-pass PCG); only where spmv_fuses_pcg_pass() is true.
template <typename I>
static int launch_pcg_direction_pass(const lapis_b200_csr *h, int64_t p_off, double *pw0, double *pw1, double *Ap,
                                     double *blk_partial, cudaStream_t st, const PcgExchange &ex) {
  const int64_t ntiles = (h->nrows + 255) / 256;
  unsigned grid = 1;
  LAPIS_TRY(pcg_pass_grid<I>(h, &grid));
  pcg_spmv_direction_kernel<I><<<grid, 256, 0, st>>>(static_cast<const I *>(h->pos), static_cast<const I *>(h->crd),
                                                                    h->val, h->base & ~(int64_t)3, h->nrows, ntiles, p_off, pw0,
                                                                    pw1, Ap, blk_partial, ex);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}
int spmv_launch_pcg_direction_pass(const lapis_b200_csr *h, int64_t p_off, double *pw0, double *pw1, double *Ap,
                                   double *blk_partial, cudaStream_t st, const PcgExchange &ex) {
  if (!spmv_fuses_pcg_pass(h)) return fail(LAPIS_EBADARG, "pcg: the two-pass form needs the one-thread-per-row SpMV kernel");
  if (h->idx_bytes == 4) return launch_pcg_direction_pass<int32_t>(h, p_off, pw0, pw1, Ap, blk_partial, st, ex);
  return launch_pcg_direction_pass<int64_t>(h, p_off, pw0, pw1, Ap, blk_partial, st, ex);
}

template <typename I, int WARPS, int UNROLL>
static void launch_spmm_variant(const lapis_b200_csr *h, int64_t k, const double *B, double *C, int accumulate,
                                cudaStream_t st) {
  const I *pos = static_cast<const I *>(h->pos);
  const I *crd = static_cast<const I *>(h->crd);
  const unsigned grid = (unsigned)((h->nrows + WARPS - 1) / WARPS);
  const bool vec2 = (k % 2 == 0) && ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 == 0);
  if (vec2)
    spmm_row_kernel<I, true, WARPS, UNROLL><<<grid, WARPS * 32, 0, st>>>(pos, crd, h->val, h->nrows, k, B, C, accumulate);
  else
    spmm_row_kernel<I, false, WARPS, UNROLL><<<grid, WARPS * 32, 0, st>>>(pos, crd, h->val, h->nrows, k, B, C, accumulate);
}

// The direct-load kernel (four rows of B in flight per lane) needs k even and 16-byte aligned B, C; other
// operands take the shuffle-broadcast kernel.  Measured on the 2^21-row, 32-per-row, k = 64 case: direct 5.10 ms
// (5.12 ms with eight rows in flight), shuffle-broadcast 6.6 ms.
template <typename I>
static int launch_spmm(const lapis_b200_csr *h, int64_t k, const double *B, double *C, int accumulate,
                       cudaStream_t st) {
  const bool vec2 = (k % 2 == 0) && ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 == 0);
  if (vec2) {
    const I *pos = static_cast<const I *>(h->pos);
    const I *crd = static_cast<const I *>(h->crd);
    const unsigned grid = (unsigned)((h->nrows + 7) / 8);
    spmm_row_direct_kernel<I, 8, 4><<<grid, 256, 0, st>>>(pos, crd, h->val, h->nrows, k / 2,
                                                          reinterpret_cast<const double2 *>(B),
                                                          reinterpret_cast<double2 *>(C), accumulate);
  } else {
    launch_spmm_variant<I, 8, 4>(h, k, B, C, accumulate, st);
  }
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

}  // namespace lapis_b200

using namespace lapis_b200;

extern "C" int lapis_b200_csr_create(lapis_b200_csr_t *out, int idx_bytes, int64_t nrows, int64_t ncols,
                                     const void *d_pos, const void *d_crd, const double *d_val,
                                     void *stream) {
  clear_error();
  if (out == nullptr) return fail(LAPIS_EBADARG, "csr_create: out is null");
  *out = nullptr;
  if (idx_bytes != 4 && idx_bytes != 8) return fail(LAPIS_EBADARG, "csr_create: idx_bytes must be 4 or 8");
  if (nrows < 0 || ncols < 0) return fail(LAPIS_EBADSHAPE, "csr_create: negative dimension");
  if (d_pos == nullptr) return fail(LAPIS_EBADARG, "csr_create: pos is null");
  if ((reinterpret_cast<uintptr_t>(d_val) % 16) || (reinterpret_cast<uintptr_t>(d_crd) % 16))
    return fail(LAPIS_EBADARG, "csr_create: val and crd must be 16-byte aligned");
  cudaStream_t st = as_stream(stream);
  int dev = 0;
  LAPIS_CUDA_TRY(cudaGetDevice(&dev));

  // pos[0] and pos[nrows] define the nnz range addressed by this matrix.
  int64_t ends[2] = {0, 0};
  if (idx_bytes == 4) {
    int32_t e32[2];
    LAPIS_CUDA_TRY(cudaMemcpyAsync(&e32[0], d_pos, 4, cudaMemcpyDeviceToHost, st));
    LAPIS_CUDA_TRY(cudaMemcpyAsync(&e32[1], static_cast<const int32_t *>(d_pos) + nrows, 4,
                                   cudaMemcpyDeviceToHost, st));
    LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
    ends[0] = e32[0];
    ends[1] = e32[1];
  } else {
    LAPIS_CUDA_TRY(cudaMemcpyAsync(&ends[0], d_pos, 8, cudaMemcpyDeviceToHost, st));
    LAPIS_CUDA_TRY(cudaMemcpyAsync(&ends[1], static_cast<const int64_t *>(d_pos) + nrows, 8,
                                   cudaMemcpyDeviceToHost, st));
    LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  }
  if (ends[1] < ends[0] || ends[0] < 0) return fail(LAPIS_EBADSHAPE, "csr_create: pos is not non-decreasing");
  const int64_t nnz = ends[1] - ends[0];
  if (nnz > 0 && (d_crd == nullptr || d_val == nullptr)) return fail(LAPIS_EBADARG, "csr_create: crd/val null");
  int64_t nblk = (ends[1] - (ends[0] & ~(int64_t)3) + SPMV_TILE - 1) / SPMV_TILE;
  if (nblk < 1) nblk = 1;
  if (nblk > 0x7fffffffLL) return fail(LAPIS_ETOOBIG, "csr_create: more than 2^31 chunks");

  lapis_b200_csr *h = new lapis_b200_csr();
  h->idx_bytes = idx_bytes;
  h->nrows = nrows;
  h->ncols = ncols;
  h->nnz = nnz;
  h->base = ends[0];
  h->pos = d_pos;
  h->crd = d_crd;
  h->val = d_val;
  h->nblk = nblk;
  h->blk_row = nullptr;
  h->blk_partial = nullptr;
  h->carry = nullptr;
  h->tuned_threads = h->tuned_minb = h->tuned_hint = 0;
  h->max_row_len = -1;
  h->device = dev;
  h->walk_plan = nullptr;
  h->walk_carry = nullptr;
  h->walk_nblk = 0;
  h->walk_tile = 0;
  // The warp-walk kernel gives one warp a range of entries.  With 2048-entry ranges a matrix needs about eight
  // times as many ranges as the GPU holds warps (32 per SM) before the last, partly filled round of warps stops
  // mattering; smaller matrices (a row block of a partitioned one) get a second plan of 512-entry ranges.
  const int64_t resident_warps = (int64_t)sm_count() * 32;
  if (nblk > 1 && nblk < 8 * resident_warps) {
    h->walk_tile = SPMV_WALK_FINE_TILE;
    h->walk_nblk = (ends[1] - (ends[0] & ~(int64_t)3) + h->walk_tile - 1) / h->walk_tile;
  }
  cudaError_t e = cudaMalloc(&h->blk_row, (size_t)(nblk + 1) * sizeof(int64_t));
  if (e == cudaSuccess) e = cudaMalloc(&h->blk_partial, (size_t)nblk * sizeof(double));
  if (e == cudaSuccess) e = cudaMalloc(&h->carry, (size_t)nblk * sizeof(double));
  if (e == cudaSuccess && h->walk_nblk > 0) e = cudaMalloc(&h->walk_plan, (size_t)(h->walk_nblk + 1) * sizeof(int64_t));
  if (e == cudaSuccess && h->walk_nblk > 0) e = cudaMalloc(&h->walk_carry, (size_t)h->walk_nblk * sizeof(double));
  if (e != cudaSuccess) {
    cudaFree(h->blk_row);
    cudaFree(h->blk_partial);
    cudaFree(h->carry);
    cudaFree(h->walk_plan);
    cudaFree(h->walk_carry);
    delete h;
    return fail(LAPIS_ECUDA, "csr_create: cudaMalloc failed: %s", cudaGetErrorString(e));
  }
  const unsigned pgrid = (unsigned)((nblk + 1 + 255) / 256);
  if (idx_bytes == 4)
    spmv_plan_kernel<int32_t><<<pgrid, 256, 0, st>>>(static_cast<const int32_t *>(d_pos), nrows, nblk, h->blk_row);
  else
    spmv_plan_kernel<int64_t><<<pgrid, 256, 0, st>>>(static_cast<const int64_t *>(d_pos), nrows, nblk, h->blk_row);
  if (h->walk_nblk > 0) {
    const unsigned wgrid = (unsigned)((h->walk_nblk + 1 + 255) / 256);
    if (idx_bytes == 4)
      spmv_plan_kernel<int32_t><<<wgrid, 256, 0, st>>>(static_cast<const int32_t *>(d_pos), nrows, h->walk_nblk, h->walk_plan,
                                                       h->walk_tile);
    else
      spmv_plan_kernel<int64_t><<<wgrid, 256, 0, st>>>(static_cast<const int64_t *>(d_pos), nrows, h->walk_nblk, h->walk_plan,
                                                       h->walk_tile);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    cudaFree(h->blk_row);
    cudaFree(h->blk_partial);
    cudaFree(h->carry);
    cudaFree(h->walk_plan);
    cudaFree(h->walk_carry);
    delete h;
    return fail(LAPIS_ECUDA, "csr_create: plan kernel launch failed: %s", cudaGetErrorString(e));
  }
  *out = h;
  return LAPIS_OK;
}

extern "C" int lapis_b200_spmv_select_kernel(int threads, int blocks_per_sm, int l2_hint) {
  clear_error();
  if (threads == 0) {  // back to automatic: the handle's tuned choice, else the default
    spmv_override() = SpmvVariant{0, 0, 0};
    return LAPIS_OK;
  }
  if (!spmv_variant_known(threads, blocks_per_sm)) return fail(LAPIS_EBADARG, "spmv_select_kernel: unknown kernel variant");
  spmv_override() = SpmvVariant{threads, blocks_per_sm, l2_hint ? 1 : 0};
  return LAPIS_OK;
}

// Times the candidate kernels on this matrix (y = A x with scratch x = 0, y) and keeps the fastest.
// relaxed: the segmented-scan kernel is a candidate too (row sums in scan order: within the 1e-12 bound of
// the sequential sum, not the bits of the other variants).
static int csr_tune_impl(lapis_b200_csr_t h, void *stream, bool relaxed) {
  clear_error();
  if (h == nullptr) return fail(LAPIS_EBADARG, "csr_tune: null matrix handle");
  if (h->nrows == 0 || h->nnz == 0) return LAPIS_OK;
  cudaStream_t st = as_stream(stream);
  double *x = nullptr, *y = nullptr;
  LAPIS_CUDA_TRY(cudaMalloc(&x, (size_t)(h->ncols > 0 ? h->ncols : 1) * 8));
  cudaError_t e = cudaMalloc(&y, (size_t)h->nrows * 8);
  if (e != cudaSuccess) {
    cudaFree(x);
    return fail(LAPIS_ECUDA, "csr_tune: cudaMalloc failed: %s", cudaGetErrorString(e));
  }
  cudaMemsetAsync(x, 0, (size_t)(h->ncols > 0 ? h->ncols : 1) * 8, st);
  if (h->max_row_len < 0) {  // the longest row decides whether the one-thread-per-row kernel is a candidate
    unsigned long long *d_max = reinterpret_cast<unsigned long long *>(y), h_max = 0;
    cudaMemsetAsync(d_max, 0, 8, st);
    const unsigned g = (unsigned)std::min<int64_t>((h->nrows + 255) / 256, (int64_t)sm_count() * 8);
    if (h->idx_bytes == 4)
      max_row_len_kernel<int32_t><<<g, 256, 0, st>>>(static_cast<const int32_t *>(h->pos), h->nrows, d_max);
    else
      max_row_len_kernel<int64_t><<<g, 256, 0, st>>>(static_cast<const int64_t *>(h->pos), h->nrows, d_max);
    if (cudaMemcpyAsync(&h_max, d_max, 8, cudaMemcpyDeviceToHost, st) == cudaSuccess && cudaStreamSynchronize(st) == cudaSuccess)
      h->max_row_len = (int64_t)h_max;
  }
  const int pipe_blocks = h->idx_bytes == 4 ? 4 : 3;  // what fits in shared memory
  const bool short_rows = h->max_row_len >= 0 && h->max_row_len <= SPMV_ROWTHREAD_MAX_LEN;
  const SpmvVariant cand[] = {{256, 4, 1}, {256, 6, 1}, {512, 3, 1}, {-256, pipe_blocks, 1}, {1, 0, 1},
                              {2, 5, 1}, {2, 5, 0}, {3, 4, 1}, {3, 4, 0}, {4, 0, 0}};
  const SpmvVariant saved = spmv_override();
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float best = 0.f;
  int status = LAPIS_OK;
  for (const SpmvVariant &c : cand) {
    if (c.threads == 1 && !short_rows) continue;
    if ((c.threads == 2 || c.threads == 3 || c.threads == 4) && !relaxed) continue;
    if (c.threads == 4 && ((reinterpret_cast<uintptr_t>(h->val) | reinterpret_cast<uintptr_t>(h->crd)) & 31) != 0) continue;
    if (!spmv_variant_known(c.threads, c.minb)) continue;
    spmv_override() = c;
    status = spmv_launch(h, x, y, 0, nullptr, nullptr, nullptr, st);  // warm-up
    if (status != LAPIS_OK) break;
    cudaEventRecord(e0, st);
    for (int r = 0; r < 3 && status == LAPIS_OK; ++r) status = spmv_launch(h, x, y, 0, nullptr, nullptr, nullptr, st);
    cudaEventRecord(e1, st);
    if (status != LAPIS_OK || cudaEventSynchronize(e1) != cudaSuccess) {
      if (status == LAPIS_OK) status = fail(LAPIS_ECUDA, "csr_tune: timing run failed");
      break;
    }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (h->tuned_threads == 0 || ms < best) {
      best = ms;
      h->tuned_threads = c.threads;
      h->tuned_minb = c.minb;
      h->tuned_hint = c.hint;
    }
  }
  spmv_override() = saved;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(x);
  cudaFree(y);
  return status;
}

extern "C" int lapis_b200_csr_tune(lapis_b200_csr_t h, void *stream) { return csr_tune_impl(h, stream, false); }
extern "C" int lapis_b200_csr_tune_relaxed(lapis_b200_csr_t h, void *stream) { return csr_tune_impl(h, stream, true); }

extern "C" int lapis_b200_csr_tuned_kernel(lapis_b200_csr_t h, int *threads, int *blocks_per_sm) {
  if (h == nullptr) return LAPIS_EBADARG;
  if (threads) *threads = h->tuned_threads;
  if (blocks_per_sm) *blocks_per_sm = h->tuned_minb;
  return LAPIS_OK;
}

// Reads and clears the flag a persistent SpMV block sets when one of its bounded waits gives up.
extern "C" int lapis_b200_spmv_status(void *stream) {
  clear_error();
  LAPIS_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
  int flag = 0;
  LAPIS_CUDA_TRY(cudaMemcpyFromSymbol(&flag, g_spmv_error, sizeof(int)));
  if (flag != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_spmv_error, &zero, sizeof(int));
    return fail(LAPIS_ECUDA, "spmv: a bulk copy did not complete within the wait limit; y is not valid");
  }
  return LAPIS_OK;
}

extern "C" int lapis_b200_csr_destroy(lapis_b200_csr_t h) {
  // does not touch the recorded status: it runs while an error of the enclosing call unwinds
  if (h == nullptr) return LAPIS_OK;
  cudaFree(h->blk_row);
  cudaFree(h->blk_partial);
  cudaFree(h->carry);
  cudaFree(h->walk_plan);
  cudaFree(h->walk_carry);
  delete h;
  return LAPIS_OK;
}

extern "C" int64_t lapis_b200_csr_nnz(lapis_b200_csr_t h) { return h ? h->nnz : -1; }

extern "C" int lapis_b200_spmv_f64(lapis_b200_csr_t h, const double *d_x, double *d_y, int accumulate,
                                   void *stream) {
  clear_error();
  if (h == nullptr) return fail(LAPIS_EBADARG, "spmv: null matrix handle");
  if (h->nrows > 0 && d_y == nullptr) return fail(LAPIS_EBADARG, "spmv: y is null");
  if (h->nnz > 0 && d_x == nullptr) return fail(LAPIS_EBADARG, "spmv: x is null");
  return spmv_launch(h, d_x, d_y, accumulate, nullptr, nullptr, nullptr, as_stream(stream));
}

extern "C" int lapis_b200_spmm_f64(lapis_b200_csr_t h, int64_t k, const double *d_B, double *d_C,
                                   int accumulate, void *stream) {
  clear_error();
  if (h == nullptr) return fail(LAPIS_EBADARG, "spmm: null matrix handle");
  if (k < 0) return fail(LAPIS_EBADSHAPE, "spmm: negative k");
  if (h->nrows == 0 || k == 0) return LAPIS_OK;
  if (d_C == nullptr || (h->nnz > 0 && d_B == nullptr)) return fail(LAPIS_EBADARG, "spmm: null operand");
  if (h->idx_bytes == 4) return launch_spmm<int32_t>(h, k, d_B, d_C, accumulate, as_stream(stream));
  return launch_spmm<int64_t>(h, k, d_B, d_C, accumulate, as_stream(stream));
}

// ---------------------------------------------------------------------------
// SpMV without any allocation.
//
// Some callers must not allocate device memory when they call in: a solver that
// runs inside a memory pool another component has already sized to the whole GPU,
// or a service whose steady state is forbidden to touch the allocator because a
// cudaMalloc may synchronise the device or fail long after start-up.
// lapis_b200_csr_create allocates the streaming plan (8 bytes per 2048 stored
// entries); this entry point keeps that plan in a fixed array in the library's own
// device image instead.  The price is a size limit and one shared buffer: every
// GPU that loads the library holds the array until exit, every call overwrites all
// entries it uses (nothing needs to start at zero), and two calls in flight on the
// same device at the same time would overwrite each other's plan.
// ---------------------------------------------------------------------------
constexpr int64_t NOALLOC_MAX_TILES = 1 << 18;  // matrices of up to 2^29 stored entries
// [0, MAX]: the plan (int64); (MAX, 2*MAX]: the per-chunk carries (doubles, same width).  4 MiB.
static __device__ __align__(256) int64_t g_noalloc_plan[2 * NOALLOC_MAX_TILES + 1];

// Device address of g_noalloc_plan per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel may use; cudaGetSymbolAddress returns the
// address in the device that is current when it is called.  Plain statics without a lock, like
// the rest of the library: one caller thread per process at a time.
static int64_t *g_noalloc_plan_addr[64] = {nullptr};

static int noalloc_plan_ptr(int64_t **out, int *device) {
  int dev = 0;
  LAPIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return lapis_b200::fail(LAPIS_EBADARG, "spmv_noalloc: device index %d not supported", dev);
  if (g_noalloc_plan_addr[dev] == nullptr) {
    void *p = nullptr;
    LAPIS_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_plan));
    g_noalloc_plan_addr[dev] = static_cast<int64_t *>(p);
  }
  *out = g_noalloc_plan_addr[dev];
  *device = dev;
  return LAPIS_OK;
}

extern "C" int lapis_b200_spmv_f64_noalloc(int idx_bytes, int64_t nrows, int64_t ncols, const void *d_pos,
                                           const void *d_crd, const double *d_val, const double *d_x, double *d_y,
                                           int accumulate, void *stream) {
  clear_error();
  if (idx_bytes != 4 && idx_bytes != 8) return fail(LAPIS_EBADARG, "spmv_noalloc: idx_bytes must be 4 or 8");
  if (nrows < 0 || ncols < 0) return fail(LAPIS_EBADSHAPE, "spmv_noalloc: negative dimension");
  if (d_pos == nullptr) return fail(LAPIS_EBADARG, "spmv_noalloc: pos is null");
  if ((reinterpret_cast<uintptr_t>(d_val) % 16) || (reinterpret_cast<uintptr_t>(d_crd) % 16))
    return fail(LAPIS_EBADARG, "spmv_noalloc: val and crd must be 16-byte aligned");
  if (nrows == 0) return LAPIS_OK;
  if (d_y == nullptr) return fail(LAPIS_EBADARG, "spmv_noalloc: y is null");
  cudaStream_t st = as_stream(stream);
  int64_t *plan = nullptr;
  int dev = 0;
  LAPIS_TRY(noalloc_plan_ptr(&plan, &dev));

  // pos[0] and pos[nrows] (copied into host variables: no allocation involved)
  int64_t ends[2] = {0, 0};
  if (idx_bytes == 4) {
    int32_t e32[2] = {0, 0};
    LAPIS_CUDA_TRY(cudaMemcpyAsync(&e32[0], d_pos, 4, cudaMemcpyDeviceToHost, st));
    LAPIS_CUDA_TRY(cudaMemcpyAsync(&e32[1], static_cast<const int32_t *>(d_pos) + nrows, 4, cudaMemcpyDeviceToHost, st));
    LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
    ends[0] = e32[0];
    ends[1] = e32[1];
  } else {
    LAPIS_CUDA_TRY(cudaMemcpyAsync(&ends[0], d_pos, 8, cudaMemcpyDeviceToHost, st));
    LAPIS_CUDA_TRY(cudaMemcpyAsync(&ends[1], static_cast<const int64_t *>(d_pos) + nrows, 8, cudaMemcpyDeviceToHost, st));
    LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  }
  if (ends[1] < ends[0] || ends[0] < 0) return fail(LAPIS_EBADSHAPE, "spmv_noalloc: pos is not non-decreasing");
  const int64_t nnz = ends[1] - ends[0];
  if (nnz > 0 && (d_crd == nullptr || d_val == nullptr || d_x == nullptr))
    return fail(LAPIS_EBADARG, "spmv_noalloc: crd/val/x null");
  int64_t nblk = (ends[1] - (ends[0] & ~(int64_t)3) + SPMV_TILE - 1) / SPMV_TILE;
  if (nblk < 1) nblk = 1;
  if (nblk > NOALLOC_MAX_TILES)
    return fail(LAPIS_ETOOBIG,
                "spmv_noalloc: %lld stored entries starting at offset %lld need %lld chunks of %d, the fixed plan "
                "buffer holds %lld (at most %lld entries when pos[0] is a multiple of 4, up to 3 fewer otherwise); "
                "use lapis_b200_csr_create + lapis_b200_spmv_f64 for larger matrices",
                (long long)nnz, (long long)ends[0], (long long)nblk, SPMV_TILE, (long long)NOALLOC_MAX_TILES,
                (long long)(NOALLOC_MAX_TILES * (int64_t)SPMV_TILE));

  lapis_b200_csr h;
  h.idx_bytes = idx_bytes;
  h.nrows = nrows;
  h.ncols = ncols;
  h.nnz = nnz;
  h.base = ends[0];
  h.pos = d_pos;
  h.crd = d_crd;
  h.val = d_val;
  h.nblk = nblk;
  h.blk_row = plan;
  h.blk_partial = nullptr;
  h.carry = reinterpret_cast<double *>(plan + NOALLOC_MAX_TILES + 1);
  h.tuned_threads = h.tuned_minb = h.tuned_hint = 0;
  h.max_row_len = -1;
  h.device = dev;
  h.walk_plan = nullptr;
  h.walk_carry = nullptr;
  h.walk_nblk = 0;
  h.walk_tile = 0;
  const unsigned pgrid = (unsigned)((nblk + 1 + 255) / 256);
  if (idx_bytes == 4)
    spmv_plan_kernel<int32_t><<<pgrid, 256, 0, st>>>(static_cast<const int32_t *>(d_pos), nrows, nblk, plan);
  else
    spmv_plan_kernel<int64_t><<<pgrid, 256, 0, st>>>(static_cast<const int64_t *>(d_pos), nrows, nblk, plan);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return spmv_launch(&h, d_x, d_y, accumulate, nullptr, nullptr, nullptr, st);
}
