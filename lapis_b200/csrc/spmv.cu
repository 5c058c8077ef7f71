// CSR SpMV and SpMM for sm_100a.
//
// Replaces the loop the LAPIS emitter prints for `linalg.matvec` on a CSR operand
// (tests/Dialect/Kokkos/loop_mapping_2.mlir.gold:12-37; emitted by
// mlir/lib/Target/KokkosCpp/TranslateToKokkosCpp.cpp:1966-2064 and :1692-1845):
// one row per Kokkos thread with a vector length taken from the *average* row
// length.  That shape streams val/crd uncoalesced for short rows and serialises
// long ones.  Here the nonzeros are the unit of work instead:
//
//   * The nnz range is cut into tiles of SPMV_TILE entries.  Thread block b owns
//     the rows whose start offset falls into tile b (found once per matrix by a
//     binary-search kernel; 8 bytes of plan per block).  A block therefore
//     streams ~SPMV_TILE consecutive (val, crd) pairs with 16-byte loads that are
//     fully coalesced whatever the row lengths are, gathers x through the
//     read-only path, and parks the products in shared memory.
//   * The rows overlapping the tile are then reduced out of shared memory by
//     groups of L lanes (L = 1..32 chosen per tile from its average row length)
//     with warp shuffles.  A row longer than a tile is carried from tile to tile
//     inside the block; no atomics, so results are run-to-run identical.
//
// Arithmetic: products and sums use explicit round-to-nearest multiplies and adds
// (no FMA contraction), as the emitted code has separate arith.mulf / arith.addf.
// The summation order inside a row differs from the sequential CPU order when
// L > 1 (documented tolerance 1e-12 of the row's magnitude); with L == 1 the
// result is bit-identical to the sequential order.
#include "common.h"

namespace lapis_b200 {

constexpr int SPMV_THREADS = 256;
constexpr int SPMV_TILE = 2048;       // nonzeros per tile (products staged in 16 KB of shared memory)
constexpr int SPMV_POS_CACHE = 1024;  // row offsets staged per block; further rows read global memory

// ---------------------------------------------------------------------------
// Plan: blk_row[b] = first row r in [0, nrows] with pos[r] >= pos[0] + b*TILE.
// ---------------------------------------------------------------------------
template <typename I>
__global__ void spmv_plan_kernel(const I *__restrict__ pos, int64_t nrows, int64_t nblk,
                                 int64_t *__restrict__ blk_row) {
  int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b > nblk) return;
  if (b == nblk) {
    blk_row[b] = nrows;
    return;
  }
  const int64_t target = (int64_t)pos[0] + b * (int64_t)SPMV_TILE;
  int64_t lo = 0, hi = nrows;
  while (lo < hi) {
    int64_t mid = lo + ((hi - lo) >> 1);
    if ((int64_t)pos[mid] < target)
      lo = mid + 1;
    else
      hi = mid;
  }
  blk_row[b] = lo;
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

// Reduces the rows [ra, rb] that overlap the current tile out of s_prod with L
// lanes per row.  Returns this thread's contribution to the fused dot product.
template <typename I, int L, bool FUSE_DOT>
__device__ __forceinline__ double spmv_reduce_tile(
    const I *__restrict__ pos, const I *s_pos, int64_t r0, int ncached, const double *s_prod,
    int64_t ra, int64_t rb, int64_t tile_lo, int64_t tile_hi, double carry_in, double *carry_out,
    double *__restrict__ y, int accumulate, const double *__restrict__ dotvec) {
  const int tid = threadIdx.x;
  const int grp = tid / L, lane = tid % L;
  constexpr int NGRP = SPMV_THREADS / L;
  double dot_local = 0.0;
  for (int64_t rbase = ra; rbase <= rb; rbase += NGRP) {
    const int64_t r = rbase + grp;
    const bool valid = r <= rb;
    double acc = 0.0, yin = 0.0;
    int64_t s = 0, e = 0;
    if (valid) {
      const int64_t i = r - r0;
      s = (i < ncached) ? (int64_t)s_pos[i] : (int64_t)pos[r];
      e = (i + 1 < ncached) ? (int64_t)s_pos[i + 1] : (int64_t)pos[r + 1];
      if (accumulate && lane == 0 && e <= tile_hi) yin = y[r];
      const int64_t sc = s > tile_lo ? s : tile_lo;
      const int64_t ec = e < tile_hi ? e : tile_hi;
      const double *p = s_prod - tile_lo;
#pragma unroll 4
      for (int64_t j = sc + lane; j < ec; j += L) acc = __dadd_rn(acc, p[j]);
    }
#pragma unroll
    for (int off = L / 2; off > 0; off >>= 1) acc = __dadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if (valid && lane == 0) {
      if (s < tile_lo) acc = __dadd_rn(carry_in, acc);  // the row began in an earlier tile
      if (e > tile_hi) {
        *carry_out = acc;  // continues in the next tile (at most one such row per tile)
      } else {
        const double out = __dadd_rn(acc, yin);
        y[r] = out;
        if (FUSE_DOT) dot_local = __dadd_rn(dot_local, __dmul_rn(out, dotvec[r]));
      }
    }
  }
  return dot_local;
}

// y = (accumulate ? y : 0) + A x.  With FUSE_DOT, blk_partial[b] receives this
// block's part of sum_r y[r] * dotvec[r] (the p.Ap of a PCG iteration).
template <typename I, bool FUSE_DOT>
__global__ void __launch_bounds__(SPMV_THREADS, 4)
spmv_stream_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const double *__restrict__ val,
                   const int64_t *__restrict__ blk_row, int64_t nnz_end, const double *__restrict__ x,
                   double *__restrict__ y, int accumulate, const double *__restrict__ dotvec,
                   double *__restrict__ blk_partial, const int *__restrict__ skip_flag) {
  __shared__ __align__(16) double s_prod[SPMV_TILE];
  __shared__ I s_pos[SPMV_POS_CACHE + 1];
  __shared__ double s_carry[2];
  __shared__ double s_red[SPMV_THREADS / 32];
  using Pair = typename IndexPair<I>::type;

  if (skip_flag != nullptr && *skip_flag != 0) return;

  const int tid = threadIdx.x;
  const int64_t r0 = blk_row[blockIdx.x], r1 = blk_row[blockIdx.x + 1];
  double dot_local = 0.0;

  if (r0 < r1) {
    const int64_t nrows_b = r1 - r0;
    const int ncached = (int)(nrows_b < SPMV_POS_CACHE ? nrows_b : SPMV_POS_CACHE) + 1;
    for (int i = tid; i < ncached; i += SPMV_THREADS) s_pos[i] = pos[r0 + i];
    const int64_t lo = (int64_t)pos[r0], hi = (int64_t)pos[r1];

    int64_t tile_lo = lo & ~(int64_t)1;  // even offset: 16-byte aligned val/crd pairs
    int64_t ra = r0;                     // first row that can overlap the current tile
    int parity = 0;
    if (tid == 0) s_carry[0] = 0.0;
    do {
      const bool last = tile_lo + SPMV_TILE >= hi;
      const int64_t tile_hi = last ? hi : tile_lo + SPMV_TILE;

      // ---- stream phase: coalesced 16-byte loads, gather x, stage products --------
      double2 v[SPMV_TILE / (2 * SPMV_THREADS)];
      Pair c[SPMV_TILE / (2 * SPMV_THREADS)];
#pragma unroll
      for (int k = 0; k < SPMV_TILE / (2 * SPMV_THREADS); ++k) {
        const int64_t j = tile_lo + 2 * (int64_t)(tid + k * SPMV_THREADS);
        v[k] = make_double2(0.0, 0.0);
        c[k].x = 0;
        c[k].y = 0;
        if (j < tile_hi) {
          if (j + 1 < nnz_end) {
            v[k] = __ldcs(reinterpret_cast<const double2 *>(val + j));
            c[k] = __ldcs(reinterpret_cast<const Pair *>(crd + j));
          } else {  // the very last entry of the arrays
            v[k].x = __ldcs(val + j);
            c[k].x = __ldcs(crd + j);
          }
        }
      }
#pragma unroll
      for (int k = 0; k < SPMV_TILE / (2 * SPMV_THREADS); ++k) {
        const int64_t j = tile_lo + 2 * (int64_t)(tid + k * SPMV_THREADS);
        if (j < tile_hi) {
          double2 p;
          p.x = __dmul_rn(v[k].x, __ldg(x + c[k].x));
          p.y = __dmul_rn(v[k].y, __ldg(x + c[k].y));
          *reinterpret_cast<double2 *>(s_prod + (j - tile_lo)) = p;
        }
      }
      __syncthreads();  // products and s_pos visible

      // ---- rows overlapping this tile ----------------------------------------------
      int64_t rb;
      if (last) {
        rb = r1 - 1;
      } else {  // last row whose start offset is below tile_hi
        int64_t a = ra, b = r1;
        while (a < b) {
          const int64_t mid = a + ((b - a) >> 1);
          const int64_t i = mid - r0;
          const int64_t pm = (i < ncached) ? (int64_t)s_pos[i] : (int64_t)pos[mid];
          if (pm < tile_hi)
            a = mid + 1;
          else
            b = mid;
        }
        rb = a - 1;
      }
      const int64_t nrows_t = rb - ra + 1;
      const int64_t avg = (tile_hi - tile_lo) / (nrows_t > 0 ? nrows_t : 1);
      const double carry_in = s_carry[parity];
      double *carry_out = &s_carry[parity ^ 1];
#define LAPIS_REDUCE(LANES)                                                                          \
  dot_local = __dadd_rn(dot_local, spmv_reduce_tile<I, LANES, FUSE_DOT>(                             \
                                       pos, s_pos, r0, ncached, s_prod, ra, rb, tile_lo, tile_hi,    \
                                       carry_in, carry_out, y, accumulate, dotvec))
      if (avg <= 2)
        LAPIS_REDUCE(1);
      else if (avg <= 4)
        LAPIS_REDUCE(2);
      else if (avg <= 8)
        LAPIS_REDUCE(4);
      else if (avg <= 16)
        LAPIS_REDUCE(8);
      else if (avg <= 32)
        LAPIS_REDUCE(16);
      else
        LAPIS_REDUCE(32);
#undef LAPIS_REDUCE
      if (!last) {
        // the row that crosses tile_hi (if any) is reduced again in the next tile
        const int64_t i = rb + 1 - r0;
        const int64_t e = (i < ncached) ? (int64_t)s_pos[i] : (int64_t)pos[rb + 1];
        ra = e > tile_hi ? rb : rb + 1;
      }
      parity ^= 1;
      tile_lo += SPMV_TILE;
      __syncthreads();  // s_prod is overwritten by the next tile; carry_out visible
      if (last) break;
    } while (true);
  }

  if (FUSE_DOT) {
    const double t = block_sum(dot_local, s_red);
    if (tid == 0) blk_partial[blockIdx.x] = t;
  }
}

// ---------------------------------------------------------------------------
// SpMM: C[r, :] = (accumulate ? C[r, :] : 0) + sum_j val[j] * B[crd[j], :].
// One warp per row; lane l owns columns {2l, 2l+1} of a 64-column panel, so a B
// row is fetched as one coalesced 512-byte request and every output element is
// summed in ascending j by a single lane: bit-identical to the sequential row
// loop (examples/bspmm.py:15-23, spmm_dcsr_opdsl.py:132-135 outer-loop-only
// parallelism).  Eight B rows are in flight per warp.
// ---------------------------------------------------------------------------
constexpr int SPMM_WARPS = 8;
constexpr int SPMM_UNROLL = 8;

template <typename I, bool VEC2>
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

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
template <typename I>
static int launch_spmv(const lapis_b200_csr *h, const double *x, double *y, int accumulate,
                       const double *dotvec, double *blk_partial, const int *skip_flag,
                       cudaStream_t st) {
  const I *pos = static_cast<const I *>(h->pos);
  const I *crd = static_cast<const I *>(h->crd);
  const int64_t nnz_end = h->base + h->nnz;
  if (dotvec != nullptr)
    spmv_stream_kernel<I, true><<<(unsigned)h->nblk, SPMV_THREADS, 0, st>>>(
        pos, crd, h->val, h->blk_row, nnz_end, x, y, accumulate, dotvec, blk_partial, skip_flag);
  else
    spmv_stream_kernel<I, false><<<(unsigned)h->nblk, SPMV_THREADS, 0, st>>>(
        pos, crd, h->val, h->blk_row, nnz_end, x, y, accumulate, nullptr, nullptr, skip_flag);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

int spmv_launch(const lapis_b200_csr *h, const double *x, double *y, int accumulate,
                const double *dotvec, double *blk_partial, const int *skip_flag, cudaStream_t st) {
  if (h->nrows == 0) return LAPIS_OK;
  if (h->idx_bytes == 4)
    return launch_spmv<int32_t>(h, x, y, accumulate, dotvec, blk_partial, skip_flag, st);
  return launch_spmv<int64_t>(h, x, y, accumulate, dotvec, blk_partial, skip_flag, st);
}

template <typename I>
static int launch_spmm(const lapis_b200_csr *h, int64_t k, const double *B, double *C, int accumulate,
                       cudaStream_t st) {
  const I *pos = static_cast<const I *>(h->pos);
  const I *crd = static_cast<const I *>(h->crd);
  const unsigned grid = (unsigned)((h->nrows + SPMM_WARPS - 1) / SPMM_WARPS);
  const bool vec2 = (k % 2 == 0) && ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 == 0);
  if (vec2)
    spmm_row_kernel<I, true><<<grid, SPMM_WARPS * 32, 0, st>>>(pos, crd, h->val, h->nrows, k, B, C, accumulate);
  else
    spmm_row_kernel<I, false><<<grid, SPMM_WARPS * 32, 0, st>>>(pos, crd, h->val, h->nrows, k, B, C, accumulate);
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
  int64_t nblk = (nnz + SPMV_TILE - 1) / SPMV_TILE;
  if (nblk < 1) nblk = 1;
  if (nblk > 0x7fffffffLL) return fail(LAPIS_ETOOBIG, "csr_create: more than 2^31 tiles");

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
  h->device = dev;
  cudaError_t e = cudaMalloc(&h->blk_row, (size_t)(nblk + 1) * sizeof(int64_t));
  if (e == cudaSuccess) e = cudaMalloc(&h->blk_partial, (size_t)nblk * sizeof(double));
  if (e != cudaSuccess) {
    cudaFree(h->blk_row);
    delete h;
    return fail(LAPIS_ECUDA, "csr_create: cudaMalloc failed: %s", cudaGetErrorString(e));
  }
  const unsigned pgrid = (unsigned)((nblk + 1 + 255) / 256);
  if (idx_bytes == 4)
    spmv_plan_kernel<int32_t><<<pgrid, 256, 0, st>>>(static_cast<const int32_t *>(d_pos), nrows, nblk, h->blk_row);
  else
    spmv_plan_kernel<int64_t><<<pgrid, 256, 0, st>>>(static_cast<const int64_t *>(d_pos), nrows, nblk, h->blk_row);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    cudaFree(h->blk_row);
    cudaFree(h->blk_partial);
    delete h;
    return fail(LAPIS_ECUDA, "csr_create: plan kernel launch failed: %s", cudaGetErrorString(e));
  }
  *out = h;
  return LAPIS_OK;
}

extern "C" int lapis_b200_csr_destroy(lapis_b200_csr_t h) {
  clear_error();
  if (h == nullptr) return LAPIS_OK;
  cudaFree(h->blk_row);
  cudaFree(h->blk_partial);
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
constexpr int64_t NOALLOC_MAX_TILES = 1 << 18;  // 2 MiB of plan: matrices of up to 2^29 stored entries
static __device__ __align__(256) int64_t g_noalloc_plan[NOALLOC_MAX_TILES + 1];

// Device address of g_noalloc_plan per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel may use; cudaGetSymbolAddress returns the
// address in the device that is current when it is called.
static int64_t *g_noalloc_plan_addr[64] = {nullptr};

static int noalloc_plan_ptr(int64_t **out) {
  int dev = 0;
  LAPIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return lapis_b200::fail(LAPIS_EBADARG, "spmv_noalloc: device index %d not supported", dev);
  if (g_noalloc_plan_addr[dev] == nullptr) {
    void *p = nullptr;
    LAPIS_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_plan));
    g_noalloc_plan_addr[dev] = static_cast<int64_t *>(p);
  }
  *out = g_noalloc_plan_addr[dev];
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
  LAPIS_TRY(noalloc_plan_ptr(&plan));

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
  int64_t nblk = (nnz + SPMV_TILE - 1) / SPMV_TILE;
  if (nblk < 1) nblk = 1;
  if (nblk > NOALLOC_MAX_TILES)
    return fail(LAPIS_ETOOBIG,
                "spmv_noalloc: %lld stored entries exceed the fixed plan buffer (limit %lld entries); "
                "use lapis_b200_csr_create + lapis_b200_spmv_f64 for larger matrices",
                (long long)nnz, (long long)(NOALLOC_MAX_TILES * (int64_t)SPMV_TILE));

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
  h.device = 0;
  const unsigned pgrid = (unsigned)((nblk + 1 + 255) / 256);
  if (idx_bytes == 4)
    spmv_plan_kernel<int32_t><<<pgrid, 256, 0, st>>>(static_cast<const int32_t *>(d_pos), nrows, nblk, plan);
  else
    spmv_plan_kernel<int64_t><<<pgrid, 256, 0, st>>>(static_cast<const int64_t *>(d_pos), nrows, nblk, plan);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return spmv_launch(&h, d_x, d_y, accumulate, nullptr, nullptr, nullptr, st);
}
