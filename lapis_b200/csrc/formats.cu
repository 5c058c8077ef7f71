// Neighbouring sparse formats of the same front end: batched SpMM over a CSRV tensor and SpMM over a DCSR
// matrix.
//
// CSRV (examples/bspmm.py:14-52 in the LAPIS project): a 3-D tensor A[n1, n2, nh] stored as
// (dense, compressed, dense) -- a CSR pattern (pos, crd) whose stored entry j carries a fiber of nh values
// val[j*nh .. j*nh+nh).  out[n1, dh, nh] = sum_n2 A[n1, n2, nh] * B[n2, dh, nh], fp32, all batches share the
// pattern.  The emitted loop nest is rows -> stored entries -> dh -> nh with the two inner loops dense and
// parallel, so every output element is updated in place once per stored entry, in ascending entry order:
// out = a*b + out.  One thread owns an output element for the whole row here, which keeps that order.
//
// DCSR (examples/spmm_dcsr_opdsl.py:46-101, 137-160): both levels compressed -- p1 = {0, stored rows},
// i1 = their row numbers, p2 / i2 / val a CSR over the stored rows only.  C[i1[r], :] += sum_j val[j] *
// B[i2[j], :] in ascending j, updated in place; rows that are not stored are not touched.  i1 ascends (a number
// may repeat).
#include <cstdint>

#include "common.h"

namespace lapis_b200 {

constexpr int BSPMM_THREADS = 128;

// GROUP threads share one row (GROUP = 32: four rows per block; GROUP = 128: one); each thread owns EPT
// output elements per pass, GROUP apart, so that B rows and C rows are read and written coalesced.
template <typename I, int GROUP, int EPT>
__global__ void __launch_bounds__(BSPMM_THREADS)
bspmm_csrv_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const float *__restrict__ val, int64_t nrows,
                  int64_t nh, int64_t E, const float *__restrict__ B, float *__restrict__ C, int accumulate) {
  const int g = threadIdx.x % GROUP;
  const int64_t row = (int64_t)blockIdx.x * (BSPMM_THREADS / GROUP) + threadIdx.x / GROUP;
  if (row >= nrows) return;
  const int64_t lo = (int64_t)pos[row], hi = (int64_t)pos[row + 1];
  float *crow = C + row * E;
  for (int64_t e0 = 0; e0 < E; e0 += (int64_t)GROUP * EPT) {
    int64_t e[EPT];
    int fiber[EPT];
    float acc[EPT];
#pragma unroll
    for (int q = 0; q < EPT; ++q) {
      e[q] = e0 + g + (int64_t)q * GROUP;
      fiber[q] = (int)(e[q] % nh);
      acc[q] = (accumulate && e[q] < E) ? crow[e[q]] : 0.0f;
    }
    int64_t j = lo;
    for (; j + 1 < hi; j += 2) {  // two stored entries in flight; the adds stay in entry order
      const int64_t c0 = (int64_t)crd[j], c1 = (int64_t)crd[j + 1];
      float a0[EPT], b0[EPT], a1[EPT], b1[EPT];
#pragma unroll
      for (int q = 0; q < EPT; ++q) {
        const bool in = e[q] < E;
        a0[q] = in ? val[j * nh + fiber[q]] : 0.0f;
        b0[q] = in ? __ldg(B + c0 * E + e[q]) : 0.0f;
        a1[q] = in ? val[(j + 1) * nh + fiber[q]] : 0.0f;
        b1[q] = in ? __ldg(B + c1 * E + e[q]) : 0.0f;
      }
#pragma unroll
      for (int q = 0; q < EPT; ++q) {
        acc[q] = __fadd_rn(__fmul_rn(a0[q], b0[q]), acc[q]);
        acc[q] = __fadd_rn(__fmul_rn(a1[q], b1[q]), acc[q]);
      }
    }
    if (j < hi) {
      const int64_t c0 = (int64_t)crd[j];
#pragma unroll
      for (int q = 0; q < EPT; ++q)
        if (e[q] < E) acc[q] = __fadd_rn(__fmul_rn(val[j * nh + fiber[q]], __ldg(B + c0 * E + e[q])), acc[q]);
    }
#pragma unroll
    for (int q = 0; q < EPT; ++q)
      if (e[q] < E) crow[e[q]] = acc[q];
  }
}

// The same with 16-byte accesses, for fibers whose length is a multiple of four (and 16-byte aligned arrays): a
// thread owns four consecutive output elements, which lie in one fiber, so one float4 of the entry's values
// meets one float4 of the B row.  Four stored entries are in flight per thread; the adds stay in entry order.
template <typename I, int GROUP>
__global__ void __launch_bounds__(BSPMM_THREADS)
bspmm_csrv_vec4_kernel(const I *__restrict__ pos, const I *__restrict__ crd, const float4 *__restrict__ val4,
                       int64_t nrows, int nh4, int64_t E4, const float4 *__restrict__ B4, float4 *__restrict__ C4,
                       int accumulate) {
  const int g = threadIdx.x % GROUP;
  const int64_t row = (int64_t)blockIdx.x * (BSPMM_THREADS / GROUP) + threadIdx.x / GROUP;
  if (row >= nrows) return;
  const int64_t lo = (int64_t)pos[row], hi = (int64_t)pos[row + 1];
  float4 *crow = C4 + row * E4;
  for (int64_t f = g; f < E4; f += GROUP) {  // f: index of this thread's float4 inside the row
    const float4 *vcol = val4 + (f % nh4);   // + j * nh4 selects the entry
    const float4 *bcol = B4 + f;             // + crd[j] * E4 selects the row of B
    float4 acc = accumulate ? crow[f] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    int64_t j = lo;
    for (; j + 3 < hi; j += 4) {
      float4 a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t c = (int64_t)crd[j + u];
        a[u] = __ldg(vcol + (j + u) * nh4);
        b[u] = __ldg(bcol + c * E4);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        acc.x = __fadd_rn(__fmul_rn(a[u].x, b[u].x), acc.x);
        acc.y = __fadd_rn(__fmul_rn(a[u].y, b[u].y), acc.y);
        acc.z = __fadd_rn(__fmul_rn(a[u].z, b[u].z), acc.z);
        acc.w = __fadd_rn(__fmul_rn(a[u].w, b[u].w), acc.w);
      }
    }
    for (; j < hi; ++j) {
      const float4 a = __ldg(vcol + j * nh4), b = __ldg(bcol + (int64_t)crd[j] * E4);
      acc.x = __fadd_rn(__fmul_rn(a.x, b.x), acc.x);
      acc.y = __fadd_rn(__fmul_rn(a.y, b.y), acc.y);
      acc.z = __fadd_rn(__fmul_rn(a.z, b.z), acc.z);
      acc.w = __fadd_rn(__fmul_rn(a.w, b.w), acc.w);
    }
    crow[f] = acc;
  }
}

// One warp per stored row, 16-byte accesses: a lane owns two adjacent columns of every 64-column tile and
// keeps four rows of B in flight (k even, B and C 16-byte aligned).
template <typename I>
__global__ void __launch_bounds__(256)
spmm_dcsr_vec2_kernel(const I *__restrict__ i1, const I *__restrict__ p2, const I *__restrict__ i2,
                      const double *__restrict__ val, int64_t nstored, int64_t k2, const double2 *__restrict__ B2,
                      double2 *__restrict__ C2) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= nstored) return;
  const I rowid = i1[r];
  if (r > 0 && i1[r - 1] == rowid) return;  // a repeated row number: the first warp of the run takes all of it
  int64_t rend = r + 1;
  while (rend < nstored && i1[rend] == rowid) ++rend;
  const int64_t lo = (int64_t)p2[r], hi = (int64_t)p2[rend];
  double2 *crow = C2 + (int64_t)rowid * k2;
  for (int64_t c = lane; c < k2; c += 32) {
    double2 acc = crow[c];
    int64_t j = lo;
    for (; j + 3 < hi; j += 4) {
      double a[4];
      double2 b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a[u] = __ldg(val + j + u);
        b[u] = __ldg(B2 + (int64_t)i2[j + u] * k2 + c);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        acc.x = __dadd_rn(acc.x, __dmul_rn(a[u], b[u].x));
        acc.y = __dadd_rn(acc.y, __dmul_rn(a[u], b[u].y));
      }
    }
    for (; j < hi; ++j) {
      const double a = __ldg(val + j);
      const double2 b = __ldg(B2 + (int64_t)i2[j] * k2 + c);
      acc.x = __dadd_rn(acc.x, __dmul_rn(a, b.x));
      acc.y = __dadd_rn(acc.y, __dmul_rn(a, b.y));
    }
    crow[c] = acc;
  }
}

// One warp per stored row; a lane owns the columns lane, lane + 32, ...
template <typename I>
__global__ void __launch_bounds__(256)
spmm_dcsr_kernel(const I *__restrict__ i1, const I *__restrict__ p2, const I *__restrict__ i2,
                 const double *__restrict__ val, int64_t nstored, int64_t k, const double *__restrict__ B,
                 double *__restrict__ C) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= nstored) return;
  // A row number may be listed more than once (examples/spmm_dcsr_opdsl.py:140-141 lists one twice, the second
  // time with no entries): equal numbers are adjacent, the first warp of such a run takes the whole run.
  const I rowid = i1[r];
  if (r > 0 && i1[r - 1] == rowid) return;
  int64_t rend = r + 1;
  while (rend < nstored && i1[rend] == rowid) ++rend;
  const int64_t lo = (int64_t)p2[r], hi = (int64_t)p2[rend];
  double *crow = C + (int64_t)rowid * k;
  for (int64_t c0 = 0; c0 < k; c0 += 128) {
    int64_t col[4];
    double acc[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      col[q] = c0 + lane + 32 * q;
      acc[q] = col[q] < k ? crow[col[q]] : 0.0;
    }
    for (int64_t j = lo; j < hi; ++j) {
      const double a = val[j];
      const double *brow = B + (int64_t)i2[j] * k;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (col[q] < k) acc[q] = __dadd_rn(acc[q], __dmul_rn(a, __ldg(brow + col[q])));
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (col[q] < k) crow[col[q]] = acc[q];
  }
}

template <typename I>
static void launch_bspmm(const void *pos, const void *crd, const float *val, int64_t nrows, int64_t nh, int64_t E,
                         const float *B, float *C, int accumulate, cudaStream_t st) {
  const I *p = static_cast<const I *>(pos), *c = static_cast<const I *>(crd);
  const bool vec4 = nh % 4 == 0 && nh / 4 <= 0x7fffffff &&
                    ((reinterpret_cast<uintptr_t>(val) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 == 0);
  if (vec4) {
    const float4 *v4 = reinterpret_cast<const float4 *>(val), *B4 = reinterpret_cast<const float4 *>(B);
    float4 *C4 = reinterpret_cast<float4 *>(C);
    if (E / 4 <= 32)
      bspmm_csrv_vec4_kernel<I, 32><<<(unsigned)((nrows + 3) / 4), BSPMM_THREADS, 0, st>>>(p, c, v4, nrows, (int)(nh / 4), E / 4,
                                                                                          B4, C4, accumulate);
    else
      bspmm_csrv_vec4_kernel<I, 128><<<(unsigned)nrows, BSPMM_THREADS, 0, st>>>(p, c, v4, nrows, (int)(nh / 4), E / 4, B4, C4,
                                                                                accumulate);
    return;
  }
  if (E <= 128) {
    const unsigned grid = (unsigned)((nrows + 3) / 4);
    bspmm_csrv_kernel<I, 32, 4><<<grid, BSPMM_THREADS, 0, st>>>(p, c, val, nrows, nh, E, B, C, accumulate);
  } else {
    bspmm_csrv_kernel<I, 128, 4><<<(unsigned)nrows, BSPMM_THREADS, 0, st>>>(p, c, val, nrows, nh, E, B, C, accumulate);
  }
}

}  // namespace lapis_b200

using namespace lapis_b200;

extern "C" int lapis_b200_bspmm_csrv_f32(int idx_bytes, int64_t n1, int64_t n2, int64_t nh, int64_t dh, const void *d_pos,
                                         const void *d_crd, const float *d_val, const float *d_B, float *d_C,
                                         int accumulate, void *stream) {
  clear_error();
  if (idx_bytes != 4 && idx_bytes != 8) return fail(LAPIS_EBADARG, "bspmm: idx_bytes must be 4 or 8");
  if (n1 < 0 || n2 < 0 || nh < 0 || dh < 0) return fail(LAPIS_EBADSHAPE, "bspmm: negative dimension");
  if (n1 > 0x7fffffffLL * 4) return fail(LAPIS_ETOOBIG, "bspmm: too many rows for one launch");
  const int64_t E = dh * nh;
  if (n1 == 0 || E == 0) return LAPIS_OK;
  if (d_pos == nullptr || d_C == nullptr) return fail(LAPIS_EBADARG, "bspmm: null operand");
  cudaStream_t st = as_stream(stream);
  if (idx_bytes == 4)
    launch_bspmm<int32_t>(d_pos, d_crd, d_val, n1, nh, E, d_B, d_C, accumulate, st);
  else
    launch_bspmm<int64_t>(d_pos, d_crd, d_val, n1, nh, E, d_B, d_C, accumulate, st);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

extern "C" int lapis_b200_spmm_dcsr_f64(int idx_bytes, int64_t nrows, int64_t ncols, int64_t nstored, int64_t k,
                                        const void *d_i1, const void *d_p2, const void *d_i2, const double *d_val,
                                        const double *d_B, double *d_C, void *stream) {
  clear_error();
  if (idx_bytes != 4 && idx_bytes != 8) return fail(LAPIS_EBADARG, "spmm_dcsr: idx_bytes must be 4 or 8");
  if (nrows < 0 || ncols < 0 || nstored < 0 || k < 0)
    return fail(LAPIS_EBADSHAPE, "spmm_dcsr: bad dimensions");
  if (nstored == 0 || k == 0) return LAPIS_OK;
  if (d_i1 == nullptr || d_p2 == nullptr || d_C == nullptr) return fail(LAPIS_EBADARG, "spmm_dcsr: null operand");
  cudaStream_t st = as_stream(stream);
  const unsigned grid = (unsigned)((nstored + 7) / 8);
  if (k % 2 == 0 && (reinterpret_cast<uintptr_t>(d_B) | reinterpret_cast<uintptr_t>(d_C)) % 16 == 0) {
    const double2 *B2 = reinterpret_cast<const double2 *>(d_B);
    double2 *C2 = reinterpret_cast<double2 *>(d_C);
    if (idx_bytes == 4)
      spmm_dcsr_vec2_kernel<int32_t><<<grid, 256, 0, st>>>(static_cast<const int32_t *>(d_i1), static_cast<const int32_t *>(d_p2),
                                                           static_cast<const int32_t *>(d_i2), d_val, nstored, k / 2, B2, C2);
    else
      spmm_dcsr_vec2_kernel<int64_t><<<grid, 256, 0, st>>>(static_cast<const int64_t *>(d_i1), static_cast<const int64_t *>(d_p2),
                                                           static_cast<const int64_t *>(d_i2), d_val, nstored, k / 2, B2, C2);
    LAPIS_CUDA_TRY(cudaGetLastError());
    return LAPIS_OK;
  }
  if (idx_bytes == 4)
    spmm_dcsr_kernel<int32_t><<<grid, 256, 0, st>>>(static_cast<const int32_t *>(d_i1), static_cast<const int32_t *>(d_p2),
                                                    static_cast<const int32_t *>(d_i2), d_val, nstored, k, d_B, d_C);
  else
    spmm_dcsr_kernel<int64_t><<<grid, 256, 0, st>>>(static_cast<const int64_t *>(d_i1), static_cast<const int64_t *>(d_p2),
                                                    static_cast<const int64_t *>(d_i2), d_val, nstored, k, d_B, d_C);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}
