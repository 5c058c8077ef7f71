// Dense and batched fp32 matmul for sm_100a:  C[b] = C_in[b] + A[b] B[b].
//
// Replaces the loop nest the LAPIS pipeline makes of linalg.matmul /
// linalg.batch_matmul (tests/Dialect/Kokkos/linalg_to_loops_3.mlir.gold:6-20, from
// mlir/lib/Dialect/Kokkos/Transforms/DenseLinalgToParallelLoops.cpp:309-348): one
// output element per Kokkos thread, each reading a row of A and a strided column
// of B from global memory, no reuse.
//
// Two paths, chosen by shape only (no fallback between them at run time):
//   * general shapes: a shared-memory tiled kernel on the fp32 pipes that keeps
//     the reference's arithmetic exactly -- k ascending, separate multiply and add,
//     C_in joined last -- so small and ragged problems (the 8x7x9 and 64x5x5 cases
//     of examples/gemm_no_alloc.py and examples/batched_gemm_no_alloc.py) are
//     bit-identical to the sequential loop.
//   * tile-aligned shapes (M, N multiples of 128, K of 32): the tcgen05 kernel in
//     gemm_tcgen05.cu, fp32 emulated with three TF32 products.
#include "common.h"

namespace lapis_b200 {

int bgemm_tcgen05_supported(int64_t batch, int64_t M, int64_t N, int64_t K);
int bgemm_tcgen05_launch(int64_t batch, int64_t M, int64_t N, int64_t K, const float *A, const float *B, float *C,
                         cudaStream_t st);

constexpr int SG_TILE = 32;  // output tile edge
constexpr int SG_K = 32;     // k-slab staged per step

__global__ void __launch_bounds__(SG_TILE * SG_TILE / 4)
bgemm_simt_kernel(int64_t batch, int64_t M, int64_t N, int64_t K, const float *__restrict__ A0,
                  const float *__restrict__ B0, float *__restrict__ C0) {
  // 256 threads; thread (ty, tx) owns C[row0 + ty*2 + {0,1}, col0 + tx + {0,16}].
  __shared__ float sA[SG_TILE][SG_K + 1];
  __shared__ float sB[SG_K][SG_TILE + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t row0 = (int64_t)blockIdx.y * SG_TILE, col0 = (int64_t)blockIdx.x * SG_TILE;
  for (int64_t b = blockIdx.z; b < batch; b += gridDim.z) {
  const float *A = A0 + b * M * K;
  const float *B = B0 + b * K * N;
  float *C = C0 + b * M * N;
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int64_t k0 = 0; k0 < K; k0 += SG_K) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e >> 5, c = e & 31;
      const int64_t gr = row0 + r, gk = k0 + c;
      sA[r][c] = (gr < M && gk < K) ? A[gr * K + gk] : 0.f;
      const int64_t gkb = k0 + r, gc = col0 + c;
      sB[r][c] = (gkb < K && gc < N) ? B[gkb * N + gc] : 0.f;
    }
    __syncthreads();
    const int kmax = (int)((K - k0) < SG_K ? (K - k0) : SG_K);
    for (int k = 0; k < kmax; ++k) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(sA[ty * 2 + i][k], sB[k][tx + 16 * j]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t gr = row0 + ty * 2 + i, gc = col0 + tx + 16 * j;
      if (gr < M && gc < N) C[gr * N + gc] = __fadd_rn(acc[i][j], C[gr * N + gc]);
    }
  }
}

}  // namespace lapis_b200

using namespace lapis_b200;

extern "C" int lapis_b200_bgemm_f32(int64_t batch, int64_t M, int64_t N, int64_t K, const float *d_A, const float *d_B,
                                    float *d_C, void *stream) {
  clear_error();
  if (batch < 0 || M < 0 || N < 0 || K < 0) return fail(LAPIS_EBADSHAPE, "bgemm: negative dimension");
  if (batch == 0 || M == 0 || N == 0) return LAPIS_OK;
  if (d_C == nullptr || (K > 0 && (d_A == nullptr || d_B == nullptr))) return fail(LAPIS_EBADARG, "bgemm: null operand");
  cudaStream_t st = as_stream(stream);
  // the tensor-core kernel moves its operands with TMA, which needs 16-byte aligned bases; other pointers (a
  // slice of a larger tensor, say) take the general-shape kernel, which has no alignment rule
  const bool aligned = ((reinterpret_cast<uintptr_t>(d_A) | reinterpret_cast<uintptr_t>(d_B) | reinterpret_cast<uintptr_t>(d_C)) % 16) == 0;
  if (aligned && bgemm_tcgen05_supported(batch, M, N, K)) return bgemm_tcgen05_launch(batch, M, N, K, d_A, d_B, d_C, st);
  dim3 grid((unsigned)((N + SG_TILE - 1) / SG_TILE), (unsigned)((M + SG_TILE - 1) / SG_TILE),
            (unsigned)(batch < 65535 ? batch : 65535));
  if (grid.y > 65535) return fail(LAPIS_ETOOBIG, "bgemm: M too large for the general-shape kernel");
  bgemm_simt_kernel<<<grid, 256, 0, st>>>(batch, M, N, K, d_A, d_B, d_C);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}
