// fp32 matmul on the 5th-generation tensor cores (tcgen05 + TMEM), fp32 emulated with
// three TF32 products:  C[b] = C_in[b] + A[b] B[b]  for tile-aligned shapes.
//
// The emitted loop nest (tests/Dialect/Kokkos/linalg_to_loops_3.mlir.gold:6-20) does one
// output element per Kokkos thread with no reuse.  Here one CTA owns a 128 x 128 tile of C,
// accumulated in tensor memory (128 lanes x 128 fp32 columns), and walks K in blocks of 32:
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A block (128 x 32, K-major,
//               128-byte swizzle) and the B block (32 x 128, N-major, as four 32 x 32 boxes,
//               128-byte swizzle with 32-byte atoms) into a 3-stage shared-memory ring,
//               completion on an mbarrier.
//   warps 2-5   split: x = hi + lo with hi = the TF32 the tensor core reads from the raw
//               fp32 (its top 19 bits) and lo = x - hi (exact), written to a second pair of
//               buffers; fence.proxy.async, then arrive.
//   warp 1      MMA issuer: per 8-wide k step three tcgen05.mma.kind::tf32 into the same
//               accumulator: hi*hi (issued as soon as TMA has landed, overlapping the split),
//               then lo*hi and hi*lo (the lo*lo term is below fp32 rounding);
//               tcgen05.commit releases the stage to the producer.
//   warps 6-9   epilogue: tcgen05.ld the accumulator, add C_in, store C.
//
// Blocks are persistent (one per SM) and walk the output tiles; tensor memory holds two
// accumulators, so the epilogue of one tile runs while the producer, split and MMA warps are
// already in the main loop of the next (for the batched 128^3 problems the epilogue traffic is
// as large as the operand traffic, so this overlap is what keeps HBM busy).
//
// The K loop of a tile is cut into segments of 1024: each segment is accumulated in tensor memory from zero and
// added to C by the epilogue with round-to-nearest adds, because the tensor core truncates when it adds to its
// accumulator and that error grows linearly with the length of the chain (K_SEGMENT below has the numbers).
//
// Every mbarrier wait is bounded: after WAIT_LIMIT polls the thread records an error code
// in a global flag and stops waiting, the block still frees its tensor memory and exits,
// and the host turns the flag into LAPIS_ECUDA.
#include <cuda.h>

#include <cstdlib>

#include "common.h"

namespace lapis_b200 {

namespace tc {

constexpr int BM = 128;
constexpr int THREADS = 320;  // producer, MMA issuer, 4 split warps, 4 epilogue warps
constexpr uint32_t WAIT_LIMIT = 1u << 22;
// k extent accumulated in tensor memory before the epilogue adds it to C.  Measured on 8192^3 with entries in
// [-1, 1): max error / max |C| = 6.3e-5 unsegmented, 1.5e-5 / 8.2e-6 / 4.4e-6 / 2.3e-6 with segments of
// 2048 / 1024 / 512 / 256 (it grows linearly with the segment: the tensor core truncates when it adds to the
// accumulator), at 237 / 233 / 227 / 216 / 187 TFLOP/s.  1024 keeps fp32 products within 1e-5 of |C|.
constexpr int K_SEGMENT = 1024;
constexpr int EPI_PITCH = 36;                      // floats per staged epilogue row (conflict-free float4 access)
constexpr int EPI_BYTES = 4 * 32 * EPI_PITCH * 4;  // one 32 x 32 staging tile per epilogue warp

// Tile configuration.  <128, 32, 3>: 128 x 128 tiles, k blocks of 32 (A rows of 128 B, 128-byte swizzle),
// three 64 KB stages -- used for the batched 128^3 problems and whenever N is not a multiple of 256.
// <256, 16, 4>: 128 x 256 tiles, k blocks of 16 (A rows of 64 B, 64-byte swizzle), four 48 KB stages --
// per MMA the tensor core reads 4 KB of A and 8 KB of B from shared memory for twice the flops, which
// matters because 3xTF32 from fp32 operands is shared-memory-bandwidth bound.
template <int BN_, int BK_, int STAGES_>
struct Cfg {
  static constexpr int BN = BN_, BK = BK_, STAGES = STAGES_;
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BK * BN * 4;
  static constexpr int BOX_BYTES = BK * 32 * 4;  // one B box: BK k-rows x 32 columns (128 B)
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators: the epilogue of a tile overlaps the next main loop
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + EPI_BYTES;
  // instruction descriptor: D = f32, A = B = tf32, A K-major, B MN-major, N = BN, M = 128
  static constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (0u << 15) | (1u << 16) |
                                    ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  // A rows are BK*4 bytes: 128-byte swizzle (layout type 2, 8-row groups 1024 B apart) or 64-byte swizzle
  // (layout type 4, 8-row groups 512 B apart)
  static constexpr uint64_t A_LAYOUT = BK == 32 ? 2 : 4;
  static constexpr uint64_t A_SBO = (8 * BK * 4) >> 4;
  static_assert(BK == 32 || BK == 16, "A tile rows must be 128 or 64 bytes");
  static_assert(TMEM_COLS <= 512 && SMEM_BYTES <= 232448, "tile configuration does not fit");
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: false when the phase did not complete within WAIT_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
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

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// K-major operand, swizzled rows: 8-row groups `sbo` (16-byte units) apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr, uint64_t sbo, uint64_t layout) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | (sbo << 32) | (1ull << 46) | (layout << 61);
}
// MN-major 32-bit operand: the only layout the tensor core accepts is the 128-byte swizzle with
// 32-byte atoms (layout type 1; TMA mode SWIZZLE_128B_ATOM_32B): 32-column blocks BOX_BYTES
// apart (leading offset), groups of 4 k-rows 512 B apart (stride offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint64_t box_bytes) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | ((box_bytes >> 4) << 16) | (32ull << 32) | (1ull << 46) | (1ull << 61);
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

// lo = x - hi with hi = the 19 bits the tensor core reads.  An infinity has lo = 0 (inf - inf would turn a whole
// row or column of C into NaN where the fp32 loop gives an infinity); a NaN stays a NaN in lo, because truncating
// its payload may leave hi an infinity.
__device__ __forceinline__ float split_lo(float x) {
  const uint32_t u = __float_as_uint(x);
  if ((u & 0x7F800000u) == 0x7F800000u) return (u & 0x007FFFFFu) ? x : 0.0f;
  return x - __uint_as_float(u & 0xFFFFE000u);
}
__device__ __forceinline__ void split_tf32(float4 &hi_lo_in_out, float4 &lo) {
  const float4 x = hi_lo_in_out;
  lo.x = split_lo(x.x);
  lo.y = split_lo(x.y);
  lo.z = split_lo(x.z);
  lo.w = split_lo(x.w);
}

// Tile t of the persistent schedule -> (batch, m block, n block).  Within a batch entry the tiles
// are walked in groups of 8 m-blocks so that the blocks running at the same time share A and B
// panels in L2.
struct TileCoord {
  int batch, m0, n0;
};
__device__ __forceinline__ TileCoord tile_coord(int t, int tm, int tn, int bn) {
  constexpr int GROUP = 8;
  const int per = tm * tn;
  const int batch = t / per, r = t - batch * per;
  const int g = r / (GROUP * tn), first_m = g * GROUP;
  const int gsize = tm - first_m < GROUP ? tm - first_m : GROUP;
  const int q = r - g * GROUP * tn;
  return TileCoord{batch, (first_m + q % gsize) * BM, (q / gsize) * bn};
}

template <typename C_>
__global__ void __launch_bounds__(THREADS, 1)
bgemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     float *__restrict__ C, int M, int N, int K, int total_tiles, int kseg,
                     int *__restrict__ error_flag) {
  constexpr int BN = C_::BN, BK = C_::BK, STAGES = C_::STAGES, A_BYTES = C_::A_BYTES, B_BYTES = C_::B_BYTES,
                BOX_BYTES = C_::BOX_BYTES, STAGE_BYTES = C_::STAGE_BYTES, TMEM_COLS = C_::TMEM_COLS;
  constexpr uint32_t IDESC = C_::IDESC;
  constexpr uint64_t A_SBO = C_::A_SBO, A_LAYOUT = C_::A_LAYOUT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
  uint64_t *full = bars, *conv = bars + STAGES, *empty = bars + 2 * STAGES;
  uint64_t *acc_full = bars + 3 * STAGES, *acc_empty = bars + 3 * STAGES + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nk = K / BK, tm = M / BM, tn = N / BN;
  // The K loop of a tile is cut into segments of kseg k-blocks.  Every segment is accumulated in tensor memory
  // from zero and added to C by the epilogue (which adds C_in anyway): the tensor core truncates when it adds to
  // its accumulator, an error that grows with the number of additions onto a large partial sum, and the
  // epilogue's adds round to nearest.  The segments of a tile are walked by the same block in order, and an
  // epilogue thread reads back exactly the elements of C it stored for the previous segment.
  const int nseg = (nk + kseg - 1) / kseg;

  auto stage_a = [&](int s) { return smem + s * STAGE_BYTES; };
  auto stage_alo = [&](int s) { return smem + s * STAGE_BYTES + A_BYTES; };
  auto stage_b = [&](int s) { return smem + s * STAGE_BYTES + 2 * A_BYTES; };
  auto stage_blo = [&](int s) { return smem + s * STAGE_BYTES + 2 * A_BYTES + B_BYTES; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&conv[s], 128);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory: two accumulators of 128 fp32 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer: runs ahead across tiles ----------------
    if (lane == 0) {
      uint32_t g = 0;  // k blocks issued so far by this CTA
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, tm, tn, BN);
        bool ok = true;
        for (int kb = 0; kb < nk; ++kb, ++g) {  // the segments of a tile are consecutive k blocks
          const int s = g % STAGES;
          ok = mbar_wait(&empty[s], ((g / STAGES) & 1) ^ 1);
          if (!ok) break;
          mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
          tma_load_3d(stage_a(s), &map_a, &full[s], kb * BK, tc.m0, tc.batch);
#pragma unroll
          for (int j = 0; j < BN / 32; ++j)
            tma_load_3d(stage_b(s) + j * BOX_BYTES, &map_b, &full[s], tc.n0 + 32 * j, kb * BK, tc.batch);
        }
        if (!ok) {
          atomicExch(error_flag, 1);
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t g = 0, it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int sg = 0; sg < nseg && ok; ++sg, ++it) {
          const uint32_t buf = it & 1;
          ok = mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1);  // the epilogue has drained this accumulator
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int kb0 = sg * kseg, kb1 = kb0 + kseg < nk ? kb0 + kseg : nk;
          for (int kb = kb0; kb < kb1; ++kb, ++g) {
            const int s = g % STAGES;
            // hi*hi needs only what TMA wrote: issue it as soon as the stage has landed, while the split
            // warps are still producing the lo parts; the two correction products follow.
            ok = mbar_wait(&full[s], (g / STAGES) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a = smem_u32(stage_a(s)), alo = smem_u32(stage_alo(s));
            const uint32_t b = smem_u32(stage_b(s)), blo = smem_u32(stage_blo(s));
#pragma unroll
            for (int ks = 0; ks < BK / 8; ++ks)
              mma_tf32(d_tmem, desc_kmajor(a + ks * 32, A_SBO, A_LAYOUT), desc_mnmajor(b + ks * 1024, BOX_BYTES), IDESC,
                       (kb > kb0 || ks > 0) ? 1u : 0u);
            ok = mbar_wait(&conv[s], (g / STAGES) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int ks = 0; ks < BK / 8; ++ks) {
              const uint64_t da = desc_kmajor(a + ks * 32, A_SBO, A_LAYOUT), dalo = desc_kmajor(alo + ks * 32, A_SBO, A_LAYOUT);
              const uint64_t db = desc_mnmajor(b + ks * 1024, BOX_BYTES), dblo = desc_mnmajor(blo + ks * 1024, BOX_BYTES);
              mma_tf32(d_tmem, dalo, db, IDESC, 1u);
              mma_tf32(d_tmem, da, dblo, IDESC, 1u);
            }
            // releases the stage once the MMAs above have read it
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&empty[s]))
                         : "memory");
          }
          if (!ok) break;
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           smem_u32(&acc_full[buf]))
                       : "memory");
        }
      }
      if (!ok) atomicExch(error_flag, 2);
    }
  } else if (warp < 6) {
    // ---------------- split x = hi + lo ----------------
    const int t128 = threadIdx.x - 64;  // 0..127
    uint32_t g = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      for (int kb = 0; kb < nk; ++kb, ++g) {
        const int s = g % STAGES;
        ok = mbar_wait(&full[s], (g / STAGES) & 1);
        if (!ok) break;
        const float4 *a = reinterpret_cast<const float4 *>(stage_a(s));
        float4 *alo = reinterpret_cast<float4 *>(stage_alo(s));
        const float4 *b = reinterpret_cast<const float4 *>(stage_b(s));
        float4 *blo = reinterpret_cast<float4 *>(stage_blo(s));
#pragma unroll
        for (int i = 0; i < A_BYTES / 16 / 128; ++i) {
          float4 x = a[t128 + 128 * i], lo;
          split_tf32(x, lo);
          alo[t128 + 128 * i] = lo;
        }
#pragma unroll
        for (int i = 0; i < B_BYTES / 16 / 128; ++i) {
          float4 x = b[t128 + 128 * i], lo;
          split_tf32(x, lo);
          blo[t128 + 128 * i] = lo;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
        mbar_arrive(&conv[s]);
      }
    }
    if (!ok) atomicExch(error_flag, 3);
  } else {
    // ---------------- epilogue: overlaps the main loop of the next tile ----------------
    // accumulator row = TMEM lane; a warp may touch lanes 32*(warp%4)..+31
    const int q = warp & 3;
    float *stile = reinterpret_cast<float *>(smem + STAGES * STAGE_BYTES + 256) + (warp - 6) * 32 * EPI_PITCH;
    constexpr int NC = BN / 32;  // 32-column chunks of a tile
    static_assert(NC % 2 == 0 && NC >= 2, "the epilogue walks the chunks in pairs");
    auto warp_rows = [&](int t) {  // this warp's 32 rows of tile t in C
      const TileCoord tc = tile_coord(t, tm, tn, BN);
      return C + ((size_t)tc.batch * M + tc.m0 + 32 * q) * (size_t)N + tc.n0;
    };
    // C_in chunk (32 rows x 32 columns), coalesced: 8 lanes cover the 128 bytes of one row.  Two chunks are
    // requested together, so that the latency of these loads is paid once per pair.
    auto load_cin = [&](float4(&cin)[8], const float *cwarp, int c) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        cin[i] = *reinterpret_cast<const float4 *>(cwarp + (size_t)(4 * i + (lane >> 3)) * N + 32 * c + 4 * (lane & 7));
    };
    auto drain = [&](const float4(&cin)[8], float *cwarp, int c, uint32_t buf, bool last) {
      // thread = row in tensor memory; transpose through shared memory so that stores are coalesced.  The 32
      // columns come in two halves of 16 (the registers of a half are free before the next is read).
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c);
      __syncwarp();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr + 16u * half));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (last && half == 1) {  // the accumulator is in registers: hand it back to the MMA warp
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          mbar_arrive(&acc_empty[buf]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<float4 *>(stile + lane * EPI_PITCH + 16 * half + 4 * i) =
              make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                          __uint_as_float(r[4 * i + 3]));
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = 4 * i + (lane >> 3);
        const float4 a = *reinterpret_cast<const float4 *>(stile + row * EPI_PITCH + 4 * (lane & 7));
        float4 o = cin[i];
        o.x = __fadd_rn(a.x, o.x);
        o.y = __fadd_rn(a.y, o.y);
        o.z = __fadd_rn(a.z, o.z);
        o.w = __fadd_rn(a.w, o.w);
        *reinterpret_cast<float4 *>(cwarp + (size_t)row * N + 32 * c + 4 * (lane & 7)) = o;
      }
    };
    uint32_t it = 0;
    bool ok = true;
    for (int u = 0, t = blockIdx.x; t < total_tiles && ok; ++it) {
      // unit of work: one K segment of one tile; u counts the segments of tile t
      float *cwarp = warp_rows(t);
      if (++u == nseg) {
        u = 0;
        t += gridDim.x;
      }
      const uint32_t buf = it & 1;
      ok = mbar_wait(&acc_full[buf], (it >> 1) & 1);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (BN == 128) {
#pragma unroll 1
        for (int c = 0; c < NC; c += 2) {
          float4 cin_a[8], cin_b[8];
          load_cin(cin_a, cwarp, c);
          load_cin(cin_b, cwarp, c + 1);
          drain(cin_a, cwarp, c, buf, false);
          drain(cin_b, cwarp, c + 1, buf, c + 2 == NC);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < NC; ++c) {
          float4 cin_a[8];
          load_cin(cin_a, cwarp, c);
          drain(cin_a, cwarp, c, buf, c + 1 == NC);
        }
      }
    }
    if (!ok) atomicExch(error_flag, 4);
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    // resolved through the runtime so that the library does not link libcuda directly
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Row-major [batch][rows][cols] fp32 tensor, box = box_rows x box_cols, swizzled.
static int make_map(CUtensorMap *map, const float *base, int64_t batch, int64_t rows, int64_t cols, int box_rows,
                    int box_cols, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(LAPIS_ECUDA, "bgemm: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 4, (cuuint64_t)cols * rows * 4};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LAPIS_ECUDA, "bgemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return LAPIS_OK;
}

}  // namespace tc

static int *error_flag[64] = {nullptr};

template <typename C_>
static int launch_cfg(int64_t batch, int64_t M, int64_t N, int64_t K, const float *A, const float *B, float *C,
                      int dev, cudaStream_t st) {
  static bool attr_set[64] = {false};
  CUtensorMap map_a, map_b;
  LAPIS_TRY(tc::make_map(&map_a, A, batch, M, K, tc::BM, C_::BK,
                         C_::BK == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B));
  LAPIS_TRY(tc::make_map(&map_b, B, batch, K, N, C_::BK, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B));
  if (!attr_set[dev]) {
    LAPIS_CUDA_TRY(cudaFuncSetAttribute(tc::bgemm_tcgen05_kernel<C_>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        C_::SMEM_BYTES));
    attr_set[dev] = true;
  }
  const int64_t total = batch * (M / tc::BM) * (N / C_::BN);
  const int64_t grid = total < sm_count() ? total : sm_count();  // persistent: one block per SM
  const int kseg = tc::K_SEGMENT / C_::BK;
  tc::bgemm_tcgen05_kernel<C_><<<(unsigned)grid, tc::THREADS, C_::SMEM_BYTES, st>>>(map_a, map_b, C, (int)M, (int)N,
                                                                                  (int)K, (int)total, kseg, error_flag[dev]);
  LAPIS_CUDA_TRY(cudaGetLastError());
  return LAPIS_OK;
}

using CfgSmall = tc::Cfg<128, 32, 3>;
using CfgWide = tc::Cfg<256, 16, 4>;

int bgemm_tcgen05_supported(int64_t batch, int64_t M, int64_t N, int64_t K) {
  return batch >= 1 && M >= tc::BM && N >= CfgSmall::BN && K >= CfgSmall::BK && M % tc::BM == 0 &&
         N % CfgSmall::BN == 0 && K % CfgSmall::BK == 0 && M <= (1 << 30) && N <= (1 << 30) && K <= (1 << 30) &&
         batch * (M / tc::BM) * (N / CfgSmall::BN) < (1ll << 31) && batch < (1ll << 31);
}

int bgemm_tcgen05_launch(int64_t batch, int64_t M, int64_t N, int64_t K, const float *A, const float *B, float *C,
                         cudaStream_t st) {
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16)
    return fail(LAPIS_EBADARG, "bgemm: operands must be 16-byte aligned");
  int dev = 0;
  LAPIS_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(LAPIS_EBADARG, "bgemm: device index %d not supported", dev);
  if (error_flag[dev] == nullptr) {
    LAPIS_CUDA_TRY(cudaMalloc(&error_flag[dev], sizeof(int)));
    LAPIS_CUDA_TRY(cudaMemset(error_flag[dev], 0, sizeof(int)));
  }
  // 128 x 256 tiles when N allows and there are enough of them to fill the SMs; LAPIS_B200_GEMM_TILE=128 forces
  // the 128 x 128 configuration.
  static const int forced = [] {
    const char *e = std::getenv("LAPIS_B200_GEMM_TILE");
    return e ? atoi(e) : 0;
  }();
  const bool wide = forced != 128 && N % CfgWide::BN == 0 && K >= 8 * CfgWide::BK &&
                    batch * (M / tc::BM) * (N / CfgWide::BN) >= sm_count();
  if (wide) return launch_cfg<CfgWide>(batch, M, N, K, A, B, C, dev, st);
  return launch_cfg<CfgSmall>(batch, M, N, K, A, B, C, dev, st);
}

}  // namespace lapis_b200

// Reads and clears the tensor-core kernel's error flag; synchronises `stream`.  A non-zero flag
// means a bounded wait inside the kernel gave up (1 producer, 2 MMA issuer, 3 split warps,
// 4 epilogue) and the output of that launch is not valid.
extern "C" int lapis_b200_bgemm_status(void *stream) {
  using namespace lapis_b200;
  clear_error();
  int dev = 0;
  LAPIS_CUDA_TRY(cudaGetDevice(&dev));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
  if (dev < 0 || dev >= 64 || error_flag[dev] == nullptr) return LAPIS_OK;
  int flag = 0;
  LAPIS_CUDA_TRY(cudaMemcpy(&flag, error_flag[dev], sizeof(int), cudaMemcpyDeviceToHost));
  if (flag != 0) {
    cudaMemset(error_flag[dev], 0, sizeof(int));
    return fail(LAPIS_ECUDA, "bgemm: tensor-core kernel gave up waiting (role %d)", flag);
  }
  return LAPIS_OK;
}
