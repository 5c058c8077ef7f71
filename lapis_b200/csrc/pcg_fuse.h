// Device-side pieces shared by the PCG passes (pcg.cu) and the SpMV kernels that can carry them (spmv.cu):
// the scalar block of a solver workspace, the mailbox protocol of the row-partitioned solver, bounded waits,
// and the "last block done" tail that turns per-block partial sums into the iteration's scalars inside the
// pass that produced them.
//
// One PCG iteration (examples/pcg_solve.py:74-98 in the LAPIS project) is three launches:
//
//   pass A  Ap = A p, partial sums of p.Ap
//           tail: p.Ap summed; one rank: alpha derived; several ranks: {p.Ap, seq} stored into every mailbox
//   pass B  [wait for every rank's p.Ap; alpha]   x += alpha p, r -= alpha Ap, z = r*dinv, partial r.r and r.z;
//           the rows of z that neighbours need are also stored into their halo buffers
//           tail: sums; one rank: stop test and beta; several ranks: {r.r, r.z, seq} stored into every mailbox
//           (after the z rows: a rank that sees the sequence number also sees the rows)
//   pass C  [wait for every rank's r.r, r.z; stop test; beta]   p = z + beta p on the own rows AND on the halo
//           entries of the window, from the neighbours' z rows and the old halo of p (the same operation the
//           owner performs, so the same bits) -- the halo of p needs no exchange of its own
//           tail: several ranks: iteration counter advanced
//
// Two points per iteration at which a rank waits for the others, not three.
//
// Two-pass form (matrices served by the one-thread-per-row SpMV kernel): pass C is folded into the next
// iteration's pass A.  That kernel's head is pass C's head (wait for r.r / r.z, stop test, beta); its SpMV reads
// z + beta * p_old at every column it gathers (the values pass C would have stored, the same bits), stores the
// own rows and the halo entries of the new p into the second p buffer (the buffers alternate; SC_PCUR names the
// current one), and its tail is pass C's bookkeeping followed by pass A's tail.  Before the first SpMV of a solve
// (SC_STAGE == 0) p is read as initialised.  Pass B keeps z in the window-indexed z buffer, own rows included,
// so that the SpMV can gather from it.  Two launches per iteration; with several ranks the stop test of an
// iteration runs at the head of the launch after it.
//
// A "tail" runs in the block that finishes last (an atomic ticket per pass) and adds the partial sums in a
// fixed order, so results do not depend on which block that is.  Heads that wait poll this rank's own mailbox
// (local memory) with a bound; every block of a pass does its own wait and adds the ranks' values in rank
// order, so every block of every rank derives the same bits.  A wait that runs out marks the mailbox, sets the
// solver's done flag and lets the block return; nothing spins without a limit and nothing traps.
#pragma once
#include <cstdint>

namespace lapis_b200 {

// Device scalar block at the head of a PCG workspace (doubles, then flags).
enum { SC_PAP = 0, SC_RR = 1, SC_RZNEW = 2, SC_RZ = 3, SC_INITRES = 4, SC_RELRES = 5, SC_ALPHA = 6, SC_BETA = 7, SC_COUNT = 8 };
enum { FL_DONE = 0, FL_ITERS = 1, FL_COUNT = 2 };  // int64 each, at doubles 8 and 9
enum { DERIVE_NONE = 0, DERIVE_INIT = 1, DERIVE_ALPHA = 2, DERIVE_DECIDE = 3, DERIVE_ALPHA_MASKED = 4 };
constexpr int SC_EPOCH = 10;   // header slot holding epoch * 2^32 (row-partitioned solver)
constexpr int SC_DMP2 = 11;    // header slot: sum of d * (mask*p)^2 of the masked-Laplacian operator
constexpr int SC_TICKET = 12;  // header slots 12..13 reinterpreted as four unsigned tickets (one per pass)
constexpr int SC_STAGE = 14;   // header slot (int64): 0 until the first SpMV pass of a solve has run (two-pass form)
constexpr int SC_PCUR = 15;    // header slot (int64): which of the two p buffers holds the current p (two-pass form)

constexpr int P2P_MAXW = 16;
constexpr int P2P_HALO = 4 * P2P_MAXW * 4;
constexpr int P2P_ERR = P2P_HALO + P2P_MAXW;
constexpr int P2P_MBOX_DOUBLES = 512;
constexpr unsigned P2P_SPIN_LIMIT = 1u << 22;  // polls with a short sleep: a few seconds at most
enum { PH_A = 0, PH_B = 1, PH_INIT = 2 };

struct HaloPiece {  // one contiguous piece of p this rank provides to a peer
  unsigned long long dst_addr;   // address of the first destination element in the peer's p window
  long long src_off;             // offset of the first source element in this rank's p window
  long long len;
  unsigned long long flag_addr;  // address of this rank's halo flag in the peer's mailbox
};

// What a fused pass needs to know about the exchange; passed to kernels by value.
struct PcgExchange {
  double *sc;                            // scalar block of this rank's workspace
  long long *fl;                         // its flags
  double *mbox;                          // this rank's mailbox; null: no exchange, scalars derived locally
  const unsigned long long *peer_mbox;   // addresses of every rank's mailbox, own included
  const int *halo_srcs;                  // ranks whose halo pieces of p a wait in front of pass A covers (first iteration)
  const HaloPiece *pieces;               // rows of z that pass B stores into the neighbours' z halo buffers
  const long long *halo_ranges;          // {start, length} pairs: the halo parts of this rank's window
  const double *zhalo;                   // this rank's z halo buffer (window-indexed)
  int me, world, nsrc, npieces, nranges;
  unsigned spin_limit;                   // polls per bounded wait
  double tol;
  unsigned long long maxiter;
};

__device__ __forceinline__ unsigned *pcg_tickets(double *sc) { return reinterpret_cast<unsigned *>(sc + SC_TICKET); }

__device__ __forceinline__ bool p2p_wait_equal(const volatile double *flag, double expected, unsigned limit) {
  for (unsigned i = 0; i < limit; ++i) {
    if (*flag == expected) return true;
    __nanosleep(200);
  }
  return false;
}

// The same wait with acquire loads at system scope: what the producer stored before its flag is visible to this
// thread's later loads without a separate fence.
__device__ __forceinline__ bool p2p_wait_acquire(const double *flag, double expected, unsigned limit) {
  for (unsigned i = 0; i < limit; ++i) {
    double v;
    asm volatile("ld.acquire.sys.global.f64 %0, [%1];" : "=d"(v) : "l"(flag) : "memory");
    if (v == expected) return true;
    __nanosleep(100);
  }
  return false;
}

// Sequence number of the iteration in flight: epoch * 2^32 + completed iterations + 1.
__device__ __forceinline__ double pcg_seq(const PcgExchange &ex) { return ex.sc[SC_EPOCH] + (double)(ex.fl[FL_ITERS] + 1); }

// A wait ran out: leave a mark for the host (1 + phase for scalar sums, 9 for the halo) and stop the solve.
__device__ __forceinline__ void pcg_give_up(const PcgExchange &ex, double mark) {
  ex.mbox[P2P_ERR] = mark;
  ex.fl[FL_DONE] = 1;
}

// Head of pass A on several ranks: warp 0 of the block waits for the halo flags of this iteration.
// Returns false (in every thread) when the block has to return.  s_flag: one int of shared memory.
__device__ __forceinline__ bool pcg_wait_halo(const PcgExchange &ex, int *s_flag) {
  if (ex.nsrc == 0) return true;
  if (threadIdx.x < 32) {
    const double expected = pcg_seq(ex);
    bool ok = true;
    if ((int)threadIdx.x < ex.nsrc) ok = p2p_wait_acquire(ex.mbox + P2P_HALO + ex.halo_srcs[threadIdx.x], expected, ex.spin_limit);
    const bool all_ok = __all_sync(0xffffffffu, ok);
    if (all_ok) __threadfence_system();  // the pieces were stored before their flag; the barrier below orders the
                                         // other warps' reads behind this one
    if (threadIdx.x == 0) {
      if (!all_ok) pcg_give_up(ex, 9.0);
      *s_flag = all_ok ? 1 : 0;
    }
  }
  __syncthreads();
  return *s_flag != 0;
}

// Head of passes B and C on several ranks: warp 0 waits for every rank's values of `phase` and adds them in
// rank order.  Returns false when the block has to return; v0, v1 are valid in every thread otherwise.
// s_vals: three doubles of shared memory.
__device__ __forceinline__ bool pcg_wait_sums(const PcgExchange &ex, int phase, double *s_vals, double &v0, double &v1) {
  if (threadIdx.x < 32) {
    const int j = threadIdx.x;
    const double expected = pcg_seq(ex);
    const volatile double *slot = ex.mbox + (phase * P2P_MAXW + (j < ex.world ? j : 0)) * 4;
    bool ok = true;
    if (j < ex.world) ok = p2p_wait_acquire(const_cast<const double *>(slot) + 2, expected, ex.spin_limit);
    const bool all_ok = __all_sync(0xffffffffu, ok);
    double a = 0.0, b = 0.0;
    if (all_ok) {
      // the values were stored before their sequence number, which this lane read with an acquire load
      const double mine0 = j < ex.world ? slot[0] : 0.0, mine1 = j < ex.world ? slot[1] : 0.0;  // one load per lane
      for (int r = 0; r < ex.world; ++r) {  // added in rank order, on every block of every rank
        a = __dadd_rn(a, __shfl_sync(0xffffffffu, mine0, r));
        b = __dadd_rn(b, __shfl_sync(0xffffffffu, mine1, r));
      }
    }
    if (j == 0) {
      if (!all_ok) pcg_give_up(ex, 1.0 + phase);
      s_vals[0] = a;
      s_vals[1] = b;
      s_vals[2] = all_ok ? 1.0 : 0.0;
    }
  }
  __syncthreads();
  v0 = s_vals[0];
  v1 = s_vals[1];
  return s_vals[2] != 0.0;
}

// Stores this rank's values of `phase` into every rank's mailbox (threads j < world of the calling block).
__device__ __forceinline__ void pcg_push_sums(const PcgExchange &ex, int phase, double v0, double v1, double seq) {
  const int j = threadIdx.x;
  if (j < ex.world) {
    volatile double *slot = reinterpret_cast<volatile double *>(ex.peer_mbox[j]) + (phase * P2P_MAXW + ex.me) * 4;
    slot[0] = v0;
    slot[1] = v1;
    __threadfence_system();  // values before the sequence number, system-wide
    slot[2] = seq;
  }
}

// True in every thread of the block that takes the last ticket of this launch (all other blocks have
// written their partial sums and made them visible).  Resets the ticket for the next launch.
__device__ __forceinline__ bool pcg_last_block(unsigned *ticket, unsigned nblocks, int *s_flag) {
  __syncthreads();  // this block's partial sums are written
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned t = atomicAdd(ticket, 1u);
    const int last = t == nblocks - 1 ? 1 : 0;
    if (last) {
      *ticket = 0u;
      __threadfence();
    }
    *s_flag = last;
  }
  __syncthreads();
  return *s_flag != 0;
}

// Sum of partials[0..nb) in a fixed order by the whole block; the result is valid in thread 0.
// s_red: blockDim.x / 32 doubles of shared memory.
__device__ __forceinline__ double pcg_block_total(const double *partials, int64_t nb, double *s_red) {
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < nb; i += blockDim.x) acc = __dadd_rn(acc, __ldcg(partials + i));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc = __dadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) s_red[warp] = acc;
  __syncthreads();
  double t = 0.0;
  if (warp == 0) {
    t = lane < (int)(blockDim.x >> 5) ? s_red[lane] : 0.0;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t = __dadd_rn(t, __shfl_xor_sync(0xffffffffu, t, off));
  }
  return t;
}

// Scalar recurrences of one PCG iteration (examples/pcg_solve.py:70-71, 78, 84-90, 96).
__device__ __forceinline__ void pcg_derive(int kind, double *sc, long long *fl, double tol, unsigned long long maxiter) {
  if (kind == DERIVE_INIT) {
    sc[SC_INITRES] = sqrt(sc[SC_RR]);
    sc[SC_RZ] = sc[SC_RZNEW];
    fl[FL_DONE] = 0;
    fl[FL_ITERS] = 0;
  } else if (kind == DERIVE_ALPHA) {
    sc[SC_ALPHA] = sc[SC_RZ] / sc[SC_PAP];
  } else if (kind == DERIVE_ALPHA_MASKED) {
    // p.(M (D - A) M p) = sum d (m p)^2 - (m p).(A (m p)): the two sums arrive separately
    sc[SC_ALPHA] = sc[SC_RZ] / __dsub_rn(sc[SC_DMP2], sc[SC_PAP]);
  } else if (kind == DERIVE_DECIDE) {
    const double relres = sqrt(sc[SC_RR]) / sc[SC_INITRES];
    sc[SC_RELRES] = relres;
    const unsigned long long iter = (unsigned long long)fl[FL_ITERS] + 1;  // i starts at 1
    fl[FL_ITERS] = (long long)iter;
    const bool not_converged = relres > tol;  // ordered compare: NaN stops the loop
    const bool below_maxiter = iter != maxiter;
    if (!(not_converged && below_maxiter)) {
      fl[FL_DONE] = 1;
    } else {
      sc[SC_BETA] = sc[SC_RZNEW] / sc[SC_RZ];
      sc[SC_RZ] = sc[SC_RZNEW];
    }
  }
}

// Tail of pass A in the last block: p.Ap from the per-block partial sums; alpha when there is no exchange
// (mbox == nullptr), a store into every mailbox otherwise.
__device__ __forceinline__ void pcg_tail_pass_a(const PcgExchange &ex, const double *blk_partial, int64_t nb, double *s_red) {
  const double pap = pcg_block_total(blk_partial, nb, s_red);
  __shared__ double s_pap;
  if (threadIdx.x == 0) {
    s_pap = pap;
    ex.sc[SC_PAP] = pap;  // this rank's part when the sums are exchanged
    if (ex.mbox == nullptr) pcg_derive(DERIVE_ALPHA, ex.sc, ex.fl, ex.tol, ex.maxiter);
  }
  __syncthreads();
  if (ex.mbox != nullptr) pcg_push_sums(ex, PH_A, s_pap, 0.0, pcg_seq(ex));
}

}  // namespace lapis_b200
