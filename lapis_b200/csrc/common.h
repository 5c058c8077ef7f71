// Shared host-side helpers: status recording, CUDA error checks, the CSR handle.
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/lapis_b200.h"

namespace lapis_b200 {

// Records status + message for lapis_last_error(); returns `code` so callers can
// `return fail(...)`.
int fail(int code, const char *fmt, ...);
void clear_error();

#define LAPIS_CUDA_TRY(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return ::lapis_b200::fail(LAPIS_ECUDA, "%s failed: %s (%s:%d)", #expr,              \
                                cudaGetErrorString(_e), __FILE__, __LINE__);              \
  } while (0)

#define LAPIS_TRY(expr)          \
  do {                           \
    int _s = (expr);             \
    if (_s != LAPIS_OK) return _s; \
  } while (0)

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace lapis_b200

// The CSR handle: borrowed matrix arrays + the streaming plan owned by the handle.
struct lapis_b200_csr {
  int idx_bytes;
  int64_t nrows, ncols, nnz, base;  // base = pos[0]
  const void *pos, *crd;
  const double *val;
  // Streaming plan: thread block b of the SpMV kernel processes the stored entries
  // [abase + b*TILE, abase + (b+1)*TILE), abase = base & ~1; blk_row[b] is the first row
  // that ends inside that chunk (nblk+1 entries).  carry[b] receives the partial sum of
  // the row that runs past chunk b.
  int64_t nblk;
  int64_t *blk_row;
  double *carry;
  // Scratch for the fused dot product of the PCG SpMV pass (one double per block).
  double *blk_partial;
  // Kernel variant chosen by lapis_b200_csr_tune (tuned_threads == 0: not tuned).
  int tuned_threads, tuned_minb, tuned_hint;
  // Longest row, found by lapis_b200_csr_tune (-1: not known).  The one-thread-per-row kernel is only used
  // when no row has more than 32 entries: up to there it returns the same bits as the chunk kernels.
  int64_t max_row_len;
  int device;
  // Second plan for the warp-walk kernel on small matrices: ranges of walk_tile entries (null: it uses blk_row).
  int64_t *walk_plan;
  double *walk_carry;
  int64_t walk_nblk;
  int walk_tile;
};
