// Emitted-module ABI: lapis_initialize / lapis_finalize and the py_<func> wrappers.
//
// Mirrors what mlir/lib/Target/KokkosCpp/TranslateToKokkosCpp.cpp:2541-2684 prints
// for every public function: descriptors in (host memory), results out through
// `ret` slots, device work fenced before returning.  Where the emitted wrapper
// wraps host pointers in unmanaged Kokkos views and lets LAPIS::DualView copy them
// to the device (LAPISSupport.hpp:193-282), this file stages the operands in device
// buffers with cudaMemcpyAsync, runs the kernels and copies the result back.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "common.h"

extern "C" int64_t lapis_b200_pcg_workspace_bytes(int64_t n, int64_t n_p);

namespace lapis_b200 {

static thread_local int g_status = LAPIS_OK;
static thread_local char g_message[512] = "";

int fail(int code, const char *fmt, ...) {
  g_status = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_message, sizeof(g_message), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() {
  g_status = LAPIS_OK;
  g_message[0] = '\0';
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- module state -----------------------------------------------------------
static int g_init_count = 0;
static std::vector<void *> g_alive_host;  // result buffers handed to the caller (LAPISSupport.hpp:93-120)

// Scoped device buffer.
struct DevBuf {
  void *p = nullptr;
  ~DevBuf() {
    if (p) cudaFree(p);
  }
  int alloc(size_t bytes) {
    if (bytes == 0) bytes = 16;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return fail(LAPIS_ECUDA, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    return LAPIS_OK;
  }
};

static int require_init() {
  if (g_init_count <= 0) return fail(LAPIS_ENOTINIT, "lapis_initialize has not been called");
  return LAPIS_OK;
}

// C-contiguity check of LAPISSupport.hpp:80-89 (LayoutRight).
template <typename M, int R>
static int check_contig(const M *m, const char *what) {
  if (m == nullptr) return fail(LAPIS_EBADARG, "%s: null descriptor", what);
  int64_t expect = 1;
  for (int i = R - 1; i >= 0; --i) {
    if (m->sizes[i] < 0) return fail(LAPIS_EBADSHAPE, "%s: negative extent", what);
    if (m->sizes[i] > 1 && m->strides[i] != expect)
      return fail(LAPIS_ELAYOUT, "%s: descriptor is not contiguous row-major", what);
    expect *= m->sizes[i];
  }
  if (expect > 0 && m->data == nullptr) return fail(LAPIS_EBADARG, "%s: null data pointer", what);
  return LAPIS_OK;
}

template <typename T, typename M>
static T *elem_ptr(const M *m) {
  return static_cast<T *>(m->data) + m->offset;
}

struct CsrArgs {
  int64_t nrows, ncols, npos, nnz;
};

static int check_csr(const lapis_memref1 *pos, const lapis_memref1 *crd, const lapis_memref1 *val,
                     const lapis_csr_spec *spec, CsrArgs *out) {
  LAPIS_TRY((check_contig<lapis_memref1, 1>(pos, "pos")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(crd, "crd")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(val, "val")));
  if (spec == nullptr) return fail(LAPIS_EBADARG, "null storage specifier");
  out->nrows = spec->dims[0];
  out->ncols = spec->dims[1];
  out->npos = spec->mem_sizes[0];
  out->nnz = spec->mem_sizes[2];
  if (out->nrows < 0 || out->ncols < 0) return fail(LAPIS_EBADSHAPE, "negative matrix dimension");
  if (out->npos != out->nrows + 1 || pos->sizes[0] < out->npos)
    return fail(LAPIS_EBADSHAPE, "pos must have rows+1 entries");
  if (spec->mem_sizes[1] != out->nnz || crd->sizes[0] < out->nnz || val->sizes[0] < out->nnz)
    return fail(LAPIS_EBADSHAPE, "crd/val shorter than the specifier says");
  return LAPIS_OK;
}

// Validates pos on the host (non-decreasing, ends at nnz) before any kernel trusts it.
template <typename I>
static int check_pos_host(const I *pos, int64_t nrows, int64_t nnz) {
  if (pos[0] != 0) return fail(LAPIS_EBADSHAPE, "pos[0] must be 0");
  for (int64_t r = 0; r < nrows; ++r)
    if (pos[r + 1] < pos[r]) return fail(LAPIS_EBADSHAPE, "pos is not non-decreasing at row %lld", (long long)r);
  if ((int64_t)pos[nrows] != nnz) return fail(LAPIS_EBADSHAPE, "pos[rows] != number of stored entries");
  return LAPIS_OK;
}

// Validates the column indices on the host: 0 <= crd[j] < ncols for every stored entry.  The emitted code
// indexes x with them unchecked (a bad index is undefined behaviour there); here a bad index must not
// reach a gather on the device.  Min and max over slices of the array on a few host threads.
template <typename I>
static int check_crd_host(const I *crd, int64_t nnz, int64_t ncols) {
  if (nnz <= 0) return LAPIS_OK;
  const int nthreads = nnz < (1 << 20) ? 1 : (int)std::min<int64_t>(8, std::max(1u, std::thread::hardware_concurrency()));
  std::vector<I> lo(nthreads), hi(nthreads);
  auto scan = [&](int t) {
    const int64_t b = nnz * t / nthreads, e = nnz * (t + 1) / nthreads;
    I mn = crd[b], mx = crd[b];
    for (int64_t j = b; j < e; ++j) {
      mn = crd[j] < mn ? crd[j] : mn;
      mx = crd[j] > mx ? crd[j] : mx;
    }
    lo[t] = mn;
    hi[t] = mx;
  };
  if (nthreads == 1) {
    scan(0);
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < nthreads; ++t) pool.emplace_back(scan, t);
    for (auto &th : pool) th.join();
  }
  I mn = lo[0], mx = hi[0];
  for (int t = 1; t < nthreads; ++t) {
    mn = lo[t] < mn ? lo[t] : mn;
    mx = hi[t] > mx ? hi[t] : mx;
  }
  if ((int64_t)mn < 0 || (int64_t)mx >= ncols)
    return fail(LAPIS_EBADSHAPE, "column index out of range: crd holds values in [%lld, %lld], the matrix has %lld columns",
                (long long)mn, (long long)mx, (long long)ncols);
  return LAPIS_OK;
}

// Uploads a CSR matrix and builds its handle.
struct DeviceCsr {
  DevBuf pos, crd, val;
  lapis_b200_csr_t h = nullptr;
  ~DeviceCsr() { lapis_b200_csr_destroy(h); }
};

template <typename I>
static int upload_csr(const lapis_memref1 *pos, const lapis_memref1 *crd, const lapis_memref1 *val, const CsrArgs &a,
                      DeviceCsr *d, cudaStream_t st) {
  const I *hpos = elem_ptr<I>(pos);
  LAPIS_TRY(d->pos.alloc((size_t)a.npos * sizeof(I)));
  LAPIS_TRY(d->crd.alloc((size_t)a.nnz * sizeof(I)));
  LAPIS_TRY(d->val.alloc((size_t)a.nnz * sizeof(double)));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(d->pos.p, hpos, (size_t)a.npos * sizeof(I), cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(d->crd.p, elem_ptr<I>(crd), (size_t)a.nnz * sizeof(I), cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(d->val.p, elem_ptr<double>(val), (size_t)a.nnz * sizeof(double), cudaMemcpyHostToDevice, st));
  // validated on the host while the copies are in flight (they are asynchronous from pinned memory);
  // no kernel has been given the offsets yet
  if (check_pos_host<I>(hpos, a.nrows, a.nnz) != LAPIS_OK || check_crd_host<I>(elem_ptr<I>(crd), a.nnz, a.ncols) != LAPIS_OK) {
    const int code = lapis_last_error();
    char msg[512];
    snprintf(msg, sizeof(msg), "%s", lapis_last_error_message());
    cudaStreamSynchronize(st);
    return fail(code, "%s", msg);
  }
  return lapis_b200_csr_create(&d->h, (int)sizeof(I), a.nrows, a.ncols, d->pos.p, d->crd.p,
                               static_cast<const double *>(d->val.p), st);
}

template <typename I>
static int spmv_host(lapis_memref1 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                     const lapis_csr_spec *spec, lapis_memref1 *x, lapis_memref1 *y) {
  clear_error();
  LAPIS_TRY(require_init());
  CsrArgs a;
  LAPIS_TRY(check_csr(pos, crd, val, spec, &a));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(x, "x")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(y, "y")));
  if (x->sizes[0] != a.ncols || y->sizes[0] != a.nrows) return fail(LAPIS_EBADSHAPE, "spmv: x/y length mismatch");
  cudaStream_t st = nullptr;
  DeviceCsr d;
  LAPIS_TRY(upload_csr<I>(pos, crd, val, a, &d, st));
  DevBuf dx, dy;
  LAPIS_TRY(dx.alloc((size_t)a.ncols * 8));
  LAPIS_TRY(dy.alloc((size_t)a.nrows * 8));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dx.p, elem_ptr<double>(x), (size_t)a.ncols * 8, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dy.p, elem_ptr<double>(y), (size_t)a.nrows * 8, cudaMemcpyHostToDevice, st));
  LAPIS_TRY(lapis_b200_spmv_f64(d.h, static_cast<const double *>(dx.p), static_cast<double *>(dy.p), 1, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(elem_ptr<double>(y), dy.p, (size_t)a.nrows * 8, cudaMemcpyDeviceToHost, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));  // results host-visible on return (emitted fence, :2682)
  if (ret0 != nullptr && *ret0 != nullptr) **ret0 = *y;  // the function returns its outs argument
  return LAPIS_OK;
}

template <typename I>
static int spmm_host(lapis_memref2 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                     const lapis_csr_spec *spec, lapis_memref2 *B, lapis_memref2 *C) {
  clear_error();
  LAPIS_TRY(require_init());
  CsrArgs a;
  LAPIS_TRY(check_csr(pos, crd, val, spec, &a));
  LAPIS_TRY((check_contig<lapis_memref2, 2>(B, "B")));
  LAPIS_TRY((check_contig<lapis_memref2, 2>(C, "C")));
  const int64_t k = B->sizes[1];
  if (B->sizes[0] != a.ncols || C->sizes[0] != a.nrows || C->sizes[1] != k)
    return fail(LAPIS_EBADSHAPE, "spmm: B/C shape mismatch");
  cudaStream_t st = nullptr;
  DeviceCsr d;
  LAPIS_TRY(upload_csr<I>(pos, crd, val, a, &d, st));
  DevBuf dB, dC;
  const size_t bB = (size_t)a.ncols * k * 8, bC = (size_t)a.nrows * k * 8;
  LAPIS_TRY(dB.alloc(bB));
  LAPIS_TRY(dC.alloc(bC));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dB.p, elem_ptr<double>(B), bB, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dC.p, elem_ptr<double>(C), bC, cudaMemcpyHostToDevice, st));
  LAPIS_TRY(lapis_b200_spmm_f64(d.h, k, static_cast<const double *>(dB.p), static_cast<double *>(dC.p), 1, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(elem_ptr<double>(C), dC.p, bC, cudaMemcpyDeviceToHost, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  if (ret0 != nullptr && *ret0 != nullptr) **ret0 = *C;
  return LAPIS_OK;
}

static int gemm_host(int64_t batch, int64_t M, int64_t N, int64_t K, const float *A, const float *B, float *C) {
  cudaStream_t st = nullptr;
  DevBuf dA, dB, dC;
  const size_t bA = (size_t)batch * M * K * 4, bB = (size_t)batch * K * N * 4, bC = (size_t)batch * M * N * 4;
  LAPIS_TRY(dA.alloc(bA));
  LAPIS_TRY(dB.alloc(bB));
  LAPIS_TRY(dC.alloc(bC));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dA.p, A, bA, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dB.p, B, bB, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dC.p, C, bC, cudaMemcpyHostToDevice, st));
  LAPIS_TRY(lapis_b200_bgemm_f32(batch, M, N, K, static_cast<const float *>(dA.p), static_cast<const float *>(dB.p),
                                 static_cast<float *>(dC.p), st));
  LAPIS_TRY(lapis_b200_bgemm_status(st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(C, dC.p, bC, cudaMemcpyDeviceToHost, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  return LAPIS_OK;
}

template <typename I>
static int pcg_host(lapis_memref1 **ret0, size_t *ret1, double *ret2, lapis_memref1 *pos, lapis_memref1 *crd,
                    lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *b, lapis_memref1 *dinv, double tol,
                    size_t maxiter) {
  clear_error();
  LAPIS_TRY(require_init());
  CsrArgs a;
  LAPIS_TRY(check_csr(pos, crd, val, spec, &a));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(b, "b")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(dinv, "dinv")));
  const int64_t n = b->sizes[0];
  if (a.nrows != n || a.ncols != n || dinv->sizes[0] != n) return fail(LAPIS_EBADSHAPE, "pcg: A, b, dinv sizes differ");
  if (ret0 == nullptr || *ret0 == nullptr) return fail(LAPIS_EBADARG, "pcg: null result slot");
  cudaStream_t st = nullptr;
  DeviceCsr d;
  LAPIS_TRY(upload_csr<I>(pos, crd, val, a, &d, st));
  DevBuf db, ddinv, dx;
  LAPIS_TRY(db.alloc((size_t)n * 8));
  LAPIS_TRY(ddinv.alloc((size_t)n * 8));
  LAPIS_TRY(dx.alloc((size_t)n * 8));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(db.p, elem_ptr<double>(b), (size_t)n * 8, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(ddinv.p, elem_ptr<double>(dinv), (size_t)n * 8, cudaMemcpyHostToDevice, st));
  uint64_t iters = 0;
  double relres = 0.0;
  LAPIS_TRY(lapis_b200_pcg_f64(d.h, static_cast<const double *>(db.p), static_cast<const double *>(ddinv.p), tol,
                               (uint64_t)maxiter, static_cast<double *>(dx.p), &iters, &relres, st));
  // x is a new tensor of the module: owned here until lapis_finalize (LAPISSupport.hpp:93-120).
  double *hx = static_cast<double *>(std::malloc(n > 0 ? (size_t)n * 8 : 8));
  if (hx == nullptr) return fail(LAPIS_ECUDA, "pcg: host allocation failed");
  g_alive_host.push_back(hx);
  LAPIS_CUDA_TRY(cudaMemcpyAsync(hx, dx.p, (size_t)n * 8, cudaMemcpyDeviceToHost, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  lapis_memref1 out;
  out.basePtr = hx;
  out.data = hx;
  out.offset = 0;
  out.sizes[0] = n;
  out.strides[0] = 1;
  **ret0 = out;
  if (ret1) *ret1 = (size_t)iters;
  if (ret2) *ret2 = relres;
  return LAPIS_OK;
}

// A result vector owned by the module until lapis_finalize (LAPISSupport.hpp:93-120), filled from the device.
static int result_vector(const void *d_src, int64_t n, lapis_memref1 *out, cudaStream_t st) {
  double *hx = static_cast<double *>(std::malloc(n > 0 ? (size_t)n * 8 : 8));
  if (hx == nullptr) return fail(LAPIS_ECUDA, "host allocation failed");
  g_alive_host.push_back(hx);
  if (n > 0) LAPIS_CUDA_TRY(cudaMemcpyAsync(hx, d_src, (size_t)n * 8, cudaMemcpyDeviceToHost, st));
  out->basePtr = hx;
  out->data = hx;
  out->offset = 0;
  out->sizes[0] = n;
  out->strides[0] = 1;
  return LAPIS_OK;
}

// examples/hitting_times.py:151-194 (@mht), call at :216
template <typename I>
static int mht_host(lapis_memref1 **ret0, lapis_memref1 **ret1, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                    const lapis_csr_spec *spec, lapis_memref1 *mask, lapis_memref1 *dvec, double alpha, double tol,
                    size_t maxiter) {
  clear_error();
  LAPIS_TRY(require_init());
  CsrArgs a;
  LAPIS_TRY(check_csr(pos, crd, val, spec, &a));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(mask, "mask")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(dvec, "d")));
  const int64_t n = dvec->sizes[0];
  if (a.nrows != n || a.ncols != n || mask->sizes[0] != n) return fail(LAPIS_EBADSHAPE, "mht: A, mask, d sizes differ");
  if (ret0 == nullptr || *ret0 == nullptr || ret1 == nullptr || *ret1 == nullptr)
    return fail(LAPIS_EBADARG, "mht: null result slot");
  cudaStream_t st = nullptr;
  DeviceCsr d;
  LAPIS_TRY(upload_csr<I>(pos, crd, val, a, &d, st));
  DevBuf dmask, dd, dm1, dm2;
  LAPIS_TRY(dmask.alloc((size_t)n * 8));
  LAPIS_TRY(dd.alloc((size_t)n * 8));
  LAPIS_TRY(dm1.alloc((size_t)n * 8));
  LAPIS_TRY(dm2.alloc((size_t)n * 8));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dmask.p, elem_ptr<double>(mask), (size_t)n * 8, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dd.p, elem_ptr<double>(dvec), (size_t)n * 8, cudaMemcpyHostToDevice, st));
  LAPIS_TRY(lapis_b200_mht_f64(d.h, static_cast<const double *>(dmask.p), static_cast<const double *>(dd.p), alpha, tol,
                               (uint64_t)maxiter, static_cast<double *>(dm1.p), static_cast<double *>(dm2.p), nullptr,
                               nullptr, st));
  LAPIS_TRY(result_vector(dm1.p, n, *ret0, st));
  LAPIS_TRY(result_vector(dm2.p, n, *ret1, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  return LAPIS_OK;
}

// examples/hitting_times.py:196-218 (@normalize_mom2), call at :218
static int normalize_mom2_host(lapis_memref1 **ret0, lapis_memref1 *mom1, lapis_memref1 *mom2) {
  clear_error();
  LAPIS_TRY(require_init());
  LAPIS_TRY((check_contig<lapis_memref1, 1>(mom1, "mom1")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(mom2, "mom2")));
  const int64_t n = mom1->sizes[0];
  if (mom2->sizes[0] != n) return fail(LAPIS_EBADSHAPE, "normalize_mom2: lengths differ");
  if (ret0 == nullptr || *ret0 == nullptr) return fail(LAPIS_EBADARG, "normalize_mom2: null result slot");
  cudaStream_t st = nullptr;
  DevBuf d1, d2, dout;
  LAPIS_TRY(d1.alloc((size_t)n * 8));
  LAPIS_TRY(d2.alloc((size_t)n * 8));
  LAPIS_TRY(dout.alloc((size_t)n * 8));
  if (n > 0) {
    LAPIS_CUDA_TRY(cudaMemcpyAsync(d1.p, elem_ptr<double>(mom1), (size_t)n * 8, cudaMemcpyHostToDevice, st));
    LAPIS_CUDA_TRY(cudaMemcpyAsync(d2.p, elem_ptr<double>(mom2), (size_t)n * 8, cudaMemcpyHostToDevice, st));
  }
  LAPIS_TRY(lapis_b200_normalize_mom2_f64(n, static_cast<const double *>(d1.p), static_cast<const double *>(d2.p),
                                          static_cast<double *>(dout.p), st));
  LAPIS_TRY(result_vector(dout.p, n, *ret0, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  return LAPIS_OK;
}

// examples/bspmm.py:26-52, call at :103
template <typename I>
static int bspmm_host(lapis_memref3 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                      const lapis_csrv_spec *spec, lapis_memref3 *B) {
  clear_error();
  LAPIS_TRY(require_init());
  LAPIS_TRY((check_contig<lapis_memref1, 1>(pos, "pos")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(crd, "crd")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(val, "val")));
  LAPIS_TRY((check_contig<lapis_memref3, 3>(B, "B")));
  if (spec == nullptr) return fail(LAPIS_EBADARG, "null storage specifier");
  if (ret0 == nullptr || *ret0 == nullptr) return fail(LAPIS_EBADARG, "bspmm: null result slot");
  const int64_t n1 = spec->dims[0], n2 = spec->dims[1], nh = spec->dims[2];
  const int64_t npos = spec->mem_sizes[0], nnz = spec->mem_sizes[1], nval = spec->mem_sizes[2];
  if (n1 < 0 || n2 < 0 || nh < 0) return fail(LAPIS_EBADSHAPE, "negative tensor dimension");
  if (npos != n1 + 1 || pos->sizes[0] < npos) return fail(LAPIS_EBADSHAPE, "pos must have rows+1 entries");
  if (nval != nnz * nh || crd->sizes[0] < nnz || val->sizes[0] < nval)
    return fail(LAPIS_EBADSHAPE, "crd/val shorter than the specifier says");
  if (B->sizes[0] != n2 || B->sizes[2] != nh) return fail(LAPIS_EBADSHAPE, "bspmm: B must be [n2, dh, nh]");
  const int64_t dh = B->sizes[1];
  const I *hpos = elem_ptr<I>(pos);
  LAPIS_TRY(check_pos_host<I>(hpos, n1, nnz));
  const I *hcrd = elem_ptr<I>(crd);
  for (int64_t j = 0; j < nnz; ++j)
    if (hcrd[j] < 0 || (int64_t)hcrd[j] >= n2) return fail(LAPIS_EBADSHAPE, "bspmm: column index out of range at entry %lld", (long long)j);
  cudaStream_t st = nullptr;
  DevBuf dpos, dcrd, dval, dB, dC;
  const size_t bB = (size_t)n2 * dh * nh * 4, bC = (size_t)n1 * dh * nh * 4;
  LAPIS_TRY(dpos.alloc((size_t)npos * sizeof(I)));
  LAPIS_TRY(dcrd.alloc((size_t)nnz * sizeof(I)));
  LAPIS_TRY(dval.alloc((size_t)nval * 4));
  LAPIS_TRY(dB.alloc(bB));
  LAPIS_TRY(dC.alloc(bC));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dpos.p, hpos, (size_t)npos * sizeof(I), cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dcrd.p, hcrd, (size_t)nnz * sizeof(I), cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dval.p, elem_ptr<float>(val), (size_t)nval * 4, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dB.p, elem_ptr<float>(B), bB, cudaMemcpyHostToDevice, st));
  LAPIS_TRY(lapis_b200_bspmm_csrv_f32((int)sizeof(I), n1, n2, nh, dh, dpos.p, dcrd.p, static_cast<const float *>(dval.p),
                                      static_cast<const float *>(dB.p), static_cast<float *>(dC.p), 0, st));
  float *hc = static_cast<float *>(std::malloc(bC > 0 ? bC : 8));
  if (hc == nullptr) return fail(LAPIS_ECUDA, "bspmm: host allocation failed");
  g_alive_host.push_back(hc);
  if (bC > 0) LAPIS_CUDA_TRY(cudaMemcpyAsync(hc, dC.p, bC, cudaMemcpyDeviceToHost, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  lapis_memref3 out;
  out.basePtr = hc;
  out.data = hc;
  out.offset = 0;
  out.sizes[0] = n1;
  out.sizes[1] = dh;
  out.sizes[2] = nh;
  out.strides[0] = dh * nh;
  out.strides[1] = nh;
  out.strides[2] = 1;
  **ret0 = out;
  return LAPIS_OK;
}

// examples/spmm_dcsr_opdsl.py:59-101, call at :160 (decomposed arguments)
template <typename I>
static int spmm_dcsr_host(lapis_memref2 **ret0, lapis_memref1 *p1, lapis_memref1 *i1, lapis_memref1 *p2, lapis_memref1 *i2,
                          lapis_memref1 *val, const lapis_dcsr_spec *spec, lapis_memref2 *B, lapis_memref2 *C) {
  clear_error();
  LAPIS_TRY(require_init());
  LAPIS_TRY((check_contig<lapis_memref1, 1>(p1, "p1")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(i1, "i1")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(p2, "p2")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(i2, "i2")));
  LAPIS_TRY((check_contig<lapis_memref1, 1>(val, "val")));
  LAPIS_TRY((check_contig<lapis_memref2, 2>(B, "B")));
  LAPIS_TRY((check_contig<lapis_memref2, 2>(C, "C")));
  if (spec == nullptr) return fail(LAPIS_EBADARG, "null storage specifier");
  const int64_t nrows = spec->dims[0], ncols = spec->dims[1];
  const int64_t nstored = spec->mem_sizes[1], nnz = spec->mem_sizes[4];
  if (nrows < 0 || ncols < 0) return fail(LAPIS_EBADSHAPE, "negative matrix dimension");
  if (spec->mem_sizes[0] != 2 || p1->sizes[0] < 2 || spec->mem_sizes[2] != nstored + 1 || p2->sizes[0] < nstored + 1 ||
      i1->sizes[0] < nstored || spec->mem_sizes[3] != nnz || i2->sizes[0] < nnz || val->sizes[0] < nnz)
    return fail(LAPIS_EBADSHAPE, "spmm_dcsr: buffers do not match the specifier");
  const int64_t k = B->sizes[1];
  if (B->sizes[0] != ncols || C->sizes[0] != nrows || C->sizes[1] != k) return fail(LAPIS_EBADSHAPE, "spmm_dcsr: B/C shape mismatch");
  const I *hp1 = elem_ptr<I>(p1), *hi1 = elem_ptr<I>(i1), *hp2 = elem_ptr<I>(p2), *hi2 = elem_ptr<I>(i2);
  if (hp1[0] != 0 || (int64_t)hp1[1] != nstored) return fail(LAPIS_EBADSHAPE, "spmm_dcsr: p1 must be {0, stored rows}");
  LAPIS_TRY(check_pos_host<I>(hp2, nstored, nnz));
  for (int64_t r = 0; r < nstored; ++r)  // ascending row numbers: equal ones are adjacent and one warp takes the run
    if (hi1[r] < 0 || (int64_t)hi1[r] >= nrows || (r > 0 && hi1[r] < hi1[r - 1]))
      return fail(LAPIS_EBADSHAPE, "spmm_dcsr: stored row numbers must ascend within [0, rows)");
  for (int64_t j = 0; j < nnz; ++j)
    if (hi2[j] < 0 || (int64_t)hi2[j] >= ncols) return fail(LAPIS_EBADSHAPE, "spmm_dcsr: column index out of range at entry %lld", (long long)j);
  cudaStream_t st = nullptr;
  DevBuf di1, dp2, di2, dval, dB, dC;
  const size_t bB = (size_t)ncols * k * 8, bC = (size_t)nrows * k * 8;
  LAPIS_TRY(di1.alloc((size_t)nstored * sizeof(I)));
  LAPIS_TRY(dp2.alloc((size_t)(nstored + 1) * sizeof(I)));
  LAPIS_TRY(di2.alloc((size_t)nnz * sizeof(I)));
  LAPIS_TRY(dval.alloc((size_t)nnz * 8));
  LAPIS_TRY(dB.alloc(bB));
  LAPIS_TRY(dC.alloc(bC));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(di1.p, hi1, (size_t)nstored * sizeof(I), cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dp2.p, hp2, (size_t)(nstored + 1) * sizeof(I), cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(di2.p, hi2, (size_t)nnz * sizeof(I), cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dval.p, elem_ptr<double>(val), (size_t)nnz * 8, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dB.p, elem_ptr<double>(B), bB, cudaMemcpyHostToDevice, st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(dC.p, elem_ptr<double>(C), bC, cudaMemcpyHostToDevice, st));
  LAPIS_TRY(lapis_b200_spmm_dcsr_f64((int)sizeof(I), nrows, ncols, nstored, k, di1.p, dp2.p, di2.p,
                                     static_cast<const double *>(dval.p), static_cast<const double *>(dB.p),
                                     static_cast<double *>(dC.p), st));
  LAPIS_CUDA_TRY(cudaMemcpyAsync(elem_ptr<double>(C), dC.p, bC, cudaMemcpyDeviceToHost, st));
  LAPIS_CUDA_TRY(cudaStreamSynchronize(st));
  if (ret0 != nullptr && *ret0 != nullptr) **ret0 = *C;
  return LAPIS_OK;
}

}  // namespace lapis_b200

using namespace lapis_b200;

extern "C" int lapis_last_error(void) { return g_status; }
extern "C" const char *lapis_last_error_message(void) { return g_message; }

extern "C" void lapis_initialize(void) {
  clear_error();
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev <= 0) {
    fail(LAPIS_ECUDA, "lapis_initialize: no usable CUDA device (%s); this library has no CPU path",
         e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    return;
  }
  e = cudaFree(nullptr);  // brings the primary context up, as Kokkos::initialize does (:4289)
  if (e != cudaSuccess) {
    fail(LAPIS_ECUDA, "lapis_initialize: %s", cudaGetErrorString(e));
    return;
  }
  ++g_init_count;
}

extern "C" void lapis_finalize(void) {
  clear_error();
  if (g_init_count <= 0) return;
  if (--g_init_count == 0) {
    for (void *p : g_alive_host) std::free(p);
    g_alive_host.clear();
    cudaDeviceSynchronize();
  }
}

extern "C" void py_spmv_f64_i32(lapis_memref1 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                                const lapis_csr_spec *spec, lapis_memref1 *x, lapis_memref1 *y) {
  spmv_host<int32_t>(ret0, pos, crd, val, spec, x, y);
}
extern "C" void py_spmv_f64_i64(lapis_memref1 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                                const lapis_csr_spec *spec, lapis_memref1 *x, lapis_memref1 *y) {
  spmv_host<int64_t>(ret0, pos, crd, val, spec, x, y);
}
extern "C" void py_spmm_f64_i32(lapis_memref2 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                                const lapis_csr_spec *spec, lapis_memref2 *B, lapis_memref2 *C) {
  spmm_host<int32_t>(ret0, pos, crd, val, spec, B, C);
}
extern "C" void py_spmm_f64_i64(lapis_memref2 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                                const lapis_csr_spec *spec, lapis_memref2 *B, lapis_memref2 *C) {
  spmm_host<int64_t>(ret0, pos, crd, val, spec, B, C);
}

extern "C" void py_matmul_f32(lapis_memref2 **ret0, lapis_memref2 *A, lapis_memref2 *B, lapis_memref2 *C) {
  clear_error();
  if (require_init() != LAPIS_OK) return;
  if (check_contig<lapis_memref2, 2>(A, "A") || check_contig<lapis_memref2, 2>(B, "B") ||
      check_contig<lapis_memref2, 2>(C, "C"))
    return;
  // cf.assert of benchmarks/gemm/gemm.mlir:10-11
  if (A->sizes[1] != B->sizes[0]) {
    fail(LAPIS_EBADSHAPE, "mismatching contracting dimension for torch.aten.mm");
    return;
  }
  if (C->sizes[0] != A->sizes[0] || C->sizes[1] != B->sizes[1]) {
    fail(LAPIS_EBADSHAPE, "matmul: output shape mismatch");
    return;
  }
  if (gemm_host(1, A->sizes[0], B->sizes[1], A->sizes[1], elem_ptr<float>(A), elem_ptr<float>(B), elem_ptr<float>(C)))
    return;
  if (ret0 != nullptr && *ret0 != nullptr) **ret0 = *C;
}

extern "C" void py_batch_matmul_f32(lapis_memref3 **ret0, lapis_memref3 *A, lapis_memref3 *B, lapis_memref3 *C) {
  clear_error();
  if (require_init() != LAPIS_OK) return;
  if (check_contig<lapis_memref3, 3>(A, "A") || check_contig<lapis_memref3, 3>(B, "B") ||
      check_contig<lapis_memref3, 3>(C, "C"))
    return;
  // cf.assert pair of benchmarks/batched_gemm/batched_gemm.mlir:14-20
  if (A->sizes[0] != B->sizes[0] || A->sizes[2] != B->sizes[1]) {
    fail(LAPIS_EBADSHAPE, "mismatching contracting dimension");
    return;
  }
  if (C->sizes[0] != A->sizes[0] || C->sizes[1] != A->sizes[1] || C->sizes[2] != B->sizes[2]) {
    fail(LAPIS_EBADSHAPE, "batch_matmul: output shape mismatch");
    return;
  }
  if (gemm_host(A->sizes[0], A->sizes[1], B->sizes[2], A->sizes[2], elem_ptr<float>(A), elem_ptr<float>(B),
                elem_ptr<float>(C)))
    return;
  if (ret0 != nullptr && *ret0 != nullptr) **ret0 = *C;
}

extern "C" void py_pcg_f64_i32(lapis_memref1 **ret0, size_t *ret1, double *ret2, lapis_memref1 *pos,
                               lapis_memref1 *crd, lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *b,
                               lapis_memref1 *dinv, double tol, size_t maxiter) {
  pcg_host<int32_t>(ret0, ret1, ret2, pos, crd, val, spec, b, dinv, tol, maxiter);
}
extern "C" void py_pcg_f64_i64(lapis_memref1 **ret0, size_t *ret1, double *ret2, lapis_memref1 *pos,
                               lapis_memref1 *crd, lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *b,
                               lapis_memref1 *dinv, double tol, size_t maxiter) {
  pcg_host<int64_t>(ret0, ret1, ret2, pos, crd, val, spec, b, dinv, tol, maxiter);
}

extern "C" void py_mht_f64_i32(lapis_memref1 **ret0, lapis_memref1 **ret1, lapis_memref1 *pos, lapis_memref1 *crd,
                               lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *mask, lapis_memref1 *d,
                               double alpha, double tol, size_t maxiter) {
  mht_host<int32_t>(ret0, ret1, pos, crd, val, spec, mask, d, alpha, tol, maxiter);
}
extern "C" void py_mht_f64_i64(lapis_memref1 **ret0, lapis_memref1 **ret1, lapis_memref1 *pos, lapis_memref1 *crd,
                               lapis_memref1 *val, const lapis_csr_spec *spec, lapis_memref1 *mask, lapis_memref1 *d,
                               double alpha, double tol, size_t maxiter) {
  mht_host<int64_t>(ret0, ret1, pos, crd, val, spec, mask, d, alpha, tol, maxiter);
}
extern "C" void py_normalize_mom2_f64(lapis_memref1 **ret0, lapis_memref1 *mom1, lapis_memref1 *mom2) {
  normalize_mom2_host(ret0, mom1, mom2);
}

extern "C" void py_bspmm_f32_i32(lapis_memref3 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                                 const lapis_csrv_spec *spec, lapis_memref3 *B) {
  bspmm_host<int32_t>(ret0, pos, crd, val, spec, B);
}
extern "C" void py_bspmm_f32_i64(lapis_memref3 **ret0, lapis_memref1 *pos, lapis_memref1 *crd, lapis_memref1 *val,
                                 const lapis_csrv_spec *spec, lapis_memref3 *B) {
  bspmm_host<int64_t>(ret0, pos, crd, val, spec, B);
}
extern "C" void py_spmm_dcsr_f64_i32(lapis_memref2 **ret0, lapis_memref1 *p1, lapis_memref1 *i1, lapis_memref1 *p2,
                                     lapis_memref1 *i2, lapis_memref1 *val, const lapis_dcsr_spec *spec,
                                     lapis_memref2 *B, lapis_memref2 *C) {
  spmm_dcsr_host<int32_t>(ret0, p1, i1, p2, i2, val, spec, B, C);
}
extern "C" void py_spmm_dcsr_f64_i64(lapis_memref2 **ret0, lapis_memref1 *p1, lapis_memref1 *i1, lapis_memref1 *p2,
                                     lapis_memref1 *i2, lapis_memref1 *val, const lapis_dcsr_spec *spec,
                                     lapis_memref2 *B, lapis_memref2 *C) {
  spmm_dcsr_host<int64_t>(ret0, p1, i1, p2, i2, val, spec, B, C);
}

// ---- host-side partition rule ------------------------------------------------
template <typename I>
static void partition_rows(int64_t nrows, const I *pos, int G, int64_t *bounds) {
  const int64_t base = (int64_t)pos[0];
  const int64_t nnz = (int64_t)pos[nrows] - base;
  for (int g = 0; g <= G; ++g) {
    if (g == G) {
      bounds[g] = nrows;
      continue;
    }
    const int64_t target = base + (int64_t)(((__int128)nnz * g) / G);
    int64_t lo = 0, hi = nrows;
    while (lo < hi) {
      const int64_t mid = lo + (hi - lo) / 2;
      if ((int64_t)pos[mid] < target)
        lo = mid + 1;
      else
        hi = mid;
    }
    bounds[g] = lo;
  }
}

extern "C" int lapis_b200_validate_csr_host(int idx_bytes, int64_t nrows, int64_t ncols, int64_t nnz, const void *pos,
                                           const void *crd) {
  clear_error();
  if ((idx_bytes != 4 && idx_bytes != 8) || nrows < 0 || ncols < 0 || nnz < 0 || pos == nullptr || (nnz > 0 && crd == nullptr))
    return fail(LAPIS_EBADARG, "validate_csr_host: bad arguments");
  if (idx_bytes == 4) {
    LAPIS_TRY(check_pos_host<int32_t>(static_cast<const int32_t *>(pos), nrows, nnz));
    return check_crd_host<int32_t>(static_cast<const int32_t *>(crd), nnz, ncols);
  }
  LAPIS_TRY(check_pos_host<int64_t>(static_cast<const int64_t *>(pos), nrows, nnz));
  return check_crd_host<int64_t>(static_cast<const int64_t *>(crd), nnz, ncols);
}

extern "C" int lapis_b200_partition_rows(int idx_bytes, int64_t nrows, const void *pos, int G, int64_t *bounds) {
  clear_error();
  if (pos == nullptr || bounds == nullptr || G < 1 || nrows < 0) return fail(LAPIS_EBADARG, "partition_rows: bad arguments");
  if (idx_bytes == 4)
    partition_rows<int32_t>(nrows, static_cast<const int32_t *>(pos), G, bounds);
  else if (idx_bytes == 8)
    partition_rows<int64_t>(nrows, static_cast<const int64_t *>(pos), G, bounds);
  else
    return fail(LAPIS_EBADARG, "partition_rows: idx_bytes must be 4 or 8");
  return LAPIS_OK;
}
