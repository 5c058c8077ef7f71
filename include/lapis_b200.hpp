// C++ call surface of an emitted LAPIS module, without Kokkos.
//
// A LAPIS-emitted module is also used from C++: drivers include the emitted header and call
// `spmv(DualView...)`, `forward(DualView...)` directly, keeping data on the device between calls
// (benchmarks/spmv/main.cpp:42-62, benchmarks/gemm/main.cpp:18-35, benchmarks/batched_gemm/main.cpp:22-38
// in the LAPIS project).  This header gives such a driver the same names over liblapis_b200.so:
//
//   LAPIS::DualView<T*, Kokkos::LayoutRight>    host + device copy of a rank-1..3 array with the
//                                               modify / sync protocol of LAPISSupport.hpp:136-426
//                                               (modified flags, lazy deep copy on syncHost / syncDevice)
//   Struct0                                     the flattened CSR storage specifier
//                                               (mlir/lib/Target/KokkosCpp/TranslateToKokkosCpp.cpp:4495-4546)
//   lapis_initialize / lapis_finalize           from lapis_b200.h
//   spmv, spmm, forward, pcg, mht, normalize_mom2   the emitted functions of the accelerated path
//
// What is not here: Kokkos itself (views are plain pointer + extents, no subviews, LayoutRight only),
// Kokkos::Timer / fill_random used by the drivers' set-up code, and any function outside the
// accelerated path.  Errors throw std::runtime_error instead of Kokkos::abort.
#ifndef LAPIS_B200_HPP
#define LAPIS_B200_HPP

#include <cuda_runtime_api.h>

#include <array>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>
#include <type_traits>

#include "lapis_b200.h"

#ifndef KOKKOS_CORE_HPP
namespace Kokkos {
struct LayoutRight {};
}  // namespace Kokkos
#endif

namespace LAPIS {

inline void check(int status, const char *what) {
  if (status != LAPIS_OK) throw std::runtime_error(std::string(what) + ": " + lapis_last_error_message());
}
inline void check_cuda(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// Rank-R view over contiguous row-major memory (what the emitted code gets from device_view()/host_view()).
template <typename T, int R>
struct View {
  T *ptr = nullptr;
  std::array<size_t, 3> ext{{1, 1, 1}};
  T *data() const { return ptr; }
  size_t extent(int i) const { return i < R ? ext[i] : 1; }
  size_t size() const { return ext[0] * ext[1] * ext[2]; }
  T &operator()(size_t i) const { return ptr[i]; }
  T &operator()(size_t i, size_t j) const { return ptr[i * ext[1] + j]; }
  T &operator()(size_t i, size_t j, size_t k) const { return ptr[(i * ext[1] + j) * ext[2] + k]; }
};

template <typename D>
struct DataTraits;
template <typename T>
struct DataTraits<T *> {
  using value_type = T;
  static constexpr int rank = 1;
};
template <typename T>
struct DataTraits<T **> {
  using value_type = T;
  static constexpr int rank = 2;
};
template <typename T>
struct DataTraits<T ***> {
  using value_type = T;
  static constexpr int rank = 3;
};

// Host + device copy with modify flags shared by all copies of the handle (LAPISSupport.hpp:136-426).
template <typename DataType, typename Layout = Kokkos::LayoutRight>
class DualView {
 public:
  using value_type = typename DataTraits<DataType>::value_type;
  static constexpr int rank = DataTraits<DataType>::rank;
  using HostView = View<value_type, rank>;
  using DeviceView = View<value_type, rank>;

  DualView() = default;
  // Allocates both copies, zero-initialised like a labelled Kokkos::View.
  explicit DualView(const std::string &label, size_t n0 = 1, size_t n1 = 1, size_t n2 = 1) : impl_(std::make_shared<Impl>()) {
    impl_->label = label;
    impl_->ext = {{n0, rank > 1 ? n1 : 1, rank > 2 ? n2 : 1}};
    const size_t bytes = impl_->bytes();
    impl_->host = static_cast<value_type *>(std::calloc(bytes ? bytes : 1, 1));
    check_cuda(cudaMalloc(reinterpret_cast<void **>(&impl_->dev), bytes ? bytes : 1), "DualView cudaMalloc");
    check_cuda(cudaMemset(impl_->dev, 0, bytes), "DualView cudaMemset");
    impl_->own_host = impl_->own_dev = true;
  }
  // Wraps caller-owned host memory (the py_ wrappers do this with unmanaged views); device copy allocated here.
  static DualView from_host(value_type *host, size_t n0, size_t n1 = 1, size_t n2 = 1) {
    DualView v;
    v.impl_ = std::make_shared<Impl>();
    v.impl_->ext = {{n0, rank > 1 ? n1 : 1, rank > 2 ? n2 : 1}};
    v.impl_->host = host;
    const size_t bytes = v.impl_->bytes();
    check_cuda(cudaMalloc(reinterpret_cast<void **>(&v.impl_->dev), bytes ? bytes : 1), "DualView cudaMalloc");
    v.impl_->own_dev = true;
    v.impl_->modified_host = true;
    return v;
  }

  size_t extent(int i) const { return i < rank ? impl_->ext[i] : 1; }
  HostView host_view() const { return HostView{impl_->host, impl_->ext}; }
  DeviceView device_view() const { return DeviceView{impl_->dev, impl_->ext}; }
  void modifyHost() { impl_->modified_host = true; impl_->modified_dev = false; }
  void modifyDevice() { impl_->modified_dev = true; impl_->modified_host = false; ++impl_->device_generation; }
  void syncHost() {
    if (impl_->modified_dev) {
      check_cuda(cudaMemcpy(impl_->host, impl_->dev, impl_->bytes(), cudaMemcpyDeviceToHost), "DualView syncHost");
      impl_->modified_dev = false;
    }
  }
  void syncDevice() {
    if (impl_->modified_host) {
      check_cuda(cudaMemcpy(impl_->dev, impl_->host, impl_->bytes(), cudaMemcpyHostToDevice), "DualView syncDevice");
      impl_->modified_host = false;
      ++impl_->device_generation;
    }
  }
  // Changes whenever the device copy may have changed: lets callers cache work derived from it.
  uint64_t device_generation() const { return impl_->device_generation; }
  explicit operator bool() const { return static_cast<bool>(impl_); }

 private:
  struct Impl {
    std::string label;
    std::array<size_t, 3> ext{{1, 1, 1}};
    value_type *host = nullptr, *dev = nullptr;
    bool own_host = false, own_dev = false, modified_host = false, modified_dev = false;
    uint64_t device_generation = 0;
    size_t bytes() const { return ext[0] * ext[1] * ext[2] * sizeof(value_type); }
    ~Impl() {
      if (own_host) std::free(host);
      if (own_dev) cudaFree(dev);
    }
  };
  std::shared_ptr<Impl> impl_;
};

}  // namespace LAPIS

// {{rows, cols}, {len(pos), len(crd), len(val)}} -- benchmarks/spmv/main.cpp:48-51.
struct Struct0 {
  std::array<int64_t, 2> m0;
  std::array<int64_t, 3> m1;
};

namespace lapis_b200_detail {
template <typename I>
struct PlanCache {  // one cached handle per index type: rebuilt when the matrix arrays change
  lapis_b200_csr_t handle = nullptr;
  const void *pos = nullptr, *crd = nullptr, *val = nullptr;
  uint64_t gen = ~0ull;
  int64_t rows = -1;
  ~PlanCache() { lapis_b200_csr_destroy(handle); }
};
template <typename I>
inline lapis_b200_csr_t plan_for(LAPIS::DualView<I *, Kokkos::LayoutRight> &pos, LAPIS::DualView<I *, Kokkos::LayoutRight> &crd,
                                 LAPIS::DualView<double *, Kokkos::LayoutRight> &val, const Struct0 &shape) {
  static_assert(sizeof(I) == 4 || sizeof(I) == 8, "pos/crd must be 32- or 64-bit integers");
  static PlanCache<I> cache;
  pos.syncDevice();
  crd.syncDevice();
  val.syncDevice();
  const void *p = pos.device_view().data(), *c = crd.device_view().data(), *v = val.device_view().data();
  const uint64_t gen = pos.device_generation() * 1315423911ull + crd.device_generation();
  if (cache.handle == nullptr || cache.pos != p || cache.crd != c || cache.val != v || cache.gen != gen ||
      cache.rows != shape.m0[0]) {
    lapis_b200_csr_destroy(cache.handle);
    cache.handle = nullptr;
    LAPIS::check(lapis_b200_csr_create(&cache.handle, (int)sizeof(I), shape.m0[0], shape.m0[1], p, c,
                                       static_cast<const double *>(v), nullptr),
                 "spmv: csr_create");
    LAPIS::check(lapis_b200_csr_tune(cache.handle, nullptr), "spmv: csr_tune");
    cache.pos = p;
    cache.crd = c;
    cache.val = v;
    cache.gen = gen;
    cache.rows = shape.m0[0];
  }
  return cache.handle;
}
}  // namespace lapis_b200_detail

// y += A x; returns y (device-modified), as the emitted `spmv` does (benchmarks/spmv/main.cpp:2-11).
template <typename I>
inline LAPIS::DualView<double *, Kokkos::LayoutRight> spmv(LAPIS::DualView<I *, Kokkos::LayoutRight> pos,
                                                          LAPIS::DualView<I *, Kokkos::LayoutRight> crd,
                                                          LAPIS::DualView<double *, Kokkos::LayoutRight> val, Struct0 shape,
                                                          LAPIS::DualView<double *, Kokkos::LayoutRight> x,
                                                          LAPIS::DualView<double *, Kokkos::LayoutRight> y) {
  if ((int64_t)x.extent(0) != shape.m0[1] || (int64_t)y.extent(0) != shape.m0[0])
    throw std::runtime_error("spmv: x/y length mismatch");
  lapis_b200_csr_t h = lapis_b200_detail::plan_for<I>(pos, crd, val, shape);
  x.syncDevice();
  y.syncDevice();
  LAPIS::check(lapis_b200_spmv_f64(h, x.device_view().data(), y.device_view().data(), 1, nullptr), "spmv");
  y.modifyDevice();
  return y;
}

// C += A B with CSR A, dense row-major B and C.
template <typename I>
inline LAPIS::DualView<double **, Kokkos::LayoutRight> spmm(LAPIS::DualView<I *, Kokkos::LayoutRight> pos,
                                                           LAPIS::DualView<I *, Kokkos::LayoutRight> crd,
                                                           LAPIS::DualView<double *, Kokkos::LayoutRight> val, Struct0 shape,
                                                           LAPIS::DualView<double **, Kokkos::LayoutRight> B,
                                                           LAPIS::DualView<double **, Kokkos::LayoutRight> C) {
  if ((int64_t)B.extent(0) != shape.m0[1] || (int64_t)C.extent(0) != shape.m0[0] || B.extent(1) != C.extent(1))
    throw std::runtime_error("spmm: B/C shape mismatch");
  lapis_b200_csr_t h = lapis_b200_detail::plan_for<I>(pos, crd, val, shape);
  B.syncDevice();
  C.syncDevice();
  LAPIS::check(lapis_b200_spmm_f64(h, (int64_t)B.extent(1), B.device_view().data(), C.device_view().data(), 1, nullptr), "spmm");
  C.modifyDevice();
  return C;
}

// C += A B (benchmarks/gemm/main.cpp:29-35) and C[b] += A[b] B[b] (benchmarks/batched_gemm/main.cpp:32-38).
inline LAPIS::DualView<float **, Kokkos::LayoutRight> forward(LAPIS::DualView<float **, Kokkos::LayoutRight> A,
                                                            LAPIS::DualView<float **, Kokkos::LayoutRight> B,
                                                            LAPIS::DualView<float **, Kokkos::LayoutRight> C) {
  if (A.extent(1) != B.extent(0)) throw std::runtime_error("mismatching contracting dimension for torch.aten.mm");
  if (C.extent(0) != A.extent(0) || C.extent(1) != B.extent(1)) throw std::runtime_error("forward: output shape mismatch");
  A.syncDevice();
  B.syncDevice();
  C.syncDevice();
  LAPIS::check(lapis_b200_bgemm_f32(1, (int64_t)A.extent(0), (int64_t)B.extent(1), (int64_t)A.extent(1), A.device_view().data(),
                                    B.device_view().data(), C.device_view().data(), nullptr),
               "forward");
  C.modifyDevice();
  return C;
}
inline LAPIS::DualView<float ***, Kokkos::LayoutRight> forward(LAPIS::DualView<float ***, Kokkos::LayoutRight> A,
                                                             LAPIS::DualView<float ***, Kokkos::LayoutRight> B,
                                                             LAPIS::DualView<float ***, Kokkos::LayoutRight> C) {
  if (A.extent(0) != B.extent(0) || A.extent(2) != B.extent(1)) throw std::runtime_error("mismatching contracting dimension");
  if (C.extent(0) != A.extent(0) || C.extent(1) != A.extent(1) || C.extent(2) != B.extent(2))
    throw std::runtime_error("forward: output shape mismatch");
  A.syncDevice();
  B.syncDevice();
  C.syncDevice();
  LAPIS::check(lapis_b200_bgemm_f32((int64_t)A.extent(0), (int64_t)A.extent(1), (int64_t)B.extent(2), (int64_t)A.extent(2),
                                    A.device_view().data(), B.device_view().data(), C.device_view().data(), nullptr),
               "forward");
  C.modifyDevice();
  return C;
}

// Jacobi-preconditioned CG (examples/pcg_solve.py:52-101): returns (x, iterations, relative residual).
template <typename I>
inline std::tuple<LAPIS::DualView<double *, Kokkos::LayoutRight>, size_t, double> pcg(
    LAPIS::DualView<I *, Kokkos::LayoutRight> pos, LAPIS::DualView<I *, Kokkos::LayoutRight> crd,
    LAPIS::DualView<double *, Kokkos::LayoutRight> val, Struct0 shape, LAPIS::DualView<double *, Kokkos::LayoutRight> b,
    LAPIS::DualView<double *, Kokkos::LayoutRight> dinv, double tol, size_t maxiter) {
  lapis_b200_csr_t h = lapis_b200_detail::plan_for<I>(pos, crd, val, shape);
  b.syncDevice();
  dinv.syncDevice();
  LAPIS::DualView<double *, Kokkos::LayoutRight> x("x", b.extent(0));
  uint64_t iters = 0;
  double relres = 0.0;
  LAPIS::check(lapis_b200_pcg_f64(h, b.device_view().data(), dinv.device_view().data(), tol, (uint64_t)maxiter,
                                  x.device_view().data(), &iters, &relres, nullptr),
               "pcg");
  x.modifyDevice();
  return std::make_tuple(x, (size_t)iters, relres);
}

// Hitting-time moments (examples/hitting_times.py:151-194): returns (first moment, second moment).
template <typename I>
inline std::tuple<LAPIS::DualView<double *, Kokkos::LayoutRight>, LAPIS::DualView<double *, Kokkos::LayoutRight>> mht(
    LAPIS::DualView<I *, Kokkos::LayoutRight> pos, LAPIS::DualView<I *, Kokkos::LayoutRight> crd,
    LAPIS::DualView<double *, Kokkos::LayoutRight> val, Struct0 shape, LAPIS::DualView<double *, Kokkos::LayoutRight> mask,
    LAPIS::DualView<double *, Kokkos::LayoutRight> d, double alpha, double tol, size_t maxiter) {
  lapis_b200_csr_t h = lapis_b200_detail::plan_for<I>(pos, crd, val, shape);
  mask.syncDevice();
  d.syncDevice();
  LAPIS::DualView<double *, Kokkos::LayoutRight> mom1("mom1", d.extent(0)), mom2("mom2", d.extent(0));
  LAPIS::check(lapis_b200_mht_f64(h, mask.device_view().data(), d.device_view().data(), alpha, tol, (uint64_t)maxiter,
                                  mom1.device_view().data(), mom2.device_view().data(), nullptr, nullptr, nullptr),
               "mht");
  mom1.modifyDevice();
  mom2.modifyDevice();
  return std::make_tuple(mom1, mom2);
}

// sqrt(mom2 - mom1^2) (examples/hitting_times.py:196-218).
inline LAPIS::DualView<double *, Kokkos::LayoutRight> normalize_mom2(LAPIS::DualView<double *, Kokkos::LayoutRight> mom1,
                                                                     LAPIS::DualView<double *, Kokkos::LayoutRight> mom2) {
  mom1.syncDevice();
  mom2.syncDevice();
  LAPIS::DualView<double *, Kokkos::LayoutRight> out("nm2", mom1.extent(0));
  LAPIS::check(lapis_b200_normalize_mom2_f64((int64_t)mom1.extent(0), mom1.device_view().data(), mom2.device_view().data(),
                                             out.device_view().data(), nullptr),
               "normalize_mom2");
  out.modifyDevice();
  return out;
}

#endif  // LAPIS_B200_HPP
