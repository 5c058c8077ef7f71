// A C++ driver in the style of the reference's benchmark drivers (benchmarks/spmv/main.cpp,
// benchmarks/gemm/main.cpp in the LAPIS project) written against include/lapis_b200.hpp:
// DualViews that stay on the device, repeated calls, results read back with syncHost().
#include <cmath>
#include <cstdio>
#include <vector>

#include "lapis_b200.hpp"

using IntDV = LAPIS::DualView<int32_t *, Kokkos::LayoutRight>;
using VecDV = LAPIS::DualView<double *, Kokkos::LayoutRight>;

static int fail(const char *what) {
  std::printf("FAIL: %s\n", what);
  return 1;
}

int main() {
  lapis_initialize();
  if (lapis_last_error() != LAPIS_OK) return fail(lapis_last_error_message());
  int rc = 0;
  {
    // the 5 x 5 known answer of examples/spmv_noalloc.py:16-32
    const int32_t rowptrs[] = {0, 1, 5, 6, 8, 8}, colinds[] = {1, 0, 2, 3, 4, 2, 0, 1};
    const double values[] = {1.1, 0.3, 2.2, 3.7, -4, -19, -2, 1}, expect[] = {1.1, 2.2, -19, -1, 0};
    IntDV pos("pos", 6), crd("crd", 8);
    VecDV val("val", 8), x("x", 5), y("y", 5);
    for (int i = 0; i < 6; i++) pos.host_view()(i) = rowptrs[i];
    for (int i = 0; i < 8; i++) crd.host_view()(i) = colinds[i], val.host_view()(i) = values[i];
    for (int i = 0; i < 5; i++) x.host_view()(i) = 1.0;
    pos.modifyHost(); crd.modifyHost(); val.modifyHost(); x.modifyHost();
    Struct0 shape = {{5, 5}, {6, 8, 8}};
    for (int trial = 1; trial <= 3; trial++) {   // y accumulates: trial * expect
      spmv(pos, crd, val, shape, x, y);
      cudaDeviceSynchronize();
      y.syncHost();
      for (int i = 0; i < 5; i++)
        if (std::fabs(y.host_view()(i) - trial * expect[i]) > 1e-12) rc |= fail("spmv known answer");
    }
  }
  {
    // dense and batched matmul: small integers, exact
    using M2 = LAPIS::DualView<float **, Kokkos::LayoutRight>;
    using M3 = LAPIS::DualView<float ***, Kokkos::LayoutRight>;
    M2 A("A", 8, 7), B("B", 7, 9), C("C", 8, 9);
    for (int i = 0; i < 8; i++) for (int k = 0; k < 7; k++) A.host_view()(i, k) = float(i + k);
    for (int k = 0; k < 7; k++) for (int j = 0; j < 9; j++) B.host_view()(k, j) = float(k - j);
    A.modifyHost(); B.modifyHost();
    forward(A, B, C);
    C.syncHost();
    for (int i = 0; i < 8; i++) for (int j = 0; j < 9; j++) {
      float s = 0; for (int k = 0; k < 7; k++) s += float(i + k) * float(k - j);
      if (C.host_view()(i, j) != s) rc |= fail("forward 2-D");
    }
    M3 A3("A", 4, 128, 128), B3("B", 4, 128, 128), C3("C", 4, 128, 128);   // tile-aligned: tensor-core path
    for (int b = 0; b < 4; b++) for (int i = 0; i < 128; i++) for (int k = 0; k < 128; k++) {
      A3.host_view()(b, i, k) = float((i + k + b) % 3);
      B3.host_view()(b, i, k) = float((i * k + b) % 2);
    }
    A3.modifyHost(); B3.modifyHost();
    forward(A3, B3, C3);
    if (lapis_b200_bgemm_status(nullptr) != LAPIS_OK) rc |= fail(lapis_last_error_message());
    C3.syncHost();
    for (int b = 0; b < 4; b++) for (int i = 0; i < 128; i += 17) for (int j = 0; j < 128; j += 13) {
      float s = 0; for (int k = 0; k < 128; k++) s += float((i + k + b) % 3) * float((k * j + b) % 2);
      if (C3.host_view()(b, i, j) != s) rc |= fail("forward 3-D");
    }
  }
  {
    // PCG on a 1-D Laplacian (tridiagonal 2, -1): converges to the exact solution
    const int n = 64;
    std::vector<int32_t> p(n + 1), c;
    std::vector<double> v;
    for (int i = 0; i < n; i++) {
      p[i] = (int32_t)c.size();
      if (i > 0) { c.push_back(i - 1); v.push_back(-1); }
      c.push_back(i); v.push_back(2);
      if (i < n - 1) { c.push_back(i + 1); v.push_back(-1); }
    }
    p[n] = (int32_t)c.size();
    IntDV pos("pos", n + 1), crd("crd", c.size());
    VecDV val("val", v.size()), b("b", n), dinv("dinv", n);
    for (int i = 0; i <= n; i++) pos.host_view()(i) = p[i];
    for (size_t i = 0; i < c.size(); i++) crd.host_view()(i) = c[i], val.host_view()(i) = v[i];
    for (int i = 0; i < n; i++) b.host_view()(i) = (i == 0 || i == n - 1) ? 1.0 : 0.0, dinv.host_view()(i) = 0.5;  // A * ones
    pos.modifyHost(); crd.modifyHost(); val.modifyHost(); b.modifyHost(); dinv.modifyHost();
    Struct0 shape = {{n, n}, {n + 1, (int64_t)c.size(), (int64_t)v.size()}};
    auto [x, iters, relres] = pcg(pos, crd, val, shape, b, dinv, 1e-12, (size_t)200);
    x.syncHost();
    if (!(relres <= 1e-12) || iters > 200) rc |= fail("pcg did not converge");
    for (int i = 0; i < n; i++) if (std::fabs(x.host_view()(i) - 1.0) > 1e-9) rc |= fail("pcg solution");
    std::printf("pcg: %zu iterations, relres %.3e\n", iters, relres);
  }
  {
    // Hitting-time moments on a 6-cycle with unit weights, node 0 absorbing: d = degree, mask[0] = 0.
    // The first moment solves mask (D - alpha A) mask m = mask d; checked by its residual on the host.
    const int n = 6;
    const double alpha = 0.9;
    IntDV pos("pos", n + 1), crd("crd", 2 * n);
    VecDV val("val", 2 * n), mask("mask", n), d("d", n);
    for (int i = 0; i < n; i++) {
      pos.host_view()(i) = 2 * i;
      const int lo = (i + n - 1) % n, hi = (i + 1) % n;
      crd.host_view()(2 * i) = lo < hi ? lo : hi;
      crd.host_view()(2 * i + 1) = lo < hi ? hi : lo;
      val.host_view()(2 * i) = val.host_view()(2 * i + 1) = 1.0;
      mask.host_view()(i) = i == 0 ? 0.0 : 1.0;
      d.host_view()(i) = 2.0;
    }
    pos.host_view()(n) = 2 * n;
    pos.modifyHost(); crd.modifyHost(); val.modifyHost(); mask.modifyHost(); d.modifyHost();
    Struct0 shape = {{n, n}, {n + 1, 2 * n, 2 * n}};
    auto [m1, m2] = mht(pos, crd, val, shape, mask, d, alpha, 1e-13, (size_t)50);
    auto sd = normalize_mom2(m1, m2);
    m1.syncHost(); m2.syncHost(); sd.syncHost(); val.syncHost();
    if (m1.host_view()(0) != 0.0) rc |= fail("mht: masked node must stay 0");
    for (int i = 1; i < n; i++) {
      const int lo = (i + n - 1) % n, hi = (i + 1) % n;
      const double nb = (lo ? m1.host_view()(lo) : 0.0) + (hi ? m1.host_view()(hi) : 0.0);
      if (std::fabs(2.0 * m1.host_view()(i) - alpha * nb - 2.0) > 1e-9) rc |= fail("mht: first moment residual");
      const double var = m2.host_view()(i) - m1.host_view()(i) * m1.host_view()(i);
      if (std::fabs(sd.host_view()(i) - std::sqrt(var)) > 1e-12) rc |= fail("normalize_mom2");
    }
    for (int j = 0; j < 2 * n; j++) if (val.host_view()(j) != 1.0) rc |= fail("mht changed the caller's values");
    std::printf("mht: m1[1] = %.6f, m1[3] = %.6f\n", m1.host_view()(1), m1.host_view()(3));
  }
  lapis_finalize();
  std::printf(rc == 0 ? "driver ok\n" : "driver failed\n");
  return rc;
}
