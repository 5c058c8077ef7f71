// MatrixMarket -> CSR reader (host code only).
//
// The step in front of the SpMV path in the reference's benchmark driver: benchmarks/spmv/main.cpp:36-38
// reads the matrix with the KokkosSparse MatrixMarket reader vendored beside it (32-bit offsets and
// ordinals, symmetric files expanded).  This is an independent implementation of the same file format
// step: coordinate files with real / integer / pattern values and general / symmetric / skew-symmetric
// storage become a CSR with ascending columns per row and duplicate entries summed, in the index width
// the caller asks for.
#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "common.h"

namespace {

struct Entry {
  int64_t row, col;
  double val;
};

std::string lower(std::string s) {
  for (char &c : s) c = (char)std::tolower((unsigned char)c);
  return s;
}

template <typename I>
int fill_csr(int64_t nrows, std::vector<Entry> &e, void **pos_out, void **crd_out, double **val_out, int64_t *nnz_out) {
  std::sort(e.begin(), e.end(), [](const Entry &a, const Entry &b) { return a.row != b.row ? a.row < b.row : a.col < b.col; });
  // merge duplicates (same row and column): values are summed, as assembling readers do
  size_t w = 0;
  for (size_t r = 0; r < e.size(); ++r) {
    if (w > 0 && e[w - 1].row == e[r].row && e[w - 1].col == e[r].col)
      e[w - 1].val += e[r].val;
    else
      e[w++] = e[r];
  }
  e.resize(w);
  I *pos = static_cast<I *>(std::calloc((size_t)nrows + 1, sizeof(I)));
  I *crd = static_cast<I *>(std::malloc(std::max<size_t>(1, e.size()) * sizeof(I)));
  double *val = static_cast<double *>(std::malloc(std::max<size_t>(1, e.size()) * sizeof(double)));
  if (!pos || !crd || !val) {
    std::free(pos);
    std::free(crd);
    std::free(val);
    return lapis_b200::fail(LAPIS_ECUDA, "read_matrix_market: out of host memory");
  }
  for (size_t k = 0; k < e.size(); ++k) {
    pos[e[k].row + 1] += 1;
    crd[k] = (I)e[k].col;
    val[k] = e[k].val;
  }
  for (int64_t r = 0; r < nrows; ++r) pos[r + 1] += pos[r];
  *pos_out = pos;
  *crd_out = crd;
  *val_out = val;
  *nnz_out = (int64_t)e.size();
  return LAPIS_OK;
}

}  // namespace

extern "C" int lapis_b200_read_matrix_market(const char *path, int idx_bytes, int64_t *nrows, int64_t *ncols,
                                             int64_t *nnz, void **pos, void **crd, double **val) {
  using lapis_b200::fail;
  lapis_b200::clear_error();
  if (!path || !nrows || !ncols || !nnz || !pos || !crd || !val) return fail(LAPIS_EBADARG, "read_matrix_market: null argument");
  if (idx_bytes != 4 && idx_bytes != 8) return fail(LAPIS_EBADARG, "read_matrix_market: idx_bytes must be 4 or 8");
  FILE *f = std::fopen(path, "r");
  if (!f) return fail(LAPIS_EBADARG, "read_matrix_market: cannot open %s: %s", path, std::strerror(errno));
  char line[1024];
  if (!std::fgets(line, sizeof(line), f)) {
    std::fclose(f);
    return fail(LAPIS_EBADSHAPE, "read_matrix_market: empty file");
  }
  char banner[64] = "", object[64] = "", format[64] = "", field[64] = "", symmetry[64] = "";
  if (std::sscanf(line, "%63s %63s %63s %63s %63s", banner, object, format, field, symmetry) != 5 ||
      lower(banner) != "%%matrixmarket" || lower(object) != "matrix") {
    std::fclose(f);
    return fail(LAPIS_EBADSHAPE, "read_matrix_market: not a MatrixMarket matrix file");
  }
  const std::string fmt = lower(format), fld = lower(field), sym = lower(symmetry);
  if (fmt != "coordinate" || (fld != "real" && fld != "integer" && fld != "pattern" && fld != "double") ||
      (sym != "general" && sym != "symmetric" && sym != "skew-symmetric")) {
    std::fclose(f);
    return fail(LAPIS_EBADSHAPE, "read_matrix_market: unsupported kind '%s %s %s'", format, field, symmetry);
  }
  do {
    if (!std::fgets(line, sizeof(line), f)) {
      std::fclose(f);
      return fail(LAPIS_EBADSHAPE, "read_matrix_market: missing size line");
    }
  } while (line[0] == '%' || line[0] == '\n' || line[0] == '\r');
  long long m = 0, n = 0, stored = 0;
  if (std::sscanf(line, "%lld %lld %lld", &m, &n, &stored) != 3 || m < 0 || n < 0 || stored < 0) {
    std::fclose(f);
    return fail(LAPIS_EBADSHAPE, "read_matrix_market: bad size line");
  }
  if (idx_bytes == 4 && (m > 0x7fffffffLL || n > 0x7fffffffLL)) {
    std::fclose(f);
    return fail(LAPIS_ETOOBIG, "read_matrix_market: dimensions need 64-bit indices");
  }
  const bool pattern = fld == "pattern", symmetric = sym != "general", skew = sym == "skew-symmetric";
  std::vector<Entry> e;
  e.reserve((size_t)stored * (symmetric ? 2 : 1));
  for (long long k = 0; k < stored; ++k) {
    long long i = 0, j = 0;
    double v = 1.0;
    const int got = pattern ? std::fscanf(f, "%lld %lld", &i, &j) : std::fscanf(f, "%lld %lld %lf", &i, &j, &v);
    if (got != (pattern ? 2 : 3) || i < 1 || j < 1 || i > m || j > n) {
      std::fclose(f);
      return fail(LAPIS_EBADSHAPE, "read_matrix_market: bad entry %lld", k + 1);
    }
    e.push_back(Entry{i - 1, j - 1, v});
    if (symmetric && i != j) e.push_back(Entry{j - 1, i - 1, skew ? -v : v});
  }
  std::fclose(f);
  if (idx_bytes == 4 && e.size() > 0x7fffffffULL) return fail(LAPIS_ETOOBIG, "read_matrix_market: entries need 64-bit offsets");
  *nrows = m;
  *ncols = n;
  return idx_bytes == 4 ? fill_csr<int32_t>(m, e, pos, crd, val, nnz) : fill_csr<int64_t>(m, e, pos, crd, val, nnz);
}

extern "C" void lapis_b200_mm_free(void *p) { std::free(p); }
