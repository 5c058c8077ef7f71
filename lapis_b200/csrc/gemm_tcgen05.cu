// tcgen05 / TMEM fp32 matmul (3xTF32).  Placeholder until the kernel lands: no shape
// is claimed, so every problem takes the general-shape kernel in gemm.cu.
#include "common.h"

namespace lapis_b200 {

int bgemm_tcgen05_supported(int64_t, int64_t, int64_t, int64_t) { return 0; }

int bgemm_tcgen05_launch(int64_t, int64_t, int64_t, int64_t, const float *, const float *, float *, cudaStream_t) {
  return fail(LAPIS_EBADSHAPE, "bgemm: tcgen05 path not available for this shape");
}

}  // namespace lapis_b200
