// placeholder until the mixed-input tcgen05 kernel lands
#include "common.cuh"
#include "kernels.h"
namespace qmm {
bool mixed_tc_supported(int, int64_t, int64_t, int64_t, int64_t, const void*, int, const void*, bool) { return false; }
int launch_mixed_tc(int, const void*, int, const void*, const float*, void*, int, int64_t, int64_t, int64_t, int64_t, cudaStream_t) {
  return fail(QMM_ERR_UNSUPPORTED, "mixed-input tcgen05 kernel is not built");
}
}  // namespace qmm
