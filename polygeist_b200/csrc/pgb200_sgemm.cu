// placeholder until the tcgen05 path lands: reports UNSUPPORTED so that the
// caller takes the SIMT kernels.
#include "pgb200_internal.h"
namespace pgb200 {
int32_t tf32x3_gemm(cudaStream_t, int64_t, int64_t, int64_t, float, const float *, int64_t,
                    const float *, int64_t, bool, float, float *, int64_t, bool, int64_t) {
  return PGB200_ERR_UNSUPPORTED;
}
}  // namespace pgb200
