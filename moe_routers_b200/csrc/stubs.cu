// Entry points whose kernels are not linked yet answer MOE_ERR_UNSUPPORTED.
#include "common.cuh"
using namespace moe;
extern "C" int moe_sinkhorn(const void*, int, int, int, int, int, float, float, int32_t*, float*, void*, size_t, void*) {
  return fail(MOE_ERR_UNSUPPORTED, "moe_sinkhorn: not built");
}
