// K2 variant for grouped scales (per_group weights and/or per_group_token activations).
#include "common.cuh"

namespace samq {

int gemm_i8_grouped_dispatch(const int8_t*, int64_t, const int8_t*, int64_t, int64_t, int64_t, int64_t,
                             const float*, int, const float*, int, int group_size,
                             const void*, const void*, int64_t, int, void*, int, int64_t, int32_t*, void*)
{
    return fail(SAMQ_ERR_UNSUPPORTED, "grouped-scale GEMM (group_size=%d) is not built yet", group_size);
}

}  // namespace samq
