// placeholder until the tcgen05 kernel lands
#include "common.cuh"
namespace b200q {
bool int4_gemm_supports(int64_t, int64_t, int64_t, int64_t, int32_t, const void*, const void*) { return false; }
}
extern "C" int32_t b200q_int4_gemm(const void*, const uint8_t*, const void*, const uint8_t*, void*, int64_t,
                                   int64_t, int64_t, int64_t, int32_t, void*) {
    return b200q::unavailable("int4_gemm: not built");
}
