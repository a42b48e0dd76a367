// Row-count dispatch of the int4 linear layer, the counterpart of the generated
// `_int4_linear` (src/backend/torch_source.cpp:1553-1570): few rows stream the
// weight once through the decode kernel, many rows go to the tcgen05 dequant-GEMM.
#include "common.cuh"

namespace b200q {
// Defined in int4_gemm_sm100.cu: whether the tcgen05 kernel takes this problem.
bool int4_gemm_supports(int64_t rows, int64_t in, int64_t out, int64_t group, int32_t dtype,
                        const void* x, const void* y);
}  // namespace b200q

using namespace b200q;

// Rows from which the tensor-memory GEMM is used; below it the decode kernel runs
// in passes of 16 rows over a weight that stays in L2.
static constexpr int64_t kGemmRows = 48;

extern "C" int32_t b200q_int4_linear(const void* x, const uint8_t* packed, const void* scale,
                                     const uint8_t* zero, void* y, int64_t rows, int64_t in,
                                     int64_t out, int64_t group, int32_t dtype, void* stream) {
    if (rows >= kGemmRows && int4_gemm_supports(rows, in, out, group, dtype, x, y))
        return b200q_int4_gemm(x, packed, scale, zero, y, rows, in, out, group, dtype, stream);
    return b200q_int4_gemv(x, packed, scale, zero, y, rows, in, out, group, dtype, stream);
}
