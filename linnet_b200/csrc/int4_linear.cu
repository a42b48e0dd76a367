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

// Rows from which the tensor-memory GEMM is used.  Measured on a B200 at K=4096, N=28672:
// the decode kernels take 33 us at 16 rows and 61 us at 32 (one pass, activations shared
// through shared memory), the GEMM 58 us from 33 to 128 rows; the decode kernel's 64-row
// pass (98 us) loses to it.
static constexpr int64_t kGemmRows = 33;

extern "C" int32_t b200q_int4_linear_ex(const void* x, const uint8_t* packed, const void* scale,
                                        const uint8_t* zero, void* y, int64_t rows, int64_t in,
                                        int64_t out, int64_t group, int32_t dtype, int32_t flags,
                                        void* stream) {
    if (rows >= kGemmRows && !(flags & B200Q_SWIGLU_INPUT) && int4_gemm_supports(rows, in, out, group, dtype, x, y))
        return b200q_int4_gemm(x, packed, scale, zero, y, rows, in, out, group, dtype, stream);
    return b200q_int4_gemv_ex(x, packed, scale, zero, y, rows, in, out, group, dtype, flags, stream);
}

extern "C" int32_t b200q_int4_linear(const void* x, const uint8_t* packed, const void* scale,
                                     const uint8_t* zero, void* y, int64_t rows, int64_t in,
                                     int64_t out, int64_t group, int32_t dtype, void* stream) {
    return b200q_int4_linear_ex(x, packed, scale, zero, y, rows, in, out, group, dtype, 0, stream);
}
