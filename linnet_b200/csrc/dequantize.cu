// Whole-weight dequantization kernels (HBM-bound elementwise passes).
//
// int4: stands in for the generated `_int4_weight` / Triton `_int4_unpack`
// (src/backend/torch_source.cpp:1519-1551): w = (q - zero) * scale in f32, rounded
// once to the output type.  int8: stands in for `dequantize8`
// (python/linnet/src/linnet/torch/kernels.py:595-666): w = f32(q) * scale.
#include "mma.cuh"

namespace b200q {
namespace {

template <typename T>
__global__ void __launch_bounds__(256)
int4_dequantize_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scale,
                       const uint8_t* __restrict__ zero, uint16_t* __restrict__ out,
                       int64_t words, int64_t half_group_words) {
    using H = Half16<T>;
    // One 32-bit word (8 weights) per thread per step; a group is G/8 words.
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < words;
         i += int64_t(gridDim.x) * blockDim.x) {
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(packed) + i);
        const int64_t grp = i / half_group_words;
        const float s = H::to_float(__ldg(scale + grp));
        const float z = float(__ldg(zero + grp));
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float lo = (float((w >> (8 * j)) & 15) - z) * s;
            const float hi = (float((w >> (8 * j + 4)) & 15) - z) * s;
            o[j] = uint32_t(H::from_float(lo)) | (uint32_t(H::from_float(hi)) << 16);
        }
        reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// Groups that are not a multiple of 8 weights, or unaligned tensors.
template <typename T>
__global__ void int4_dequantize_bytes_kernel(const uint8_t* __restrict__ packed,
                                             const uint16_t* __restrict__ scale,
                                             const uint8_t* __restrict__ zero,
                                             uint16_t* __restrict__ out, int64_t bytes,
                                             int64_t half_group) {
    using H = Half16<T>;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < bytes;
         i += int64_t(gridDim.x) * blockDim.x) {
        const uint32_t b = packed[i];
        const int64_t grp = i / half_group;
        const float s = H::to_float(scale[grp]);
        const float z = float(zero[grp]);
        out[2 * i] = H::from_float((float(b & 15) - z) * s);
        out[2 * i + 1] = H::from_float((float(b >> 4) - z) * s);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
int8_dequantize_kernel(const int8_t* __restrict__ w, const float* __restrict__ scale,
                       uint16_t* __restrict__ out, int64_t total, int64_t in, int64_t group) {
    using H = Half16<T>;
    const int64_t groups = in / group;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t row = i / in, col = i % in;
        out[i] = H::from_float(float(w[i]) * __ldg(scale + row * groups + col / group));
    }
}

int blocks_for(int64_t items) {
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = int64_t(sm_count()) * 32;
    return int(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_int4_dequantize(const uint8_t* packed, const void* scale,
                                         const uint8_t* zero, void* weight, int64_t out,
                                         int64_t in, int64_t group, int32_t dtype, void* stream) {
    B200Q_REQUIRE(dtype == B200Q_BF16 || dtype == B200Q_F16, "int4_dequantize: the weight is bf16 or f16");
    B200Q_REQUIRE(out >= 0 && in >= 0 && group > 0 && group % 2 == 0 && in % group == 0,
                  "int4_dequantize: a group of %lld must be even and divide the %lld inputs",
                  (long long)group, (long long)in);
    if (out * in == 0) return B200Q_OK;
    B200Q_REQUIRE(packed && scale && zero && weight, "int4_dequantize: null tensor");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint16_t* sc = static_cast<const uint16_t*>(scale);
    uint16_t* dst = static_cast<uint16_t*>(weight);
    const int64_t bytes = out * in / 2;
    if (group % 8 == 0 && aligned(packed, 4) && aligned(weight, 16)) {
        const int64_t words = bytes / 4;
        if (dtype == B200Q_BF16)
            int4_dequantize_kernel<__nv_bfloat16><<<blocks_for(words), 256, 0, s>>>(packed, sc, zero, dst, words, group / 8);
        else
            int4_dequantize_kernel<__half><<<blocks_for(words), 256, 0, s>>>(packed, sc, zero, dst, words, group / 8);
    } else {
        if (dtype == B200Q_BF16)
            int4_dequantize_bytes_kernel<__nv_bfloat16><<<blocks_for(bytes), 256, 0, s>>>(packed, sc, zero, dst, bytes, group / 2);
        else
            int4_dequantize_bytes_kernel<__half><<<blocks_for(bytes), 256, 0, s>>>(packed, sc, zero, dst, bytes, group / 2);
    }
    return launched("int4_dequantize");
}

extern "C" int32_t b200q_int8_dequantize(const int8_t* w, const float* scale, void* weight,
                                         int64_t out, int64_t in, int64_t group, int32_t dtype,
                                         void* stream) {
    B200Q_REQUIRE(dtype == B200Q_BF16 || dtype == B200Q_F16, "int8_dequantize: the weight is bf16 or f16");
    B200Q_REQUIRE(out >= 0 && in >= 0 && group >= 0 && (group == 0 || in % group == 0),
                  "int8_dequantize: groups of %lld must divide the %lld inputs", (long long)group, (long long)in);
    if (out * in == 0) return B200Q_OK;
    B200Q_REQUIRE(w && scale && weight, "int8_dequantize: null tensor");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t total = out * in;
    const int64_t g = group == 0 ? in : group;
    if (dtype == B200Q_BF16)
        int8_dequantize_kernel<__nv_bfloat16><<<blocks_for(total), 256, 0, s>>>(w, scale, static_cast<uint16_t*>(weight), total, in, g);
    else
        int8_dequantize_kernel<__half><<<blocks_for(total), 256, 0, s>>>(w, scale, static_cast<uint16_t*>(weight), total, in, g);
    return launched("int8_dequantize");
}
