// Warp-level m16n8k16 tensor-core product and the element-type traits the decode
// (few-row) kernels share.  The decode kernels are HBM-bound; the tensor cores
// are used so that one pass over the weight bytes serves up to 16 activation
// rows without spending CUDA-core issue slots on the multiply-adds.
#pragma once

#include "common.cuh"

namespace b200q {

template <typename T>
struct Half16;  // traits of the two 16-bit activation types

template <>
struct Half16<__nv_bfloat16> {
    using pair = __nv_bfloat162;
    // 128 + q: the nibble sits in the low mantissa bits of 128.0 (ulp 1).
    static constexpr uint32_t kMagic = 0x43004300u;
    static constexpr float kBias = 128.0f;
    static constexpr uint32_t kOnes = 0x3F803F80u;  // (1.0, 1.0)
    static constexpr int kDtype = B200Q_BF16;
    __device__ static __forceinline__ float to_float(uint32_t bits16) {
        return __uint_as_float(bits16 << 16);
    }
    __device__ static __forceinline__ uint16_t from_float(float v) {
        return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&p);
    }
    __device__ static __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4],
                                               uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

template <>
struct Half16<__half> {
    using pair = __half2;
    static constexpr uint32_t kMagic = 0x64006400u;  // 1024 + q
    static constexpr float kBias = 1024.0f;
    static constexpr uint32_t kOnes = 0x3C003C00u;  // (1.0, 1.0)
    static constexpr int kDtype = B200Q_F16;
    __device__ static __forceinline__ float to_float(uint32_t bits16) {
        return __half2float(__ushort_as_half(uint16_t(bits16)));
    }
    __device__ static __forceinline__ uint16_t from_float(float v) {
        return __half_as_ushort(__float2half_rn(v));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 p = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&p);
    }
    __device__ static __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4],
                                               uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

// (v - bias) * scale on a pair of 16-bit floats, each step rounded once in the
// 16-bit type.  With v = magic + q and bias = magic + zero the difference is the
// exact integer q - zero, and the product is the reference's f32 product rounded
// once to the 16-bit type (an integer of at most 5 bits times a 16-bit float is
// exact in f32).
template <typename T>
__device__ __forceinline__ uint32_t sub_mul(uint32_t v, uint32_t bias, uint32_t scale) {
    using P = typename Half16<T>::pair;
    P r = __hmul2(__hsub2(*reinterpret_cast<P*>(&v), *reinterpret_cast<P*>(&bias)),
                  *reinterpret_cast<P*>(&scale));
    return *reinterpret_cast<uint32_t*>(&r);
}

}  // namespace b200q
