// Group quantize / pack kernels, bit-exact with the reference's NumPy quantizer
// (python/linnet/src/linnet/quant.py:83-120, :242-248).
//
// Everything is IEEE binary32 with explicit round-to-nearest intrinsics: a true
// division (the reference divides; multiplying by a reciprocal flips codes), rintf
// for NumPy's half-to-even `round`, and no fused multiply-add.  This translation
// unit must be compiled with -fmad=false -prec-div=true -ftz=false.
//
// HBM-bound by its bytes (2 B read + 0.52 B written per weight for int4-g128 from bf16,
// 2 B + 1 B for int8) but with some twenty instructions a weight when written naively, so
// the instruction count is what the kernels are built around:
//   * the common case of round(v / s) is three additions and a multiply-add per weight (the
//     1.5 * 2^23 trick), with one test per eight weights for the rare near tie, which takes
//     the true division; levels are packed arithmetically (four nibbles are one f32 sum);
//   * per-group work (the shuffles of the min/max reduction, two divisions and a reciprocal)
//     is spread over 32 weights a lane instead of 8.
// Two kernels:
//   * team kernel  - groups of 16..256 elements: a team of 1..8 lanes holds one group in
//     registers, each lane up to four consecutive 8-weight chunks (64 bytes of bf16),
//     reduces min/max with shuffles and writes its 16 packed bytes (or 32 int8) at once.
//   * group kernel - any other group size: one warp or one 256-thread block per
//     group; the group stays in registers (up to 8 chunks per thread) between the
//     reduction and the rounding, the rest is read again (from L2).
#include "common.cuh"

namespace b200q {
namespace {

constexpr int kInt4 = 0;
constexpr int kInt8 = 1;

struct Chunk {  // eight consecutive weights as f32
    float v[8];
};

__device__ __forceinline__ Chunk widen(const uint4& raw) {  // 8 x bf16
    Chunk c;
    c.v[0] = __uint_as_float(raw.x << 16);
    c.v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
    c.v[2] = __uint_as_float(raw.y << 16);
    c.v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
    c.v[4] = __uint_as_float(raw.z << 16);
    c.v[5] = __uint_as_float(raw.z & 0xFFFF0000u);
    c.v[6] = __uint_as_float(raw.w << 16);
    c.v[7] = __uint_as_float(raw.w & 0xFFFF0000u);
    return c;
}

__device__ __forceinline__ float min3(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

template <typename In>
struct Raw;  // the bytes of one chunk as loaded
template <>
struct Raw<__nv_bfloat16> {
    uint4 a;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { a = __ldg(reinterpret_cast<const uint4*>(p)); }
    __device__ __forceinline__ void clear() { a = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ Chunk get() const { return widen(a); }
    // smallest and largest of the eight values, two at a time in the 16-bit type (exact: min and
    // max only select), which keeps the eight f32 values out of the registers until the second pass
    __device__ __forceinline__ void range(float& lo, float& hi) const {
        const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162 l = __hmin2(__hmin2(v[0], v[1]), __hmin2(v[2], v[3]));
        const __nv_bfloat162 h = __hmax2(__hmax2(v[0], v[1]), __hmax2(v[2], v[3]));
        lo = min3(lo, __low2float(l), __high2float(l));
        hi = max3(hi, __low2float(h), __high2float(h));
    }
};
template <>
struct Raw<float> {
    uint4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = __ldg(reinterpret_cast<const uint4*>(p));
        b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    }
    __device__ __forceinline__ void clear() { a = b = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ void range(float& lo, float& hi) const {
        const Chunk v = get();
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            lo = min3(lo, v.v[j], v.v[j + 1]);
            hi = max3(hi, v.v[j], v.v[j + 1]);
        }
    }
    __device__ __forceinline__ Chunk get() const {
        Chunk c;
        c.v[0] = __uint_as_float(a.x); c.v[1] = __uint_as_float(a.y);
        c.v[2] = __uint_as_float(a.z); c.v[3] = __uint_as_float(a.w);
        c.v[4] = __uint_as_float(b.x); c.v[5] = __uint_as_float(b.y);
        c.v[6] = __uint_as_float(b.z); c.v[7] = __uint_as_float(b.w);
        return c;
    }
};

__device__ __forceinline__ float widen_one(const float* p) { return *p; }
__device__ __forceinline__ float widen_one(const __nv_bfloat16* p) {
    return __uint_as_float(uint32_t(*reinterpret_cast<const uint16_t*>(p)) << 16);
}

// ---- the reference's arithmetic ---------------------------------------------

// quant.py:93-94: scale = (high - low) / 15, replaced by 1 where not positive.
__device__ __forceinline__ float int4_step(float lo, float hi) {
    float s = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
    return s > 0.0f ? s : 1.0f;
}
// quant.py:95: zero = clip(round(-low / scale), 0, 15).
__device__ __forceinline__ float int4_zero(float lo, float step) {
    float z = rintf(__fdiv_rn(-lo, step));
    return fminf(fmaxf(z, 0.0f), 15.0f);
}
// round(v / s) exactly as NumPy computes it (a correctly rounded f32 division, then
// round-half-even), at a fraction of the division's cost: v * (1/s) is within 1.2e-7
// relative of the true quotient, so for |quotient| < 256 it is within 4.6e-5 of the
// rounded quotient NumPy sees; unless it lies within 1e-4 of a half-integer both round to
// the same integer.  The rare near-tie, huge or non-finite quotients take the division.
__device__ __forceinline__ float rint_div(float v, float s, float inv_s) {
    const float t = __fmul_rn(v, inv_s);
    float n = rintf(t);
    const float to_half = fabsf(fabsf(__fsub_rn(t, n)) - 0.5f);
    if (!(fabsf(t) < 256.0f) || to_half < 1e-4f) n = rintf(__fdiv_rn(v, s));
    return n;
}
// quant.py:96: q = clip(round(g / scale) + zero, 0, 15).
__device__ __forceinline__ uint32_t int4_level(float v, float step, float inv_step, float zero) {
    float q = __fadd_rn(rint_div(v, step, inv_step), zero);
    return uint32_t(fminf(fmaxf(q, 0.0f), 15.0f));
}
// weights.py:74-79: bf16 bits, round to nearest even by the integer trick.
__device__ __forceinline__ uint32_t bf16_bits_rne(float v) {
    uint32_t bits = __float_as_uint(v);
    return (bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16;
}
// quant.py:115-118: absmax / 127, 1 where not positive, through the stored dtype.
__device__ __forceinline__ float int8_scale(float absmax, int scale_dtype) {
    float s = __fdiv_rn(absmax, 127.0f);
    s = s > 0.0f ? s : 1.0f;
    if (scale_dtype == B200Q_BF16) return __uint_as_float(bf16_bits_rne(s) << 16);
    if (scale_dtype == B200Q_F16) return __half2float(__float2half_rn(s));
    return s;
}
// quant.py:119: q = clip(round(g / scale), -127, 127).
__device__ __forceinline__ int int8_level(float v, float scale, float inv_scale) {
    float q = rint_div(v, scale, inv_scale);
    return int(fminf(fmaxf(q, -127.0f), 127.0f));
}

// Adding 1.5 * 2^23 to |t| < 2^22 rounds t to an integer, half to even, in the sum's low bits.
constexpr float kRound = 12582912.0f;
// A quotient within 1e-4 of a half-integer is rounded by the true division; the test is on the
// squared distance from the nearest integer (0.4999^2 = 0.24990001).
constexpr float kTie2 = 0.2499f;

__device__ __forceinline__ void store_scale(void* dst, int dtype, int64_t i, float s) {
    if (dst == nullptr) return;
    if (dtype == B200Q_BF16) {
        reinterpret_cast<uint16_t*>(dst)[i] = uint16_t(bf16_bits_rne(s));
    } else if (dtype == B200Q_F16) {
        reinterpret_cast<__half*>(dst)[i] = __float2half_rn(s);
    } else {
        reinterpret_cast<float*>(dst)[i] = s;
    }
}

// Eight levels clip(round(v / step) + zero, 0, 15) as one little-endian word (byte j/2 holds
// element j low, j+1 high).  t = v * (1/step) + zero is within 1e-5 of the reference's
// quotient plus zero wherever the clip does not decide the level anyway (|v / step| < 32),
// so away from half-integers both round alike; zero is an integer, so adding it before the
// rounding only matters at exact ties, which take the division with every near tie.
// INSIDE: the group's range straddles zero (low < 0 < high), so its zero point is not clipped
// and every t lies in [-0.5, 15.5]: away from ties (the only case kept here) it rounds into
// 0..15 without the clip.
// The arithmetic runs two weights an instruction (fma / add .f32x2 of sm_100, each half an IEEE
// operation of its own): weight j is paired with weight j + 4, so that the packing sums of the
// low and the high four levels are the two halves of one chain.
template <bool INSIDE = false>
__device__ __forceinline__ uint32_t pack8_int4(const Chunk& c, float step, float zero, float inv) {
    const float2 inv2 = make_float2(inv, inv), zero2 = make_float2(zero, zero);
    const float2 up = make_float2(kRound, kRound), down = make_float2(-kRound, -kRound);
    const float2 minus = make_float2(-1.0f, -1.0f), sixteen = make_float2(16.0f, 16.0f);
    float2 q[4], dd[4];
    float worst = 0.0f;  // largest squared distance of a t from its integer
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 t = __ffma2_rn(make_float2(c.v[j], c.v[j + 4]), inv2, zero2);
        const float2 r = __fadd2_rn(__fadd2_rn(t, up), down);
        const float2 d = __ffma2_rn(r, minus, t);  // t - r (the product is exact)
        dd[j] = __fmul2_rn(d, d);
        worst = max3(worst, dd[j].x, dd[j].y);
        q[j] = INSIDE ? r : make_float2(fminf(fmaxf(r.x, 0.0f), 15.0f), fminf(fmaxf(r.y, 0.0f), 15.0f));
    }
    if (!(worst < kTie2)) {  // rare (one chunk in 600), but a warp takes it when any lane does: only the near ties
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (!(dd[j].x < kTie2)) q[j].x = float(int4_level(c.v[j], step, inv, zero));
            if (!(dd[j].y < kTie2)) q[j].y = float(int4_level(c.v[j + 4], step, inv, zero));
        }
    }
    // four levels are one exact f32 sum; 2^23 + sum has them in its low 16 bits
    float2 sum = __ffma2_rn(q[3], sixteen, q[2]);
    sum = __ffma2_rn(sum, sixteen, q[1]);
    sum = __ffma2_rn(sum, sixteen, q[0]);
    sum = __fadd2_rn(sum, make_float2(8388608.0f, 8388608.0f));
    return __byte_perm(__float_as_uint(sum.x), __float_as_uint(sum.y), 0x5410);
}
__device__ __forceinline__ uint32_t pack8_int4(const Chunk& c, float step, float zero) {
    return pack8_int4<false>(c, step, zero, __frcp_rn(step));
}

// Eight levels clip(round(v / scale), -127, 127) as bytes: kRound + level has the level's
// two's complement in its low byte.
__device__ __forceinline__ uint2 pack8_int8(const Chunk& c, float scale, float inv) {
    // Two weights an instruction, as in pack8_int4.  No clip here: the scale is the group's own
    // largest magnitude / 127, so |t| <= 127.3 for every finite group; a quotient that is out
    // of range all the same (a subnormal scale, a non-finite weight) shows in the largest
    // squared level and takes the division with the near ties.
    const float2 inv2 = make_float2(inv, inv), up = make_float2(kRound, kRound), down = make_float2(-kRound, -kRound);
    const float2 minus = make_float2(-1.0f, -1.0f);
    uint32_t b[8];
    float worst = 0.0f, largest = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
        const float2 t = __fmul2_rn(make_float2(c.v[j], c.v[j + 1]), inv2);
        const float2 s = __fadd2_rn(t, up);
        const float2 r = __fadd2_rn(s, down);      // the level
        const float2 d = __ffma2_rn(r, minus, t);  // t - r
        const float2 dd = __fmul2_rn(d, d), rr = __fmul2_rn(r, r);
        worst = max3(worst, dd.x, dd.y);
        largest = max3(largest, rr.x, rr.y);
        b[j] = __float_as_uint(s.x);
        b[j + 1] = __float_as_uint(s.y);
    }
    if (!(worst < kTie2) || !(largest <= 127.0f * 127.0f)) {
#pragma unroll
        for (int j = 0; j < 8; ++j) b[j] = uint32_t(int8_level(c.v[j], scale, inv));
    }
    return make_uint2(__byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410),
                      __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410));
}
__device__ __forceinline__ uint2 pack8_int8(const Chunk& c, float scale) {
    return pack8_int8(c, scale, __frcp_rn(scale));
}

struct Outputs {
    uint8_t* packed;    // int4: [groups, G/2] bytes; int8: [groups, G] bytes
    float* scale;       // [groups]
    void* scale_store;  // int4 only, may be null
    int store_dtype;    // int4: dtype of scale_store; int8: dtype the scale is rounded through
    uint8_t* zero;      // int4 only
};

// ---- team kernel ------------------------------------------------------------
// T lanes per group, C consecutive 8-weight chunks per lane (G == 8 * T * C).
template <int MODE, int T, int C, typename In>
__global__ void __launch_bounds__(256, 4)  // at most 64 registers: 32 warps per multiprocessor
quantize_team_kernel(const In* __restrict__ w, int64_t lanes, Outputs o) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const bool leader = (threadIdx.x % T) == 0;
    int64_t l = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    Raw<In> next[C];  // the following iteration's chunks, asked for before this one's arithmetic
    auto fetch = [&](int64_t at) {
        if (at < lanes) {
#pragma unroll
            for (int u = 0; u < C; ++u) next[u].load(w + (at * C + u) * 8);
        } else {
#pragma unroll
            for (int u = 0; u < C; ++u) next[u].clear();
        }
    };
    fetch(l);
    for (; l - threadIdx.x % 32 < lanes; l += stride) {
        const bool live = l < lanes;  // uniform over a team: lanes % T == 0
        Raw<In> raw[C];
#pragma unroll
        for (int u = 0; u < C; ++u) raw[u] = next[u];
        fetch(l + stride);
        float lo = __int_as_float(0x7F800000), hi = __int_as_float(0xFF800000);
#pragma unroll
        for (int u = 0; u < C; ++u) raw[u].range(lo, hi);
#pragma unroll
        for (int d = T / 2; d >= 1; d >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, d));
            hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, d));
        }
        if (!live) continue;
        if (MODE == kInt4) {
            const float step = int4_step(lo, hi);
            const float zero = int4_zero(lo, step);
            const float inv = __frcp_rn(step);
            uint32_t word[C];
            if (lo < 0.0f && hi > 0.0f) {
#pragma unroll
                for (int u = 0; u < C; ++u) word[u] = pack8_int4<true>(raw[u].get(), step, zero, inv);
            } else {
#pragma unroll
                for (int u = 0; u < C; ++u) word[u] = pack8_int4<false>(raw[u].get(), step, zero, inv);
            }
            uint32_t* dst = reinterpret_cast<uint32_t*>(o.packed) + l * C;
            if (C == 4) {
                *reinterpret_cast<uint4*>(dst) = make_uint4(word[0], word[1], word[2], word[3]);
            } else if (C == 2) {
                *reinterpret_cast<uint2*>(dst) = make_uint2(word[0], word[1 % C]);
            } else {
#pragma unroll
                for (int u = 0; u < C; ++u) dst[u] = word[u];
            }
            if (leader) {
                const int64_t g = l / T;
                o.scale[g] = step;
                o.zero[g] = uint8_t(zero);
                store_scale(o.scale_store, o.store_dtype, g, step);
            }
        } else {
            const float scale = int8_scale(fmaxf(-lo, hi), o.store_dtype);  // the largest magnitude
            const float inv = __frcp_rn(scale);
            uint2 pair[C];
#pragma unroll
            for (int u = 0; u < C; ++u) pair[u] = pack8_int8(raw[u].get(), scale, inv);
            uint2* dst = reinterpret_cast<uint2*>(o.packed) + l * C;
            if (C % 2 == 0) {
#pragma unroll
                for (int u = 0; u < C; u += 2)
                    *reinterpret_cast<uint4*>(dst + u) = make_uint4(pair[u].x, pair[u].y, pair[(u + 1) % C].x, pair[(u + 1) % C].y);
            } else {
#pragma unroll
                for (int u = 0; u < C; ++u) dst[u] = pair[u];
            }
            if (leader) o.scale[l / T] = scale;
        }
    }
}

// ---- group kernel -----------------------------------------------------------
// THREADS == 32: one warp per group (blocks of 4 warps); otherwise one block per
// group.  VEC: the group is a whole number of aligned 8-element chunks.
template <int THREADS>
__device__ __forceinline__ float reduce_max(float v, float* scratch) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
    if (THREADS > 32) {
        const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
        __syncthreads();  // scratch may still be read from the previous use
        if (lane == 0) scratch[warp] = v;
        __syncthreads();
        v = scratch[0];
#pragma unroll
        for (int i = 1; i < THREADS / 32; ++i) v = fmaxf(v, scratch[i]);
    }
    return v;
}

template <int MODE, int THREADS, typename In, bool VEC>
__global__ void __launch_bounds__(THREADS == 32 ? 128 : THREADS)
quantize_group_kernel(const In* __restrict__ w, int64_t groups, int64_t G, Outputs o) {
    constexpr int CACHED = 8;
    __shared__ float scratch[32];
    const int lane = THREADS == 32 ? threadIdx.x % 32 : threadIdx.x;
    const int64_t first = THREADS == 32 ? int64_t(blockIdx.x) * 4 + threadIdx.x / 32 : blockIdx.x;
    const int64_t step_groups = THREADS == 32 ? int64_t(gridDim.x) * 4 : gridDim.x;
    for (int64_t g = first; g < groups; g += step_groups) {
        const In* src = w + g * G;
        float lo = __int_as_float(0x7F800000), hi = __int_as_float(0xFF800000), top = 0.0f;
        Raw<In> cache[CACHED];
        const int64_t nchunks = G / 8;
        if (VEC) {
#pragma unroll
            for (int i = 0; i < CACHED; ++i) {
                const int64_t c = lane + int64_t(i) * THREADS;
                if (c < nchunks) cache[i].load(src + c * 8);
            }
#pragma unroll
            for (int i = 0; i < CACHED; ++i) {
                const int64_t c = lane + int64_t(i) * THREADS;
                if (c < nchunks) {
                    const Chunk v = cache[i].get();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        lo = fminf(lo, v.v[j]);
                        hi = fmaxf(hi, v.v[j]);
                        top = fmaxf(top, fabsf(v.v[j]));
                    }
                }
            }
            for (int64_t c = lane + int64_t(CACHED) * THREADS; c < nchunks; c += THREADS) {
                Raw<In> r;
                r.load(src + c * 8);
                const Chunk v = r.get();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    lo = fminf(lo, v.v[j]);
                    hi = fmaxf(hi, v.v[j]);
                    top = fmaxf(top, fabsf(v.v[j]));
                }
            }
        } else {
            for (int64_t e = lane; e < G; e += THREADS) {
                const float v = widen_one(src + e);
                lo = fminf(lo, v);
                hi = fmaxf(hi, v);
                top = fmaxf(top, fabsf(v));
            }
        }
        if (MODE == kInt4) {
            lo = -reduce_max<THREADS>(-lo, scratch);
            hi = reduce_max<THREADS>(hi, scratch);
            const float step = int4_step(lo, hi);
            const float zero = int4_zero(lo, step);
            if (lane == 0) {
                o.scale[g] = step;
                o.zero[g] = uint8_t(zero);
                store_scale(o.scale_store, o.store_dtype, g, step);
            }
            uint8_t* dst = o.packed + g * (G / 2);
            if (VEC) {
#pragma unroll
                for (int i = 0; i < CACHED; ++i) {
                    const int64_t c = lane + int64_t(i) * THREADS;
                    if (c < nchunks)
                        reinterpret_cast<uint32_t*>(dst)[c] = pack8_int4(cache[i].get(), step, zero);
                }
                for (int64_t c = lane + int64_t(CACHED) * THREADS; c < nchunks; c += THREADS) {
                    Raw<In> r;
                    r.load(src + c * 8);
                    reinterpret_cast<uint32_t*>(dst)[c] = pack8_int4(r.get(), step, zero);
                }
            } else {
                for (int64_t b = lane; b < G / 2; b += THREADS) {
                    const float inv = __frcp_rn(step);
                    const uint32_t even = int4_level(widen_one(src + 2 * b), step, inv, zero);
                    const uint32_t odd = int4_level(widen_one(src + 2 * b + 1), step, inv, zero);
                    dst[b] = uint8_t(even | (odd << 4));
                }
            }
        } else {
            top = reduce_max<THREADS>(top, scratch);
            const float scale = int8_scale(top, o.store_dtype);
            if (lane == 0) o.scale[g] = scale;
            uint8_t* dst = o.packed + g * G;
            if (VEC) {
#pragma unroll
                for (int i = 0; i < CACHED; ++i) {
                    const int64_t c = lane + int64_t(i) * THREADS;
                    if (c < nchunks)
                        reinterpret_cast<uint2*>(dst)[c] = pack8_int8(cache[i].get(), scale);
                }
                for (int64_t c = lane + int64_t(CACHED) * THREADS; c < nchunks; c += THREADS) {
                    Raw<In> r;
                    r.load(src + c * 8);
                    reinterpret_cast<uint2*>(dst)[c] = pack8_int8(r.get(), scale);
                }
            } else {
                for (int64_t e = lane; e < G; e += THREADS)
                    dst[e] = uint8_t(int8_level(widen_one(src + e), scale, __frcp_rn(scale)));
            }
        }
    }
}

template <int MODE, typename In>
int32_t launch_quantize(const In* w, int64_t out, int64_t in, int64_t G, Outputs o,
                        cudaStream_t stream) {
    const int64_t total = out * in;
    if (total == 0) return B200Q_OK;
    const int64_t groups = total / G;
    const bool vec = (G % 8 == 0) && aligned(w, 16) &&
                     aligned(o.packed, MODE == kInt4 ? 4 : 8);
    const int sms = sm_count();
    const bool wide = aligned(o.packed, 16);  // a lane's 16 (int4) or 32 (int8) output bytes in one or two stores
    if (vec && wide && (G == 16 || G == 32 || G == 64 || G == 128 || G == 256)) {
        // a lane holds up to four consecutive chunks (64 bytes of bf16): lanes at a 64-byte
        // stride read half a sector per load, the other half is the next load's (L1 keeps it)
        const int C = G >= 32 ? 4 : 2;
        const int64_t lanes = total / (8 * C);
        int64_t blocks = (lanes + 255) / 256;
        const int64_t cap = int64_t(sms) * 32;
        if (blocks > cap) blocks = cap;
        const dim3 grid{unsigned(blocks)};
        switch (G) {
            case 16: quantize_team_kernel<MODE, 1, 2, In><<<grid, 256, 0, stream>>>(w, lanes, o); break;
            case 32: quantize_team_kernel<MODE, 1, 4, In><<<grid, 256, 0, stream>>>(w, lanes, o); break;
            case 64: quantize_team_kernel<MODE, 2, 4, In><<<grid, 256, 0, stream>>>(w, lanes, o); break;
            case 128: quantize_team_kernel<MODE, 4, 4, In><<<grid, 256, 0, stream>>>(w, lanes, o); break;
            default: quantize_team_kernel<MODE, 8, 4, In><<<grid, 256, 0, stream>>>(w, lanes, o); break;
        }
        return launched("quantize (team kernel)");
    }
    if (G < 2048) {
        int64_t blocks = (groups + 3) / 4;
        if (blocks > int64_t(sms) * 64) blocks = int64_t(sms) * 64;
        if (vec)
            quantize_group_kernel<MODE, 32, In, true><<<unsigned(blocks), 128, 0, stream>>>(w, groups, G, o);
        else
            quantize_group_kernel<MODE, 32, In, false><<<unsigned(blocks), 128, 0, stream>>>(w, groups, G, o);
    } else {
        int64_t blocks = groups;
        if (blocks > int64_t(sms) * 32) blocks = int64_t(sms) * 32;
        if (vec)
            quantize_group_kernel<MODE, 256, In, true><<<unsigned(blocks), 256, 0, stream>>>(w, groups, G, o);
        else
            quantize_group_kernel<MODE, 256, In, false><<<unsigned(blocks), 256, 0, stream>>>(w, groups, G, o);
    }
    return launched("quantize (group kernel)");
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_quantize_int4_groups(const void* weight, int32_t weight_dtype,
                                              int64_t out, int64_t in, int64_t group,
                                              uint8_t* packed, float* scale, void* scale_store,
                                              int32_t store_dtype, uint8_t* zero, void* stream) {
    B200Q_REQUIRE(out >= 0 && in >= 0, "quantize_int4_groups: a linear weight is [Out, In]; got [%lld, %lld]",
                  (long long)out, (long long)in);
    B200Q_REQUIRE(group > 0 && group % 2 == 0 && in % group == 0,
                  "quantize_int4_groups: groups of %lld must be even and divide the %lld inputs",
                  (long long)group, (long long)in);
    B200Q_REQUIRE(weight_dtype == B200Q_F32 || weight_dtype == B200Q_BF16,
                  "quantize_int4_groups: weights are f32 or bf16");
    B200Q_REQUIRE(store_dtype == B200Q_F32 || store_dtype == B200Q_BF16 || store_dtype == B200Q_F16,
                  "quantize_int4_groups: scales are stored as bf16, f16, or f32");
    if (out * in == 0) return B200Q_OK;
    B200Q_REQUIRE(weight && packed && scale && zero, "quantize_int4_groups: null tensor");
    Outputs o{packed, scale, scale_store, store_dtype, zero};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (weight_dtype == B200Q_BF16)
        return launch_quantize<kInt4>(static_cast<const __nv_bfloat16*>(weight), out, in, group, o, s);
    return launch_quantize<kInt4>(static_cast<const float*>(weight), out, in, group, o, s);
}

extern "C" int32_t b200q_quantize_int8_groups(const void* weight, int32_t weight_dtype,
                                              int64_t out, int64_t in, int64_t group,
                                              int32_t scale_dtype, int8_t* q, float* scale,
                                              void* stream) {
    B200Q_REQUIRE(out >= 0 && in >= 0, "quantize_int8_groups: a linear weight is [Out, In]; got [%lld, %lld]",
                  (long long)out, (long long)in);
    B200Q_REQUIRE(group > 0 && in % group == 0,
                  "quantize_int8_groups: groups of %lld must divide the %lld inputs",
                  (long long)group, (long long)in);
    B200Q_REQUIRE(weight_dtype == B200Q_F32 || weight_dtype == B200Q_BF16,
                  "quantize_int8_groups: weights are f32 or bf16");
    B200Q_REQUIRE(scale_dtype == B200Q_F32 || scale_dtype == B200Q_BF16 || scale_dtype == B200Q_F16,
                  "quantize_int8_groups: scales are stored as bf16, f16, or f32");
    if (out * in == 0) return B200Q_OK;
    B200Q_REQUIRE(weight && q && scale, "quantize_int8_groups: null tensor");
    Outputs o{reinterpret_cast<uint8_t*>(q), scale, nullptr, scale_dtype, nullptr};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (weight_dtype == B200Q_BF16)
        return launch_quantize<kInt8>(static_cast<const __nv_bfloat16*>(weight), out, in, group, o, s);
    return launch_quantize<kInt8>(static_cast<const float*>(weight), out, in, group, o, s);
}
