// int8 weight-only decode product for up to 16 activation rows.
//
//   y[m, n] = sum_k x[m, k] * w[n, k] * scale[n (, k/G)]
//
// Stands in for linnet::gemv8 (python/linnet/src/linnet/torch/kernels.py:336-434,
// one row) and linnet::w8a16 (:437-592, a few rows) for the int8 formats:
// w [N, K] i8, scale f32 [N] (group == 0) or [N, K/G].
//
// HBM-bound at 1 B per weight.  Same structure as the int4 decode kernel: every
// thread streams 16-byte pieces of rows g and g+8 of a 16-row tile into registers
// (D k-blocks of 64 inputs in flight), widens the bytes exactly (2^23 + 128 + w
// read as f32, less 2^23 + 128 -- the reference's `_widen8`, kernels.py:326-333 --
// then packed to 16-bit pairs, which every int8 value fits), and feeds them to
// mma.m16n8k16 as A fragments with the activations, staged once per block in
// shared memory, as B fragments.  A per-row scale is applied to the final sum, a
// per-group scale (G a multiple of 64) to each k-block's sum, both in f32; smaller
// groups scale each weight in f32 before the one rounding to the 16-bit type.
#include "gemv_common.cuh"
#include "int8_gemv_tma.cuh"

namespace b200q {
namespace {

enum { kScaleRow = 0, kScaleBlock = 1, kScaleElement = 2 };

struct Gemv8Args {
    const void* x;       // [M, K]
    const int8_t* w;     // [N, K]
    const float* scale;  // [N] or [N, K/G]
    void* y;             // [M, N]
    int M, K, N, G;      // G == 0: one scale per row
    int kblocks;         // K / 64
    int kb_per_cta;
    int ksplit;
    int flags;           // B200Q_EXACT_WEIGHTS | B200Q_EARLY_DEPENDENTS
};

template <int NT>
struct Stage8 {
    uint4 q[NT][2];
    float s[NT][2];
};

// Four int8 of `word` as two 16-bit pairs (v0, v1), (v2, v3), each times `scale`.
template <typename T, bool SCALED>
__device__ __forceinline__ void widen4(uint32_t word, float scale, uint32_t& p01, uint32_t& p23) {
    const uint32_t u = word ^ 0x80808080u;  // w + 128 in each byte
    const float bias = 8388736.0f;          // 2^23 + 128
    float v0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)) - bias;
    float v1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)) - bias;
    float v2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)) - bias;
    float v3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)) - bias;
    if (SCALED) {
        v0 *= scale; v1 *= scale; v2 *= scale; v3 *= scale;
    }
    p01 = Half16<T>::pack(v0, v1);
    p23 = Half16<T>::pack(v2, v3);
}

template <typename T, int MODE, int MB, int NT, int W, int D>
__global__ void __launch_bounds__(W * 32)
int8_gemv_kernel(const Gemv8Args a) {
    using H = Half16<T>;
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
    const int M = a.M, K = a.K, N = a.N;
    const int G = MODE == kScaleRow ? K : a.G;
    const int groups = K / G;
    const int tile_row = blockIdx.x * (16 * NT);
    const int kb0 = min(int(blockIdx.y) * a.kb_per_cta, a.kblocks);
    const int kb1 = min(kb0 + a.kb_per_cta, a.kblocks);
    const int nkb = kb1 - kb0;
    const int per_warp = (nkb + W - 1) / W;
    const int wb0 = min(warp * per_warp, nkb), wb1 = min(wb0 + per_warp, nkb);

    // Shared memory: activations [nkb][2 halves][M][4 lanes] x 16 B, then the
    // reduction buffer (same offset in every block of a cluster).
    uint4* xs = reinterpret_cast<uint4*>(smem);
    float* red = reinterpret_cast<float*>(xs + size_t(a.kb_per_cta) * 8 * M);

    const int8_t* rowp[NT][2];
    size_t srow[NT][2];
    bool real[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = tile_row + nt * 16 + h * 8 + g;
            real[nt][h] = r < N;
            const int rc = min(r, N - 1);
            rowp[nt][h] = a.w + size_t(rc) * K + t * 16;
            srow[nt][h] = size_t(rc) * groups;
        }

    auto load_stage = [&](Stage8<NT>& s, int kb_local) {
        const int kb = kb0 + kb_local;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int h = 0; h < 2; ++h) s.q[nt][h] = ldg_stream(rowp[nt][h] + size_t(kb) * 64);
        if (MODE == kScaleBlock) {
            const int grp = (kb * 64) / G;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h) s.s[nt][h] = __ldg(a.scale + srow[nt][h] + grp);
        }
    };

    Stage8<NT> st[D];
#pragma unroll
    for (int d = 0; d < D; ++d)
        if (wb0 + d < wb1) load_stage(st[d], wb0 + d);

    pdl_launch_dependents();
    pdl_wait();  // activations may come from the kernel before this one
    {
        const uint4* xg = static_cast<const uint4*>(a.x);
        const int per_row = nkb * 8;  // 16-byte pieces per activation row
        const int total = M * per_row;
        for (int e = threadIdx.x; e < total; e += W * 32) {
            const int m = e / per_row, rem = e % per_row;
            const int j = rem / 8, c = rem % 8;
            const uint4 raw = ld_mutable(xg + (size_t(m) * K + size_t(kb0 + j) * 64) / 8 + c);
            xs[(size_t(j * 2 + (c & 1)) * M + m) * 4 + (c >> 1)] = raw;
        }
    }
    __syncthreads();

    float total[NT][MB][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 4; ++i) total[nt][mb][i] = 0.0f;

    for (int base = wb0; base < wb1; base += D) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const int j = base + d;
            if (j < wb1) {
                const Stage8<NT> cur = st[d];
                if (j + D < wb1) load_stage(st[d], j + D);
                uint4 b[MB][2];
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    const int m = mb * 8 + g;
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        b[mb][h] = m < M ? xs[(size_t(j * 2 + h) * M + m) * 4 + t]
                                         : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float acc[MB][4];
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[mb][i] = 0.0f;
                    const uint32_t w0[4] = {cur.q[nt][0].x, cur.q[nt][0].y, cur.q[nt][0].z, cur.q[nt][0].w};
                    const uint32_t w1[4] = {cur.q[nt][1].x, cur.q[nt][1].y, cur.q[nt][1].z, cur.q[nt][1].w};
                    float e0 = 1.0f, e1 = 1.0f;
                    if (MODE == kScaleElement) {
                        const int grp = ((kb0 + j) * 64 + t * 16) / G;
                        e0 = __ldg(a.scale + srow[nt][0] + grp);
                        e1 = __ldg(a.scale + srow[nt][1] + grp);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t frag[4];  // a0 (row g, k 0..1), a1 (row g+8), a2 (row g, k 2..3), a3
                        widen4<T, MODE == kScaleElement>(w0[i], e0, frag[0], frag[2]);
                        widen4<T, MODE == kScaleElement>(w1[i], e1, frag[1], frag[3]);
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb) {
                            const uint4 bb = b[mb][i / 2];
                            const uint32_t b0 = (i & 1) ? bb.z : bb.x, b1 = (i & 1) ? bb.w : bb.y;
                            if (MODE == kScaleBlock)
                                H::mma(acc[mb], frag, b0, b1);
                            else
                                H::mma(total[nt][mb], frag, b0, b1);
                        }
                    }
                    if (MODE == kScaleBlock) {
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb) {
                            total[nt][mb][0] = fmaf(cur.s[nt][0], acc[mb][0], total[nt][mb][0]);
                            total[nt][mb][1] = fmaf(cur.s[nt][0], acc[mb][1], total[nt][mb][1]);
                            total[nt][mb][2] = fmaf(cur.s[nt][1], acc[mb][2], total[nt][mb][2]);
                            total[nt][mb][3] = fmaf(cur.s[nt][1], acc[mb][3], total[nt][mb][3]);
                        }
                    }
                }
            }
        }
    }
    if (MODE == kScaleRow) {
        // The row's scale distributes over the K split, so each partial sum takes it.
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float s0 = real[nt][0] ? __ldg(a.scale + srow[nt][0]) : 0.0f;
            const float s1 = real[nt][1] ? __ldg(a.scale + srow[nt][1]) : 0.0f;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                total[nt][mb][0] *= s0;
                total[nt][mb][1] *= s0;
                total[nt][mb][2] *= s1;
                total[nt][mb][3] *= s1;
            }
        }
    }
    reduce_and_store<H, MB, NT, W>(total, red, a.ksplit, tile_row, M, N, static_cast<uint16_t*>(a.y));
}

// Shapes the tensor-core kernel does not take (K not a multiple of 64).
template <typename T>
__global__ void int8_linear_simple_kernel(const Gemv8Args a, int m0) {
    using H = Half16<T>;
    const int n = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (n >= a.N) return;
    const int rows = min(8, a.M - m0);
    const uint16_t* x = static_cast<const uint16_t*>(a.x);
    const int G = a.G == 0 ? a.K : a.G;
    const int groups = a.K / G;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = lane; k < a.K; k += 32) {
        const float s = a.scale[size_t(n) * groups + k / G];
        const float w = H::to_float(H::from_float(float(a.w[size_t(n) * a.K + k]) * s));
        for (int r = 0; r < rows; ++r)
            acc[r] = fmaf(H::to_float(x[size_t(m0 + r) * a.K + k]), w, acc[r]);
    }
    uint16_t* y = static_cast<uint16_t*>(a.y);
    for (int r = 0; r < rows; ++r) {
        float v = acc[r];
        for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
        if (lane == 0) y[size_t(m0 + r) * a.N + n] = H::from_float(v);
    }
}

template <typename T, int MODE, int MB, int NT, int W, int D>
int32_t launch_gemv8(const Gemv8Args& args, int ksplit, cudaStream_t stream) {
    Gemv8Args a = args;
    a.ksplit = ksplit;
    a.kb_per_cta = (a.kblocks + ksplit - 1) / ksplit;
    const int tiles = (a.N + 16 * NT - 1) / (16 * NT);
    const size_t smem = size_t(a.kb_per_cta) * 8 * a.M * 16 + size_t(W) * NT * 16 * MB * 8 * 4;
    return launch_clustered("int8_gemv", int8_gemv_kernel<T, MODE, MB, NT, W, D>, a, tiles, ksplit,
                            W * 32, smem, stream, true);
}

template <typename T, int MODE>
int32_t dispatch_gemv8(const Gemv8Args& a, cudaStream_t stream) {
    const int sms = sm_count();
    const int nt = a.M <= 8 ? 1 : 2;
    const int tiles = (a.N + 16 * nt - 1) / (16 * nt);
    int ksplit = 1;
    while (ksplit < 8 && a.kblocks / (ksplit * 2) >= 4 &&
           (tiles * ksplit < 3 * sms || size_t(a.kblocks / ksplit) * 128 * a.M > 48 * 1024))
        ksplit *= 2;
    if (a.M <= 8) return launch_gemv8<T, MODE, 1, 1, 4, 3>(a, ksplit, stream);
    return launch_gemv8<T, MODE, 2, 2, 4, 2>(a, ksplit, stream);
}

// One scale a row, one or two activation rows, and no request for the per-weight rounding:
// the kernel of int8_gemv_tma.cuh, which applies the scale to the finished sum as the
// reference's own GPU kernel does (python/linnet/src/linnet/torch/kernels.py:352-371).
template <typename T>
bool run_tma8(const Gemv8Args& a, cudaStream_t stream, int32_t* status) {
    if ((a.G != 0 && a.G != a.K) || a.M > 2 || (a.flags & B200Q_EXACT_WEIGHTS)) return false;
    if (size_t(a.N) * size_t(a.K) >= (size_t(1) << 40)) return false;
    int* word = gemm_error_word();
    if (word == nullptr) return false;
    Tma8Args p{a.x, a.scale, a.y, a.M, a.K, a.N, (a.N + 15) / 16, 1, 1, 1, 0, 1,
               (a.flags & B200Q_EARLY_DEPENDENTS) ? 1 : 0, word};
    size_t smem = 0;
    const int sms = sm_count();
    if (tma8_plan<16, 8>(p, &smem)) {
        *status = launch_tma8<T, 16, 8>(p, a.w, smem, sms, stream);
        return true;
    }
    if (tma8_plan<16, 4>(p, &smem)) {
        *status = launch_tma8<T, 16, 4>(p, a.w, smem, sms, stream);
        return true;
    }
    return false;
}

template <typename T>
int32_t run_gemv8(Gemv8Args a, int64_t rows, cudaStream_t stream) {
    const uint8_t* x = static_cast<const uint8_t*>(a.x);
    uint8_t* y = static_cast<uint8_t*>(a.y);
    for (int64_t m0 = 0; m0 < rows; m0 += 16) {
        a.M = int(rows - m0 < 16 ? rows - m0 : 16);
        a.x = x + size_t(m0) * a.K * 2;
        a.y = y + size_t(m0) * a.N * 2;
        int32_t status = B200Q_OK;
        if (run_tma8<T>(a, stream, &status)) {
            // scale applied to the sum
        } else if (a.K % 64 == 0 && (a.G == 0 || a.G % 16 == 0)) {
            // Every weight is scaled in f32 and rounded once to the 16-bit type before the
            // product, which is the reference's arithmetic ((w.float() * scale).to(dtype),
            // python/linnet/src/linnet/torch/quantized.py:193); applying the scale to the
            // sums instead is cheaper but rounds differently.
            Gemv8Args e = a;
            if (e.G == 0) e.G = e.K;
            status = dispatch_gemv8<T, kScaleElement>(e, stream);
        } else {
            for (int sub = 0; sub < a.M; sub += 8)
                int8_linear_simple_kernel<T><<<(a.N + 3) / 4, 128, 0, stream>>>(a, sub);
            status = launched("int8_linear (general kernel)");
        }
        if (status != B200Q_OK) return status;
    }
    return B200Q_OK;
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_int8_linear_ex(const void* x, const int8_t* w, const float* scale, void* y,
                                        int64_t rows, int64_t in, int64_t out, int64_t group,
                                        int32_t dtype, int32_t flags, void* stream) {
    B200Q_REQUIRE((flags & ~(B200Q_EXACT_WEIGHTS | B200Q_EARLY_DEPENDENTS)) == 0, "int8_linear: unknown flag bits %d", flags);
    B200Q_REQUIRE(dtype == B200Q_BF16 || dtype == B200Q_F16, "int8_linear: activations are bf16 or f16");
    B200Q_REQUIRE(rows >= 0 && in > 0 && out > 0, "int8_linear: bad shape rows=%lld in=%lld out=%lld",
                  (long long)rows, (long long)in, (long long)out);
    B200Q_REQUIRE(group >= 0 && (group == 0 || in % group == 0),
                  "int8_linear: groups of %lld must divide the %lld inputs", (long long)group, (long long)in);
    B200Q_REQUIRE(in < (int64_t(1) << 30) && out < (int64_t(1) << 30), "int8_linear: dimension too large");
    if (rows == 0) return B200Q_OK;
    B200Q_REQUIRE(x && w && scale && y, "int8_linear: null tensor");
    B200Q_REQUIRE(aligned(x, 16) && aligned(w, 16) && aligned(scale, 4) && aligned(y, 2),
                  "int8_linear: x and w must be 16-byte aligned");
    Gemv8Args a{x, w, scale, y, 0, int(in), int(out), int(group), int(in / 64), 0, 1, flags};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == B200Q_BF16 ? run_gemv8<__nv_bfloat16>(a, rows, s) : run_gemv8<__half>(a, rows, s);
}

extern "C" int32_t b200q_int8_linear(const void* x, const int8_t* w, const float* scale, void* y,
                                     int64_t rows, int64_t in, int64_t out, int64_t group,
                                     int32_t dtype, void* stream) {
    return b200q_int8_linear_ex(x, w, scale, y, rows, in, out, group, dtype, 0, stream);
}
