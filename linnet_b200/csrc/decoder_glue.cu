// The small kernels between the quantized linears of a decode step: residual add +
// RMSNorm, rotary embedding + KV-cache write, single-query attention over the cache
// (split over the keys, then merged) and SwiGLU's silu(gate) * up.
//
// In the reference these are stdlib ops lowered to PyTorch calls inside the captured
// decode graph (rms_norm, rope, index_put_ cache write, scaled_dot_product_attention,
// silu * mul: examples/01-llama/src/{lib,attention}.linnet run by
// python/linnet/src/linnet/torch/compiled.py:430-503); run that way a batch-1 step on a
// B200 spends three quarters of its time in ~50 tiny elementwise launches per layer, so
// the decode benchmark fuses them into six launches per layer.  Arithmetic follows the
// PyTorch ops (f32 math on bf16 values, one rounding where PyTorch rounds).
#include "common.cuh"

namespace b200q {
namespace {

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t bf16_pack(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ---- x (+= delta); y = rms_norm(x) * w --------------------------------------------
// One block per row; hidden is a multiple of 8.  x is updated in place when delta != null.
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(uint16_t* __restrict__ x, const uint16_t* __restrict__ delta,
                   const uint16_t* __restrict__ w, uint16_t* __restrict__ y, int hidden, float eps) {
    __shared__ float partial[8];
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x, chunks = hidden / 8;
    uint4* xr = reinterpret_cast<uint4*>(x + size_t(row) * hidden);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + size_t(row) * hidden) : nullptr;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        uint4 v = xr[c];
        if (dr) {
            const uint4 d = dr[c];
            v.x = bf16_pack(bf16_lo(v.x) + bf16_lo(d.x), bf16_hi(v.x) + bf16_hi(d.x));
            v.y = bf16_pack(bf16_lo(v.y) + bf16_lo(d.y), bf16_hi(v.y) + bf16_hi(d.y));
            v.z = bf16_pack(bf16_lo(v.z) + bf16_lo(d.z), bf16_hi(v.z) + bf16_hi(d.z));
            v.w = bf16_pack(bf16_lo(v.w) + bf16_lo(d.w), bf16_hi(v.w) + bf16_hi(d.w));
            xr[c] = v;
        }
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) sum += bf16_lo(u[i]) * bf16_lo(u[i]) + bf16_hi(u[i]) * bf16_hi(u[i]);
    }
    for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
    if (threadIdx.x % 32 == 0) partial[threadIdx.x / 32] = sum;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < int(blockDim.x) / 32; ++i) total += partial[i];
    const float rstd = rsqrtf(total / float(hidden) + eps);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    uint4* yr = reinterpret_cast<uint4*>(y + size_t(row) * hidden);
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        const uint4 v = xr[c], g = wr[c];
        uint4 o;
        o.x = bf16_pack(bf16_lo(v.x) * rstd * bf16_lo(g.x), bf16_hi(v.x) * rstd * bf16_hi(g.x));
        o.y = bf16_pack(bf16_lo(v.y) * rstd * bf16_lo(g.y), bf16_hi(v.y) * rstd * bf16_hi(g.y));
        o.z = bf16_pack(bf16_lo(v.z) * rstd * bf16_lo(g.z), bf16_hi(v.z) * rstd * bf16_hi(g.z));
        o.w = bf16_pack(bf16_lo(v.w) * rstd * bf16_lo(g.w), bf16_hi(v.w) * rstd * bf16_hi(g.w));
        yr[c] = o;
    }
}

// ---- rotary embedding of q and k, cache write of k and v -----------------------------
// qkv [B, (nq + 2 nkv) * hd]; q_out [B, nq, hd]; cache_{k,v} [B, nkv, S, hd]; halves rotated.
__global__ void rope_cache_kernel(const uint16_t* __restrict__ qkv, const int64_t* __restrict__ positions,
                                  uint16_t* __restrict__ q_out, uint16_t* __restrict__ cache_k,
                                  uint16_t* __restrict__ cache_v, int nq, int nkv, int hd, int S,
                                  float theta) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.y, head = blockIdx.x;  // head < nq: q; < nq + nkv: k; else v
    const int half = hd / 2;
    const int64_t pos = positions[b];
    const uint16_t* src = qkv + (size_t(b) * (nq + 2 * nkv) + head) * hd;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        if (head < nq + nkv) {
            const float freq = powf(theta, -float(i) / float(half));
            float s, c;
            sincosf(float(pos) * freq, &s, &c);
            const float a = bf16_lo(src[i]), bb = bf16_lo(src[i + half]);
            const uint16_t lo = uint16_t(bf16_pack(a * c - bb * s, 0.0f) & 0xFFFF);
            const uint16_t hi = uint16_t(bf16_pack(bb * c + a * s, 0.0f) & 0xFFFF);
            uint16_t* dst = head < nq ? q_out + (size_t(b) * nq + head) * hd
                                      : cache_k + ((size_t(b) * nkv + (head - nq)) * S + pos) * hd;
            dst[i] = lo;
            dst[i + half] = hi;
        } else {
            uint16_t* dst = cache_v + ((size_t(b) * nkv + (head - nq - nkv)) * S + pos) * hd;
            dst[i] = src[i];
            dst[i + half] = src[i + half];
        }
    }
}

// ---- single-query attention, split over the keys --------------------------------------
// Block (split, kv head, batch row): one warp per query head of the KV head's group (REP
// warps).  The block streams its keys and values through shared memory in chunks of 64
// positions with cp.async, two chunks in flight, so every K/V byte is read from HBM once
// for all REP heads and many bytes are in flight per multiprocessor; a group of HD/16
// lanes owns one position at a time (two 16-byte pieces per lane, laid out so a quarter
// warp reads 128 contiguous bytes) and keeps its own running softmax; the groups of a
// warp and finally the splits are merged with the usual (max, sum, weighted accumulator)
// rule.  partial: [B, nq, splits, HD + 2] f32.
constexpr int kAttnChunk = 64;

template <int HD, int REP>
__global__ void __launch_bounds__(32 * REP)
attention_partial_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ cache_k,
                         const uint16_t* __restrict__ cache_v, const int64_t* __restrict__ positions,
                         float* __restrict__ partial, int nq, int nkv, int S, int splits, float scale) {
    constexpr int LPK = HD / 16;             // lanes per position
    constexpr int KPW = 32 / LPK;            // positions per warp step
    constexpr int kRowBytes = HD * 2;
    constexpr int kStage = kAttnChunk * kRowBytes;  // bytes of K (or V) per chunk
    extern __shared__ __align__(16) uint8_t attn_smem[];  // [2 stages][K chunk | V chunk]
    pdl_wait();
    pdl_launch_dependents();
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int sub = lane / LPK, part = lane % LPK;
    const int keys = int(positions[b]) + 1;  // attend to positions 0 .. pos
    const int per_split = (keys + splits - 1) / splits;
    const int k0 = split * per_split, k1 = min(k0 + per_split, keys);
    const int chunks = k1 > k0 ? (k1 - k0 + kAttnChunk - 1) / kAttnChunk : 0;
    const size_t base = (size_t(b) * nkv + kvh) * S * HD;

    auto issue = [&](int c) {  // chunk c of this split -> stage c % 2
        uint8_t* dst = attn_smem + (c % 2) * 2 * kStage;
        const int first = k0 + c * kAttnChunk;
        for (int piece = threadIdx.x; piece < 2 * kStage / 16; piece += 32 * REP) {
            const int which = piece / (kStage / 16), within = piece % (kStage / 16);
            const int key = min(first + within / (kRowBytes / 16), k1 - 1);  // the tail repeats the last key
            const uint16_t* src = (which ? cache_v : cache_k) + base + size_t(key) * HD + (within % (kRowBytes / 16)) * 8;
            const uint32_t d = uint32_t(__cvta_generic_to_shared(dst + size_t(piece) * 16));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (chunks > 0) issue(0);
    if (chunks > 1) issue(1);

    // This warp's query head, scaled; the lane's 16 elements are [part*8, +8) of each half.
    float qv[16];
    {
        const uint16_t* qp = q + (size_t(b) * nq + kvh * REP + warp) * HD;
        const uint4 lo = *reinterpret_cast<const uint4*>(qp + part * 8);
        const uint4 hi = *reinterpret_cast<const uint4*>(qp + HD / 2 + part * 8);
        const uint32_t u[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            qv[2 * i] = bf16_lo(u[i]) * scale;
            qv[2 * i + 1] = bf16_hi(u[i]) * scale;
        }
    }
    float m = -INFINITY, l = 0.0f, acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;

    for (int c = 0; c < chunks; ++c) {
        if (c + 1 < chunks) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const uint8_t* ks = attn_smem + (c % 2) * 2 * kStage;
        const uint8_t* vs = ks + kStage;
        const int first = k0 + c * kAttnChunk;
#pragma unroll 2
        for (int s0 = 0; s0 < kAttnChunk; s0 += KPW) {
            const int slot = s0 + sub;
            const bool live = first + slot < k1;
            const uint4 ka = *reinterpret_cast<const uint4*>(ks + slot * kRowBytes + part * 16);
            const uint4 kb = *reinterpret_cast<const uint4*>(ks + slot * kRowBytes + HD + part * 16);
            const uint32_t ku[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) dot += qv[2 * i] * bf16_lo(ku[i]) + qv[2 * i + 1] * bf16_hi(ku[i]);
#pragma unroll
            for (int d = LPK / 2; d >= 1; d >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, d);
            if (live) {
                const uint4 va = *reinterpret_cast<const uint4*>(vs + slot * kRowBytes + part * 16);
                const uint4 vb = *reinterpret_cast<const uint4*>(vs + slot * kRowBytes + HD + part * 16);
                const uint32_t vu[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
                const float m_new = fmaxf(m, dot);
                const float corr = __expf(m - m_new), p = __expf(dot - m_new);
                m = m_new;
                l = l * corr + p;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    acc[2 * i] = acc[2 * i] * corr + p * bf16_lo(vu[i]);
                    acc[2 * i + 1] = acc[2 * i + 1] * corr + p * bf16_hi(vu[i]);
                }
            }
        }
        __syncthreads();  // everyone is done with this stage before it is refilled
        if (c + 2 < chunks) issue(c + 2);
    }
    // Merge the position slots of the warp (lanes with the same `part`).
#pragma unroll
    for (int d = LPK; d < 32; d <<= 1) {
        const float m_o = __shfl_xor_sync(0xFFFFFFFFu, m, d);
        const float l_o = __shfl_xor_sync(0xFFFFFFFFu, l, d);
        const float m_new = fmaxf(m, m_o);
        const float c_s = m == -INFINITY ? 0.0f : __expf(m - m_new);
        const float c_o = m_o == -INFINITY ? 0.0f : __expf(m_o - m_new);
        l = l * c_s + l_o * c_o;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float a_o = __shfl_xor_sync(0xFFFFFFFFu, acc[i], d);
            acc[i] = acc[i] * c_s + a_o * c_o;
        }
        m = m_new;
    }
    if (sub == 0) {
        float* out = partial + ((size_t(b) * nq + kvh * REP + warp) * splits + split) * (HD + 2);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            out[part * 8 + i] = acc[i];
            out[HD / 2 + part * 8 + i] = acc[8 + i];
        }
        if (part == 0) {
            out[HD] = m;
            out[HD + 1] = l;
        }
    }
}

template <int HD>
__global__ void attention_merge_kernel(const float* __restrict__ partial, uint16_t* __restrict__ out,
                                       int splits) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t head = blockIdx.x;  // b * nq + query head
    const float* p = partial + head * splits * (HD + 2);
    float m_all = -INFINITY;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, p[s * (HD + 2) + HD]);
    for (int dcol = threadIdx.x; dcol < HD; dcol += blockDim.x) {
        float l_all = 0.0f, a_all = 0.0f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            const float ms = p[s * (HD + 2) + HD];
            const float c = ms == -INFINITY ? 0.0f : __expf(ms - m_all);
            l_all += p[s * (HD + 2) + HD + 1] * c;
            a_all += p[s * (HD + 2) + dcol] * c;
        }
        out[head * HD + dcol] = uint16_t(bf16_pack(a_all / l_all, 0.0f) & 0xFFFF);
    }
}

// ---- silu(gate) * up ---------------------------------------------------------------------
// gate_up [B, 2 I] -> out [B, I]; silu is rounded to bf16 before the product, as the two
// PyTorch ops do.
__global__ void silu_mul_kernel(const uint16_t* __restrict__ gate_up, uint16_t* __restrict__ out,
                                int inner, int64_t total) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += int64_t(gridDim.x) * blockDim.x) {
        const int64_t row = e / inner, col = e % inner;
        const float g = bf16_lo(gate_up[row * 2 * inner + col]);
        const float u = bf16_lo(gate_up[row * 2 * inner + inner + col]);
        const float s = bf16_round(g / (1.0f + expf(-g)));
        out[e] = uint16_t(bf16_pack(s * u, 0.0f) & 0xFFFF);
    }
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_add_rmsnorm(void* x, const void* delta, const void* weight, void* y,
                                     int64_t rows, int64_t hidden, float eps, void* stream) {
    B200Q_REQUIRE(rows >= 0 && hidden > 0 && hidden % 8 == 0, "add_rmsnorm: hidden must be a multiple of 8");
    if (rows == 0) return B200Q_OK;
    B200Q_REQUIRE(x && weight && y && aligned(x, 16) && aligned(weight, 16) && aligned(y, 16) &&
                      (!delta || aligned(delta, 16)),
                  "add_rmsnorm: tensors must be 16-byte aligned");
    return launch_status("add_rmsnorm", launch_overlapped(
        add_rmsnorm_kernel, dim3(unsigned(rows)), dim3(256), 0, static_cast<cudaStream_t>(stream),
        static_cast<uint16_t*>(x), static_cast<const uint16_t*>(delta), static_cast<const uint16_t*>(weight),
        static_cast<uint16_t*>(y), int(hidden), eps));
}

extern "C" int32_t b200q_rope_cache(const void* qkv, const int64_t* positions, void* q_out, void* cache_k,
                                    void* cache_v, int64_t batch, int64_t nq, int64_t nkv, int64_t head_dim,
                                    int64_t max_seq, float theta, void* stream) {
    B200Q_REQUIRE(batch >= 0 && nq > 0 && nkv > 0 && head_dim % 2 == 0, "rope_cache: bad shape");
    if (batch == 0) return B200Q_OK;
    return launch_status("rope_cache", launch_overlapped(
        rope_cache_kernel, dim3(unsigned(nq + 2 * nkv), unsigned(batch)), dim3(64), 0,
        static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(qkv), positions,
        static_cast<uint16_t*>(q_out), static_cast<uint16_t*>(cache_k), static_cast<uint16_t*>(cache_v), int(nq),
        int(nkv), int(head_dim), int(max_seq), theta));
}

extern "C" int64_t b200q_decode_attention_scratch_bytes(int64_t batch, int64_t nq, int64_t head_dim,
                                                        int64_t splits) {
    return batch * nq * splits * (head_dim + 2) * 4;
}

namespace b200q {
namespace {

int32_t launch_attention(const char* who, const void* q, const void* cache_k, const void* cache_v,
                         const int64_t* positions, void* out, void* scratch, int64_t batch, int64_t nq,
                         int64_t nkv, int64_t head_dim, int64_t max_seq, int64_t splits, void* stream) {
    B200Q_REQUIRE(batch >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0 && splits >= 1 && splits <= 65535,
                  "%s: bad shape", who);
    if (batch == 0) return B200Q_OK;
    const int rep = int(nq / nkv);
    B200Q_REQUIRE((head_dim == 128 || head_dim == 64) && (rep == 1 || rep == 2 || rep == 4 || rep == 8),
                  "%s: head_dim is 64 or 128 and heads / kv_heads is 1, 2, 4 or 8", who);
    B200Q_REQUIRE(q && cache_k && cache_v && positions && out && scratch && aligned(q, 16) &&
                      aligned(cache_k, 16) && aligned(cache_v, 16) && aligned(scratch, 16),
                  "%s: tensors must be 16-byte aligned", who);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid{unsigned(splits), unsigned(nkv), unsigned(batch)};
    const float scale = 1.0f / sqrtf(float(head_dim));
#define B200Q_ATTN(HD, REP) do {                                                                      \
    cudaFuncSetAttribute(attention_partial_kernel<HD, REP>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                         4 * kAttnChunk * HD * 2);                                                    \
    launch_overlapped(attention_partial_kernel<HD, REP>, grid, dim3(32 * REP),                        \
                      size_t(4) * kAttnChunk * HD * 2, s,                                             \
                      static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(cache_k),         \
                      static_cast<const uint16_t*>(cache_v), positions, static_cast<float*>(scratch), \
                      int(nq), int(nkv), int(max_seq), int(splits), scale); } while (0)
    if (head_dim == 128) {
        if (rep == 1) B200Q_ATTN(128, 1); else if (rep == 2) B200Q_ATTN(128, 2);
        else if (rep == 4) B200Q_ATTN(128, 4); else B200Q_ATTN(128, 8);
        launch_overlapped(attention_merge_kernel<128>, dim3(unsigned(batch * nq)), dim3(128), 0, s,
                          static_cast<const float*>(scratch), static_cast<uint16_t*>(out), int(splits));
    } else {
        if (rep == 1) B200Q_ATTN(64, 1); else if (rep == 2) B200Q_ATTN(64, 2);
        else if (rep == 4) B200Q_ATTN(64, 4); else B200Q_ATTN(64, 8);
        launch_overlapped(attention_merge_kernel<64>, dim3(unsigned(batch * nq)), dim3(64), 0, s,
                          static_cast<const float*>(scratch), static_cast<uint16_t*>(out), int(splits));
    }
#undef B200Q_ATTN
    return launched(who);
}

}  // namespace
}  // namespace b200q

extern "C" int32_t b200q_decode_attention(const void* q, const void* cache_k, const void* cache_v,
                                          const int64_t* positions, void* out, void* scratch,
                                          int64_t batch, int64_t nq, int64_t nkv, int64_t head_dim,
                                          int64_t max_seq, int64_t splits, void* stream) {
    return launch_attention("decode_attention", q, cache_k, cache_v, positions, out, scratch, batch, nq,
                            nkv, head_dim, max_seq, splits, stream);
}

// ---- the same attention for callers that cannot allocate device memory ----------------
// Some hosts of this library have no way to hand it scratch memory: a runtime that owns a
// fixed arena sized before the model is known, a plug-in loaded into a server whose
// allocator is off limits to it, code running while a stream is being captured (no
// cudaMalloc there).  For them the splits' partial results live in a fixed array inside
// the library image instead: 4 MiB that every GPU which loads the library keeps until
// the process exits.
constexpr int64_t kStaticScratchBytes = int64_t(4) << 20;
static __device__ __align__(256) unsigned char g_attention_scratch[kStaticScratchBytes];

namespace b200q {
namespace {

// In host code `g_attention_scratch` is only a handle for the runtime, not a device
// address; the address is asked for once per device, with that device current.
void* static_scratch_address() {
    static void* cached[64] = {nullptr};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (cached[device] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_attention_scratch) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cached[device] = p;
    }
    return cached[device];
}

}  // namespace
}  // namespace b200q

extern "C" int64_t b200q_decode_attention_static_scratch_limit(void) { return kStaticScratchBytes; }

extern "C" int32_t b200q_decode_attention_static(const void* q, const void* cache_k, const void* cache_v,
                                                 const int64_t* positions, void* out, int64_t batch,
                                                 int64_t nq, int64_t nkv, int64_t head_dim, int64_t max_seq,
                                                 int64_t splits, void* stream) {
    B200Q_REQUIRE(batch >= 0 && nq > 0 && head_dim > 0 && splits >= 1, "decode_attention_static: bad shape");
    const int64_t need = b200q_decode_attention_scratch_bytes(batch, nq, head_dim, splits);
    B200Q_REQUIRE(need <= kStaticScratchBytes,
                  "decode_attention_static: batch %lld x %lld heads x %lld splits needs %lld bytes of scratch, "
                  "the built-in array holds %lld; use fewer splits or b200q_decode_attention with your own scratch",
                  (long long)batch, (long long)nq, (long long)splits, (long long)need,
                  (long long)kStaticScratchBytes);
    void* scratch = static_scratch_address();
    B200Q_REQUIRE(scratch != nullptr, "decode_attention_static: cudaGetSymbolAddress failed on this device");
    return launch_attention("decode_attention_static", q, cache_k, cache_v, positions, out, scratch, batch, nq,
                            nkv, head_dim, max_seq, splits, stream);
}

extern "C" int32_t b200q_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t inner, void* stream) {
    B200Q_REQUIRE(rows >= 0 && inner > 0, "silu_mul: bad shape");
    const int64_t total = rows * inner;
    if (total == 0) return B200Q_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > int64_t(sm_count()) * 16) blocks = int64_t(sm_count()) * 16;
    return launch_status("silu_mul", launch_overlapped(
        silu_mul_kernel, dim3(unsigned(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
        static_cast<const uint16_t*>(gate_up), static_cast<uint16_t*>(out), int(inner), total));
}
