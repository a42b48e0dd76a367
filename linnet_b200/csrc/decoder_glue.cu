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

static __device__ int g_decoder_error = 0;

namespace b200q {

int* decoder_error_word() {
    // In host code the symbol is a handle, not an address: ask once per device.
    static int* cached[64] = {nullptr};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (cached[device] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_decoder_error) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cached[device] = static_cast<int*>(p);
    }
    return cached[device];
}

namespace {

// ---- x (+= delta); y = rms_norm(x) * w --------------------------------------------
// One block per row; hidden is a multiple of 8.  x is updated in place when delta != null.
// A decode step runs this on a handful of rows, so what counts is the length of the chain
// of dependent memory round trips: the norm weights do not depend on the kernel before, so
// they are fetched before waiting for it, and the row stays in registers between the sum of
// squares and the scaling (CPT 16-byte pieces per thread; CPT = 0 re-reads x, any width).
template <int CPT>
__global__ void __launch_bounds__(512)
add_rmsnorm_kernel(uint16_t* x, const uint16_t* delta,  // read with ld_mutable()
                   const uint16_t* __restrict__ w, uint16_t* __restrict__ y, int hidden, float eps) {
    __shared__ float partial[16];
    constexpr int kHeld = CPT > 0 ? CPT : 1;
    const int row = blockIdx.x, chunks = hidden / 8;
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    uint4 g[kHeld], v[kHeld];
    if (CPT > 0) {
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            g[u] = c < chunks ? __ldg(wr + c) : make_uint4(0, 0, 0, 0);
        }
    }
    pdl_launch_dependents();  // the next kernel may start its own prologue (a product: its weight fetch) at once
    pdl_wait();
    uint4* xr = reinterpret_cast<uint4*>(x + size_t(row) * hidden);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + size_t(row) * hidden) : nullptr;
    float sum = 0.0f;
    auto add_and_square = [&](int c) {
        uint4 t = ld_mutable(xr + c);
        if (dr) {
            const uint4 d = ld_mutable(dr + c);
            t.x = bf16_pack(bf16_lo(t.x) + bf16_lo(d.x), bf16_hi(t.x) + bf16_hi(d.x));
            t.y = bf16_pack(bf16_lo(t.y) + bf16_lo(d.y), bf16_hi(t.y) + bf16_hi(d.y));
            t.z = bf16_pack(bf16_lo(t.z) + bf16_lo(d.z), bf16_hi(t.z) + bf16_hi(d.z));
            t.w = bf16_pack(bf16_lo(t.w) + bf16_lo(d.w), bf16_hi(t.w) + bf16_hi(d.w));
            xr[c] = t;
        }
        const uint32_t e[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) sum += bf16_lo(e[i]) * bf16_lo(e[i]) + bf16_hi(e[i]) * bf16_hi(e[i]);
        return t;
    };
    if (CPT > 0) {
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            v[u] = c < chunks ? add_and_square(c) : make_uint4(0, 0, 0, 0);
        }
    } else {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) add_and_square(c);
    }
    for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
    if (threadIdx.x % 32 == 0) partial[threadIdx.x / 32] = sum;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < int(blockDim.x) / 32; ++i) total += partial[i];
    const float rstd = rsqrtf(total / float(hidden) + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + size_t(row) * hidden);
    auto scaled = [&](const uint4& t, const uint4& gw) {
        uint4 o;
        o.x = bf16_pack(bf16_lo(t.x) * rstd * bf16_lo(gw.x), bf16_hi(t.x) * rstd * bf16_hi(gw.x));
        o.y = bf16_pack(bf16_lo(t.y) * rstd * bf16_lo(gw.y), bf16_hi(t.y) * rstd * bf16_hi(gw.y));
        o.z = bf16_pack(bf16_lo(t.z) * rstd * bf16_lo(gw.z), bf16_hi(t.z) * rstd * bf16_hi(gw.z));
        o.w = bf16_pack(bf16_lo(t.w) * rstd * bf16_lo(gw.w), bf16_hi(t.w) * rstd * bf16_hi(gw.w));
        return o;
    };
    if (CPT > 0) {
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            if (c < chunks) yr[c] = scaled(v[u], g[u]);
        }
    } else {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) yr[c] = scaled(ld_mutable(xr + c), wr[c]);
    }
}

// ---- rotary embedding of q and k, cache write of k and v -----------------------------
// qkv [B, (nq + 2 nkv) * hd]; q_out [B, nq, hd]; cache_{k,v} [B, nkv, S, hd]; halves rotated.
__global__ void rope_cache_kernel(const uint16_t* qkv, const int64_t* positions,
                                  uint16_t* __restrict__ q_out, uint16_t* __restrict__ cache_k,
                                  uint16_t* __restrict__ cache_v, int nq, int nkv, int hd, int S,
                                  float theta, int* status) {
    pdl_launch_dependents();  // the next kernel may start its own prologue (a product: its weight fetch) at once
    pdl_wait();
    const int b = blockIdx.y, head = blockIdx.x;  // head < nq: q; < nq + nkv: k; else v
    const int half = hd / 2;
    int64_t pos = ld_mutable(positions + b);
    const bool bad = pos < 0 || pos >= S;  // outside the cache: nothing is written for this row
    if (bad) {
        if (threadIdx.x == 0 && head == 0) record_bad_position(status, b);
        if (head >= nq) return;
        pos = 0;
    }
    const uint16_t* src = qkv + (size_t(b) * (nq + 2 * nkv) + head) * hd;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        if (head < nq + nkv) {
            const float freq = powf(theta, -float(i) / float(half));
            float s, c;
            sincosf(float(pos) * freq, &s, &c);
            const float a = bf16_lo(ld_mutable(src + i)), bb = bf16_lo(ld_mutable(src + i + half));
            const uint16_t lo = uint16_t(bf16_pack(a * c - bb * s, 0.0f) & 0xFFFF);
            const uint16_t hi = uint16_t(bf16_pack(bb * c + a * s, 0.0f) & 0xFFFF);
            uint16_t* dst = head < nq ? q_out + (size_t(b) * nq + head) * hd
                                      : cache_k + ((size_t(b) * nkv + (head - nq)) * S + pos) * hd;
            dst[i] = lo;
            dst[i + half] = hi;
        } else {
            uint16_t* dst = cache_v + ((size_t(b) * nkv + (head - nq - nkv)) * S + pos) * hd;
            dst[i] = ld_mutable(src + i);
            dst[i + half] = ld_mutable(src + i + half);
        }
    }
}

// ---- silu(gate) * up ---------------------------------------------------------------------
// gate_up [B, 2 I] -> out [B, I]; silu is rounded to bf16 before the product, as the two
// PyTorch ops do.
__global__ void silu_mul_kernel(const uint16_t* gate_up, uint16_t* __restrict__ out,
                                int inner, int64_t total) {
    pdl_launch_dependents();  // the next kernel may start its own prologue (a product: its weight fetch) at once
    pdl_wait();
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += int64_t(gridDim.x) * blockDim.x) {
        const int64_t row = e / inner, col = e % inner;
        const float g = bf16_lo(ld_mutable(gate_up + row * 2 * inner + col));
        const float u = bf16_lo(ld_mutable(gate_up + row * 2 * inner + inner + col));
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
    const int chunks = int(hidden / 8);
    int threads = ((chunks + 31) / 32) * 32;
    threads = threads > 512 ? 512 : threads;
    const int held = (chunks + threads - 1) / threads;
    const dim3 grid{unsigned(rows)}, block{unsigned(threads)};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint16_t* xp = static_cast<uint16_t*>(x);
    const uint16_t* dp = static_cast<const uint16_t*>(delta);
    const uint16_t* wp = static_cast<const uint16_t*>(weight);
    uint16_t* yp = static_cast<uint16_t*>(y);
    cudaError_t err;
    if (held <= 1) err = launch_overlapped(add_rmsnorm_kernel<1>, grid, block, 0, s, xp, dp, wp, yp, int(hidden), eps);
    else if (held <= 2) err = launch_overlapped(add_rmsnorm_kernel<2>, grid, block, 0, s, xp, dp, wp, yp, int(hidden), eps);
    else if (held <= 4) err = launch_overlapped(add_rmsnorm_kernel<4>, grid, block, 0, s, xp, dp, wp, yp, int(hidden), eps);
    else err = launch_overlapped(add_rmsnorm_kernel<0>, grid, block, 0, s, xp, dp, wp, yp, int(hidden), eps);
    return launch_status("add_rmsnorm", err);
}

extern "C" int32_t b200q_rope_cache(const void* qkv, const int64_t* positions, void* q_out, void* cache_k,
                                    void* cache_v, int64_t batch, int64_t nq, int64_t nkv, int64_t head_dim,
                                    int64_t max_seq, float theta, void* stream) {
    B200Q_REQUIRE(batch >= 0 && nq > 0 && nkv > 0 && head_dim % 2 == 0 && max_seq > 0, "rope_cache: bad shape");
    B200Q_REQUIRE(batch == 0 || (qkv && positions && q_out && cache_k && cache_v && aligned(positions, 8)),
                  "rope_cache: null tensor, or positions not int64");
    if (batch == 0) return B200Q_OK;
    return launch_status("rope_cache", launch_overlapped(
        rope_cache_kernel, dim3(unsigned(nq + 2 * nkv), unsigned(batch)), dim3(64), 0,
        static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(qkv), positions,
        static_cast<uint16_t*>(q_out), static_cast<uint16_t*>(cache_k), static_cast<uint16_t*>(cache_v), int(nq),
        int(nkv), int(head_dim), int(max_seq), theta, decoder_error_word()));
}

extern "C" int32_t b200q_decoder_status(void) {
    int flag = 0;
    cudaError_t err = cudaMemcpyFromSymbol(&flag, g_decoder_error, sizeof(int));
    if (err != cudaSuccess) return fail("decoder_status: %s", cudaGetErrorString(err));
    if (flag != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_decoder_error, &zero, sizeof(int));
        return fail("decode step: the position of batch row %d lies outside its cache; that row's keys and "
                    "values were not stored", flag - 1);
    }
    return B200Q_OK;
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
