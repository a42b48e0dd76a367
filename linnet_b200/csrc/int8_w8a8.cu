// 8-bit activations times 8-bit weights (W8A8): the reference's route for int8 layers under
// `numerics="fast"` past 32 rows (python/linnet/src/linnet/torch/quantized.py:187-189).
//
//   int8_rows  (linnet::rows8, python/linnet/src/linnet/torch/kernels.py:669-753)
//       every row of x gets a scale of its own, max|row| / 127 (at least 1e-12 / 127), and is
//       rounded to int8 levels: x / scale, half away from zero, clamped to +-127.
//   int8_mm    (linnet::int8_mm, kernels.py:805-915)
//       y[m, n] = (sum_k xq[m, k] * w[n, k]) * x_scale[m] * w_scale[n], the sum exact in int32,
//       the two scales applied in f32 in that order, one rounding to the output type.
//
// int8_mm runs on the Blackwell tensor cores: tcgen05.mma kind::i8 with the int32 accumulator
// in tensor memory.  Both operands are plain int8 row-major tensors, so both come straight
// from global memory by TMA (128-byte swizzle, no register stage in between): warp 4 is the
// TMA producer, one thread of warp 5 issues the MMAs (128 x BN x 32 per instruction, four per
// 128-byte stage), warps 0-3 are the epilogue (tcgen05.ld -> f32 -> scales -> 16-bit -> y).
// One persistent block per multiprocessor walks over the 128 x BN tiles; the accumulators are
// double-buffered so a tile's epilogue overlaps the next tile's products.  Every mbarrier
// wait is bounded (shared with the int4 GEMM: b200q_int4_gemm_status() reports an expiry).
#include "mma.cuh"
#include "umma.cuh"

namespace b200q {


namespace {

using namespace umma;

// ---- int8_rows ------------------------------------------------------------------------------

// One block per row.  A thread keeps up to kHeld 16-byte pieces (8 values each) in registers
// between the maximum and the rounding; longer rows are read twice.
template <typename T, int kHeld>
__global__ void __launch_bounds__(256)
rows8_kernel(const uint16_t* x, int8_t* __restrict__ q, float* __restrict__ scale_out, int depth) {
    using H = Half16<T>;
    __shared__ float warp_max[8];
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x, pieces = depth / 8;
    const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * depth);
    uint4 held[kHeld];
    float top = 0.0f;
    auto absmax = [&](const uint4& v) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            top = fmaxf(top, fabsf(H::to_float(w[i] & 0xFFFFu)));
            top = fmaxf(top, fabsf(H::to_float(w[i] >> 16)));
        }
    };
#pragma unroll
    for (int u = 0; u < kHeld; ++u) {
        const int c = threadIdx.x + u * 256;
        held[u] = c < pieces ? ld_mutable(xr + c) : make_uint4(0, 0, 0, 0);
        absmax(held[u]);
    }
    for (int c = threadIdx.x + kHeld * 256; c < pieces; c += 256) absmax(ld_mutable(xr + c));
    for (int d = 16; d >= 1; d >>= 1) top = fmaxf(top, __shfl_xor_sync(0xFFFFFFFFu, top, d));
    if (threadIdx.x % 32 == 0) warp_max[threadIdx.x / 32] = top;
    __syncthreads();
    top = warp_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) top = fmaxf(top, warp_max[w]);
    const float scale = __fdiv_rn(fmaxf(top, 1e-12f), 127.0f);
    if (threadIdx.x == 0) scale_out[row] = scale;
    auto level = [&](float v) -> uint32_t {
        const float s = __fdiv_rn(v, scale);
        const float r = fminf(fmaxf(s >= 0.0f ? __fadd_rn(s, 0.5f) : __fadd_rn(s, -0.5f), -127.0f), 127.0f);
        return uint32_t(__float2int_rz(r)) & 0xFFu;
    };
    auto round8 = [&](const uint4& v) -> uint2 {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t out[2];
#pragma unroll
        for (int i = 0; i < 2; ++i)
            out[i] = level(H::to_float(w[2 * i] & 0xFFFFu)) | (level(H::to_float(w[2 * i] >> 16)) << 8) |
                     (level(H::to_float(w[2 * i + 1] & 0xFFFFu)) << 16) | (level(H::to_float(w[2 * i + 1] >> 16)) << 24);
        return make_uint2(out[0], out[1]);
    };
    uint2* qr = reinterpret_cast<uint2*>(q + size_t(row) * depth);
#pragma unroll
    for (int u = 0; u < kHeld; ++u) {
        const int c = threadIdx.x + u * 256;
        if (c < pieces) qr[c] = round8(held[u]);
    }
    for (int c = threadIdx.x + kHeld * 256; c < pieces; c += 256) qr[c] = round8(ld_mutable(xr + c));
}

// ---- int8_mm ---------------------------------------------------------------------------------

constexpr int kBM = 128;      // rows of x per tile (the MMA's M)
constexpr int kBK = 128;      // int8 inputs per stage: one 128-byte swizzle atom
constexpr int kEpilogueWarps = 4, kTmaWarp = 4, kMmaWarp = 5;
constexpr int kThreads = 6 * 32;

template <int BN>
struct Shape8 {
    static constexpr int kStages = BN == 128 ? 6 : 4;
    static constexpr int kStageBytes = kBM * kBK + BN * kBK;
    static constexpr uint32_t kTmemColumns = 2 * BN;  // two accumulators of BN columns
    static constexpr size_t kSmem = size_t(kStages) * kStageBytes + 1024 + 256;
};

struct MmArgs {
    const float* x_scale;  // [M]
    const float* w_scale;  // [N]
    uint16_t* y;           // [M, N]
    int M, K, N;
    int m_tiles, n_tiles;
    int bn;                // rows of W per tile: BN, or for BN = 256 any multiple of 16 up to it
    int f16;               // output type: 0 bf16, 1 f16
    int vec;               // y can be written 16 bytes at a time (N % 8 == 0, y aligned)
};

struct Pipe8 {
    uint64_t full[8];       // TMA bytes of both operands landed
    uint64_t empty[8];      // MMAs that read the stage completed
    uint64_t acc_full[2];   // all MMAs of a tile completed
    uint64_t acc_empty[2];  // epilogue drained the accumulator (4 warp arrivals)
    uint32_t tmem_base;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
int8_mm_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
               const MmArgs a, int* error) {
    using S = Shape8<BN>;
    constexpr int kStages = S::kStages, kStageBytes = S::kStageBytes;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Pipe8* pipe = reinterpret_cast<Pipe8*>(smem + kStages * kStageBytes);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int tiles = a.m_tiles * a.n_tiles;
    const int ksteps = a.K / kBK;
    // The tile's width is a run-time value (the W map's box has that many rows): the layout in
    // shared and tensor memory stays that of BN.
    const int bn = BN == 128 ? 128 : a.bn;
    // int32 accumulator, signed 8-bit A and B, both K-major, M = 128, N = bn
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(kBM >> 4) << 24);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&pipe->full[s], 1);
            mbar_init(&pipe->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&pipe->acc_full[b], 1);
            mbar_init(&pipe->acc_empty[b], kEpilogueWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {  // one warp allocates (and later frees) the tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&pipe->tmem_base)),
                     "r"(S::kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = pipe->tmem_base;
    pdl_wait();  // the rounded activations come from the kernel ahead of this one
    pdl_launch_dependents();

    if (warp == kTmaWarp) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            // tiles ordered with the row block fastest: blocks that share a weight tile run together
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % a.m_tiles) * kBM, n0 = (tile / a.m_tiles) * bn;
                for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
                    const int s = it % kStages;
                    if (it >= uint32_t(kStages)) ok = mbar_wait(&pipe->empty[s], ((it / kStages) - 1) & 1, error, 11);
                    if (!ok) break;
                    uint8_t* dst = smem + s * kStageBytes;
                    mbar_expect_tx(&pipe->full[s], (kBM + bn) * kBK);
                    tma_load_2d(dst, &x_map, ks * kBK, m0, &pipe->full[s]);
                    tma_load_2d(dst + kBM * kBK, &w_map, ks * kBK, n0, &pipe->full[s]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++t) {
                const uint32_t buf = t & 1;
                if (t >= 2) ok = mbar_wait(&pipe->acc_empty[buf], ((t / 2) - 1) & 1, error, 12);
                tc_fence_after();
                for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
                    const int s = it % kStages;
                    ok = mbar_wait(&pipe->full[s], (it / kStages) & 1, error, 13);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t base = smem_u32(smem + s * kStageBytes);
#pragma unroll
                    for (int kk = 0; kk < kBK / 32; ++kk)  // 32 bytes of K per instruction
                        umma_i8(tmem + buf * BN, smem_desc(base + kk * 32), smem_desc(base + kBM * kBK + kk * 32),
                                idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(&pipe->empty[s]);  // frees the stage when these MMAs retire
                }
                if (ok) umma_commit(&pipe->acc_full[buf]);
            }
        }
    } else {
        // ---- epilogue (warp w owns tensor-memory lanes 32w .. 32w+31 = rows of the tile) ----
        uint32_t t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++t) {
            const int m0 = (tile % a.m_tiles) * kBM, n0 = (tile / a.m_tiles) * bn;
            const uint32_t buf = t & 1;
            ok = mbar_wait(&pipe->acc_full[buf], (t / 2) & 1, error, 14);
            if (!ok) break;
            tc_fence_after();
            const int m = m0 + warp * 32 + lane;
            const float xs = m < a.M ? __ldg(a.x_scale + m) : 0.0f;
#pragma unroll 1
            for (int c0 = 0; c0 < bn; c0 += 32) {
                uint32_t v[32];
                tmem_load_32(v, tmem + (uint32_t(warp * 32) << 16) + buf * BN + c0);  // (past bn: not stored)
                if (m < a.M) {
                    uint16_t* dst = a.y + size_t(m) * a.N + n0 + c0;
                    const int live = min(min(bn - c0, a.N - n0 - c0), 32);  // columns of this chunk that exist
                    uint16_t out[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = n0 + c0 + j;
                        const float ws = j < live ? __ldg(a.w_scale + n) : 0.0f;
                        const float r = __fmul_rn(__fmul_rn(float(int32_t(v[j])), xs), ws);
                        out[j] = a.f16 ? Half16<__half>::from_float(r) : Half16<__nv_bfloat16>::from_float(r);
                    }
                    if (a.vec) {  // bn, n0 and N are multiples of 8: 16-byte pieces are whole or absent
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (8 * j >= live) break;
                            uint4 o;
                            o.x = uint32_t(out[8 * j + 0]) | (uint32_t(out[8 * j + 1]) << 16);
                            o.y = uint32_t(out[8 * j + 2]) | (uint32_t(out[8 * j + 3]) << 16);
                            o.z = uint32_t(out[8 * j + 4]) | (uint32_t(out[8 * j + 5]) << 16);
                            o.w = uint32_t(out[8 * j + 6]) | (uint32_t(out[8 * j + 7]) << 16);
                            reinterpret_cast<uint4*>(dst)[j] = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < live) dst[j] = out[j];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&pipe->acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(S::kTmemColumns)
                     : "memory");
    }
}

int32_t make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t depth, int box_rows, const char* who) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return unavailable("%s: the driver has no cuTensorMapEncodeTiled", who);
    const cuuint64_t dims[2] = {cuuint64_t(depth), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(depth)};
    const cuuint32_t box[2] = {cuuint32_t(kBK), cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult made = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                                 elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (made != CUDA_SUCCESS) return fail("%s: cuTensorMapEncodeTiled failed (%d)", who, int(made));
    return B200Q_OK;
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_int8_rows(const void* x, int8_t* q, float* scale, int64_t rows, int64_t in, int32_t dtype,
                                   void* stream) {
    B200Q_REQUIRE(dtype == B200Q_BF16 || dtype == B200Q_F16, "int8_rows: activations are bf16 or f16");
    B200Q_REQUIRE(rows >= 0 && in > 0 && in % 8 == 0 && in < (int64_t(1) << 30), "int8_rows: rows of a multiple of 8 inputs");
    if (rows == 0) return B200Q_OK;
    B200Q_REQUIRE(x && q && scale && aligned(x, 16) && aligned(q, 8), "int8_rows: null or misaligned tensor");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid{unsigned(rows)}, block{256};
    const int pieces = int(in / 8);
    const uint16_t* xp = static_cast<const uint16_t*>(x);
    cudaError_t err;
#define B200Q_ROWS8(T)                                                                                       \
    (pieces <= 512    ? launch_overlapped(rows8_kernel<T, 2>, grid, block, 0, s, xp, q, scale, int(in))       \
     : pieces <= 2048 ? launch_overlapped(rows8_kernel<T, 8>, grid, block, 0, s, xp, q, scale, int(in))       \
                      : launch_overlapped(rows8_kernel<T, 1>, grid, block, 0, s, xp, q, scale, int(in)))
    err = dtype == B200Q_BF16 ? B200Q_ROWS8(__nv_bfloat16) : B200Q_ROWS8(__half);
#undef B200Q_ROWS8
    return launch_status("int8_rows", err);
}

extern "C" int32_t b200q_int8_mm(const int8_t* xq, const int8_t* w, const float* x_scale, const float* w_scale,
                                 void* y, int64_t rows, int64_t in, int64_t out, int32_t dtype, void* stream) {
    B200Q_REQUIRE(dtype == B200Q_BF16 || dtype == B200Q_F16, "int8_mm: the output is bf16 or f16");
    B200Q_REQUIRE(rows >= 0 && in > 0 && out > 0 && in % kBK == 0, "int8_mm: inputs must be a multiple of %d", kBK);
    B200Q_REQUIRE(rows < (int64_t(1) << 30) && in < (int64_t(1) << 30) && out < (int64_t(1) << 30), "int8_mm: too large");
    if (rows == 0) return B200Q_OK;
    B200Q_REQUIRE(xq && w && x_scale && w_scale && y && aligned(xq, 16) && aligned(w, 16) && aligned(y, 2),
                  "int8_mm: null or misaligned tensor");
    int* error = gemm_error_word();
    B200Q_REQUIRE(error != nullptr, "int8_mm: no status word on this device");
    const int sms = sm_count();
    const int m_tiles = int((rows + kBM - 1) / kBM);
    // 256-wide tiles halve the traffic of x when there are enough tiles to go round
    const bool wide = int64_t(m_tiles) * ((out + 255) / 256) >= sms;
    // ... and of the wide tiles (144 to 256 rows of W in steps of 16) the width that fills the
    // blocks' last round best: every block takes ceil(tiles / blocks) tiles in turn, and a tile's
    // time goes about as its width plus 64 columns.
    int bn = wide ? 256 : 128;
    if (wide) {
        double best = 0.0;
        for (int width = 256; width >= 144; width -= 16) {
            const int64_t count = int64_t(m_tiles) * ((out + width - 1) / width);
            const double cost = double(width + 64) * double((count + sms - 1) / sms);
            if (width == 256 || cost < best) bn = width, best = cost;
        }
    }
    CUtensorMap x_map, w_map;
    int32_t status = make_map(&x_map, xq, rows, in, kBM, "int8_mm");
    if (status != B200Q_OK) return status;
    status = make_map(&w_map, w, out, in, bn, "int8_mm");
    if (status != B200Q_OK) return status;
    MmArgs a{x_scale, w_scale, static_cast<uint16_t*>(y), int(rows), int(in), int(out), m_tiles,
             int((out + bn - 1) / bn), bn, dtype == B200Q_F16 ? 1 : 0, (out % 8 == 0 && aligned(y, 16)) ? 1 : 0};
    const int tiles = a.m_tiles * a.n_tiles;
    const int grid = tiles < sms ? tiles : sms;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err;
    if (wide) {
        ensure_dynamic_smem(reinterpret_cast<const void*>(int8_mm_kernel<256>), Shape8<256>::kSmem);
        err = launch_overlapped(int8_mm_kernel<256>, dim3(unsigned(grid)), dim3(kThreads), Shape8<256>::kSmem, s, x_map,
                                w_map, a, error);
    } else {
        ensure_dynamic_smem(reinterpret_cast<const void*>(int8_mm_kernel<128>), Shape8<128>::kSmem);
        err = launch_overlapped(int8_mm_kernel<128>, dim3(unsigned(grid)), dim3(kThreads), Shape8<128>::kSmem, s, x_map,
                                w_map, a, error);
    }
    return launch_status("int8_mm", err);
}
