// int4 group-quantized dequant-GEMM for prompt-sized row counts on Blackwell
// tensor cores (tcgen05 + tensor memory).
//
//   Y[M, N] = X[M, K] . W[N, K]^T,  W[n, k] = (q[n, k] - zero[n, k/G]) * scale[n, k/G]
//
// Stands in for the reference's many-row route, which dequantizes the whole weight
// with a Triton kernel and calls cuBLAS (`_int4_weight` + `F.linear`,
// src/backend/torch_source.cpp:1519-1566); here the weight is dequantized tile by
// tile inside the product and never written to HBM.
//
// One persistent block per multiprocessor, 22 warps with fixed roles:
//   warps 0-3   epilogue: tensor memory -> registers (tcgen05.ld) -> bf16 -> Y
//   warp  4     TMA producer: two 128 x 64 boxes of X per stage (SWIZZLE_128B)
//   warp  5     MMA issuer: one thread issues tcgen05.mma (128 x 128 x 16, bf16 -> f32)
//   warps 6-21  dequantizers (two groups of 8 taking stages in turn): packed nibbles -> registers -> the exact bf16 weight
//               ((q - zero) * scale, one rounding, as the reference) -> the 128-byte
//               swizzled K-major layout the MMA reads from shared memory
// A block tile is 256 rows of X by 128 rows of W: every dequantized 128 x 64 weight
// tile feeds two accumulators (2 x 128 columns of tensor memory), which halves the
// dequantization work per flop; the accumulators are double-buffered (4 x 128 = all
// 512 columns) so the epilogue of one tile overlaps the main loop of the next.
// Stages: 4 x (32 KB of X + 16 KB of W) of shared memory, mbarrier full/empty pairs.
// Every wait on an mbarrier is bounded: on expiry the block raises an error flag in
// global memory, stops issuing work, still releases its tensor memory and returns.
#include <cstdlib>

#include "mma.cuh"
#include "umma.cuh"

namespace b200q {
namespace {

constexpr int kBM = 128;       // rows of X per accumulator
constexpr int kBK = 64;        // inputs per stage: one 128-byte swizzle atom of bf16
constexpr int kATile = kBM * kBK * 2;               // 16 KB
constexpr int kEpilogueWarps = 4, kTmaWarp = 4, kMmaWarp = 5, kFirstDequantWarp = 6;
constexpr int kAllDequantWarps = 16;
constexpr int kThreads = (kFirstDequantWarp + kAllDequantWarps) * 32;  // 704
constexpr uint32_t kTmemColumns = 512;
constexpr int kPrefetch = 4;  // stages of packed weights each dequantizer thread keeps in flight

// The tile's width BN (rows of W = columns of Y) decides how often X is re-read from L2:
// every X element is loaded once per BN output columns.  At BN = 128 the X tiles alone
// need ~6 TB/s of L2 bandwidth at the tensor cores' speed and the kernel is L2-bound
// (measured ~0.8 PFLOP/s); BN = 256 halves that.
//   BN = 128: 4 stages of 48 KB, accumulators double-buffered (2 x 2 x 128 columns), the
//             dequantizers work as two groups of 8 warps taking stages in turn;
//   BN = 256: 3 stages of 64 KB, 2 x 256 columns used once per tile (the epilogue of a
//             tile does not overlap the next tile's products), all 16 dequantizer warps
//             fill every stage.
template <int BN>
struct Shape {
    static constexpr int kStages = BN == 128 ? 4 : 3;
    static constexpr int kStageBytes = 2 * kATile + BN * kBK * 2;
    static constexpr int kAccBufs = BN == 128 ? 2 : 1;
    static constexpr int kDequantGroups = BN == 128 ? 2 : 1;
    static constexpr int kDequantWarps = kAllDequantWarps / kDequantGroups;  // warps per stage
    static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN >> 3) << 17) |
                                       (uint32_t(kBM >> 4) << 24);
    static constexpr size_t kSmem = size_t(kStages) * kStageBytes + 1024 + 256;
};
constexpr int kMaxStages = 4;

struct GemmArgs {
    const uint8_t* packed;  // [N, K/2]
    const uint16_t* scale;  // [N, K/G] bf16
    const uint8_t* zero;    // [N, K/G]
    uint16_t* y;            // [M, N] bf16
    int M, K, N, G;
    int m_tiles, n_tiles;   // tiles of 256 rows of X, of BN rows of W
    int k_splits;           // > 1: a cluster of k_splits blocks shares one tile, each a slice of K
};

// Non-zero after a bounded wait expired in some launch on this device (the value
// names the waiting role); read back by b200q_int4_gemm_status().
__device__ int g_gemm_error = 0;

using namespace umma;

// (The kind::f16 instruction descriptor is Shape<BN>::kIdesc: f32 accumulator, bf16 A and
// B, both K-major, M = 128, N = BN.)

struct Pipeline {  // shared-memory barriers and the tensor-memory base address
    uint64_t full_a[kMaxStages];   // TMA bytes of X landed
    uint64_t full_b[kMaxStages];   // dequantized W tile written (one arrival per dequantizer warp)
    uint64_t empty[kMaxStages];    // MMAs that read the stage completed
    uint64_t acc_full[2];       // all MMAs of a tile completed
    uint64_t acc_empty[2];      // epilogue drained the accumulators (4 warp arrivals)
    uint32_t tmem_base;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
int4_gemm_kernel(const __grid_constant__ CUtensorMap x_map, const GemmArgs a) {
    using S = Shape<BN>;
    constexpr int kStages = S::kStages, kStageBytes = S::kStageBytes, kAccBufs = S::kAccBufs;
    constexpr int kDequantGroups = S::kDequantGroups, kDequantWarps = S::kDequantWarps;
    constexpr uint32_t kIdesc = S::kIdesc;
    constexpr int kBN = BN;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // The swizzled tiles need 1024-byte alignment.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Pipeline* pipe = reinterpret_cast<Pipeline*>(smem + kStages * kStageBytes);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int tiles = a.m_tiles * a.n_tiles;
    // Few rows and a narrow weight leave most multiprocessors without a tile; then a cluster
    // of k_splits blocks takes one tile, block r the r-th slice of K, and the slices' f32
    // accumulators are added through distributed shared memory at the end.  (k_splits == 1:
    // persistent blocks striding over the tiles, all of K each.)
    const int splits = a.k_splits, split = blockIdx.x % splits;
    const int tile_first = blockIdx.x / splits, tile_stride = gridDim.x / splits;
    const int k_per_split = (a.K / kBK + splits - 1) / splits;
    const int ks_begin = split * k_per_split, ks_end = min(a.K / kBK, ks_begin + k_per_split);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&pipe->full_a[s], 1);
            mbar_init(&pipe->full_b[s], kDequantWarps);
            mbar_init(&pipe->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&pipe->acc_full[b], 1);
            mbar_init(&pipe->acc_empty[b], kEpilogueWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {  // one warp allocates (and later frees) all of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&pipe->tmem_base)),
                     "r"(kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = pipe->tmem_base;

    if (warp == kTmaWarp) {
        // ---- producer of X -------------------------------------------------------
        if (lane == 0) {
            uint32_t it = 0;  // stage uses so far
            bool ok = true;
            for (int tile = tile_first; tile < tiles && ok; tile += tile_stride) {
                const int m0 = (tile % a.m_tiles) * (2 * kBM);
                const bool two = m0 + kBM < a.M;
                for (int ks = ks_begin; ks < ks_end && ok; ++ks, ++it) {
                    const int s = it % kStages;
                    if (it >= kStages) ok = mbar_wait(&pipe->empty[s], ((it / kStages) - 1) & 1, &g_gemm_error, 1);
                    if (!ok) break;
                    uint8_t* dst = smem + s * kStageBytes;
                    mbar_expect_tx(&pipe->full_a[s], two ? 2 * kATile : kATile);
                    tma_load_2d(dst, &x_map, ks * kBK, m0, &pipe->full_a[s]);
                    if (two) tma_load_2d(dst + kATile, &x_map, ks * kBK, m0 + kBM, &pipe->full_a[s]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---- MMA issuer ----------------------------------------------------------
        if (lane == 0) {
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (int tile = tile_first; tile < tiles && ok; tile += tile_stride, ++t) {
                const int m0 = (tile % a.m_tiles) * (2 * kBM);
                const bool two = m0 + kBM < a.M;
                const uint32_t buf = t % kAccBufs;
                if (t >= uint32_t(kAccBufs))
                    ok = mbar_wait(&pipe->acc_empty[buf], ((t / kAccBufs) - 1) & 1, &g_gemm_error, 2);
                tc_fence_after();
                for (int ks = ks_begin; ks < ks_end && ok; ++ks, ++it) {
                    const int s = it % kStages;
                    const uint32_t parity = (it / kStages) & 1;
                    ok = mbar_wait(&pipe->full_a[s], parity, &g_gemm_error, 3) &&
                         mbar_wait(&pipe->full_b[s], parity, &g_gemm_error, 4);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t base = smem_u32(smem + s * kStageBytes);
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk) {
                        const uint64_t b_desc = smem_desc(base + 2 * kATile + kk * 32);
                        const uint32_t acc = (ks > ks_begin || kk > 0) ? 1u : 0u;
                        umma_bf16(tmem + buf * (2 * kBN), smem_desc(base + kk * 32), b_desc, kIdesc, acc);
                        if (two) umma_bf16(tmem + buf * (2 * kBN) + kBN, smem_desc(base + kATile + kk * 32), b_desc, kIdesc, acc);
                    }
                    umma_commit(&pipe->empty[s]);  // frees the stage when these MMAs retire
                }
                if (ok) umma_commit(&pipe->acc_full[buf]);
            }
        }
    } else if (warp >= kFirstDequantWarp) {
        // ---- dequantizers --------------------------------------------------------
        const int d = (threadIdx.x - kFirstDequantWarp * 32) % (kDequantWarps * 32);  // (row, half) of a stage
        const int group_id = (threadIdx.x - kFirstDequantWarp * 32) / (kDequantWarps * 32);
        const int row = d >> 1, half = d & 1;                // W row of the tile, 32-input half
        const int groups = a.K / a.G;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = tile_first; tile < tiles && ok; tile += tile_stride) {
            const int n = min((tile / a.m_tiles) * kBN + row, a.N - 1);  // ragged tile: clamp
            const uint8_t* src = a.packed + size_t(n) * (a.K / 2) + half * 16;
            const uint16_t* srow = a.scale + size_t(n) * groups;
            const uint8_t* zrow = a.zero + size_t(n) * groups;
            // With few rows the weights stream from HBM exactly once, and what bounds the
            // kernel is how many bytes each multiprocessor keeps in flight: the loads of this
            // thread's next kPrefetch stages are always outstanding (16 bytes each, 512 or
            // 256 threads a stage), so the HBM latency hides behind several stages of work.
            auto fetch = [&](int ks, uint4& q, uint32_t& sc, uint32_t& bias) {
                q = __ldg(reinterpret_cast<const uint4*>(src + size_t(ks) * (kBK / 2)));
                const int grp = (ks * kBK) / a.G;
                // raw values only: any arithmetic here would make the thread wait for these two
                // loads at once instead of when the stage is dequantized, kPrefetch stages later
                sc = __ldg(srow + grp);
                bias = __ldg(zrow + grp);
            };
            const int first = ks_begin + int((group_id + kDequantGroups - it % kDequantGroups) % kDequantGroups);
            uint4 q_ring[kPrefetch];
            uint32_t sc_ring[kPrefetch], bias_ring[kPrefetch];
#pragma unroll
            for (int u = 0; u < kPrefetch; ++u) {
                q_ring[u] = make_uint4(0, 0, 0, 0);
                sc_ring[u] = bias_ring[u] = 0;
                if (first + u * kDequantGroups < ks_end) fetch(first + u * kDequantGroups, q_ring[u], sc_ring[u], bias_ring[u]);
            }
            for (int ks0 = first; ks0 < ks_end && ok; ks0 += kPrefetch * kDequantGroups) {
#pragma unroll
                for (int u = 0; u < kPrefetch; ++u) {
                    const int ks = ks0 + u * kDequantGroups;
                    if (ks >= ks_end || !ok) break;
                    const uint32_t mine = it + uint32_t(ks - ks_begin);  // this stage's use number
                    const int s = mine % kStages;
                    const uint4 q = q_ring[u];
                    const uint32_t sc = sc_ring[u] * 0x00010001u;               // (scale, scale)
                    const uint32_t bias = 0x43004300u + bias_ring[u] * 0x00010001u;  // (128 + zero) twice
                    if (ks + kPrefetch * kDequantGroups < ks_end)
                        fetch(ks + kPrefetch * kDequantGroups, q_ring[u], sc_ring[u], bias_ring[u]);
                    if (mine >= uint32_t(kStages))
                        ok = mbar_wait(&pipe->empty[s], ((mine / kStages) - 1) & 1, &g_gemm_error, 5);
                    if (!ok) break;
                    uint8_t* tile_b = smem + s * kStageBytes + 2 * kATile + row * 128;
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        // (k0,k4) (k1,k5) (k2,k6) (k3,k7): magic + q, then exactly (q - zero) * scale
                        uint32_t f[4];
                        f[0] = lop3_and_or(w[i], 0x000F000Fu, 0x43004300u);
                        f[1] = lop3_and_or(w[i] >> 4, 0x000F000Fu, 0x43004300u);
                        f[2] = lop3_and_or(w[i] >> 8, 0x000F000Fu, 0x43004300u);
                        f[3] = lop3_and_or(w[i] >> 12, 0x000F000Fu, 0x43004300u);
#pragma unroll
                        for (int e = 0; e < 4; ++e) f[e] = sub_mul<__nv_bfloat16>(f[e], bias, sc);
                        uint4 out;  // natural order (k0,k1) (k2,k3) (k4,k5) (k6,k7)
                        out.x = __byte_perm(f[0], f[1], 0x5410);
                        out.y = __byte_perm(f[2], f[3], 0x5410);
                        out.z = __byte_perm(f[0], f[1], 0x7632);
                        out.w = __byte_perm(f[2], f[3], 0x7632);
                        const int chunk = half * 4 + i;  // 16-byte chunk of the 128-byte row
                        *reinterpret_cast<uint4*>(tile_b + ((chunk ^ (row & 7)) * 16)) = out;
                    }
                    fence_proxy_async();  // generic-proxy stores -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&pipe->full_b[s]);
                }
            }
            it += uint32_t(ks_end - ks_begin);
        }
    } else {
        // ---- epilogue (warps 0-3; warp w owns tensor-memory lanes 32w .. 32w+31) ---
        uint32_t t = 0;
        bool ok = true;
        for (int tile = tile_first; tile < tiles && ok; tile += tile_stride, ++t) {
            const int m0 = (tile % a.m_tiles) * (2 * kBM);
            const int n0 = (tile / a.m_tiles) * kBN;
            const uint32_t buf = t % kAccBufs;
            ok = mbar_wait(&pipe->acc_full[buf], (t / kAccBufs) & 1, &g_gemm_error, 6);
            if (!ok || splits > 1) break;  // a K slice: the cluster adds the slices below
            tc_fence_after();
#pragma unroll 1
            for (int acc = 0; acc < 2; ++acc) {
                const int m = m0 + acc * kBM + warp * 32 + lane;
                if (m0 + acc * kBM >= a.M) break;  // second accumulator unused (warp-uniform)
#pragma unroll 1
                for (int c0 = 0; c0 < kBN; c0 += 32) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem + (uint32_t(warp * 32) << 16) + buf * (2 * kBN) + acc * kBN + c0;
                    tmem_load_32(v, taddr);
                    if (m < a.M) {
                        uint16_t* dst = a.y + size_t(m) * a.N + n0 + c0;
                        if (n0 + c0 + 32 <= a.N && (a.N % 8) == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint4 o;
                                o.x = Half16<__nv_bfloat16>::pack(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
                                o.y = Half16<__nv_bfloat16>::pack(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                                o.z = Half16<__nv_bfloat16>::pack(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                                o.w = Half16<__nv_bfloat16>::pack(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                                reinterpret_cast<uint4*>(dst)[j] = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n0 + c0 + j < a.N)
                                    dst[j] = Half16<__nv_bfloat16>::from_float(__uint_as_float(v[j]));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&pipe->acc_empty[buf]);
        }
    }

    // Every role falls through to here, also after an expired wait.
    if (splits > 1) {
        // The epilogue warps have seen acc_full, so once every thread of the cluster is here
        // no tensor core, TMA or dequantizer of any block touches the stages any more:
        // they become the exchange buffer [source block][128 rows][BN / splits columns] f32.
        cluster_sync();
        const int cps = kBN / splits;  // columns this block owns and reduces
        float* exchange = reinterpret_cast<float*>(smem);
        if (warp < kEpilogueWarps) {
            tc_fence_after();
            const int row = warp * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < kBN; c0 += 32) {
                uint32_t v[32];
                tmem_load_32(v, tmem + (uint32_t(warp * 32) << 16) + c0);
                if (row < a.M) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int col = c0 + 4 * j, owner = col / cps, within = col % cps;
                        const uint32_t local = smem_u32(exchange + (size_t(split) * kBM + row) * cps + within);
                        uint32_t remote;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(owner));
                        asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(remote), "r"(v[4 * j]),
                                     "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                                     : "memory");
                    }
                }
            }
            tc_fence_before();
        }
        cluster_sync();  // every slice of my columns has arrived
        const int n_base = (tile_first / a.m_tiles) * kBN + split * cps;
        for (int item = threadIdx.x; item < kBM * cps; item += kThreads) {
            const int row = item / cps, col = item % cps;
            if (row < a.M && n_base + col < a.N) {
                float sum = 0.0f;
                for (int src = 0; src < splits; ++src) sum += exchange[(size_t(src) * kBM + row) * cps + col];
                a.y[size_t(row) * a.N + n_base + col] = Half16<__nv_bfloat16>::from_float(sum);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns)
                     : "memory");
    }
}

}  // namespace

bool int4_gemm_supports(int64_t rows, int64_t in, int64_t out, int64_t group, int32_t dtype,
                        const void* x, const void* y) {
    return dtype == B200Q_BF16 && rows > 0 && in % kBK == 0 && group % kBK == 0 && in >= kBK &&
           (in * 2) % 16 == 0 && aligned(x, 16) && aligned(y, 2) && out > 0;
}

}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_int4_gemm(const void* x, const uint8_t* packed, const void* scale,
                                   const uint8_t* zero, void* y, int64_t rows, int64_t in, int64_t out,
                                   int64_t group, int32_t dtype, void* stream) {
    const int32_t ok = check_int4_args("int4_gemm", x, packed, scale, zero, y, rows, in, out, group, dtype);
    if (ok != B200Q_OK || rows == 0) return ok;
    B200Q_REQUIRE(int4_gemm_supports(rows, in, out, group, dtype, x, y),
                  "int4_gemm: needs bf16, inputs and group multiples of %d (got in=%lld group=%lld)", kBK,
                  (long long)in, (long long)group);
    B200Q_REQUIRE(rows < (int64_t(1) << 30), "int4_gemm: too many rows");
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return unavailable("int4_gemm: the driver has no cuTensorMapEncodeTiled");

    CUtensorMap x_map;
    const cuuint64_t dims[2] = {cuuint64_t(in), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(in) * 2};
    const cuuint32_t box[2] = {cuuint32_t(kBK), cuuint32_t(kBM)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult made = encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims,
                                 strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200Q_REQUIRE(made == CUDA_SUCCESS, "int4_gemm: cuTensorMapEncodeTiled failed (%d)", int(made));

    // Tile width: 256 unless the narrower tile's better fit to the SM count outweighs its
    // L2-bound main loop (a 256-wide tile takes about 1.25x the time of a 128-wide one).
    const int sms = sm_count();
    const int m_tiles = int((rows + 2 * kBM - 1) / (2 * kBM));
    const int64_t tiles128 = int64_t(m_tiles) * ((out + 127) / 128), tiles256 = int64_t(m_tiles) * ((out + 255) / 256);
    const double cost128 = double((tiles128 + sms - 1) / sms), cost256 = 1.25 * double((tiles256 + sms - 1) / sms);
    // Up to 128 rows over a narrow weight: split K over a cluster while the tiles alone would
    // leave more than half of the multiprocessors idle (every slice keeps >= 2 steps of 64).
    int k_splits = 1;
    const int ksteps = int(in / kBK);
    if (rows <= kBM) {
        const int64_t n_tiles = (out + 127) / 128;
        while (k_splits < 8 && n_tiles * k_splits * 2 <= sms && ksteps / (k_splits * 2) >= 2) k_splits *= 2;
        while (k_splits > 1 && (k_splits - 1) * ((ksteps + k_splits - 1) / k_splits) >= ksteps) k_splits /= 2;
    }
    const bool wide = k_splits == 1 && cost256 <= cost128;
    GemmArgs a{packed, static_cast<const uint16_t*>(scale), zero, static_cast<uint16_t*>(y),
               int(rows), int(in), int(out), int(group), m_tiles, int(wide ? (out + 255) / 256 : (out + 127) / 128),
               k_splits};
    const int tiles = a.m_tiles * a.n_tiles;
    const int grid = k_splits > 1 ? tiles * k_splits : (tiles < sms ? tiles : sms);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (k_splits > 1) {
        ensure_dynamic_smem(reinterpret_cast<const void*>(int4_gemm_kernel<128>), Shape<128>::kSmem);
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(unsigned(grid));
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = Shape<128>::kSmem;
        config.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = unsigned(k_splits);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
        return launch_status("int4_gemm", cudaLaunchKernelEx(&config, int4_gemm_kernel<128>, x_map, a));
    }
    if (wide) {
        ensure_dynamic_smem(reinterpret_cast<const void*>(int4_gemm_kernel<256>), Shape<256>::kSmem);
        int4_gemm_kernel<256><<<grid, kThreads, Shape<256>::kSmem, s>>>(x_map, a);
    } else {
        ensure_dynamic_smem(reinterpret_cast<const void*>(int4_gemm_kernel<128>), Shape<128>::kSmem);
        int4_gemm_kernel<128><<<grid, kThreads, Shape<128>::kSmem, s>>>(x_map, a);
    }
    return launched("int4_gemm");
}

namespace b200q {
// Device address of the bounded-wait flag (also used by int8_w8a8.cu); asked for once per device.
int* gemm_error_word() {
    static int* cached[64] = {nullptr};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (cached[device] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_gemm_error) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cached[device] = static_cast<int*>(p);
    }
    return cached[device];
}
}  // namespace b200q

extern "C" int32_t b200q_int4_gemm_status(void) {
    int flag = 0;
    const cudaError_t err = cudaMemcpyFromSymbol(&flag, g_gemm_error, sizeof(int));
    if (err != cudaSuccess) return fail("int4_gemm_status: %s", cudaGetErrorString(err));
    if (flag != 0) {
        // Reported once: cleared so that later launches wait their full time again.
        const int zero = 0;
        cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
        return fail("int4_gemm: a bounded wait expired (role %d)", flag);
    }
    return B200Q_OK;
}
