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
//   warp  5     MMA issuer: one thread issues tcgen05.mma (128 x bn x 16, bf16 -> f32)
//   warps 6-21  dequantizers, two threads a row of W: packed nibbles -> registers -> the
//               exact bf16 weight ((q - zero) * scale, one rounding, as the reference) ->
//               the 128-byte swizzled K-major layout the MMA reads from shared memory
// A block tile is 256 rows of X by bn rows of W: every dequantized bn x 64 weight tile
// feeds two accumulators, which halves the dequantization work per flop.  Two kernels:
//   general (BN = 256): bn is any multiple of 16 from 64 to 256, chosen per launch so that
//     the tiles fill the multiprocessors' last round; 2 x bn columns of tensor memory used
//     once per tile; stages of 32 KB of X + bn x 128 bytes of W, as many as fit 192 KB;
//   128-wide (BN = 128): accumulators double-buffered (4 x 128 = all 512 columns) so the
//     epilogue of a tile overlaps the next tile's products, the dequantizers as two groups
//     of 8 warps taking stages in turn; it runs the K-split case (few rows, narrow weight).
// mbarrier full/empty pairs per stage.  Every wait on an mbarrier is bounded: on expiry the
// block raises an error flag in global memory, stops issuing work, still releases its
// tensor memory and returns.
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
constexpr int kRing = 192 * 1024;  // shared memory of the stages
constexpr int kMaxStages = 5;
constexpr int kTileFixed = 120;  // a tile's time is as that of its width plus this many columns
constexpr int kPrefetch = 4;  // stages of packed weights each dequantizer thread keeps in flight

// The tile's width (rows of W = columns of Y) decides how often X is re-read from L2: every
// X element is loaded once per tile width of output columns, 32 KB a stage whatever the
// width, so narrow tiles are bound by that traffic and wide ones by the products.
template <int BN>
struct Shape {
    static constexpr int kAccBufs = BN == 128 ? 2 : 1;
    static constexpr int kDequantGroups = BN == 128 ? 2 : 1;
    static constexpr int kDequantWarps = kAllDequantWarps / kDequantGroups;  // warps per stage
    static constexpr size_t kSmem = size_t(kRing) + 1024 + 256;
};


struct GemmArgs {
    const uint8_t* packed;  // [N, K/2]
    const uint16_t* scale;  // [N, K/G] bf16
    const uint8_t* zero;    // [N, K/G]
    uint16_t* y;            // [M, N] bf16
    int M, K, N, G;
    int m_tiles, n_tiles;   // tiles of 256 rows of X, of bn rows of W
    int bn;                 // rows of W per tile: BN, or for BN = 256 any multiple of 16 up to it
    int vec;                // y can be written 16 bytes at a time (N % 8 == 0, y aligned)
    int stages, stage_bytes;  // of the ring: 2 x 16 KB of X and bn x 128 bytes of W each
    int group_shift;          // log2 of the stages a quantization group lasts
    int k_splits;           // > 1: a cluster of k_splits blocks shares one tile, each a slice of K
};

// Non-zero after a bounded wait expired in some launch on this device (the value
// names the waiting role); read back by b200q_int4_gemm_status().
__device__ int g_gemm_error = 0;

using namespace umma;

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
    constexpr int kAccBufs = S::kAccBufs;
    const int stages = a.stages;
    const uint32_t stage_bytes = uint32_t(a.stage_bytes);
    constexpr int kDequantGroups = S::kDequantGroups, kDequantWarps = S::kDequantWarps;
    constexpr int kBN = BN;
    // kind::f16 instruction descriptor: f32 accumulator, bf16 A and B, both K-major, M = 128, N = bn
    const int bn = BN == 128 ? 128 : a.bn;
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // The swizzled tiles need 1024-byte alignment.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Pipeline* pipe = reinterpret_cast<Pipeline*>(smem + kRing);
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
    const int span = ks_end - ks_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&pipe->full_a[s], 1);
            mbar_init(&pipe->full_b[s], bn / 16);  // the warps that fill a stage: two threads a row
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
            int s = 0;            // ring slot of the next stage
            uint32_t lap = 0;     // times the ring has been gone round
            bool ok = true;
            for (int tile = tile_first; tile < tiles && ok; tile += tile_stride) {
                const int m0 = (tile % a.m_tiles) * (2 * kBM);
                const bool two = m0 + kBM < a.M;
                for (int ks = ks_begin; ks < ks_end && ok; ++ks) {
                    if (lap > 0) ok = mbar_wait(&pipe->empty[s], (lap - 1) & 1, &g_gemm_error, 1);
                    if (!ok) break;
                    uint8_t* dst = smem + s * stage_bytes;
                    mbar_expect_tx(&pipe->full_a[s], two ? 2 * kATile : kATile);
                    tma_load_2d(dst, &x_map, ks * kBK, m0, &pipe->full_a[s]);
                    if (two) tma_load_2d(dst + kATile, &x_map, ks * kBK, m0 + kBM, &pipe->full_a[s]);
                    if (++s == stages) s = 0, ++lap;
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---- MMA issuer ----------------------------------------------------------
        if (lane == 0) {
            uint32_t t = 0, lap = 0;
            int s = 0;
            bool ok = true;
            for (int tile = tile_first; tile < tiles && ok; tile += tile_stride, ++t) {
                const int m0 = (tile % a.m_tiles) * (2 * kBM);
                const bool two = m0 + kBM < a.M;
                const uint32_t buf = t % kAccBufs;
                if (t >= uint32_t(kAccBufs))
                    ok = mbar_wait(&pipe->acc_empty[buf], ((t / kAccBufs) - 1) & 1, &g_gemm_error, 2);
                tc_fence_after();
                for (int j = 0; j < span && ok; ++j) {
                    ok = mbar_wait(&pipe->full_a[s], lap & 1, &g_gemm_error, 3) &&
                         mbar_wait(&pipe->full_b[s], lap & 1, &g_gemm_error, 4);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t base = smem_u32(smem + s * stage_bytes);
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk) {
                        const uint64_t b_desc = smem_desc(base + 2 * kATile + kk * 32);
                        const uint32_t acc = (j > 0 || kk > 0) ? 1u : 0u;
                        umma_bf16(tmem + buf * (2 * kBN), smem_desc(base + kk * 32), b_desc, idesc, acc);
                        if (two) umma_bf16(tmem + buf * (2 * kBN) + kBN, smem_desc(base + kATile + kk * 32), b_desc, idesc, acc);
                    }
                    umma_commit(&pipe->empty[s]);  // frees the stage when these MMAs retire
                    if (++s == stages) s = 0, ++lap;
                }
                if (ok) umma_commit(&pipe->acc_full[buf]);
            }
        }
    } else if (warp >= kFirstDequantWarp) {
        // ---- dequantizers --------------------------------------------------------
        const int d = (threadIdx.x - kFirstDequantWarp * 32) % (kDequantWarps * 32);  // (row, half) of a stage
        const int group_id = (threadIdx.x - kFirstDequantWarp * 32) / (kDequantWarps * 32);
        // Two threads a row of W: each takes kWords words of 8 weights of every stage.
        constexpr int kWords = 4, kDepth = kPrefetch;
        const int row = d / 2, part = d % 2;
        const int groups = a.K / a.G;
        // Everything that repeats per stage is kept as a running value (stage, lap, group,
        // addresses): the loop body is the dequantization and little else.
        // This thread's 16-byte pieces of a stage's W tile, swizzled: piece i is chunk
        // (kWords part + i) ^ (row & 7) of the 128-byte row, which is the first one with i * 16
        // XORed into its address (stages and rows start on multiples of 128).
        const uint32_t piece0 = smem_u32(smem) + 2 * kATile + row * 128 + (((part * kWords) ^ (row & 7)) * 16);
        uint32_t it = 0;
        bool ok = d < 2 * bn;  // a narrower tile leaves the last warps without a row
        for (int tile = tile_first; tile < tiles && ok; tile += tile_stride) {
            const int n = min((tile / a.m_tiles) * bn + row, a.N - 1);  // ragged tile: clamp
            // this group's first stage of the tile, its ring slot and the times the ring has been
            // gone round before it
            const int skip = int((group_id + kDequantGroups - it % kDequantGroups) % kDequantGroups);
            int todo = (span - skip + kDequantGroups - 1) / kDequantGroups;  // stages of this tile still to fill
            int ahead = todo;                                                // ... still to fetch
            int ks = ks_begin + skip;                                        // first of them
            const uint32_t mine = it + uint32_t(skip);
            int s = int(mine % uint32_t(stages));
            uint32_t lap = mine / uint32_t(stages);
            // With few rows the weights stream from HBM exactly once, and what bounds the
            // kernel is how many bytes each multiprocessor keeps in flight: the loads of this
            // thread's next kDepth stages are always outstanding, so the HBM latency hides
            // behind several stages of work.
            // (32-bit offsets from the arguments' pointers: the packed weight is under 4 GB; a
            // quantization group lasts a power-of-two number of stages)
            const uint32_t row_at = uint32_t(n) * uint32_t(a.K / 2) + part * (4 * kWords);
            const uint32_t group_at = uint32_t(n) * uint32_t(groups);
            auto fetch = [&](uint32_t (&q)[kWords], uint32_t& sc, uint32_t& bias) {
                // raw values only: any arithmetic here would make the thread wait for these
                // loads at once instead of when the stage is dequantized, kDepth stages later
                const uint8_t* src = a.packed + (row_at + uint32_t(ks) * (kBK / 2));
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
                q[0] = v.x, q[1] = v.y, q[2] = v.z, q[3] = v.w;
                const uint32_t group = group_at + (uint32_t(ks) >> a.group_shift);
                sc = __ldg(a.scale + group);
                bias = __ldg(a.zero + group);
                --ahead;
                ks += kDequantGroups;
            };
            uint32_t q_ring[kDepth][kWords];
            uint32_t sc_ring[kDepth], bias_ring[kDepth];
#pragma unroll
            for (int u = 0; u < kDepth; ++u) {
#pragma unroll
                for (int i = 0; i < kWords; ++i) q_ring[u][i] = 0;
                sc_ring[u] = bias_ring[u] = 0;
                if (ahead > 0) fetch(q_ring[u], sc_ring[u], bias_ring[u]);
            }
            while (todo > 0 && ok) {
#pragma unroll
                for (int u = 0; u < kDepth; ++u) {
                    if (todo <= 0) break;
                    uint32_t w[kWords];
#pragma unroll
                    for (int i = 0; i < kWords; ++i) w[i] = q_ring[u][i];
                    const uint32_t sc = sc_ring[u] * 0x00010001u;                    // (scale, scale)
                    const uint32_t bias = 0x43004300u + bias_ring[u] * 0x00010001u;  // (128 + zero) twice
                    if (ahead > 0) fetch(q_ring[u], sc_ring[u], bias_ring[u]);
                    if (lap > 0) ok = mbar_wait(&pipe->empty[s], (lap - 1) & 1, &g_gemm_error, 5);
                    if (!ok) break;
                    const uint32_t stage = uint32_t(s) * stage_bytes;
#pragma unroll
                    for (int i = 0; i < kWords; ++i) {
                        // (k0,k4) (k1,k5) (k2,k6) (k3,k7): magic + q, then exactly (q - zero) * scale
                        uint32_t f[4];
                        f[0] = lop3_and_or(w[i], 0x000F000Fu, 0x43004300u);
                        f[1] = lop3_and_or(w[i] >> 4, 0x000F000Fu, 0x43004300u);
                        f[2] = lop3_and_or(w[i] >> 8, 0x000F000Fu, 0x43004300u);
                        f[3] = lop3_and_or(w[i] >> 12, 0x000F000Fu, 0x43004300u);
#pragma unroll
                        for (int e = 0; e < 4; ++e) f[e] = sub_mul<__nv_bfloat16>(f[e], bias, sc);
                        // natural order (k0,k1) (k2,k3) (k4,k5) (k6,k7)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"((stage + piece0) ^ uint32_t(i * 16)),
                                     "r"(__byte_perm(f[0], f[1], 0x5410)), "r"(__byte_perm(f[2], f[3], 0x5410)),
                                     "r"(__byte_perm(f[0], f[1], 0x7632)), "r"(__byte_perm(f[2], f[3], 0x7632))
                                     : "memory");
                    }
                    fence_proxy_async();  // generic-proxy stores -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&pipe->full_b[s]);
                    --todo;
                    s += kDequantGroups;
                    if (s >= stages) s -= stages, ++lap;
                }
            }
            it += uint32_t(span);
        }
    } else {
        // ---- epilogue (warps 0-3; warp w owns tensor-memory lanes 32w .. 32w+31) ---
        uint32_t t = 0;
        bool ok = true;
        for (int tile = tile_first; tile < tiles && ok; tile += tile_stride, ++t) {
            const int m0 = (tile % a.m_tiles) * (2 * kBM);
            const int n0 = (tile / a.m_tiles) * bn;
            const uint32_t buf = t % kAccBufs;
            ok = mbar_wait(&pipe->acc_full[buf], (t / kAccBufs) & 1, &g_gemm_error, 6);
            if (!ok || splits > 1) break;  // a K slice: the cluster adds the slices below
            tc_fence_after();
#pragma unroll 1
            for (int acc = 0; acc < 2; ++acc) {
                if (m0 + acc * kBM >= a.M) break;  // second accumulator unused (warp-uniform)
                const int m = m0 + acc * kBM + warp * 32 + lane;
#pragma unroll 1
                for (int c0 = 0; c0 < bn; c0 += 32) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem + (uint32_t(warp * 32) << 16) + buf * (2 * kBN) + acc * kBN + c0;
                    tmem_load_32(v, taddr);  // (past bn: columns of the allocation nothing wrote; not stored)
                    if (m < a.M) {
                        uint16_t* dst = a.y + size_t(m) * a.N + n0 + c0;
                        const int live = min(min(bn - c0, a.N - n0 - c0), 32);  // columns of this chunk that exist
                        if (a.vec) {  // bn, n0 and N are multiples of 8: 16-byte pieces are whole or absent
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (8 * j >= live) break;
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
                                if (j < live) dst[j] = Half16<__nv_bfloat16>::from_float(__uint_as_float(v[j]));
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
           ((group / kBK) & (group / kBK - 1)) == 0 &&
           out * (in / 2) < (int64_t(1) << 32) &&
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
                  "int4_gemm: needs bf16, inputs a multiple of %d, a group of that many times a power of two, a packed weight under 4 GB (got in=%lld group=%lld)", kBK,
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

    // Tile width.  Every block takes ceil(tiles / blocks) tiles one after another, so the time is
    // that count times a tile's time; a tile's time grows with its width w as w + kTileFixed
    // (measured at 2048 rows: 256 columns take 1.26 x the time of 176), so the width that fills
    // the last round of tiles best wins: 176 for 2048 x 6144 (280 tiles, two rounds, against
    // 192 tiles of 256 that need two rounds as well), 224 for N = 28672, 240 for N = 4096.
    // The 128-wide kernel (double-buffered accumulators) takes about 0.8 of a 256-wide tile's
    // time per tile: the general kernel at the same width is never slower by this estimate, so
    // the 128-wide kernel is left with the K-split case below.
    const int sms = sm_count();
    const int m_tiles = int((rows + 2 * kBM - 1) / (2 * kBM));
    const int64_t tiles128 = int64_t(m_tiles) * ((out + 127) / 128);
    const double cost128 = 0.8 * (256 + kTileFixed) * double((tiles128 + sms - 1) / sms);
    int bn = 256;
    double cost256 = 0.0;
    for (int width = 256; width >= 64; width -= 16) {
        const int64_t count = int64_t(m_tiles) * ((out + width - 1) / width);
        const double cost = double(width + kTileFixed) * double((count + sms - 1) / sms);
        if (width == 256 || cost < cost256) bn = width, cost256 = cost;
    }
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
    GemmArgs a;
    a.packed = packed;
    a.scale = static_cast<const uint16_t*>(scale);
    a.zero = zero;
    a.y = static_cast<uint16_t*>(y);
    a.M = int(rows), a.K = int(in), a.N = int(out), a.G = int(group);
    a.bn = wide ? bn : 128;
    a.m_tiles = m_tiles;
    a.n_tiles = int((out + a.bn - 1) / a.bn);
    a.k_splits = k_splits;
    a.vec = out % 8 == 0 && aligned(y, 16);
    a.group_shift = 0;
    while ((int64_t(kBK) << a.group_shift) < group) ++a.group_shift;
    a.stage_bytes = 2 * kATile + a.bn * (kBK * 2);
    a.stages = kRing / a.stage_bytes < kMaxStages ? kRing / a.stage_bytes : kMaxStages;
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
