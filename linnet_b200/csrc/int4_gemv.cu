// int4 group-quantized decode product for up to 16 activation rows.
//
//   y[m, n] = sum_k x[m, k] * (q[n, k] - zero[n, k/G]) * scale[n, k/G]
//
// Stands in for linnet::int4_linear (python/linnet/src/linnet/torch/kernels.py:212-323)
// and for ATen's _weight_int4pack_mm as the generated source calls it
// (src/backend/torch_source.cpp:1553-1562), on the reference's own weight layout:
// packed [N, K/G, G/2] bytes (a row is K/2 contiguous bytes, even k in the low
// nibble), scale [N, K/G] in the activation type, zero [N, K/G] u8.
//
// The kernel is HBM-bound: 0.5234 B per weight at G=128.  Design:
//   * every thread streams 16-byte pieces of two weight rows (g and g+8 of a
//     16-row tile) straight into registers with L1-bypassing loads, D k-blocks
//     (128 inputs) in flight, so no shared-memory hop sits on the weight path;
//   * nibbles become 16-bit floats with one LOP3 per pair ((w >> s) & 0x000F000F
//     | magic gives magic + q for k and k + 4); (magic + q) - (magic + zero) is the
//     exact integer q - zero, and one multiply by the scale rounds it once to the
//     16-bit type: bit for bit the weight the reference multiplies by
//     ((q - zero) * scale in f32, cast once).  The pair is already an A fragment of
//     mma.m16n8k16; the activations are staged once per warp in shared memory,
//     permuted to the matching (k, k + 4) pairing, as B fragments; accumulation is
//     f32 in the tensor cores;
//   * the warps of a block split K; a cluster of blocks may split it further, the
//     partial sums meeting in (distributed) shared memory, so no global scratch
//     and no atomics are used.
#include <cstdlib>

#include "gemv_common.cuh"
#include "int4_gemv_oct.cuh"
#include "int4_gemv_tma.cuh"
#include "int4_gemv_rows.cuh"

namespace b200q {
namespace {

struct GemvArgs {
    const void* x;          // [M, K]
    const uint8_t* packed;  // [N, K/2]
    const void* scale;      // [N, K/G]
    const uint8_t* zero;    // [N, K/G]
    void* y;                // [M, N]
    int M, K, N, G;
    int kblocks;            // K / 128
    int kb_per_cta;         // k-blocks each block of a cluster handles
    int ksplit;             // blocks per cluster (along grid.y)
    int flags;              // B200Q_EXACT_WEIGHTS | B200Q_EARLY_DEPENDENTS | B200Q_SWIGLU_INPUT | B200Q_NO_OVERLAP
};

// How the zero point and scale reach the product.
//   kExactBlock: groups that are multiples of 128.  Every pair of weights is
//                dequantized exactly as the reference does ((q - zero) * scale, one
//                rounding to the 16-bit type) with one HSUB2 + one HMUL2; the group's
//                scale and zero point travel with the k-block's weight loads.
//   kExactWord:  groups of 16, 32 or 64: the same arithmetic, the scale looked up per
//                8 weights.
enum { kExactBlock = 0, kExactWord = 1 };

// One k-block of one 16-row tile as loaded: 16 bytes of rows g and g+8, and the
// (scale bits | zero << 16) words of the group the k-block lies in.
template <int NT>
struct Stage {
    uint4 q[NT][2];
    uint32_t sz[NT][2];
};

template <typename T, int MODE, int MB, int NT, int W, int D>
__global__ void __launch_bounds__(W * 32)
int4_gemv_kernel(const GemvArgs a) {
    using H = Half16<T>;
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
    const int M = a.M, K = a.K, N = a.N, G = a.G;
    const int groups = K / G;
    const int tile_row = blockIdx.x * (16 * NT);
    const int kb0 = min(int(blockIdx.y) * a.kb_per_cta, a.kblocks);
    const int kb1 = min(kb0 + a.kb_per_cta, a.kblocks);
    const int nkb = kb1 - kb0;  // k-blocks of this block (the last of a cluster may have fewer)
    // This warp's contiguous share of them.  `cap` (from kb_per_cta) sizes the shared
    // memory regions so that they sit at the same offsets in every block of a cluster.
    const int cap = (a.kb_per_cta + W - 1) / W;
    const int per_warp = (nkb + W - 1) / W;
    const int wb0 = min(warp * per_warp, nkb), wb1 = min(wb0 + per_warp, nkb);
    const int nw = wb1 - wb0;

    // Shared memory, per warp: activations as B fragments [cap][4 words][M][4 lanes] x
    // 16 B; then the block's reduction buffer [W][NT*16][MB*8].
    uint4* xs = reinterpret_cast<uint4*>(smem) + size_t(warp) * cap * 16 * M;
    float* red = reinterpret_cast<float*>(reinterpret_cast<uint4*>(smem) + size_t(W) * cap * 16 * M);

    const uint16_t* scale16 = static_cast<const uint16_t*>(a.scale);
    const uint8_t* rowp[NT][2];
    size_t srow[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = min(tile_row + nt * 16 + h * 8 + g, N - 1);  // ragged tile: clamp
            rowp[nt][h] = a.packed + size_t(r) * (K / 2) + t * 16;
            srow[nt][h] = size_t(r) * groups;
        }

    auto load_stage = [&](Stage<NT>& s, int kb_local) {
        const int kb = kb0 + kb_local;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int h = 0; h < 2; ++h) s.q[nt][h] = ldg_stream(rowp[nt][h] + size_t(kb) * 64);
        if (MODE != kExactWord) {
            const int grp = (kb * 128) / G;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    s.sz[nt][h] = uint32_t(__ldg(scale16 + srow[nt][h] + grp)) |
                                  (uint32_t(__ldg(a.zero + srow[nt][h] + grp)) << 16);
        }
    };

    // 1. Put the first weight loads in flight before anything else.
    Stage<NT> st[D];
#pragma unroll
    for (int d = 0; d < D; ++d)
        if (d < nw) load_stage(st[d], wb0 + d);

    pdl_launch_dependents();
    pdl_wait();  // activations may come from the kernel before this one

    // 2. Each warp stages the activations of its own K range (no block barrier):
    //    16-byte pieces, permuted to the (k, k+4) pairing of the A fragments.
    {
        const uint4* xg = static_cast<const uint4*>(a.x);
        const int per_row = nw * 16;  // 16-byte pieces per activation row
        const int pieces = M * per_row;
        constexpr int U = 4;
        for (int base = 0; base < pieces; base += 32 * U) {
            uint4 raw[U];
            int where[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = base + u * 32 + lane;
                where[u] = -1;
                raw[u] = make_uint4(0, 0, 0, 0);
                if (e < pieces) {
                    const int m = e / per_row, rem = e - m * per_row;
                    const int j = rem / 16, c = rem % 16;
                    raw[u] = ld_mutable(xg + (size_t(m) * K + size_t(kb0 + wb0 + j) * 128) / 8 + c);
                    where[u] = ((j * 4 + (c % 4)) * M + m) * 4 + c / 4;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (where[u] >= 0) {
                    uint4 out;
                    out.x = __byte_perm(raw[u].x, raw[u].z, 0x5410);  // (x0, x4)
                    out.y = __byte_perm(raw[u].x, raw[u].z, 0x7632);  // (x1, x5)
                    out.z = __byte_perm(raw[u].y, raw[u].w, 0x5410);  // (x2, x6)
                    out.w = __byte_perm(raw[u].y, raw[u].w, 0x7632);  // (x3, x7)
                    xs[where[u]] = out;
                }
            }
        }
    }
    __syncwarp();

    // 3. Main loop over this warp's k-blocks.
    float total[NT][MB][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 4; ++i) total[nt][mb][i] = 0.0f;

    const uint32_t kMask = 0x000F000Fu;
    for (int base = 0; base < nw; base += D) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const int j = base + d;  // this warp's j-th k-block
            if (j < nw) {
                const Stage<NT> cur = st[d];
                if (j + D < nw) load_stage(st[d], wb0 + j + D);
                // B fragments of this k-block.
                uint4 b[MB][4];
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    const int m = mb * 8 + g;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        b[mb][i] = m < M ? xs[(size_t(j * 4 + i) * M + m) * 4 + t]
                                         : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint32_t w0[4] = {cur.q[nt][0].x, cur.q[nt][0].y, cur.q[nt][0].z, cur.q[nt][0].w};
                    const uint32_t w1[4] = {cur.q[nt][1].x, cur.q[nt][1].y, cur.q[nt][1].z, cur.q[nt][1].w};
                    uint32_t bias0 = 0, bias1 = 0, sc0 = 0, sc1 = 0;  // 16-bit pairs (x, x)
                    if (MODE == kExactBlock) {
                        bias0 = H::kMagic + (cur.sz[nt][0] >> 16) * 0x00010001u;
                        bias1 = H::kMagic + (cur.sz[nt][1] >> 16) * 0x00010001u;
                        sc0 = (cur.sz[nt][0] & 0xFFFFu) * 0x00010001u;
                        sc1 = (cur.sz[nt][1] & 0xFFFFu) * 0x00010001u;
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t f0[4], f1[4];  // (k0,k4) (k1,k5) (k2,k6) (k3,k7) of rows g, g+8
                        f0[0] = lop3_and_or(w0[i], kMask, H::kMagic);
                        f0[1] = lop3_and_or(w0[i] >> 4, kMask, H::kMagic);
                        f0[2] = lop3_and_or(w0[i] >> 8, kMask, H::kMagic);
                        f0[3] = lop3_and_or(w0[i] >> 12, kMask, H::kMagic);
                        f1[0] = lop3_and_or(w1[i], kMask, H::kMagic);
                        f1[1] = lop3_and_or(w1[i] >> 4, kMask, H::kMagic);
                        f1[2] = lop3_and_or(w1[i] >> 8, kMask, H::kMagic);
                        f1[3] = lop3_and_or(w1[i] >> 12, kMask, H::kMagic);
                        if (MODE == kExactWord) {
                            const int grp = ((kb0 + wb0 + j) * 128 + t * 32 + i * 8) / G;
                            sc0 = uint32_t(__ldg(scale16 + srow[nt][0] + grp)) * 0x00010001u;
                            sc1 = uint32_t(__ldg(scale16 + srow[nt][1] + grp)) * 0x00010001u;
                            bias0 = H::kMagic + uint32_t(__ldg(a.zero + srow[nt][0] + grp)) * 0x00010001u;
                            bias1 = H::kMagic + uint32_t(__ldg(a.zero + srow[nt][1] + grp)) * 0x00010001u;
                        }
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            f0[p] = sub_mul<T>(f0[p], bias0, sc0);
                            f1[p] = sub_mul<T>(f1[p], bias1, sc1);
                        }
                        const uint32_t a_lo[4] = {f0[0], f1[0], f0[1], f1[1]};
                        const uint32_t a_hi[4] = {f0[2], f1[2], f0[3], f1[3]};
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb) {
                            H::mma(total[nt][mb], a_lo, b[mb][i].x, b[mb][i].y);
                            H::mma(total[nt][mb], a_hi, b[mb][i].z, b[mb][i].w);
                        }
                    }
                }
            }
        }
    }

    // 4. Sum the warps' partial results, then the cluster's, and write y.
    reduce_and_store<H, MB, NT, W>(total, red, a.ksplit, tile_row, M, N, static_cast<uint16_t*>(a.y));
}

// Any shape the tensor-core kernel does not take (K not a multiple of 128): one
// warp per output column, f32 multiply-adds, up to 8 activation rows at a time.
template <typename T>
__global__ void int4_linear_simple_kernel(const GemvArgs a, int m0) {
    using H = Half16<T>;
    const int n = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (n >= a.N) return;
    const int rows = min(8, a.M - m0);
    const uint16_t* x = static_cast<const uint16_t*>(a.x);
    const uint16_t* scale16 = static_cast<const uint16_t*>(a.scale);
    const int groups = a.K / a.G;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int byte = lane; byte < a.K / 2; byte += 32) {
        const uint32_t v = a.packed[size_t(n) * (a.K / 2) + byte];
        const int grp = (2 * byte) / a.G;
        const float s = H::to_float(scale16[size_t(n) * groups + grp]);
        const float z = float(a.zero[size_t(n) * groups + grp]);
        // Round the weight once to the activation type, as the reference does.
        const float w0 = H::to_float(H::from_float((float(v & 15) - z) * s));
        const float w1 = H::to_float(H::from_float((float(v >> 4) - z) * s));
        for (int r = 0; r < rows; ++r) {
            const uint16_t* xr = x + size_t(m0 + r) * a.K + 2 * byte;
            acc[r] = fmaf(H::to_float(xr[0]), w0, acc[r]);
            acc[r] = fmaf(H::to_float(xr[1]), w1, acc[r]);
        }
    }
    uint16_t* y = static_cast<uint16_t*>(a.y);
    for (int r = 0; r < rows; ++r) {
        float v = acc[r];
        for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
        if (lane == 0) y[size_t(m0 + r) * a.N + n] = H::from_float(v);
    }
}

struct Plan {
    int nt, w, d, ksplit;
};

// Launch geometry: enough warps in flight to cover HBM latency (about 24 per
// multiprocessor), each with at least two k-blocks, and activations staged in
// under ~48 KB of shared memory per block.
Plan choose_plan(int M, int K, int N) {
    const int sms = sm_count();
    const int kblocks = K / 128;
    Plan p{1, 4, 3, 1};
    if (M > 8) p.nt = 2;
    const int tiles = (N + 16 * p.nt - 1) / (16 * p.nt);
    // Split K over a cluster while the grid is short of ~3 blocks per SM or the
    // staged activations are too large.
    while (p.ksplit < 8 && kblocks / (p.ksplit * 2) >= p.w &&
           (tiles * p.ksplit < 3 * sms || size_t(kblocks / p.ksplit) * 256 * M > 48 * 1024))
        p.ksplit *= 2;
    return p;
}

template <typename T, int MODE, int MB, int NT, int W, int D>
int32_t launch_gemv(const GemvArgs& args, int ksplit, cudaStream_t stream) {
    GemvArgs a = args;
    a.ksplit = ksplit;
    a.kb_per_cta = (a.kblocks + ksplit - 1) / ksplit;
    const int tiles = (a.N + 16 * NT - 1) / (16 * NT);
    const size_t cap = (a.kb_per_cta + W - 1) / W;  // k-blocks per warp, at most
    const size_t smem = size_t(W) * cap * 16 * a.M * 16 + size_t(W) * NT * 16 * MB * 8 * 4;
    return launch_clustered("int4_gemv", int4_gemv_kernel<T, MODE, MB, NT, W, D>, a, tiles, ksplit,
                            W * 32, smem, stream, true);
}

template <typename T, int MODE>
int32_t dispatch_gemv(const GemvArgs& a, const Plan& p, cudaStream_t stream) {
    if (a.M <= 8) return launch_gemv<T, MODE, 1, 1, 4, 2>(a, p.ksplit, stream);
    return launch_gemv<T, MODE, 2, 2, 4, 2>(a, p.ksplit, stream);
}

// Three or more rows: the kernel that stages the activations once per block.  Picks the
// warps (tiles) per block so that every block of the grid is resident at once, and the
// octs per block so that the cluster has at most 8 blocks.
template <typename T, int MB>
bool run_rows(const GemvArgs& a, cudaStream_t stream, int32_t* status) {
    if (a.G != 128 || a.K % 1024 != 0 || !aligned(a.scale, 16) || !aligned(a.zero, 8)) return false;
    const int octs = a.K / 1024;
    int opc = 0;
    for (int c = 1; c <= octs; ++c)
        if (octs % c == 0 && octs / c <= 8) { opc = c; break; }
    if (opc == 0) return false;
    RowsArgs r{a.x, a.packed, a.scale, a.zero, a.y, a.M, a.K, a.N, (a.N + 15) / 16, opc, octs / opc};
    const int sms = sm_count();
    // Widest block (most sharing of the staged activations) among those that keep every
    // block resident at once and still put a block on every multiprocessor.
    const int candidates[4] = {14, 7, 4, 2};
    // warps a multiprocessor holds at this kernel's register count (72 / ~136 / ~168 a thread;
    // the 14-warp block of the 64-row kernel is held to 128)
    const int warps_by_regs = MB <= 2 ? 28 : MB <= 4 ? 14 : 12;
    int best = 4;
    double best_cost = 1e30;
    for (int w : candidates) {
        const size_t smem = size_t(MB * 8) * 2048 + size_t(w) * 16 * (MB * 8) * 4 + 1024;
        const int by_smem = int((size_t(220) << 10) / smem);
        const int by_regs = w == 14 && warps_by_regs < 14 ? 1 : warps_by_regs / w;
        if (by_smem < 1 || by_regs < 1) continue;
        const int resident = sms * (by_smem < by_regs ? by_smem : by_regs);
        const int blocks = ((r.tiles + w - 1) / w) * r.ksplit;
        const double waves = double((blocks + resident - 1) / resident);
        const double coverage = blocks >= sms ? 1.0 : double(blocks) / double(sms);
        const double cost = waves / coverage;
        if (cost < best_cost - 1e-9) { best_cost = cost; best = w; }
    }
    switch (best) {
        case 4: *status = launch_rows<T, MB, 4, 2>(r, stream); break;
        case 7: *status = launch_rows<T, MB, 7, 2>(r, stream); break;
        case 14: *status = launch_rows<T, MB, 14, 2>(r, stream); break;
        default: *status = launch_rows<T, MB, 2, 2>(r, stream); break;
    }
    return true;
}

// The short-run variants (KB = 4 or 2 k-blocks per warp) for up to 8 rows: the most warps
// per block (of 8, 4, 7, 2, 1) that divide the runs along K with at most 8 blocks per cluster.
template <typename T, int KB>
bool run_short(OctArgs o, int G, cudaStream_t stream, int32_t* status) {
    const bool deep = o.M <= 2;  // every weight load of the kernel issued up front (cp.async)
#define B200Q_SHORT(W)                                                                       \
    if (oct_plan(o.K, G, W, o.scale, o.zero, &o.ksplit, KB)) {                               \
        *status = deep ? launch_oct<T, 1, 1, W, 0, KB>(o, stream)                            \
                       : launch_oct<T, 1, 1, W, 2, KB>(o, stream);                           \
        return true;                                                                         \
    }
    B200Q_SHORT(8)
    B200Q_SHORT(4)
    B200Q_SHORT(7)
    B200Q_SHORT(2)
    B200Q_SHORT(1)
#undef B200Q_SHORT
    return false;
}

// The specialised g128 kernel when the shape allows it: the most warps per block
// (of 4, 7, 2, 1) that divide K / 1024 with at most 8 blocks per cluster.
template <typename T>
bool run_oct(const GemvArgs& a, cudaStream_t stream, int32_t* status) {
    // Every variant is launched with programmatic stream serialization: its weight
    // prefetch overlaps the tail of the kernel before it.
    OctArgs o{a.x, a.packed, a.scale, a.zero, a.y, a.M, a.K, a.N, 1, 1,
              (a.flags & B200Q_EARLY_DEPENDENTS) ? 1 : 0};
    const bool few = a.M <= 8;
    if (few && a.G == 128) {
        // A warp's run through 8 k-blocks takes ~2.7 us however little else the GPU has to
        // do; while all warps of the problem would fill less than half of the resident warp
        // slots (14 of 28 a multiprocessor), halve the run and double the warps.
        // Halving stops where it would need a cluster to split K (more than 8 runs a tile):
        // at K=4096, N=4096 two k-blocks a warp with clusters of 2 took 7.6 us, eight
        // k-blocks without a cluster 6.2.
        const int64_t tiles = (a.N + 15) / 16, slots = int64_t(14) * sm_count();
        int kb = 8;
        while (kb > 2) {
            const bool fits = a.K % (128 * kb) == 0;
            const bool half_fits = a.K % (64 * kb) == 0 && a.K / (64 * kb) <= 8;
            if (fits && (tiles * (a.K / (128 * kb)) >= slots || !half_fits)) break;
            kb /= 2;
        }
        if (kb == 4 && run_short<T, 4>(o, a.G, stream, status)) return true;
        if (kb == 2 && a.K % 256 == 0 && run_short<T, 2>(o, a.G, stream, status)) return true;
    }
    if (oct_plan(a.K, a.G, 4, a.scale, a.zero, &o.ksplit)) {
        if (a.M <= 2) {
            // One or two rows: every weight load of the kernel is issued up front (cp.async).
            *status = launch_oct<T, 1, 1, 4, 0>(o, stream);
        } else if (few) {
            *status = launch_oct<T, 1, 1, 4, 2>(o, stream);
        } else {
            *status = launch_oct<T, 2, 1, 4, 2>(o, stream);
        }
    } else if (oct_plan(a.K, a.G, 7, a.scale, a.zero, &o.ksplit)) {
        *status = few ? launch_oct<T, 1, 1, 7, 2>(o, stream) : launch_oct<T, 2, 1, 7, 2>(o, stream);
    } else if (oct_plan(a.K, a.G, 2, a.scale, a.zero, &o.ksplit)) {
        *status = few ? launch_oct<T, 1, 1, 2, 2>(o, stream) : launch_oct<T, 2, 1, 2, 2>(o, stream);
    } else if (oct_plan(a.K, a.G, 1, a.scale, a.zero, &o.ksplit)) {
        *status = few ? launch_oct<T, 1, 1, 1, 2>(o, stream) : launch_oct<T, 2, 1, 1, 2>(o, stream);
    } else {
        return false;
    }
    return true;
}

// The one-block-per-multiprocessor kernel whose weights come through the TMA unit
// (int4_gemv_tma.cuh), with post-scaled sums: group 128, one or two activation rows, where it is
// the fastest of the decode kernels (9.9 us against 12.5 us a launch on the headline shape, in a
// chain of launches).  From three rows on, staging the activations and their group sums costs
// more than the post-scaling saves, and the kernels that dequantize every weight take over.
struct NormInput {  // the input of the product is rms_norm(x + delta) * weight
    const void* delta;   // or null
    const void* weight;
    void* x_out;         // x + delta, stored by the product when delta != null
    float eps;
};

template <typename T>
bool run_tma(const GemvArgs& a, cudaStream_t stream, int32_t* status, const NormInput* norm = nullptr) {
    if (a.G != 128 || a.M > 2 || size_t(a.N) * size_t(a.K / 2) >= (size_t(1) << 40)) return false;
    int* word = gemm_error_word();
    if (word == nullptr) return false;
    TmaArgs p{a.x, a.scale, a.zero, a.y, a.M, a.K, a.N, (a.N + 15) / 16, 1, 1, 1, 0,
              (a.flags & B200Q_NO_OVERLAP) ? 0 : 1, (a.flags & B200Q_EARLY_DEPENDENTS) ? 1 : 0, (a.flags & B200Q_SWIGLU_INPUT) ? 1 : 0,
              norm ? norm->delta : nullptr, norm ? norm->weight : nullptr, norm ? norm->x_out : nullptr,
              norm ? norm->eps : 0.0f, word};
    size_t smem = 0;
    const int sms = sm_count();
    if (tma_plan<1, 16, 8>(p, a.G, &smem)) {
        *status = launch_tma<T, 1, 16, 8, false>(p, a.packed, smem, sms, stream);
        return true;
    }
    if (tma_plan<1, 16, 4>(p, a.G, &smem)) {
        *status = launch_tma<T, 1, 16, 4, false>(p, a.packed, smem, sms, stream);
        return true;
    }
    return false;
}

template <typename T>
int32_t run_gemv(GemvArgs a, int64_t rows, cudaStream_t stream) {
    const size_t elt = 2;
    const uint8_t* x = static_cast<const uint8_t*>(a.x);
    uint8_t* y = static_cast<uint8_t*>(a.y);
    int64_t step = 16;
    for (int64_t m0 = 0; m0 < rows; m0 += step) {
        // Up to 64 rows a pass when the kernel with shared activations takes the shape
        // (the weight streams from HBM once per pass), else passes of 16.
        const int64_t left = rows - m0;
        step = left > 32 ? 64 : left > 16 ? 32 : 16;
        a.M = int(left < step ? left : step);
        a.x = x + size_t(m0) * a.K * elt;
        a.y = y + size_t(m0) * a.N * elt;
        int32_t status = B200Q_OK;
        if (a.M > 32 && run_rows<T, 8>(a, stream, &status)) {
            if (status != B200Q_OK) return status;
            continue;
        }
        if (a.M > 16) {
            if (a.M <= 32 && run_rows<T, 4>(a, stream, &status)) {
                if (status != B200Q_OK) return status;
                continue;
            }
            step = 16;
            a.M = 16;
        }
        if (!(a.flags & B200Q_EXACT_WEIGHTS) && run_tma<T>(a, stream, &status)) {
            // post-scaled sums through the TMA ring: the default for one or two rows
        } else if (a.M >= 9 && run_rows<T, 2>(a, stream, &status)) {
            // 9..16 rows: activations staged once per block (15.7 us against 21.7 us at 16
            // rows, K=4096, N=14336; up to 8 rows the per-lane loads are as fast or faster)
        } else if (run_oct<T>(a, stream, &status)) {
            // the specialised g128 kernel took it
        } else if (a.K % 128 == 0) {
            const Plan p = choose_plan(a.M, a.K, a.N);
            status = a.G % 128 == 0 ? dispatch_gemv<T, kExactBlock>(a, p, stream)
                                    : dispatch_gemv<T, kExactWord>(a, p, stream);
        } else {
            for (int sub = 0; sub < a.M; sub += 8) {
                int4_linear_simple_kernel<T><<<(a.N + 3) / 4, 128, 0, stream>>>(a, sub);
            }
            status = launched("int4_linear (general kernel)");
        }
        if (status != B200Q_OK) return status;
    }
    return B200Q_OK;
}

}  // namespace

int32_t check_int4_args(const char* who, const void* x, const uint8_t* packed, const void* scale,
                        const uint8_t* zero, void* y, int64_t rows, int64_t in, int64_t out,
                        int64_t group, int32_t dtype) {
    B200Q_REQUIRE(dtype == B200Q_BF16 || dtype == B200Q_F16, "%s: activations are bf16 or f16", who);
    B200Q_REQUIRE(rows >= 0 && in > 0 && out > 0, "%s: bad shape rows=%lld in=%lld out=%lld", who,
                  (long long)rows, (long long)in, (long long)out);
    B200Q_REQUIRE(group > 0 && group % 2 == 0 && in % group == 0,
                  "%s: a group of %lld must be even and divide the %lld inputs", who, (long long)group,
                  (long long)in);
    B200Q_REQUIRE(in < (int64_t(1) << 30) && out < (int64_t(1) << 30), "%s: dimension too large", who);
    if (rows == 0) return B200Q_OK;
    B200Q_REQUIRE(x && packed && scale && zero && y, "%s: null tensor", who);
    B200Q_REQUIRE(aligned(x, 16) && aligned(packed, 16) && aligned(scale, 2) && aligned(y, 2),
                  "%s: x and packed must be 16-byte aligned", who);
    return B200Q_OK;
}

}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_int4_gemv_ex(const void* x, const uint8_t* packed, const void* scale,
                                      const uint8_t* zero, void* y, int64_t rows, int64_t in,
                                      int64_t out, int64_t group, int32_t dtype, int32_t flags,
                                      void* stream) {
    const int32_t ok = check_int4_args("int4_gemv", x, packed, scale, zero, y, rows, in, out, group, dtype);
    if (ok != B200Q_OK || rows == 0) return ok;
    B200Q_REQUIRE((flags & ~(B200Q_EXACT_WEIGHTS | B200Q_EARLY_DEPENDENTS | B200Q_SWIGLU_INPUT | B200Q_NO_OVERLAP)) == 0,
                  "int4_gemv: unknown flag bits %d", flags);
    GemvArgs a{x, packed, scale, zero, y, 0, int(in), int(out), int(group), int(in / 128), 0, 1, flags};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (flags & B200Q_SWIGLU_INPUT) {
        // only the kernel that stages the activations once per block forms them on the way
        a.M = int(rows);
        int32_t status = B200Q_OK;
        const bool taken = rows <= 2 && !(flags & B200Q_EXACT_WEIGHTS) &&
                           (dtype == B200Q_BF16 ? run_tma<__nv_bfloat16>(a, s, &status) : run_tma<__half>(a, s, &status));
        if (!taken)
            return unavailable("int4_gemv: B200Q_SWIGLU_INPUT is taken for one or two rows, groups of 128 and the "
                               "default numerics");
        return status;
    }
    return dtype == B200Q_BF16 ? run_gemv<__nv_bfloat16>(a, rows, s) : run_gemv<__half>(a, rows, s);
}

extern "C" int32_t b200q_int4_gemv_norm(const void* x, const void* delta, const void* norm_weight, float eps,
                                        void* x_out, const uint8_t* packed, const void* scale,
                                        const uint8_t* zero, void* y, int64_t rows, int64_t in, int64_t out,
                                        int64_t group, int32_t dtype, int32_t flags, void* stream) {
    const int32_t ok = check_int4_args("int4_gemv_norm", x, packed, scale, zero, y, rows, in, out, group, dtype);
    if (ok != B200Q_OK || rows == 0) return ok;
    B200Q_REQUIRE((flags & ~B200Q_EARLY_DEPENDENTS) == 0, "int4_gemv_norm: unknown flag bits %d", flags);
    B200Q_REQUIRE(norm_weight && aligned(norm_weight, 16) && (!delta || (aligned(delta, 16) && x_out && aligned(x_out, 16))),
                  "int4_gemv_norm: norm weights (and delta with x_out) must be given, 16-byte aligned");
    B200Q_REQUIRE(!delta || x_out != x, "int4_gemv_norm: x_out must not be x (every block reads x)");
    if (dtype != B200Q_BF16 || rows > 2 || group != 128 || in > 8192)
        return unavailable("int4_gemv_norm: taken for bf16, one or two rows, groups of 128, up to 8192 inputs");
    GemvArgs a{x, packed, scale, zero, y, int(rows), int(in), int(out), int(group), int(in / 128), 0, 1, flags};
    NormInput norm{delta, norm_weight, x_out, eps};
    int32_t status = B200Q_OK;
    if (!run_tma<__nv_bfloat16>(a, static_cast<cudaStream_t>(stream), &status, &norm))
        return unavailable("int4_gemv_norm: the shape is not one the kernel that stages its input once takes");
    return status;
}

extern "C" int32_t b200q_int4_gemv(const void* x, const uint8_t* packed, const void* scale,
                                   const uint8_t* zero, void* y, int64_t rows, int64_t in,
                                   int64_t out, int64_t group, int32_t dtype, void* stream) {
    return b200q_int4_gemv_ex(x, packed, scale, zero, y, rows, in, out, group, dtype, 0, stream);
}
