// int4-g128 decode kernel, up to 16 activation rows: ONE block per multiprocessor, the weights
// brought in by the TMA unit, the arithmetic on warps that never issue a weight load.
//
//   y[m, n] = sum_g scale[n, g] * ( sum_{k in g} x[m, k] (magic + q[n, k])  -  (magic + zero[n, g]) X[m, g] )
//   X[m, g] = sum_{k in g} x[m, k]
//
// magic + q (128 + q in bf16, 1024 + q in f16) is what one LOP3 makes of a pair of nibbles,
// and it is exact, so the tensor-core sums are sums of exact products in f32; the zero point
// costs one multiply-add per k-block with X, which the block computes once in f32 while it
// stages the activations.  The result differs from the reference's torch path ((q - zero) *
// scale rounded to the 16-bit type per weight, python/linnet/src/linnet/torch/native.py:417-424)
// by the rounding noise of its weights only; EXACT = true keeps that rounding, weight for
// weight, in the same kernel.
//
// Layout of the work (weights in the checkpoint layout, nothing repacked):
//   * W is seen through a 3-D tensor map: 64 bytes of a k-block (128 inputs) innermost, then
//     the rows (stride K/2 bytes), then the k-blocks of a row (stride 64 bytes).  One box is
//     an ITEM: 16 rows x KB k-blocks, landing in shared memory as [KB][16 rows][64 bytes], so
//     that the 16-byte reads of a quarter warp (rows g, g+1 and the four quarters of a k-block)
//     cover all 32 banks once;
//   * the grid has one block per multiprocessor; block b owns the 16-row tiles
//     [b * tiles / grid, (b + 1) * tiles / grid).  WPT warps share a tile, each taking OPC
//     consecutive items of its K, and TPC = WARPS / WPT tiles are in work at a time;
//   * one extra warp is the producer: a single thread issues every item's box into a ring of
//     shared-memory stages, in the order the consumers will want them, as deep as shared
//     memory allows (the whole share of a multiprocessor, some 200 KB, is in flight from the
//     first microsecond, ahead even of the wait on the previous kernel: weights are constants);
//   * the block stages ALL activations once: [rows x K] 16-bit values, permuted to the
//     (k, k+4) pairing of the A fragments and stored as B fragments of mma.m16n8k16, with the
//     per-group sums X beside them;
//   * a warp hands a stage back to the producer the moment it has read the item in it, so the
//     ring only holds what is being read or is on its way (a block whose share of W is larger
//     than the ring would otherwise wait, round after round, for the stages of the round
//     before);
//   * the warps of a tile add up their partial sums in a small shared-memory area of their own,
//     behind a named barrier of their own: no thread-block cluster, no atomics, no global scratch.
//
// Every wait on a shared-memory barrier is bounded: after about a second the waiting warp
// records a code in the device's status word, and it and every other warp finish without
// further waiting (the output is then incomplete and the status says so).
#pragma once

#include <cuda.h>

#include "tma_ring.cuh"

namespace b200q {

struct TmaArgs {
    const void* x;          // [M, K]
    const void* scale;      // [N, K/128]
    const uint8_t* zero;    // [N, K/128]
    void* y;                // [M, N]
    int M, K, N;
    int tiles;              // ceil(N / 16)
    int wpt;                // warps per tile
    int opc;                // items per warp and tile; K == 128 * KB * opc * wpt
    int tpc;                // tiles in work at a time per block = WARPS / wpt
    int stages;             // ring stages of KB KiB
    int overlap;            // launched with programmatic stream serialization
    int early;              // dependents may start as soon as this kernel has started
    int swiglu;             // x is [M, 2 K]: the input is silu(x[:, :K]) * x[:, K:], formed while staging
    // norm != null (bf16 only): the input is rms_norm(x + delta) * norm, formed while staging; the
    // first block also stores x + delta to x_out (delta may be null: then nothing is stored)
    const void* delta;      // [M, K] or null
    const void* norm;       // [K] or null
    void* x_out;            // [M, K]
    float eps;
    int* status;            // device word of expired waits
};

// Offsets (bytes) of the shared-memory regions: ring of stages, barriers, per-warp scales
// and zero points, B fragments of the activations, their group sums.
struct TmaLayout {
    uint32_t bars, sz, xs, xsum, red, total;
    uint32_t xrow;    // bytes of one activation row in xs (padded so that rows g, g+1 fall on different banks)
    int xpairs;       // pairs of rows in xsum
};
template <int MB, int WARPS, int KB>
__host__ __device__ inline TmaLayout tma_layout(int M, int K, int stages) {
    TmaLayout l;
    const int groups = K / 128;
    l.bars = uint32_t(stages) * (KB * 1024);
    l.sz = (l.bars + uint32_t(stages + 2 * WARPS) * 8 + 15u) & ~15u;  // 16-byte stores
    l.xs = (l.sz + WARPS * 16 * KB * 3 + 127u) & ~127u;
    l.xrow = uint32_t(groups) * 256 + (M > 1 ? 64 : 0);
    l.xpairs = (M + 1) / 2;
    l.xsum = l.xs + uint32_t(M) * l.xrow;
    l.red = (l.xsum + uint32_t(l.xpairs) * groups * 8 + 128 + 15u) & ~15u;  // (+ 128: the sums of squares of the fused norm)
    l.total = l.red + 2u * WARPS * (16 * MB * 8 * 4);  // the warps' partial sums of a tile, two rounds' worth
    return l;
}

// MB: blocks of 8 activation rows (1 or 2).  WARPS: consumer warps (one more is the producer).
// KB: k-blocks per item (8 or 4).  EXACT: dequantize every weight as the reference does.
template <typename T, int MB, int WARPS, int KB, bool EXACT>
__global__ void __launch_bounds__((WARPS + 1) * 32, 1)
int4_gemv_tma_kernel(const __grid_constant__ CUtensorMap wmap, const TmaArgs a) {
    static_assert(KB == 8 || KB == 4, "k-blocks per item");
    using H = Half16<T>;
    constexpr int MP = MB * 8;
    constexpr uint32_t kItem = KB * 1024;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
    const int M = a.M, K = a.K, N = a.N;
    const int groups = K / 128;
    const int S = a.stages;
    const TmaLayout lay = tma_layout<MB, WARPS, KB>(M, K, S);
    const uint32_t smem0 = uint32_t(__cvta_generic_to_shared(smem));
    // Barriers: empty[s] (a stage has been read; the producer waits on it, lap after lap),
    // ready[w] (the bytes of consumer w's next item have landed; w waits on it, item after item)
    // and taken[w] (w has seen that; the producer waits on it before it sends w another item,
    // so that ready[w] is never two phases ahead of its waiter: a parity stands for one phase
    // only while the waiter is at most one behind).
    const uint32_t empty0 = smem0 + lay.bars, ready0 = empty0 + uint32_t(S) * 8, taken0 = ready0 + WARPS * 8;

    // This block's tiles; the consumers in use and the rounds they make.
    const int t0 = int((uint32_t(blockIdx.x) * uint32_t(a.tiles)) / gridDim.x);
    const int t1 = int((uint32_t(blockIdx.x + 1) * uint32_t(a.tiles)) / gridDim.x);
    const int active = a.tpc * a.wpt;
    const int rounds = (t1 - t0 + a.tpc - 1) / a.tpc;

    if (int(threadIdx.x) < S + 2 * WARPS) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(empty0 + threadIdx.x * 8));
        umma::fence_proxy_async();  // the TMA unit's view of the barriers
    }
    __syncthreads();

    if (warp == WARPS) {
        // ---- producer: items in the order (round, item of the tile, consumer) ----------------
        if (lane != 0) return;
        if (a.overlap) pdl_launch_dependents();  // this thread never waits on the previous kernel: weights are constants
        int s = 0;
        uint32_t lap = 0;  // times the ring has been gone round
        bool ok = true;
        int n = 0;         // items each consumer has been sent
        for (int round = 0; round < rounds && ok; ++round) {
            const int tiles_here = min(a.tpc, t1 - t0 - round * a.tpc);  // the last round may be short
            for (int o = 0; o < a.opc && ok; ++o, ++n) {
                int w = 0;
                for (int ts = 0; ts < tiles_here && ok; ++ts) {
                    const int tile = t0 + round * a.tpc + ts;
                    for (int part = 0; part < a.wpt; ++part, ++w) {
                        const uint32_t empty = empty0 + s * 8, ready = ready0 + w * 8;
                        if (lap > 0) ok = bar_wait<true>(empty, (lap - 1) & 1, a.status, 11);
                        if (ok && n > 0) ok = bar_wait<true>(taken0 + w * 8, (n - 1) & 1, a.status, 13);
                        if (!ok) break;
                        bar_expect(ready, kItem);
                        tma_item(smem0 + uint32_t(s) * kItem, &wmap, tile * 16, (part * a.opc + o) * KB, ready);
                        if (++s == S) {
                            s = 0;
                            ++lap;
                        }
                    }
                }
            }
        }
        return;
    }

    // ---- consumers ---------------------------------------------------------------------------
    const bool works = warp < active && t0 + warp / a.wpt < t1;
    const int ts = warp / a.wpt, part = warp % a.wpt;
    const uint32_t my_sz = smem0 + lay.sz + uint32_t(warp) * (16 * KB * 3);
    const uint32_t xs = smem0 + lay.xs, xsum = smem0 + lay.xsum;

    // Scales (lanes 0-15: KB x 2 bytes of row `lane`) and zero points (lanes 16-31: KB bytes of
    // row `lane - 16`) of one item, through registers.
    auto load_sz = [&](int tile, int item, uint4& v) {
        const int r = min(tile * 16 + (lane & 15), N - 1);  // ragged tile: clamp
        const size_t at = size_t(r) * groups + size_t(item) * KB;
        if (lane < 16) {
            const uint8_t* p = static_cast<const uint8_t*>(a.scale) + at * 2;
            if (KB == 8) v = __ldg(reinterpret_cast<const uint4*>(p));
            else { const uint2 h = __ldg(reinterpret_cast<const uint2*>(p)); v.x = h.x; v.y = h.y; }
        } else {
            const uint8_t* p = a.zero + at;
            if (KB == 8) { const uint2 h = __ldg(reinterpret_cast<const uint2*>(p)); v.x = h.x; v.y = h.y; }
            else v.x = __ldg(reinterpret_cast<const uint32_t*>(p));
        }
    };
    auto store_sz = [&](const uint4& v) {
        if (lane < 16) {
            const uint32_t dst = my_sz + lane * (KB * 2);
            if (KB == 8) sts128(dst, v);
            else sts64(dst, v.x, v.y);
        } else {
            const uint32_t dst = my_sz + 16 * KB * 2 + (lane - 16) * KB;
            if (KB == 8) sts64(dst, v.x, v.y);
            else sts32(dst, v.x);
        }
    };

    if (a.overlap) {
        if (a.early) pdl_launch_dependents();
        pdl_wait();  // activations may come from the kernel ahead of this one
    }

    // Activations: M * (K / 128) * 16 pieces of 16 bytes, the 16 pieces of a (row, k-block) in
    // 16 consecutive lanes, which also add up the k-block's inputs.
    uint4 szr = make_uint4(0, 0, 0, 0);
    {
        const uint4* xg = below_pdl_wait(static_cast<const uint4*>(a.x));
        const int pieces = M * groups * 16;
        constexpr int threads = WARPS * 32;
        const int me = int(threadIdx.x);
        auto where = [&](int e, int& m, int& j, int& c) {
            const int r = e >> 4;  // (row, k-block)
            m = M == 1 ? 0 : r / groups;
            j = r - m * groups;
            c = e & 15;  // piece of the k-block: lane t = c/4, word i = c%4
        };
        auto stage = [&](int e, const uint4& raw, bool live) {
            int m, j, c;
            where(e, m, j, c);
            if (!EXACT) {
                float sum = (H::to_float(raw.x & 0xFFFFu) + H::to_float(raw.x >> 16)) +
                            (H::to_float(raw.y & 0xFFFFu) + H::to_float(raw.y >> 16));
                sum += (H::to_float(raw.z & 0xFFFFu) + H::to_float(raw.z >> 16)) +
                       (H::to_float(raw.w & 0xFFFFu) + H::to_float(raw.w >> 16));
#pragma unroll
                for (int d = 8; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
                if (live && c == 0) sts32f(xsum + (uint32_t(m / 2) * groups + j) * 8 + (m % 2) * 4, sum);
            }
            if (live) {
                uint4 out;
                out.x = __byte_perm(raw.x, raw.z, 0x5410);  // (x0, x4)
                out.y = __byte_perm(raw.x, raw.z, 0x7632);  // (x1, x5)
                out.z = __byte_perm(raw.y, raw.w, 0x5410);  // (x2, x6)
                out.w = __byte_perm(raw.y, raw.w, 0x7632);  // (x3, x7)
                sts128(xs + uint32_t(m) * lay.xrow + uint32_t(j) * 256 + (c % 4) * 64 + (c / 4) * 16, out);
            }
        };
        // silu(g) rounded to the 16-bit type, times u, rounded again: what the two PyTorch ops
        // (and the stand-alone silu_mul kernel of the decode step) make of a pair of words
        auto swiglu2 = [&](uint32_t gw, uint32_t uw) {
            uint32_t out = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float gv = H::to_float((gw >> (16 * h)) & 0xFFFFu), uv = H::to_float((uw >> (16 * h)) & 0xFFFFu);
                const float sv = H::to_float(H::from_float(gv / (1.0f + expf(-gv))));
                out |= uint32_t(H::from_float(sv * uv)) << (16 * h);
            }
            return out;
        };
        auto load = [&](int e) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (e < pieces) {
                int m, j, c;
                where(e, m, j, c);
                if (!a.swiglu) {
                    raw = ld_mutable(xg + (size_t(m) * K + size_t(j) * 128) / 8 + c);
                } else {
                    const uint4 gq = ld_mutable(xg + (size_t(m) * 2 * K + size_t(j) * 128) / 8 + c);
                    const uint4 uq = ld_mutable(xg + (size_t(m) * 2 * K + K + size_t(j) * 128) / 8 + c);
                    raw = make_uint4(swiglu2(gq.x, uq.x), swiglu2(gq.y, uq.y), swiglu2(gq.z, uq.z), swiglu2(gq.w, uq.w));
                }
            }
            return raw;
        };
        constexpr int kFirst = MB == 1 ? 4 : 8;  // pieces a thread has in flight at first
        if (MB == 1 && a.norm != nullptr) {
            // x + delta, its RMS norm times the norm weights, with the arithmetic and the order of
            // sums of the stand-alone kernel of the decode step (decoder_glue.cu): thread c takes
            // the pieces c, c + 512, ... of every row; up to two rows of up to 1024 pieces.
            constexpr int kHeld = 2;
            const int chunks = groups * 16;
            const uint4* dg = below_pdl_wait(static_cast<const uint4*>(a.delta));
            const uint4* ng = static_cast<const uint4*>(a.norm);
            uint4* xo = static_cast<uint4*>(a.x_out);
            const uint32_t squares = xsum + uint32_t(lay.xpairs) * groups * 8;  // [2 rows][16 warps] f32
            uint4 v[2][kHeld], gw[kHeld];
#pragma unroll
            for (int u = 0; u < kHeld; ++u) {
                const int c = me + u * threads;
                gw[u] = c < chunks ? __ldg(ng + c) : make_uint4(0, 0, 0, 0);
            }
            if (works) load_sz(t0 + ts, part * a.opc, szr);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                float sum = 0.0f;
#pragma unroll
                for (int u = 0; u < kHeld; ++u) {
                    const int c = me + u * threads;
                    uint4 tv = make_uint4(0, 0, 0, 0);
                    if (m < M && c < chunks) {
                        tv = ld_mutable(xg + size_t(m) * chunks + c);
                        if (dg != nullptr) {
                            const uint4 d = ld_mutable(dg + size_t(m) * chunks + c);
                            tv.x = bf16_pack(bf16_lo(tv.x) + bf16_lo(d.x), bf16_hi(tv.x) + bf16_hi(d.x));
                            tv.y = bf16_pack(bf16_lo(tv.y) + bf16_lo(d.y), bf16_hi(tv.y) + bf16_hi(d.y));
                            tv.z = bf16_pack(bf16_lo(tv.z) + bf16_lo(d.z), bf16_hi(tv.z) + bf16_hi(d.z));
                            tv.w = bf16_pack(bf16_lo(tv.w) + bf16_lo(d.w), bf16_hi(tv.w) + bf16_hi(d.w));
                            if (blockIdx.x == 0) xo[size_t(m) * chunks + c] = tv;
                        }
                        const uint32_t e4[4] = {tv.x, tv.y, tv.z, tv.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) sum += bf16_lo(e4[i]) * bf16_lo(e4[i]) + bf16_hi(e4[i]) * bf16_hi(e4[i]);
                    }
                    v[m][u] = tv;
                }
                for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
                if (lane == 0) sts32f(squares + (m * 16 + warp) * 4, sum);
            }
            named_barrier(15, WARPS * 32);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                float total = 0.0f;
                for (int i = 0; i < WARPS; ++i) total += lds32f(squares + (m * 16 + i) * 4);
                const float rstd = rsqrtf(total / float(K) + a.eps);
#pragma unroll
                for (int u = 0; u < kHeld; ++u) {
                    const int c = me + u * threads;
                    if (u * threads >= chunks || m >= M) continue;  // uniform over the block
                    const uint4 tv = v[m][u];
                    uint4 o;
                    o.x = bf16_pack(bf16_lo(tv.x) * rstd * bf16_lo(gw[u].x), bf16_hi(tv.x) * rstd * bf16_hi(gw[u].x));
                    o.y = bf16_pack(bf16_lo(tv.y) * rstd * bf16_lo(gw[u].y), bf16_hi(tv.y) * rstd * bf16_hi(gw[u].y));
                    o.z = bf16_pack(bf16_lo(tv.z) * rstd * bf16_lo(gw[u].z), bf16_hi(tv.z) * rstd * bf16_hi(gw[u].z));
                    o.w = bf16_pack(bf16_lo(tv.w) * rstd * bf16_lo(gw[u].w), bf16_hi(tv.w) * rstd * bf16_hi(gw[u].w));
                    stage(m * chunks + c, o, c < chunks);
                }
            }
        } else {
            uint4 raw[kFirst];
#pragma unroll
            for (int u = 0; u < kFirst; ++u) raw[u] = load(u * threads + me);
            if (works) load_sz(t0 + ts, part * a.opc, szr);
#pragma unroll
            for (int u = 0; u < kFirst; ++u)
                if (u * threads < pieces) stage(u * threads + me, raw[u], u * threads + me < pieces);
            for (int base = kFirst * threads; base < pieces; base += 4 * threads) {  // four loads in flight a thread
                uint4 more[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) more[u] = load(base + u * threads + me);
#pragma unroll
                for (int u = 0; u < 4; ++u) stage(base + u * threads + me, more[u], base + u * threads + me < pieces);
            }
        }
    }
    named_barrier(15, WARPS * 32);  // the consumers only: the producer is on its own way
    if (!works) return;

    // ---- this warp's items --------------------------------------------------------------------
    const uint32_t kMask = 0x000F000Fu;
    uint16_t* y = static_cast<uint16_t*>(a.y);
    const uint32_t wl = uint32_t(g) * 64 + t * 16;                      // this lane's bytes of a k-block's row g
    const uint32_t x_lane0 = xs + uint32_t(min(g, M - 1)) * lay.xrow + t * 16;
    const uint32_t x_lane1 = xs + uint32_t(min(8 + g, M - 1)) * lay.xrow + t * 16;
    const uint32_t xsum_lane0 = xsum + uint32_t(min(t, lay.xpairs - 1)) * groups * 8;
    const uint32_t xsum_lane1 = xsum + uint32_t(min(4 + t, lay.xpairs - 1)) * groups * 8;
    const uint32_t my_sc = my_sz + g * (KB * 2), my_zp = my_sz + 16 * KB * 2 + g * KB;
    bool ok = true;
    int n = 0;                      // items this warp has taken
    int s = warp % S;               // stage of its next item: the items before it in the producer's order, modulo S
    const int s_step = active % S;  // a full round's items between two of this warp's
    const int s_last = (min(a.tpc, t1 - t0 - (rounds - 1) * a.tpc) * a.wpt) % S;  // the last round's
    const uint32_t ready = ready0 + warp * 8;
    for (int tile = t0 + ts, round = 0; tile < t1; tile += a.tpc, ++round) {
        float acc[MB][2][4];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int s = 0; s < 2; ++s)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mb][s][i] = 0.0f;
        uint32_t stage_addr = 0;
        int s_mine = 0;
        for (int o = 0; o < a.opc; ++o, ++n) {
            const int item = part * a.opc + o;
            // scales and zero points: this item's from the registers, the next one's on their way
            __syncwarp();
            store_sz(szr);
            __syncwarp();
            {
                const bool more_here = o + 1 < a.opc;
                const int next_tile = more_here ? tile : tile + a.tpc;
                if (next_tile < t1) load_sz(next_tile, more_here ? item + 1 : part * a.opc, szr);
            }
            s_mine = s;
            s += tile + a.tpc >= t1 ? s_last : s_step;
            if (s >= S) s -= S;
            stage_addr = smem0 + uint32_t(s_mine) * kItem;
            if (ok) ok = bar_wait(ready, uint32_t(n) & 1, a.status, 12);
            __syncwarp();  // every lane has seen the phase
            if (lane == 0) bar_arrive(taken0 + warp * 8);
            const uint32_t wq = stage_addr + wl;
            const uint32_t xq0 = x_lane0 + uint32_t(item) * (KB * 256), xq1 = x_lane1 + uint32_t(item) * (KB * 256);
            const uint32_t xsq0 = xsum_lane0 + uint32_t(item) * (KB * 8), xsq1 = xsum_lane1 + uint32_t(item) * (KB * 8);
            // the item's scales and zero points of rows g and g+8: KB 16-bit values and KB bytes each
            uint32_t scw[2][KB / 2], zpw[2][KB / 4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (KB == 8) {
                    const uint4 sv = lds128(my_sc + h * 8 * KB * 2);
                    scw[h][0] = sv.x; scw[h][1] = sv.y; scw[h][2 % (KB / 2)] = sv.z; scw[h][3 % (KB / 2)] = sv.w;
                    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(zpw[h][0]), "=r"(zpw[h][1 % (KB / 4)]) : "r"(my_zp + h * 8 * KB));
                } else {
                    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(scw[h][0]), "=r"(scw[h][1]) : "r"(my_sc + h * 8 * KB * 2));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zpw[h][0]) : "r"(my_zp + h * 8 * KB));
                }
            }
#pragma unroll
            for (int j = 0; j < KB; ++j) {
                const uint4 q0 = lds128(wq + j * 1024), q1 = lds128(wq + j * 1024 + 512);
                uint32_t sc[2] = {0, 0}, bias[2] = {0, 0};
                if (EXACT) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        sc[h] = __byte_perm(scw[h][j / 2], 0, j % 2 ? 0x3232 : 0x1010);  // (scale, scale)
                        bias[h] = H::kMagic + __byte_perm(zpw[h][j / 4], 0, 0x4040 | (j % 4) | (j % 4) << 8);  // (magic + zero) x 2
                    }
                }
                float ka[MB][4], kb[MB][4];  // !EXACT: this k-block's sums, in two chains of MMAs
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // rows past the last one re-read the last row: their columns are never stored
                    uint4 b[MB];
                    b[0] = lds128(xq0 + j * 256 + i * 64);
                    if (MB > 1) b[MB - 1] = lds128(xq1 + j * 256 + i * 64);
                    const uint32_t w0 = i == 0 ? q0.x : i == 1 ? q0.y : i == 2 ? q0.z : q0.w;
                    const uint32_t w1 = i == 0 ? q1.x : i == 1 ? q1.y : i == 2 ? q1.z : q1.w;
                    uint32_t f0[4], f1[4];  // (k0,k4) (k1,k5) (k2,k6) (k3,k7) of rows g, g+8
                    f0[0] = lop3_and_or(w0, kMask, H::kMagic);
                    f0[1] = lop3_and_or(w0 >> 4, kMask, H::kMagic);
                    f0[2] = lop3_and_or(w0 >> 8, kMask, H::kMagic);
                    f0[3] = lop3_and_or(w0 >> 12, kMask, H::kMagic);
                    f1[0] = lop3_and_or(w1, kMask, H::kMagic);
                    f1[1] = lop3_and_or(w1 >> 4, kMask, H::kMagic);
                    f1[2] = lop3_and_or(w1 >> 8, kMask, H::kMagic);
                    f1[3] = lop3_and_or(w1 >> 12, kMask, H::kMagic);
                    if (EXACT) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            f0[e] = sub_mul<T>(f0[e], bias[0], sc[0]);
                            f1[e] = sub_mul<T>(f1[e], bias[1], sc[1]);
                        }
                    }
                    const uint32_t a_lo[4] = {f0[0], f1[0], f0[1], f1[1]};
                    const uint32_t a_hi[4] = {f0[2], f1[2], f0[3], f1[3]};
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) {
                        if (EXACT) {
                            H::mma(acc[mb][0], a_lo, b[mb].x, b[mb].y);
                            H::mma(acc[mb][1], a_hi, b[mb].z, b[mb].w);
                        } else if (i == 0) {
                            mma_first<T>(ka[mb], a_lo, b[mb].x, b[mb].y);
                            mma_first<T>(kb[mb], a_hi, b[mb].z, b[mb].w);
                        } else {
                            H::mma(ka[mb], a_lo, b[mb].x, b[mb].y);
                            H::mma(kb[mb], a_hi, b[mb].z, b[mb].w);
                        }
                    }
                }
                if (!EXACT) {
                    // y += scale * (sums - (magic + zero) * X), rows g (0, 1) and g+8 (2, 3)
                    float sf[2], nz[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        sf[h] = scale_of<T>(scw[h][j / 2], j % 2);
                        // 2^23 + zero as f32 bits, then (2^23 - magic) - that = -(magic + zero)
                        nz[h] = (8388608.0f - H::kBias) - __uint_as_float(__byte_perm(zpw[h][j / 4], 0x4B000000u, 0x7440 | (j % 4)));
                    }
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) {
                        const float2 X = lds64f((mb == 0 ? xsq0 : xsq1) + j * 8);
                        acc[mb][0][0] = fmaf(sf[0], fmaf(nz[0], X.x, ka[mb][0] + kb[mb][0]), acc[mb][0][0]);
                        acc[mb][0][1] = fmaf(sf[0], fmaf(nz[0], X.y, ka[mb][1] + kb[mb][1]), acc[mb][0][1]);
                        acc[mb][0][2] = fmaf(sf[1], fmaf(nz[1], X.x, ka[mb][2] + kb[mb][2]), acc[mb][0][2]);
                        acc[mb][0][3] = fmaf(sf[1], fmaf(nz[1], X.y, ka[mb][3] + kb[mb][3]), acc[mb][0][3]);
                    }
                }
            }
            __syncwarp();  // every lane has read the item: the stage goes back to the producer at once
            if (lane == 0) bar_arrive(empty0 + s_mine * 8);
        }
        const bool last_tile = tile + a.tpc >= t1;
        if (last_tile && a.overlap && !a.early) pdl_launch_dependents();

        // The tile's partial sums meet in a small area of their own (16 x MP floats a warp, two
        // rounds' worth: a warp can only write a buffer again after the tile's first warp has
        // passed the next round's barrier, that is after it has read this round's): the tile's
        // first warp adds them up and stores y.
        const uint32_t red = smem0 + lay.red + uint32_t(round & 1) * (WARPS * 16 * MP * 4);
        {
            const uint32_t dst0 = red + uint32_t(warp) * (16 * MP * 4);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const uint32_t dst = dst0 + (g * MP + mb * 8 + 2 * t) * 4;
                sts32f(dst, acc[mb][0][0] + (EXACT ? acc[mb][1][0] : 0.0f));
                sts32f(dst + 4, acc[mb][0][1] + (EXACT ? acc[mb][1][1] : 0.0f));
                sts32f(dst + 8 * MP * 4, acc[mb][0][2] + (EXACT ? acc[mb][1][2] : 0.0f));
                sts32f(dst + 8 * MP * 4 + 4, acc[mb][0][3] + (EXACT ? acc[mb][1][3] : 0.0f));
            }
        }
        if (a.wpt > 1) named_barrier(1 + ts, a.wpt * 32);
        else __syncwarp();
        if (part == 0) {
            for (int e = lane; e < 16 * M; e += 32) {
                const int row = e % 16, m = e / 16;
                float sum = 0.0f;
                for (int w = 0; w < a.wpt; ++w)  // the tile's warps are this one and the wpt - 1 after it
                    sum += lds32f(red + uint32_t(warp + w) * (16 * MP * 4) + (row * MP + m) * 4);
                const int nrow = tile * 16 + row;
                if (nrow < N) y[size_t(m) * N + nrow] = H::from_float(sum);
            }
        }
    }
}

// Launch geometry; false when the kernel does not take the shape.
template <int MB, int WARPS, int KB>
inline bool tma_plan(TmaArgs& a, int G, size_t* smem) {
    if (G != 128 || a.K % (128 * KB) != 0 || a.M > MB * 8 || a.M < 1) return false;
    if (!aligned(a.scale, KB * 2) || !aligned(a.zero, KB) || !aligned(a.x, 16)) return false;
    const int runs = a.K / (128 * KB);
    // as many warps per tile as there are items, up to the block; else whole items per warp
    int opc = 1;
    while (runs % opc != 0 || runs / opc > WARPS) ++opc;
    a.opc = opc;
    a.wpt = runs / opc;
    if (a.wpt > 32) return false;  // the tile's first warp hands one stage back per lane
    a.tpc = WARPS / a.wpt;
    if (a.wpt > 1 && a.tpc > 14) a.tpc = 14;  // named barriers 1..14 (15 is the consumers')
    const TmaLayout fixed = tma_layout<MB, WARPS, KB>(a.M, a.K, 0);
    const long budget = 226L * 1024 - long(fixed.total);
    long stages = (budget - 2 * WARPS * 8 - 16) / (KB * 1024 + 8);
    // A shallow ring is another kernel's shape (and every warp of a tile wants a stage of its own).
    if (stages < 4 || stages <= a.wpt) return false;
    if (stages > 96) stages = 96;
    a.stages = int(stages);
    *smem = tma_layout<MB, WARPS, KB>(a.M, a.K, a.stages).total;
    return true;
}

// The weights [N, K/2] as 64-byte pieces: (byte of the k-block, row, k-block of the row).
template <int KB>
inline bool tma_weight_map(CUtensorMap* map, const uint8_t* packed, int N, int K) {
    const umma::EncodeTiled encode = umma::encode_tiled();
    if (encode == nullptr || !aligned(packed, 16)) return false;
    const cuuint64_t dims[3] = {64, cuuint64_t(N), cuuint64_t(K / 128)};
    const cuuint64_t strides[2] = {cuuint64_t(K / 2), 64};
    const cuuint32_t box[3] = {64, 16, KB};
    const cuuint32_t elem[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(packed), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int MB, int WARPS, int KB, bool EXACT>
int32_t launch_tma(const TmaArgs& a, const uint8_t* packed, size_t smem, int sms, cudaStream_t stream) {
    auto kernel = int4_gemv_tma_kernel<T, MB, WARPS, KB, EXACT>;
    CUtensorMap map;
    if (!tma_weight_map<KB>(&map, packed, a.N, a.K)) return fail("int4_gemv: the weight tensor map was refused");
    const cudaError_t attr_err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    if (attr_err != cudaSuccess) {
        cudaGetLastError();
        return fail("int4_gemv: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(attr_err));
    }
    // One block per multiprocessor (each takes an equal share of the tiles, several rounds of
    // `tpc` if need be), fewer when there are fewer tiles than multiprocessors.
    const int grid = a.tiles < sms ? a.tiles : sms;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(unsigned(grid), 1, 1);
    config.blockDim = dim3((WARPS + 1) * 32, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = a.overlap ? 1 : 0;
    const cudaError_t err = cudaLaunchKernelEx(&config, kernel, map, a);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail("int4_gemv: launch failed: %s", cudaGetErrorString(err));
    }
    return B200Q_OK;
}

}  // namespace b200q
