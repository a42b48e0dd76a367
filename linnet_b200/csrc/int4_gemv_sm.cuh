// int4-g128 decode kernel, up to 16 activation rows: ONE block per multiprocessor, the
// activations staged once per multiprocessor, zero point and scale applied to group sums.
//
//   y[m, n] = sum_g scale[n, g] * ( sum_{k in g} x[m, k] (magic + q[n, k])  -  (magic + zero[n, g]) X[m, g] )
//   X[m, g] = sum_{k in g} x[m, k]
//
// magic + q (128 + q in bf16, 1024 + q in f16) is what one LOP3 makes of a pair of nibbles,
// and it is exact, so the tensor-core sums are sums of exact products in f32; the zero point
// costs one multiply-add per k-block with X, which the block computes once in f32 while it
// stages the activations.  Per 8 weights that is 7 integer instructions, against 15 when
// every weight is first rounded to the 16-bit type as the reference's torch path does
// ((q - zero) * scale, cast once: python/linnet/src/linnet/torch/native.py:417-424).  The
// result differs from that path by the rounding noise of its weights only (about 2^-9
// relative per weight); EXACT = true keeps the reference's rounding, weight for weight, in
// the same kernel.
//
// Layout of the work (weights in the checkpoint layout, nothing repacked):
//   * the grid has one block per multiprocessor; block b owns the 16-row tiles
//     [b * tiles / grid, (b + 1) * tiles / grid) of W.  A tile's K is cut into runs of KB
//     k-blocks (128 inputs each); WPT warps share a tile, each taking OPC consecutive runs,
//     and TPC = WARPS / WPT tiles are in work at a time;
//   * the block stages ALL activations once: [rows x K] 16-bit values, permuted to the
//     (k, k+4) pairing of the A fragments and stored as B fragments of mma.m16n8k16, with
//     the per-group sums X beside them;
//   * lane (g, t) streams 16 bytes of rows g and g+8 per k-block with cp.async.cg into a ring
//     of R lane-private shared-memory slots (a lane reads back only what it asked for, so
//     cp.async.wait_group is all the synchronisation the weight path has);
//   * the warps of a tile add up their partial sums in shared memory behind a named barrier
//     of their own: no thread-block cluster, no atomics, no global scratch.
//
// Order of the memory requests.  A multiprocessor serves its requests in the order they were
// made (its share of the weight stream is some 200 KB, 5 us at its share of the HBM rate), and a
// warp that asks for more than the memory pipeline has room for stalls at the request itself.
// Measured with per-block timestamps on the headline shape: activation loads issued behind a
// full ring arrive 3 to 4 us late, and a warp that fills a deep ring first does not even look
// at them before that, so the arithmetic starts when the memory traffic is nearly over
// instead of running under it.  Hence: the activation loads go out first, the ring is filled
// behind them, and it is only as deep as it takes to keep HBM busy (84 KB a multiprocessor
// at three slots; bandwidth times latency is about 45 KB), the rest being requested as slots
// are consumed.  PRE ring slots can still be asked for before the wait on the previous kernel.
#pragma once

#include "gemv_common.cuh"

namespace b200q {

struct SmArgs {
    const void* x;          // [M, K]
    const uint8_t* packed;  // [N, K/2]
    const void* scale;      // [N, K/128]
    const uint8_t* zero;    // [N, K/128]
    void* y;                // [M, N]
    int M, K, N;
    int tiles;              // ceil(N / 16)
    int wpt;                // warps per tile
    int opc;                // runs of KB k-blocks per warp; K == 128 * KB * opc * wpt
    int tpc;                // tiles in work at a time per block = WARPS / wpt
    int overlap;            // launched with programmatic stream serialization
    int early;              // dependents may start as soon as this kernel has started
};

template <int N>
__device__ __forceinline__ void cp_async_wait_n() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Shared memory by its 32-bit address (one register instead of a generic pointer's two).
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds32f(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts32f(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// d = a * b (accumulator starts at zero).
template <typename T>
__device__ __forceinline__ void mma_first(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_first<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}
template <>
__device__ __forceinline__ void mma_first<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                  uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

// Bytes of the shared-memory regions, in order: ring, scales + zero points, B fragments, sums.
struct SmLayout {
    uint32_t ring, sz, xs, xsum, total;
    int sz_per_warp;  // bytes
    int xstride;      // floats per k-block in xsum (rows rounded up to even)
};
template <int MB, int WARPS, int KB, int R>
__host__ __device__ inline SmLayout sm_layout(int M, int K, int opc) {
    SmLayout l;
    l.ring = 0;
    l.sz = WARPS * R * 1024;
    l.sz_per_warp = 16 * KB * opc * 3;
    l.xs = l.sz + WARPS * l.sz_per_warp;
    l.xs = (l.xs + 15u) & ~15u;
    l.xstride = (M + 1) & ~1;
    l.xsum = l.xs + (K / 128) * 256 * M;
    l.total = l.xsum + (K / 128) * l.xstride * 4 + (MB > 1 ? 64 : 0);
    return l;
}

// MB: blocks of 8 activation rows (1 or 2).  WARPS: warps per block.  KB: k-blocks per run
// (8 or 4).  R: ring slots per lane.  EXACT: dequantize every weight as the reference does.
// PRE: ring slots requested ahead of the wait on the previous kernel and of the activations.
// SW: extra warps that do nothing but load and stage the activations, while the WARPS others
// fill their rings (a warp stalls at a request the memory pipeline has no room for, and could
// not look at the activations meanwhile); 0: every warp stages its share after its requests.
template <typename T, int MB, int WARPS, int KB, int R, bool EXACT, int PRE = 0, int SW = 0>
__global__ void __launch_bounds__((WARPS + SW) * 32, 1)
int4_gemv_sm_kernel(const SmArgs a) {
    static_assert(KB == 8 || KB == 4, "k-blocks per run");
    using H = Half16<T>;
    constexpr int MP = MB * 8;
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
    const int M = a.M, K = a.K, N = a.N;
    const int groups = K / 128;
    const SmLayout lay = sm_layout<MB, WARPS, KB, R>(M, K, a.opc);
    const uint32_t smem0 = uint32_t(__cvta_generic_to_shared(smem));
    const uint32_t ring = smem0 + lay.ring + uint32_t(warp) * (R * 1024) + lane * 16;  // + (slot * 2 + row) * 512
    const uint32_t my_sz = smem0 + lay.sz + uint32_t(warp) * lay.sz_per_warp;
    const uint32_t xs = smem0 + lay.xs;      // + index * 16
    const uint32_t xsum = smem0 + lay.xsum;  // + index * 4
    const int XS = lay.xstride;

    // This block's tiles, and this warp's place among the tiles in work.
    const int t0 = int((int64_t(blockIdx.x) * a.tiles) / gridDim.x);
    const int t1 = int((int64_t(blockIdx.x + 1) * a.tiles) / gridDim.x);
    const bool works = warp < a.tpc * a.wpt;
    const int ts = warp / a.wpt, part = warp % a.wpt;
    const int steps = a.opc * KB;        // k-blocks of one task
    const int kbase = part * steps;      // first k-block of this warp's tasks
    int tile = t0 + ts;

    const uint8_t* rowp[2];
    auto set_rows = [&](int tl) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = min(tl * 16 + h * 8 + g, N - 1);  // ragged tile: clamp
            rowp[h] = a.packed + size_t(r) * (K / 2) + size_t(kbase) * 64 + t * 16;
        }
    };
    auto request = [&](int slot, int step) {  // both rows of k-block `step` -> ring slot
        if (step < steps) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t dst = ring + (slot * 2 + h) * 512;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(rowp[h] + size_t(step) * 64)
                             : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per step, empty past the end
    };
    // The task's scales ([16 rows][steps] x 2 B) and zero points ([16][steps] x 1 B) -> this
    // warp's part of shared memory, 4 bytes at a time: loads first (up to kSzWords words a
    // lane in registers), stores later.
    constexpr int kSzWords = 4;
    auto sz_word = [&](int tl, int i, bool store, uint32_t& v) {
        const int sw = steps / 2, zw = steps / 4;  // words per row
        if (i >= 16 * (sw + zw)) return;
        const bool is_zero = i >= 16 * sw;
        const int j = is_zero ? i - 16 * sw : i;
        const int per = is_zero ? zw : sw;
        const int row = j / per, word = j % per;
        if (!store) {
            const int r = min(tl * 16 + row, N - 1);
            const size_t at = size_t(r) * groups + kbase;  // element index of the row's first group
            v = is_zero ? __ldg(reinterpret_cast<const uint32_t*>(a.zero) + at / 4 + word)
                        : __ldg(reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(a.scale)) + at / 2 + word);
        } else {
            sts32(my_sz + (is_zero ? 16 * steps * 2 : 0) + j * 4, v);
        }
    };
    auto fetch_sz = [&](int tl) {  // load and store at once (tasks after the first)
        for (int i = lane; i < 16 * (steps / 2 + steps / 4); i += 32) {
            uint32_t v = 0;
            sz_word(tl, i, false, v);
            sz_word(tl, i, true, v);
        }
    };
    const bool sz_in_registers = 16 * (steps / 2 + steps / 4) <= 32 * kSzWords;

    // 1. Requests, in the order they should be served: (PRE ring slots, which may run ahead of
    //    the previous kernel in the stream;) the activations; the first task's scales and zero
    //    points; the rest of the ring.  Nothing loaded is touched before all of it is asked for.
    const bool has_task = works && tile < t1;
    uint32_t szr[kSzWords] = {0, 0, 0, 0};
    constexpr int kPre = R < PRE ? R : PRE;
    if (has_task) {
        set_rows(tile);
#pragma unroll
        for (int s = 0; s < kPre; ++s) request(s, s);
    }
    if (a.overlap) {
        if (a.early) pdl_launch_dependents();
        pdl_wait();  // activations may come from the kernel ahead of this one
    }

    // 2. Activations: M * (K / 128) * 16 pieces of 16 bytes, the 16 pieces of a (row, k-block)
    //    in 16 consecutive lanes, which also add up the k-block's inputs.
    {
        const uint4* xg = below_pdl_wait(static_cast<const uint4*>(a.x));
        const int pieces = M * groups * 16;
        const bool stager = SW == 0 || warp >= WARPS;
        const int threads = SW == 0 ? WARPS * 32 : SW * 32;
        const int me = SW == 0 ? int(threadIdx.x) : int(threadIdx.x) - WARPS * 32;  // among the staging threads
        auto where = [&](int e, int& m, int& j, int& c) {
            m = e / (groups * 16);
            const int rem = e - m * (groups * 16);
            j = rem / 16;
            c = rem % 16;  // piece of the k-block: lane t = c/4, word i = c%4
        };
        auto stage = [&](int e, const uint4& raw) {
            const bool live = e < pieces;
            int m, j, c;
            where(e, m, j, c);
            if (!EXACT) {
                float sum = (H::to_float(raw.x & 0xFFFFu) + H::to_float(raw.x >> 16)) +
                            (H::to_float(raw.y & 0xFFFFu) + H::to_float(raw.y >> 16));
                sum += (H::to_float(raw.z & 0xFFFFu) + H::to_float(raw.z >> 16)) +
                       (H::to_float(raw.w & 0xFFFFu) + H::to_float(raw.w >> 16));
#pragma unroll
                for (int d = 8; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
                if (live && c == 0) sts32f(xsum + (j * XS + m) * 4, sum);
            }
            if (live) {
                uint4 out;
                out.x = __byte_perm(raw.x, raw.z, 0x5410);  // (x0, x4)
                out.y = __byte_perm(raw.x, raw.z, 0x7632);  // (x1, x5)
                out.z = __byte_perm(raw.y, raw.w, 0x5410);  // (x2, x6)
                out.w = __byte_perm(raw.y, raw.w, 0x7632);  // (x3, x7)
                sts128(xs + (((j * 4 + (c % 4)) * M + m) * 4 + c / 4) * 16, out);
            }
        };
        auto load = [&](int e) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (e < pieces) {
                int m, j, c;
                where(e, m, j, c);
                raw = ld_mutable(xg + (size_t(m) * K + size_t(j) * 128) / 8 + c);
            }
            return raw;
        };
        // Up to kFirst pieces a thread are in flight at once: registers are plentiful before the
        // main loop (and all a staging warp needs).
        constexpr int kFirst = SW > 0 ? 8 : MB == 1 ? 5 : 10;
        uint4 raw[kFirst];
        if (stager) {
#pragma unroll
            for (int u = 0; u < kFirst; ++u) raw[u] = load(u * threads + me);
        }
        if (has_task) {
            if (sz_in_registers) {
#pragma unroll
                for (int u = 0; u < kSzWords; ++u) sz_word(tile, lane + 32 * u, false, szr[u]);
            }
#pragma unroll
            for (int s = kPre; s < R; ++s) request(s, s);  // the (rest of the) ring
        }
        if (stager) {
#pragma unroll
            for (int u = 0; u < kFirst; ++u)
                if (u * threads < pieces) stage(u * threads + me, raw[u]);
            for (int base = kFirst * threads; base < pieces; base += 4 * threads) {  // four loads in flight a thread
                uint4 more[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) more[u] = load(base + u * threads + me);
#pragma unroll
                for (int u = 0; u < 4; ++u) stage(base + u * threads + me, more[u]);
            }
        }
        if (has_task) {
            if (sz_in_registers) {
#pragma unroll
                for (int u = 0; u < kSzWords; ++u) sz_word(tile, lane + 32 * u, true, szr[u]);
            } else {
                fetch_sz(tile);
            }
        }
    }
    __syncthreads();
    if (!works) return;

    // 3. This warp's tasks: one tile each, `steps` k-blocks.
    const uint32_t kMask = 0x000F000Fu;
    uint16_t* y = static_cast<uint16_t*>(a.y);
    bool first_task = true;
    for (; tile < t1; tile += a.tpc) {
        if (!first_task) {
            set_rows(tile);
            fetch_sz(tile);
#pragma unroll
            for (int s = 0; s < R; ++s) request(s, s);
        }
        first_task = false;
        __syncwarp();  // the task's scales and zero points are in shared memory

        float acc[MB][2][4];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int s = 0; s < 2; ++s)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mb][s][i] = 0.0f;

        const uint32_t my_sc = my_sz + g * steps * 2, my_zp = my_sz + 16 * steps * 2 + g * steps;
        const uint32_t my_x = xs + (min(g, M - 1) * 4 + t) * 16;        // + ((kb * 4 + i) * M + mb * 8 rows) * 64
        const uint32_t my_xsum = xsum + min(2 * t, XS - 2) * 4;          // + (kb * XS + mb * 8) * 4
        int slot = 0;
#pragma unroll 1
        for (int j = 0; j < steps; ++j) {
            cp_async_wait_n<R - 1>();  // the oldest request of this lane has landed
            const uint4 q0 = lds128(ring + slot * 1024), q1 = lds128(ring + slot * 1024 + 512);
            const int kb = kbase + j;
            // scale and zero point of rows g and g+8 in this k-block
            uint32_t sbits[2], zbyte[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sbits[h]) : "r"(my_sc + (h * 8 * steps + j) * 2));
                asm volatile("ld.shared.u8 %0, [%1];" : "=r"(zbyte[h]) : "r"(my_zp + h * 8 * steps + j));
            }
            uint32_t sc[2] = {0, 0}, bias[2] = {0, 0};
            if (EXACT) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    sc[h] = sbits[h] * 0x00010001u;
                    bias[h] = H::kMagic + zbyte[h] * 0x00010001u;  // (magic + zero, magic + zero)
                }
            }
            float ka[MB][4];  // !EXACT: this k-block's sums
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 b[MB];
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    // rows past the last one re-read the last row: their columns are never stored
                    const uint32_t at = mb == 0 ? my_x : xs + (min(8 + g, M - 1) * 4 + t) * 16;
                    b[mb] = lds128(at + uint32_t((kb * 4 + i) * M) * 64);
                }
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
                    } else {
                        if (i == 0) mma_first<T>(ka[mb], a_lo, b[mb].x, b[mb].y);
                        else H::mma(ka[mb], a_lo, b[mb].x, b[mb].y);
                        H::mma(ka[mb], a_hi, b[mb].z, b[mb].w);
                    }
                }
            }
            if (!EXACT) {
                // y += scale * (sums - (magic + zero) * X), rows g (0, 1) and g+8 (2, 3)
                float s[2], nz[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    s[h] = H::to_float(sbits[h]);
                    // 2^23 + zero as f32 bits, then (2^23 - magic) - that = -(magic + zero)
                    nz[h] = (8388608.0f - H::kBias) - __uint_as_float(zbyte[h] | 0x4B000000u);
                }
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    const float2 X = lds64f(my_xsum + (kb * XS + mb * 8) * 4);
                    acc[mb][0][0] = fmaf(s[0], fmaf(nz[0], X.x, ka[mb][0]), acc[mb][0][0]);
                    acc[mb][0][1] = fmaf(s[0], fmaf(nz[0], X.y, ka[mb][1]), acc[mb][0][1]);
                    acc[mb][0][2] = fmaf(s[1], fmaf(nz[1], X.x, ka[mb][2]), acc[mb][0][2]);
                    acc[mb][0][3] = fmaf(s[1], fmaf(nz[1], X.y, ka[mb][3]), acc[mb][0][3]);
                }
            }
            request(slot, j + R);  // refill the slot just consumed
            slot = slot + 1 == R ? 0 : slot + 1;
        }
        const bool last_task = tile + a.tpc >= t1;
        if (last_task && a.overlap && !a.early) pdl_launch_dependents();

        // 4. The tile's partial sums meet in shared memory (each warp writes into its own, now
        //    idle, part of the ring); the tile's first warp adds them up and stores y.
        cp_async_wait_n<0>();
        const uint32_t red_of_tile = smem0 + lay.ring + uint32_t(ts * a.wpt) * (R * 1024);  // + warp-in-tile * R * 1024
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            const uint32_t dst = red_of_tile + uint32_t(part) * (R * 1024) + (g * MP + mb * 8 + 2 * t) * 4;
            sts32f(dst, acc[mb][0][0] + (EXACT ? acc[mb][1][0] : 0.0f));
            sts32f(dst + 4, acc[mb][0][1] + (EXACT ? acc[mb][1][1] : 0.0f));
            sts32f(dst + 8 * MP * 4, acc[mb][0][2] + (EXACT ? acc[mb][1][2] : 0.0f));
            sts32f(dst + 8 * MP * 4 + 4, acc[mb][0][3] + (EXACT ? acc[mb][1][3] : 0.0f));
        }
        if (a.wpt > 1) named_barrier(1 + ts, a.wpt * 32);
        else __syncwarp();
        if (part == 0) {
            for (int e = lane; e < 16 * M; e += 32) {
                const int row = e % 16, m = e / 16;
                float sum = 0.0f;
                for (int w = 0; w < a.wpt; ++w) sum += lds32f(red_of_tile + uint32_t(w) * (R * 1024) + (row * MP + m) * 4);
                const int n = tile * 16 + row;
                if (n < N) y[size_t(m) * N + n] = H::from_float(sum);
            }
        }
        if (!last_task) {  // the next task's requests overwrite the partial sums
            if (a.wpt > 1) named_barrier(1 + ts, a.wpt * 32);
            else __syncwarp();
        }
    }
}

// Launch geometry; false when the kernel does not take the shape.
template <int MB, int WARPS, int KB, int R>
inline bool sm_plan(SmArgs& a, int G, int sms, size_t* smem) {
    if (G != 128 || a.K % (128 * KB) != 0 || a.M > MB * 8) return false;
    if (!aligned(a.scale, 4) || !aligned(a.zero, 4)) return false;
    const int runs = a.K / (128 * KB);
    // as many warps per tile as there are runs, up to the block; else whole runs per warp
    int opc = 1;
    while (runs % opc != 0 || runs / opc > WARPS) ++opc;
    a.opc = opc;
    a.wpt = runs / opc;
    a.tpc = WARPS / a.wpt;
    if (a.wpt > 1 && a.tpc > 15) return false;  // named barriers 1..15
    if ((a.opc * KB) % 4 != 0) return false;
    const SmLayout l = sm_layout<MB, WARPS, KB, R>(a.M, a.K, a.opc);
    *smem = l.total;
    (void)sms;
    return l.total <= 226 * 1024;
}

template <typename T, int MB, int WARPS, int KB, int R, bool EXACT, int PRE = 0, int SW = 0>
int32_t launch_sm(const SmArgs& a, size_t smem, int sms, cudaStream_t stream) {
    auto kernel = int4_gemv_sm_kernel<T, MB, WARPS, KB, R, EXACT, PRE, SW>;
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
    config.blockDim = dim3((WARPS + SW) * 32, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = a.overlap ? 1 : 0;
    const cudaError_t err = cudaLaunchKernelEx(&config, kernel, a);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail("int4_gemv: launch failed: %s", cudaGetErrorString(err));
    }
    return B200Q_OK;
}

}  // namespace b200q
