// The fast int4-g128 decode kernel: every warp owns one "oct" -- 8 consecutive
// k-blocks (1024 inputs, 512 weight bytes per row) -- of NT 16-row tiles.
//
// It is the kernel of int4_gemv.cu specialised for group == 128 and K a multiple of
// 1024 so that everything indexed by the k-block is a compile-time constant:
//   * the oct's 8 scales (one 16-byte load) and 8 zero points (one 8-byte load) of a
//     row arrive with the first weight loads; one PRMT each turns them into the
//     (scale, scale) and (magic + zero, magic + zero) pairs of a k-block;
//   * the 8 * NT k-block steps are fully unrolled around a D-deep register pipeline
//     of 16-byte weight loads (L1-bypassing, straight into A-fragment position);
//   * activations are not staged at all: each lane reads the 16 bytes of its
//     activation row it needs for a pair of products straight from global memory
//     (they stay in L1, which the weight loads bypass) and permutes them with four
//     PRMTs to the (k, k+4) pairing of the A fragments; every B fragment is used
//     exactly once per warp, so a shared-memory copy would only add traffic;
//   * two accumulator sets alternate to halve the tensor-core dependency chains.
// Dequantization is the reference's arithmetic exactly: (magic + q) - (magic + zero)
// is the integer q - zero, and one multiply by the scale rounds once to the 16-bit
// type.  Per k-block and 16-row tile that is 56 LOP3/SHF + 64 HSUB2/HMUL2 + 8 MMA.
// This is the kernel behind B200Q_EXACT_WEIGHTS; int4_gemv_post.cuh is the default.
#pragma once

#include "gemv_common.cuh"

namespace b200q {

struct OctArgs {
    const void* x;          // [M, K]
    const uint8_t* packed;  // [N, K/2]
    const void* scale;      // [N, K/128]
    const uint8_t* zero;    // [N, K/128]
    void* y;                // [M, N]
    int M, K, N;
    int ksplit;             // blocks per cluster; K == 128 * KB * W * ksplit
    int overlap;            // launched with programmatic stream serialization
    int early;              // dependents may start as soon as this kernel has started
};

// Waits until at most `pending` of this thread's cp.async groups are in flight
// (`pending` is a constant once the caller's loop is unrolled).
__device__ __forceinline__ void cp_async_wait(int pending) {
    switch (pending) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    }
}

// D > 0: a D-deep register pipeline of weight loads.  D == 0 ("deep", NT == 1): the
// first k-block is loaded into registers and the other seven are requested at once
// with cp.async into lane-private shared-memory slots (each lane later reads back
// exactly the 16-byte pieces it asked for, so a wait_group is all the synchronisation
// needed): the whole weight matrix is in flight from the first cycles of the kernel
// and the arithmetic never waits on a load it has not long since issued.
// KB: k-blocks per warp (8 = an oct; 4 or 2 for small problems, where a warp's serial run
// through 8 k-blocks -- 1,500 instructions, ~2.7 us -- is the whole kernel time and most
// multiprocessors hold only a few warps: shorter runs, proportionally more warps).
// The activations are read with ordinary coherent loads (ld.global.ca).  The read-only path
// (__ldg) is about 1 us faster on the headline shape but is not safe here: launched
// programmatically inside a CUDA graph, kernels do not get that cache invalidated between
// them, and a decode step that reuses an address for a new activation tensor was served the
// old tensor's lines (found by replaying a captured step against its eager result).
// OctArgs::early: when the kernels that depend on this one may start (programmatic dependent
// launch).
//   0: after the last k-block.  Inside a decode step this is the faster order: a
//     dependent that starts early (the attention kernel with its 96-192 KB of shared memory,
//     say) only takes shared memory and warp slots from this kernel while it waits.
//   1: at once, so that a following product overlaps its weight prefetch with this
//     kernel's arithmetic (1.4 us per launch in a chain of products on the headline shape).
template <typename T, int MB, int NT, int W, int D, int KB = 8>
__global__ void __launch_bounds__(W * 32, ((NT == 1 ? 28 : 20) / W) > 0 ? (NT == 1 ? 28 : 20) / W : 1)
int4_gemv_oct_kernel(const OctArgs a) {
    static_assert(D > 0 || NT == 1, "the deep variant handles one tile per warp");
    static_assert(KB == 8 || KB == 4 || KB == 2, "k-blocks per warp");
    using H = Half16<T>;
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
    const int M = a.M, K = a.K, N = a.N;
    const int groups = K / 128;
    const int tile_row = blockIdx.x * (16 * NT);
    const int kb0 = (blockIdx.y * W + warp) * KB;  // this warp's first k-block along K

    // Shared memory: the block's reduction buffer, then (deep variant) each lane's
    // private slots [KB - 1 k-blocks][2 rows] x 16 B, laid out [slot][lane] per warp.
    float* red = reinterpret_cast<float*>(smem);
    uint4* slots = reinterpret_cast<uint4*>(smem + size_t(W) * NT * 16 * MB * 8 * 4) +
                   size_t(warp) * ((KB - 1) * 2 * 32) + lane;

    const uint8_t* rowp[NT][2];
    uint4 s8[NT][2];
    uint2 z8[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = min(tile_row + nt * 16 + h * 8 + g, N - 1);  // ragged tile: clamp
            rowp[nt][h] = a.packed + size_t(r) * (K / 2) + size_t(kb0) * 64 + t * 16;
        }

    // One pipeline step is one k-block of all NT tiles (2 * NT 16-byte loads a lane).
    uint4 st[D > 0 ? D : 1][NT][2];
    auto load_step = [&](int slot, int j) {  // compile-time arguments after unrolling
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            st[slot][nt][0] = ldg_stream(rowp[nt][0] + j * 64);
            st[slot][nt][1] = ldg_stream(rowp[nt][1] + j * 64);
        }
    };

    // 1. Weight loads first: they do not depend on the previous kernel.
    if (D > 0) {
#pragma unroll
        for (int d = 0; d < D; ++d)
            if (d < KB) load_step(d, d);
    } else {
        load_step(0, 0);
#pragma unroll
        for (int j = 1; j < KB; ++j) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t dst = uint32_t(__cvta_generic_to_shared(slots + ((j - 1) * 2 + h) * 32));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(rowp[0][h] + j * 64) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = min(tile_row + nt * 16 + h * 8 + g, N - 1);
            const size_t at = size_t(r) * groups + size_t(kb0);
            const uint16_t* sp = static_cast<const uint16_t*>(a.scale) + at;
            s8[nt][h] = make_uint4(0, 0, 0, 0);
            z8[nt][h] = make_uint2(0, 0);
            if (KB == 8) {
                s8[nt][h] = __ldg(reinterpret_cast<const uint4*>(sp));
                z8[nt][h] = __ldg(reinterpret_cast<const uint2*>(a.zero + at));
            } else if (KB == 4) {
                const uint2 s4 = __ldg(reinterpret_cast<const uint2*>(sp));
                s8[nt][h].x = s4.x;
                s8[nt][h].y = s4.y;
                z8[nt][h].x = __ldg(reinterpret_cast<const uint32_t*>(a.zero + at));
            } else {
                s8[nt][h].x = __ldg(reinterpret_cast<const uint32_t*>(sp));
                z8[nt][h].x = uint32_t(__ldg(reinterpret_cast<const uint16_t*>(a.zero + at)));
            }
        }
    if (a.overlap) {
        if (a.early) pdl_launch_dependents();
        pdl_wait();  // activations may come from the kernel before this one
    }

    // 2. This lane's activations: row mb*8 + g, inputs kb0*128 + j*128 + t*32 + i*8 ...
    // Lanes past the last row read the last row again: their columns of the product are
    // never stored, and an unconditional load needs no zeroed registers and no predicate.
    const uint4* xp[MB];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        const int m = min(mb * 8 + g, M - 1);
        xp[mb] = below_pdl_wait(static_cast<const uint4*>(a.x)) + (size_t(m) * K + size_t(kb0) * 128 + t * 32) / 8;
    }

    // 3. The KB * NT steps, fully unrolled.
    float acc[NT][MB][2][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int s = 0; s < 2; ++s)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[nt][mb][s][i] = 0.0f;

    const uint32_t kMask = 0x000F000Fu;
#pragma unroll
    for (int j = 0; j < KB; ++j) {
        uint4 q[NT][2];
        if (D > 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                q[nt][0] = st[j % (D > 0 ? D : 1)][nt][0];
                q[nt][1] = st[j % (D > 0 ? D : 1)][nt][1];
            }
            if (j + D < KB) load_step(j % (D > 0 ? D : 1), j + D);
        } else if (j == 0) {
            q[0][0] = st[0][0][0];
            q[0][1] = st[0][0][1];
        } else {
            cp_async_wait(KB - 1 - j);
            q[0][0] = slots[((j - 1) * 2 + 0) * 32];
            q[0][1] = slots[((j - 1) * 2 + 1) * 32];
        }
        // (scale, scale) and (magic + zero, magic + zero) of rows g and g+8, k-block j.
        uint32_t sc[NT][2], bias[NT][2];
        // bytes [zero, high byte of magic, zero, high byte of magic]
        const uint32_t zsel = 0x7070u | uint32_t(j & 3) | (uint32_t(j & 3) << 8);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 s = s8[nt][h];
                const uint32_t sw = j < 2 ? s.x : j < 4 ? s.y : j < 6 ? s.z : s.w;
                sc[nt][h] = __byte_perm(sw, 0, (j & 1) ? 0x3232 : 0x1010);
                bias[nt][h] = __byte_perm(j < 4 ? z8[nt][h].x : z8[nt][h].y, H::kMagic, zsel);
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 b[MB];  // (x0,x4) (x1,x5) (x2,x6) (x3,x7) of this lane's 8 inputs
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const uint4 raw = ld_activation_free(xp[mb] + j * 16 + i);
                b[mb].x = __byte_perm(raw.x, raw.z, 0x5410);
                b[mb].y = __byte_perm(raw.x, raw.z, 0x7632);
                b[mb].z = __byte_perm(raw.y, raw.w, 0x5410);
                b[mb].w = __byte_perm(raw.y, raw.w, 0x7632);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t w0 = i == 0 ? q[nt][0].x : i == 1 ? q[nt][0].y : i == 2 ? q[nt][0].z : q[nt][0].w;
                const uint32_t w1 = i == 0 ? q[nt][1].x : i == 1 ? q[nt][1].y : i == 2 ? q[nt][1].z : q[nt][1].w;
                uint32_t f0[4], f1[4];  // (k0,k4) (k1,k5) (k2,k6) (k3,k7) of rows g, g+8
                f0[0] = lop3_and_or(w0, kMask, H::kMagic);
                f0[1] = lop3_and_or(w0 >> 4, kMask, H::kMagic);
                f0[2] = lop3_and_or(w0 >> 8, kMask, H::kMagic);
                f0[3] = lop3_and_or(w0 >> 12, kMask, H::kMagic);
                f1[0] = lop3_and_or(w1, kMask, H::kMagic);
                f1[1] = lop3_and_or(w1 >> 4, kMask, H::kMagic);
                f1[2] = lop3_and_or(w1 >> 8, kMask, H::kMagic);
                f1[3] = lop3_and_or(w1 >> 12, kMask, H::kMagic);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    f0[e] = sub_mul<T>(f0[e], bias[nt][0], sc[nt][0]);
                    f1[e] = sub_mul<T>(f1[e], bias[nt][1], sc[nt][1]);
                }
                const uint32_t a_lo[4] = {f0[0], f1[0], f0[1], f1[1]};
                const uint32_t a_hi[4] = {f0[2], f1[2], f0[3], f1[3]};
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    H::mma(acc[nt][mb][0], a_lo, b[mb].x, b[mb].y);
                    H::mma(acc[nt][mb][1], a_hi, b[mb].z, b[mb].w);
                }
            }
        }
    }

    if (a.overlap && !a.early) pdl_launch_dependents();
    // 4. Sum the two accumulator sets, the warps, the cluster; write y.
    float total[NT][MB][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 4; ++i) total[nt][mb][i] = acc[nt][mb][0][i] + acc[nt][mb][1][i];
    reduce_and_store<H, MB, NT, W>(total, red, a.ksplit, tile_row, M, N, static_cast<uint16_t*>(a.y));
}

// Whether the oct kernel takes this problem with W warps per block and KB k-blocks per
// warp; sets ksplit.
inline bool oct_plan(int K, int G, int W, const void* scale, const uint8_t* zero, int* ksplit, int KB = 8) {
    if (G != 128 || K % (128 * KB) != 0) return false;
    const int runs = K / (128 * KB);
    if (runs % W != 0 || runs / W > 8) return false;
    if (!aligned(scale, 16) || !aligned(zero, 8)) return false;
    *ksplit = runs / W;
    return true;
}

template <typename T, int MB, int NT, int W, int D, int KB = 8>
int32_t launch_oct(const OctArgs& args, cudaStream_t stream) {
    const int tiles = (args.N + 16 * NT - 1) / (16 * NT);
    const size_t smem = size_t(W) * NT * 16 * MB * 8 * 4 + (D == 0 ? size_t(W) * (KB - 1) * 2 * 32 * 16 : 0);
    auto kernel = int4_gemv_oct_kernel<T, MB, NT, W, D, KB>;
    if (D == 0 && first_use_on_device(reinterpret_cast<const void*>(kernel)))
        // 7 blocks of 30 KB per multiprocessor need the largest carve-out
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    return launch_clustered("int4_gemv", kernel, args, tiles, args.ksplit, W * 32, smem, stream,
                            args.overlap != 0);
}

}  // namespace b200q
