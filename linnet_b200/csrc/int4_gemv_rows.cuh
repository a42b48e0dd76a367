// int4-g128 decode kernel for 3..64 activation rows (MB blocks of 8): the warps of a block take
// different 16-row tiles of W and the SAME inputs, so the activations are staged once
// per block in shared memory.
//
// With more than a couple of rows the per-lane activation loads of the oct kernel
// become its bottleneck (16 rows: 22 us, of which 11.6 us are those loads): every warp
// re-reads and re-permutes [rows x 1024] activations that its neighbours also need.
// Here a block of W warps owns W tiles and walks over OPC consecutive octs (1024 inputs
// each); for each oct the block's threads load the [rows x 1024] activations once,
// permute them to the (k, k+4) pairing of the A fragments and store them as B fragments
// (rows padded with zeros to 8 or 16, so no selects sit in the loop); every warp then
// reads its B fragments with conflict-free 16-byte shared-memory loads.  K is split over
// the blocks of a cluster (one block per OPC octs); the partial sums of a tile meet in
// distributed shared memory, every block adding up and writing its share of y.  Weight loads,
// dequantization and products are the oct kernel's.
#pragma once

#include "int4_gemv_oct.cuh"

namespace b200q {

struct RowsArgs {
    const void* x;          // [M, K]
    const uint8_t* packed;  // [N, K/2]
    const void* scale;      // [N, K/128]
    const uint8_t* zero;    // [N, K/128]
    void* y;                // [M, N]
    int M, K, N;
    int tiles;              // ceil(N / 16)
    int opc;                // octs per block
    int ksplit;             // blocks per cluster = K / (1024 * opc)
};

template <typename T, int MB, int W, int D>
__global__ void __launch_bounds__(W * 32, MB <= 2 ? 28 / W : 1)  // more rows: more accumulators a thread
int4_gemv_rows_kernel(const RowsArgs a) {
    using H = Half16<T>;
    constexpr int MP = MB * 8;  // activation rows as staged (zero padded)
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
    const int M = a.M, K = a.K, N = a.N;
    const int groups = K / 128;
    const int tile = min(int(blockIdx.x) * W + warp, a.tiles - 1);  // surplus warps redo the last tile
    const bool owns = int(blockIdx.x) * W + warp < a.tiles;
    const int tile_row = tile * 16;

    // Shared memory: B fragments of one oct [8 k-blocks][4 words][MP rows][4 lanes] x 16 B,
    // then the block's partial sums [W][16][MP] f32 (same offset in every block).
    uint4* xs = reinterpret_cast<uint4*>(smem);
    float* red = reinterpret_cast<float*>(smem + size_t(8) * 4 * MP * 4 * 16);

    const uint8_t* rowp[2];
    size_t srow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = min(tile_row + h * 8 + g, N - 1);  // ragged tile: clamp
        rowp[h] = a.packed + size_t(r) * (K / 2) + t * 16;
        srow[h] = size_t(r) * groups;
    }

    float acc[MB][2][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mb][s][i] = 0.0f;

    const uint32_t kMask = 0x000F000Fu;
    for (int o = 0; o < a.opc; ++o) {
        const int oct = int(blockIdx.y) * a.opc + o;
        // 1. Weight loads of this oct first, and its 8 scales / zero points per row.
        uint4 st[D][2];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            st[d][0] = ldg_stream(rowp[0] + size_t(oct) * 512 + d * 64);
            st[d][1] = ldg_stream(rowp[1] + size_t(oct) * 512 + d * 64);
        }
        uint4 s8[2];
        uint2 z8[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const size_t at = srow[h] + size_t(oct) * 8;
            s8[h] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.scale) + at));
            z8[h] = __ldg(reinterpret_cast<const uint2*>(a.zero + at));
        }
        if (o == 0) {
            pdl_launch_dependents();
            pdl_wait();  // activations may come from the kernel before this one
        } else {
            __syncthreads();  // every warp is done with the previous oct's fragments
        }
        // 2. Stage the activations of this oct: MP x 128 pieces of 16 bytes.
        {
            const uint4* xg = static_cast<const uint4*>(a.x);
            constexpr int kPieces = MP * 128;
            constexpr int kPerThread = (kPieces + W * 32 - 1) / (W * 32);
            constexpr int kBatch = kPerThread < 8 ? kPerThread : 8;
            for (int p0 = 0; p0 < kPerThread; p0 += kBatch) {
                uint4 raw[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int e = (p0 + u) * (W * 32) + threadIdx.x;
                    const int m = e / 128, piece = e % 128;
                    raw[u] = make_uint4(0, 0, 0, 0);
                    if (e < kPieces && m < M)
                        raw[u] = ld_mutable(xg + (size_t(m) * K + size_t(oct) * 1024) / 8 + piece);
                }
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int e = (p0 + u) * (W * 32) + threadIdx.x;
                    if (e < kPieces) {
                        const int m = e / 128, piece = e % 128;
                        const int j = piece / 16, c = piece % 16;  // k-block, chunk: lane t = c/4, word i = c%4
                        uint4 out;
                        out.x = __byte_perm(raw[u].x, raw[u].z, 0x5410);  // (x0, x4)
                        out.y = __byte_perm(raw[u].x, raw[u].z, 0x7632);  // (x1, x5)
                        out.z = __byte_perm(raw[u].y, raw[u].w, 0x5410);  // (x2, x6)
                        out.w = __byte_perm(raw[u].y, raw[u].w, 0x7632);  // (x3, x7)
                        xs[((j * 4 + (c % 4)) * MP + m) * 4 + c / 4] = out;
                    }
                }
            }
        }
        __syncthreads();

        // 3. The oct's 8 k-blocks.
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint4 q0 = st[j % D][0], q1 = st[j % D][1];
            if (j + D < 8) {
                st[j % D][0] = ldg_stream(rowp[0] + size_t(oct) * 512 + (j + D) * 64);
                st[j % D][1] = ldg_stream(rowp[1] + size_t(oct) * 512 + (j + D) * 64);
            }
            uint32_t sc[2], bias[2];
            const uint32_t zsel = 0x7070u | uint32_t(j & 3) | (uint32_t(j & 3) << 8);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t sw = j < 2 ? s8[h].x : j < 4 ? s8[h].y : j < 6 ? s8[h].z : s8[h].w;
                sc[h] = __byte_perm(sw, 0, (j & 1) ? 0x3232 : 0x1010);
                bias[h] = __byte_perm(j < 4 ? z8[h].x : z8[h].y, H::kMagic, zsel);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 b[MB];
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) b[mb] = xs[((j * 4 + i) * MP + mb * 8 + g) * 4 + t];
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
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    f0[e] = sub_mul<T>(f0[e], bias[0], sc[0]);
                    f1[e] = sub_mul<T>(f1[e], bias[1], sc[1]);
                }
                const uint32_t a_lo[4] = {f0[0], f1[0], f0[1], f1[1]};
                const uint32_t a_hi[4] = {f0[2], f1[2], f0[3], f1[3]};
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    H::mma(acc[mb][0], a_lo, b[mb].x, b[mb].y);
                    H::mma(acc[mb][1], a_hi, b[mb].z, b[mb].w);
                }
            }
        }
    }

    // 4. Partial sums of this block's tiles -> shared memory.
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        float* dst = red + (size_t(warp) * 16 + g) * MP + mb * 8 + 2 * t;
        dst[0] = acc[mb][0][0] + acc[mb][1][0];
        dst[1] = acc[mb][0][1] + acc[mb][1][1];
        dst[8 * MP] = acc[mb][0][2] + acc[mb][1][2];
        dst[8 * MP + 1] = acc[mb][0][3] + acc[mb][1][3];
    }
    // Every block of the cluster sums and writes its share of the tile elements (the
    // other blocks' partial sums are read through distributed shared memory, all loads
    // of an element issued before the adds), so the tail is as parallel as the cluster.
    uint16_t* y = static_cast<uint16_t*>(a.y);
    constexpr int kElems = W * 16 * MP;
    if (a.ksplit > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int rank = int(cluster.block_rank());
        const float* peers[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) peers[r] = cluster.map_shared_rank(red, r < a.ksplit ? r : 0);
        for (int e = rank * (W * 32) + threadIdx.x; e < kElems; e += a.ksplit * W * 32) {
            float v[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) v[r] = r < a.ksplit ? peers[r][e] : 0.0f;
            const float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
            const int m = e % MP, r16 = e / MP;  // red is [warp * 16 + row][MP]
            const int n = int(blockIdx.x) * W * 16 + r16;
            if (m < M && n < N && int(blockIdx.x) * W + r16 / 16 < a.tiles)
                y[size_t(m) * N + n] = H::from_float(sum);
        }
        cluster.sync();  // nobody leaves while a peer may still read its partial sums
        return;
    }
    __syncthreads();
    // red is [warp][row][col]; y is [m][n]: rows fastest so stores coalesce.
    for (int e = threadIdx.x; e < kElems; e += W * 32) {
        const int m = e / (W * 16), r = e % (W * 16);  // r = warp * 16 + row of the tile
        const int n = int(blockIdx.x) * W * 16 + r;
        if (m < M && n < N && int(blockIdx.x) * W + r / 16 < a.tiles)
            y[size_t(m) * N + n] = H::from_float(red[size_t(r) * MP + m]);
    }
    (void)owns;
}

// Launch geometry for the rows kernel: W warps (tiles) per block, OPC octs per block so
// that the cluster has at most 8 blocks; false when the shape does not fit.
template <typename T, int MB, int W, int D>
int32_t launch_rows(RowsArgs a, cudaStream_t stream) {
    const size_t smem = size_t(8) * 4 * (MB * 8) * 4 * 16 + size_t(W) * 16 * (MB * 8) * 4;
    const int blocks = (a.tiles + W - 1) / W;
    return launch_clustered("int4_gemv", int4_gemv_rows_kernel<T, MB, W, D>, a, blocks, a.ksplit, W * 32,
                            smem, stream, true);
}

}  // namespace b200q
