// int8 per-channel decode kernel for one or two activation rows: the structure of the int4
// kernel of int4_gemv_tma.cuh (one block per multiprocessor, the weights brought by the TMA
// unit into a ring of shared-memory stages, a producer thread, consumer warps that never issue
// a weight load) with each weight byte taken as two 4-bit planes.
//
//   u = w + 128 = 16 h + l  (one XOR per word makes the byte unsigned)
//   y[m, n] = scale[n] * ( sum_k x[m, k] (magic + l[n, k]) + sum_k 16 x[m, k] (magic + h[n, k])
//                          - (17 magic + 128) X[m] ),      X[m] = sum_k x[m, k]
//
// magic + nibble (128 + q in bf16, 1024 + q in f16) is what one LOP3 makes of a pair of nibbles,
// and it is exact; 16 x is exact in the 16-bit type (a power of two); the products are exact in
// f32.  So the same seven integer instructions a 32-bit word that unpack eight int4 weights
// unpack four int8 weights here, and the kernel streams int8 bytes at the rate the int4 kernel
// streams int4 bytes.  The per-row scale multiplies the finished sum, as in the kernel this one
// relieves for one and two rows (int8_gemv.cu), and as linnet::gemv8 does
// (python/linnet/src/linnet/torch/kernels.py:336-434).
//
// A k-block is 64 inputs (64 bytes of a row); an item is 16 rows x KB k-blocks, one 3-D TMA
// box landing as [KB][16 rows][64 bytes].  The activations are staged once per block as B
// fragments: for the four inputs of a word, (x0, x2), 16 (x0, x2), (x1, x3), 16 (x1, x3).
#pragma once

#include <cuda.h>

#include "tma_ring.cuh"

namespace b200q {

struct Tma8Args {
    const void* x;       // [M, K]
    const float* scale;  // [N]
    void* y;             // [M, N]
    int M, K, N;
    int tiles;           // ceil(N / 16)
    int wpt;             // warps per tile
    int opc;             // items per warp and tile; K == 64 * KB * opc * wpt
    int tpc;             // tiles in work at a time per block = WARPS / wpt
    int stages;          // ring stages of KB KiB
    int overlap;         // launched with programmatic stream serialization
    int early;           // dependents may start as soon as this kernel has started
    int* status;         // device word of expired waits
};

struct Tma8Layout {
    uint32_t bars, xs, xsum, total;
    uint32_t xrow;  // bytes of one activation row in xs
    int xpairs;     // pairs of rows in xsum
};
template <int WARPS, int KB>
__host__ __device__ inline Tma8Layout tma8_layout(int M, int K, int stages) {
    Tma8Layout l;
    const int kblocks = K / 64;
    l.bars = uint32_t(stages) * (KB * 1024);
    l.xs = (l.bars + uint32_t(stages + 2 * WARPS) * 8 + 127u) & ~127u;
    l.xrow = uint32_t(kblocks) * 256 + (M > 1 ? 64 : 0);
    l.xpairs = (M + 1) / 2;
    l.xsum = l.xs + uint32_t(M) * l.xrow;
    l.total = l.xsum + uint32_t(l.xpairs) * kblocks * 8;
    return l;
}

template <typename T, int WARPS, int KB>
__global__ void __launch_bounds__((WARPS + 1) * 32, 1)
int8_gemv_tma_kernel(const __grid_constant__ CUtensorMap wmap, const Tma8Args a) {
    using H = Half16<T>;
    using P = typename H::pair;
    constexpr int MP = 8;
    constexpr uint32_t kItem = KB * 1024;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
    const int M = a.M, K = a.K, N = a.N;
    const int kblocks = K / 64;
    const int S = a.stages;
    const Tma8Layout lay = tma8_layout<WARPS, KB>(M, K, S);
    const uint32_t smem0 = uint32_t(__cvta_generic_to_shared(smem));
    // empty[s], ready[w], taken[w]: see int4_gemv_tma.cuh
    const uint32_t empty0 = smem0 + lay.bars, ready0 = empty0 + uint32_t(S) * 8, taken0 = ready0 + WARPS * 8;

    const int t0 = int((uint32_t(blockIdx.x) * uint32_t(a.tiles)) / gridDim.x);
    const int t1 = int((uint32_t(blockIdx.x + 1) * uint32_t(a.tiles)) / gridDim.x);
    const int active = a.tpc * a.wpt;
    const int rounds = (t1 - t0 + a.tpc - 1) / a.tpc;

    if (int(threadIdx.x) < S + 2 * WARPS) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(empty0 + threadIdx.x * 8));
        umma::fence_proxy_async();
    }
    __syncthreads();

    if (warp == WARPS) {
        // ---- producer: items in the order (round, item of the tile, consumer) ----------------
        if (lane != 0) return;
        if (a.overlap) pdl_launch_dependents();  // this thread never waits on the previous kernel: weights are constants
        int s = 0;
        uint32_t lap = 0;
        bool ok = true;
        int n = 0;
        for (int round = 0; round < rounds && ok; ++round) {
            const int tiles_here = min(a.tpc, t1 - t0 - round * a.tpc);
            for (int o = 0; o < a.opc && ok; ++o, ++n) {
                int w = 0;
                for (int ts = 0; ts < tiles_here && ok; ++ts) {
                    const int tile = t0 + round * a.tpc + ts;
                    for (int part = 0; part < a.wpt; ++part, ++w) {
                        const uint32_t empty = empty0 + s * 8, ready = ready0 + w * 8;
                        if (lap > 0) ok = bar_wait<true>(empty, (lap - 1) & 1, a.status, 21);
                        if (ok && n > 0) ok = bar_wait<true>(taken0 + w * 8, (n - 1) & 1, a.status, 23);
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
    const uint32_t xs = smem0 + lay.xs, xsum = smem0 + lay.xsum;

    if (a.overlap) {
        if (a.early) pdl_launch_dependents();
        pdl_wait();  // activations may come from the kernel ahead of this one
    }

    // Activations: M * (K / 8) pieces of 16 bytes (8 inputs), the 8 pieces of a (row, k-block) in
    // 8 consecutive lanes, which also add up the k-block's inputs.
    {
        const uint4* xg = below_pdl_wait(static_cast<const uint4*>(a.x));
        const int pieces = M * kblocks * 8;
        constexpr int threads = WARPS * 32;
        const uint32_t sixteen_bits = H::pack(16.0f, 16.0f);
        const P sixteen = *reinterpret_cast<const P*>(&sixteen_bits);
        for (int base = 0; base < pieces; base += 4 * threads) {  // four loads in flight a thread
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = base + u * threads + int(threadIdx.x);
                raw[u] = make_uint4(0, 0, 0, 0);
                if (e < pieces) {
                    const int r = e >> 3, c = e & 7;
                    const int m = M == 1 ? 0 : r / kblocks, j = r - m * kblocks;
                    raw[u] = ld_mutable(xg + (size_t(m) * K + size_t(j) * 64) / 8 + c);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = base + u * threads + int(threadIdx.x);
                const bool live = e < pieces;
                const int r = e >> 3, c = e & 7;
                const int m = M == 1 ? 0 : r / kblocks, j = r - m * kblocks;
                float sum = (H::to_float(raw[u].x & 0xFFFFu) + H::to_float(raw[u].x >> 16)) +
                            (H::to_float(raw[u].y & 0xFFFFu) + H::to_float(raw[u].y >> 16));
                sum += (H::to_float(raw[u].z & 0xFFFFu) + H::to_float(raw[u].z >> 16)) +
                       (H::to_float(raw[u].w & 0xFFFFu) + H::to_float(raw[u].w >> 16));
#pragma unroll
                for (int d = 4; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
                if (live && c == 0) sts32f(xsum + (uint32_t(m / 2) * kblocks + j) * 8 + (m % 2) * 4, sum);
                if (live) {
                    // piece c: inputs 8c .. 8c+7 of the k-block, the words i = 2 (c % 2) and + 1 of lane t = c / 2
                    const uint32_t dst = xs + uint32_t(m) * lay.xrow + uint32_t(j) * 256 + (2 * (c & 1)) * 64 + (c >> 1) * 16;
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const uint32_t lo = hh == 0 ? raw[u].x : raw[u].z, hi = hh == 0 ? raw[u].y : raw[u].w;
                        uint4 out;
                        out.x = __byte_perm(lo, hi, 0x5410);  // (x0, x2)
                        out.z = __byte_perm(lo, hi, 0x7632);  // (x1, x3)
                        P p02 = __hmul2(*reinterpret_cast<P*>(&out.x), sixteen), p13 = __hmul2(*reinterpret_cast<P*>(&out.z), sixteen);
                        out.y = *reinterpret_cast<uint32_t*>(&p02);
                        out.w = *reinterpret_cast<uint32_t*>(&p13);
                        sts128(dst + hh * 64, out);
                    }
                }
            }
        }
    }
    named_barrier(15, WARPS * 32);  // the consumers only: the producer is on its own way
    if (!works) return;

    // ---- this warp's items --------------------------------------------------------------------
    const uint32_t kMask = 0x000F000Fu;
    const float kCorrection = 17.0f * H::kBias + 128.0f;  // what the magic and the +128 of the bytes add per unit of X
    uint16_t* y = static_cast<uint16_t*>(a.y);
    const uint32_t wl = uint32_t(g) * 64 + t * 16;  // this lane's bytes of a k-block's row g
    const uint32_t x_lane = xs + uint32_t(min(g, M - 1)) * lay.xrow + t * 16;
    const uint32_t xsum_lane = xsum + uint32_t(min(t, lay.xpairs - 1)) * kblocks * 8;
    bool ok = true;
    int n = 0;
    int s = warp % S;
    const int s_step = active % S;
    const int s_last = (min(a.tpc, t1 - t0 - (rounds - 1) * a.tpc) * a.wpt) % S;
    const uint32_t ready = ready0 + warp * 8;
    for (int tile = t0 + ts; tile < t1; tile += a.tpc) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint32_t stage_addr = 0;
        int s_mine = 0;
        for (int o = 0; o < a.opc; ++o, ++n) {
            const int item = part * a.opc + o;
            s_mine = s;
            s += tile + a.tpc >= t1 ? s_last : s_step;
            if (s >= S) s -= S;
            stage_addr = smem0 + uint32_t(s_mine) * kItem;
            if (ok) ok = bar_wait(ready, uint32_t(n) & 1, a.status, 22);
            __syncwarp();  // every lane has seen the phase
            if (lane == 0) bar_arrive(taken0 + warp * 8);
            const uint32_t wq = stage_addr + wl;
            const uint32_t xq = x_lane + uint32_t(item) * (KB * 256);
            const uint32_t xsq = xsum_lane + uint32_t(item) * (KB * 8);
#pragma unroll
            for (int j = 0; j < KB; ++j) {
                const uint4 q0 = lds128(wq + j * 1024), q1 = lds128(wq + j * 1024 + 512);
                float ka[4], kb[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 b = lds128(xq + j * 256 + i * 64);
                    const uint32_t w0 = (i == 0 ? q0.x : i == 1 ? q0.y : i == 2 ? q0.z : q0.w) ^ 0x80808080u;
                    const uint32_t w1 = (i == 0 ? q1.x : i == 1 ? q1.y : i == 2 ? q1.z : q1.w) ^ 0x80808080u;
                    uint32_t f0[4], f1[4];  // (l0, l2) (h0, h2) (l1, l3) (h1, h3) of rows g, g+8
                    f0[0] = lop3_and_or(w0, kMask, H::kMagic);
                    f0[1] = lop3_and_or(w0 >> 4, kMask, H::kMagic);
                    f0[2] = lop3_and_or(w0 >> 8, kMask, H::kMagic);
                    f0[3] = lop3_and_or(w0 >> 12, kMask, H::kMagic);
                    f1[0] = lop3_and_or(w1, kMask, H::kMagic);
                    f1[1] = lop3_and_or(w1 >> 4, kMask, H::kMagic);
                    f1[2] = lop3_and_or(w1 >> 8, kMask, H::kMagic);
                    f1[3] = lop3_and_or(w1 >> 12, kMask, H::kMagic);
                    const uint32_t a_lo[4] = {f0[0], f1[0], f0[1], f1[1]};
                    const uint32_t a_hi[4] = {f0[2], f1[2], f0[3], f1[3]};
                    if (i == 0) {
                        mma_first<T>(ka, a_lo, b.x, b.y);
                        mma_first<T>(kb, a_hi, b.z, b.w);
                    } else {
                        H::mma(ka, a_lo, b.x, b.y);
                        H::mma(kb, a_hi, b.z, b.w);
                    }
                }
                const float2 X = lds64f(xsq + j * 8);
                acc[0] += fmaf(-kCorrection, X.x, ka[0] + kb[0]);
                acc[1] += fmaf(-kCorrection, X.y, ka[1] + kb[1]);
                acc[2] += fmaf(-kCorrection, X.x, ka[2] + kb[2]);
                acc[3] += fmaf(-kCorrection, X.y, ka[3] + kb[3]);
            }
            if (o + 1 < a.opc) {  // hand the stage back; the tile's last one carries the partial sums first
                __syncwarp();
                if (lane == 0) bar_arrive(empty0 + s_mine * 8);
            }
        }
        const bool last_tile = tile + a.tpc >= t1;
        if (last_tile && a.overlap && !a.early) pdl_launch_dependents();

        // The tile's partial sums meet in the stages its warps have just read; the tile's first
        // warp adds them up, applies the rows' scales, stores y and hands the stages back.
        __syncwarp();
        {
            const uint32_t dst = stage_addr + (g * MP + 2 * t) * 4;
            sts32f(dst, acc[0]);
            sts32f(dst + 4, acc[1]);
            sts32f(dst + 8 * MP * 4, acc[2]);
            sts32f(dst + 8 * MP * 4 + 4, acc[3]);
        }
        umma::fence_proxy_async();  // these writes come before the TMA unit's next ones to the stage
        if (a.wpt > 1) named_barrier(1 + ts, a.wpt * 32);
        else __syncwarp();
        if (part == 0) {
            for (int e = lane; e < 16 * M; e += 32) {
                const int row = e % 16, m = e / 16;
                float sum = 0.0f;
                for (int w = 0; w < a.wpt; ++w) {
                    const int sw = s_mine + w < S ? s_mine + w : s_mine + w - S;
                    sum += lds32f(smem0 + uint32_t(sw) * kItem + (row * MP + m) * 4);
                }
                const int nrow = tile * 16 + row;
                if (nrow < N) y[size_t(m) * N + nrow] = H::from_float(sum * __ldg(a.scale + nrow));
            }
            __syncwarp();
            if (lane < a.wpt) bar_arrive(empty0 + (s_mine + lane < S ? s_mine + lane : s_mine + lane - S) * 8);
        }
    }
}

// Launch geometry; false when the kernel does not take the shape.
template <int WARPS, int KB>
inline bool tma8_plan(Tma8Args& a, size_t* smem) {
    if (a.K % (64 * KB) != 0 || a.M > 2 || a.M < 1 || !aligned(a.x, 16)) return false;
    const int runs = a.K / (64 * KB);
    int opc = 1;
    while (runs % opc != 0 || runs / opc > WARPS) ++opc;
    a.opc = opc;
    a.wpt = runs / opc;
    if (a.wpt > 32) return false;
    a.tpc = WARPS / a.wpt;
    if (a.wpt > 1 && a.tpc > 14) a.tpc = 14;
    const Tma8Layout fixed = tma8_layout<WARPS, KB>(a.M, a.K, 0);
    const long budget = 226L * 1024 - long(fixed.total);
    long stages = (budget - 2 * WARPS * 8 - 128) / (KB * 1024 + 8);
    if (stages < 4 || stages <= a.wpt) return false;
    if (stages > 96) stages = 96;
    a.stages = int(stages);
    *smem = tma8_layout<WARPS, KB>(a.M, a.K, a.stages).total;
    return true;
}

// The weights [N, K] as 64-byte pieces: (byte of the k-block, row, k-block of the row).
template <int KB>
inline bool tma8_weight_map(CUtensorMap* map, const int8_t* w, int N, int K) {
    const umma::EncodeTiled encode = umma::encode_tiled();
    if (encode == nullptr || !aligned(w, 16)) return false;
    const cuuint64_t dims[3] = {64, cuuint64_t(N), cuuint64_t(K / 64)};
    const cuuint64_t strides[2] = {cuuint64_t(K), 64};
    const cuuint32_t box[3] = {64, 16, KB};
    const cuuint32_t elem[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(w), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int WARPS, int KB>
int32_t launch_tma8(const Tma8Args& a, const int8_t* w, size_t smem, int sms, cudaStream_t stream) {
    auto kernel = int8_gemv_tma_kernel<T, WARPS, KB>;
    CUtensorMap map;
    if (!tma8_weight_map<KB>(&map, w, a.N, a.K)) return fail("int8_linear: the weight tensor map was refused");
    const cudaError_t attr_err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    if (attr_err != cudaSuccess) {
        cudaGetLastError();
        return fail("int8_linear: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(attr_err));
    }
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
        return fail("int8_linear: launch failed: %s", cudaGetErrorString(err));
    }
    return B200Q_OK;
}

}  // namespace b200q
