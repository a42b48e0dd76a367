// Single-query (decode) attention over the KV cache, split over the keys and merged.
//
// In the reference this is `scaled_dot_product_attention` with a [B, 1, 1, S] mask and
// `enable_gqa` inside the captured decode graph (examples/01-llama/src/attention.linnet run
// by python/linnet/src/linnet/torch/compiled.py:430-503).  A decode step reads every
// cached key and value once, so the kernel is bound by HBM: 2 * 2 * S * HD bytes per KV
// head and row, shared by the REP = heads / kv_heads query heads of the group.
//
// Block (split, kv head, batch row), four or eight warps.  The block streams its keys and values
// through shared memory in chunks of 64 (or 128) positions with 16-byte cp.async copies, three
// chunks deep; each warp owns 16 positions of a chunk and runs them through the tensor
// cores for all REP heads at once:
//   scores [heads x 16 positions] = Q [heads(padded to 16) x HD] . K^T   (mma m16n8k16, K
//       fragments by ldmatrix from the position-major tile),
//   running softmax in f32 on the accumulator fragments (base 2, scale folded in),
//   out [heads x HD] += P [heads x 16 positions] . V                      (V fragments by
//       ldmatrix.trans; P reuses the score registers, rounded to bf16).
// Rows of 2*HD bytes would put the eight rows of an ldmatrix on the same banks, so the
// 16-byte pieces of a row are stored at piece ^ (position % 8).  The four warps' running
// (max, sum, accumulator) are merged through shared memory into partial
// [B, nq, splits, HD + 2] f32 (max in natural-log units), and a second small kernel merges
// the splits.
#include <cooperative_groups.h>

#include "common.cuh"

namespace b200q {
namespace cg = cooperative_groups;
namespace {

// WARPS warps a block, 16 positions of a chunk each: a chunk (one shared-memory stage) is
// 16 * WARPS positions.  With more blocks than multiprocessors: 4 warps, chunks of 64, 3
// stages (two blocks fit on a multiprocessor).  With fewer: 8 warps, chunks of 128, 3
// stages (one block a multiprocessor, twice the bytes in flight, half the copies to issue
// per thread and half the block-wide barriers).
constexpr int kAttnStages = 3;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// d += a . b with rows 8..15 of a all zero (a1 = a3 = 0): only d0, d1 carry data.
__device__ __forceinline__ void mma_top(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

template <int HD, int REP, int WARPS>
__global__ void __launch_bounds__(32 * WARPS)
attention_partial_kernel(const uint16_t* q, uint16_t* cache_k,  // q and positions: ld_mutable()
                         uint16_t* cache_v, const int64_t* positions,
                         const float2* __restrict__ rope, float* __restrict__ partial,
                         uint16_t* __restrict__ out_final, int nq, int nkv, int S, int splits, int stages,
                         float scale_log2, int* status) {
    static_assert(REP <= 8 && (HD == 64 || HD == 128), "heads of a group sit in rows 0..7 of the MMA");
    constexpr int kRowBytes = HD * 2;
    constexpr int kPieces = kRowBytes / 16;          // 16-byte pieces per row
    constexpr int kAttnChunk = 16 * WARPS, kAttnWarps = WARPS;
    constexpr int kStage = kAttnChunk * kRowBytes;   // bytes of K (or V) per chunk
    constexpr int kThreads = 32 * kAttnWarps;
    constexpr float kLn2 = 0.6931471805599453f;
    extern __shared__ __align__(128) uint8_t attn_smem[];  // [stages][K chunk | V chunk]
    pdl_launch_dependents();  // the next kernel may start its own prologue (a product: its weight fetch) at once
    pdl_wait();
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
    // rope != nullptr: q is the fused projection [B, (nq + 2 nkv) * HD] straight from the
    // linear layer; this kernel rotates the query and key heads itself (cos / sin of every
    // position in `rope`), and the block whose keys end at the current position puts the new
    // key and value into its tile and into the cache.
    const bool fused = rope != nullptr;
    const int q_heads = fused ? nq + 2 * nkv : nq;  // heads per row of q
    // A position outside the cache is recorded and clamped: the row's result means nothing,
    // but no address outside the caches or the table is formed and nothing is stored for it.
    const int64_t pos_given = ld_mutable(positions + b);
    const bool bad = pos_given < 0 || pos_given >= S;
    if (bad && threadIdx.x == 0 && split == 0 && kvh == 0) record_bad_position(status, b);
    const int keys = int(bad ? 0 : pos_given) + 1;  // attend to positions 0 .. pos
    const int per_split = (keys + splits - 1) / splits;
    const int k0 = split * per_split, k1 = min(k0 + per_split, keys);
    const int chunks = k1 > k0 ? (k1 - k0 + kAttnChunk - 1) / kAttnChunk : 0;
    const size_t base = (size_t(b) * nkv + kvh) * S * HD;
    const uint32_t smem0 = uint32_t(__cvta_generic_to_shared(attn_smem));

    auto issue = [&](int c) {  // chunk c of this split -> stage c % kAttnStages (an empty group past the end)
        if (c < chunks) {
            const uint32_t dst = smem0 + (c % stages) * 2 * kStage;
            const int first = k0 + c * kAttnChunk;
            for (int piece = threadIdx.x; piece < 2 * kStage / 16; piece += kThreads) {
                const int which = piece / (kStage / 16), within = piece % (kStage / 16);
                const int row = within / kPieces, col = within % kPieces;
                // The tail repeats the last key already in the cache: with the fused rotary step
                // the row of the current position is written by this very launch.
                const int key = min(first + row, max(k1 - 1 - int(fused && k1 == keys), 0));
                const uint16_t* src = (which ? cache_v : cache_k) + base + size_t(key) * HD + col * 8;
                const uint32_t d = dst + which * kStage + row * kRowBytes + ((col ^ (row & 7)) * 16);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int c = 0; c < stages - 1; ++c) issue(c);

    // Q as the A operand: row g = head g of the group (zero rows past REP), two registers per 16 dims.
    uint32_t qa[HD / 16][2];
    {
        const uint16_t* qp = q + (size_t(b) * q_heads + kvh * REP + (g < REP ? g : 0)) * HD;
#pragma unroll
        for (int s = 0; s < HD / 16; ++s) {
            qa[s][0] = ld_mutable(reinterpret_cast<const uint32_t*>(qp + 16 * s + 2 * t));
            qa[s][1] = ld_mutable(reinterpret_cast<const uint32_t*>(qp + 16 * s + 8 + 2 * t));
        }
        if (fused) {  // dims d and d + HD/2 rotate together: registers s and s + HD/32 of this lane
            const float2* cs = rope + size_t(keys - 1) * (HD / 2);
#pragma unroll
            for (int s = 0; s < HD / 32; ++s)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int d = 16 * s + 8 * h + 2 * t;
                    const float2 c0 = __ldg(cs + d), c1 = __ldg(cs + d + 1);
                    const uint32_t lo = qa[s][h], hi = qa[s + HD / 32][h];
                    const float a0 = bf16_lo(lo), a1 = bf16_hi(lo), b0 = bf16_lo(hi), b1 = bf16_hi(hi);
                    qa[s][h] = bf16_pack(a0 * c0.x - b0 * c0.y, a1 * c1.x - b1 * c1.y);
                    qa[s + HD / 32][h] = bf16_pack(b0 * c0.x + a0 * c0.y, b1 * c1.x + a1 * c1.y);
                }
        }
#pragma unroll
        for (int s = 0; s < HD / 16; ++s) {
            qa[s][0] = g < REP ? qa[s][0] : 0u;
            qa[s][1] = g < REP ? qa[s][1] : 0u;
        }
    }
    float m = -INFINITY, l = 0.0f;  // running max (log2 units) and this lane's share of the sum, head g
    float acc[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) acc[d][0] = acc[d][1] = acc[d][2] = acc[d][3] = 0.0f;

    const int r0 = warp * 16;                       // this warp's rows of a chunk
    const int lm_row = lane & 7, lm_mat = lane >> 3;  // ldmatrix: this lane addresses row lm_row of matrix lm_mat
    for (int c = 0; c < chunks; ++c) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // stages - 2
        __syncthreads();  // chunk c has landed for everyone; everyone is done with chunk c - 1
        issue(c + stages - 1);  // into the stage chunk c - 1 used
        const int first = k0 + c * kAttnChunk;
        if (fused && k1 == keys && c == chunks - 1) {
            // The current position is the last row of this chunk: its key (rotated) and value
            // come from the projection, not from the cache, and are stored for later steps.
            const int row = keys - 1 - first, half = HD / 2;
            uint8_t* tile = attn_smem + (c % stages) * 2 * kStage;
            for (int i = threadIdx.x; i < half; i += kThreads) {
                const uint16_t* kp = q + (size_t(b) * q_heads + nq + kvh) * HD;
                const uint16_t* vp = kp + size_t(nkv) * HD;
                const float2 cs = __ldg(rope + size_t(keys - 1) * half + i);
                const float a = bf16_lo(ld_mutable(kp + i)), bb = bf16_lo(ld_mutable(kp + i + half));
                const uint16_t v_lo = ld_mutable(vp + i), v_hi = ld_mutable(vp + i + half);
                const uint16_t lo = uint16_t(bf16_pack(a * cs.x - bb * cs.y, 0.0f) & 0xFFFF);
                const uint16_t hi = uint16_t(bf16_pack(bb * cs.x + a * cs.y, 0.0f) & 0xFFFF);
                const int at_lo = row * kRowBytes + (((i / 8) ^ (row & 7)) * 16) + (i % 8) * 2;
                const int at_hi = row * kRowBytes + ((((i + half) / 8) ^ (row & 7)) * 16) + (i % 8) * 2;
                *reinterpret_cast<uint16_t*>(tile + at_lo) = lo;
                *reinterpret_cast<uint16_t*>(tile + at_hi) = hi;
                *reinterpret_cast<uint16_t*>(tile + kStage + at_lo) = v_lo;
                *reinterpret_cast<uint16_t*>(tile + kStage + at_hi) = v_hi;
                const size_t dst = base + size_t(keys - 1) * HD;
                if (!bad) {
                    cache_k[dst + i] = lo;
                    cache_k[dst + i + half] = hi;
                    cache_v[dst + i] = v_lo;
                    cache_v[dst + i + half] = v_hi;
                }
            }
            __syncthreads();
        }
        if (first + r0 >= k1) continue;  // warp-uniform: none of this warp's 16 positions exist
        const uint32_t ks = smem0 + (c % stages) * 2 * kStage, vs = ks + kStage;

        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
            const int row = r0 + 8 * j + lm_row;
#pragma unroll
            for (int p = 0; p < HD / 32; ++p) {  // two 16-dim steps per ldmatrix
                uint32_t kb[4];
                ldmatrix_x4(kb, ks + row * kRowBytes + (((4 * p + lm_mat) ^ (row & 7)) * 16));
                mma_top(sc[j], qa[2 * p][0], qa[2 * p][1], kb[0], kb[1]);
                mma_top(sc[j], qa[2 * p + 1][0], qa[2 * p + 1][1], kb[2], kb[3]);
            }
        }
        // scores of head g at positions first + r0 + 8 j + 2 t + {0, 1}
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool live = first + r0 + 8 * j + 2 * t + e < k1;
                sc[j][e] = live ? sc[j][e] * scale_log2 : -INFINITY;
                mx = fmaxf(mx, sc[j][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        const float m_new = fmaxf(m, mx);  // finite: the warp's first position exists
        const float corr = exp2f(m - m_new);
        m = m_new;
        float pr[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) pr[j][e] = exp2f(sc[j][e] - m_new);
        l = l * corr + (pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]);
        const uint32_t pa0 = bf16_pack(pr[0][0], pr[0][1]), pa2 = bf16_pack(pr[1][0], pr[1][1]);
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) {
            acc[d][0] *= corr;
            acc[d][1] *= corr;
        }
        {
            const int row = r0 + (lm_mat & 1) * 8 + lm_row;
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {  // two 8-dim blocks per ldmatrix
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, vs + row * kRowBytes + (((2 * dp + (lm_mat >> 1)) ^ (row & 7)) * 16));
                mma_top(acc[2 * dp], pa0, pa2, vb[0], vb[1]);
                mma_top(acc[2 * dp + 1], pa0, pa2, vb[2], vb[3]);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 1);
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 2);
    __syncthreads();  // the stages are free: reuse them for the warps' results

    float* merge = reinterpret_cast<float*>(attn_smem);  // [warp][head][HD + 2]
    if (g < REP) {
        float* mine = merge + (warp * REP + g) * (HD + 2);
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) {
            mine[8 * d + 2 * t] = acc[d][0];
            mine[8 * d + 2 * t + 1] = acc[d][1];
        }
        if (t == 0) {
            mine[HD] = m;
            mine[HD + 1] = l;
        }
    }
    __syncthreads();
    // partial == nullptr: the splits of a (row, kv head) form one thread-block cluster and
    // merge through distributed shared memory; otherwise a second kernel merges `partial`.
    const bool in_cluster = partial == nullptr;
    float* block_result = merge + kAttnWarps * REP * (HD + 2);  // [head][HD + 2], max in log2 units
    for (int item = threadIdx.x; item < REP * (HD + 1); item += kThreads) {
        const int head = item / (HD + 1), col = item % (HD + 1);  // col HD: the (max, sum) pair
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) m_all = fmaxf(m_all, merge[(w * REP + head) * (HD + 2) + HD]);
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float* theirs = merge + (w * REP + head) * (HD + 2);
            const float weight = theirs[HD] == -INFINITY ? 0.0f : exp2f(theirs[HD] - m_all);
            total += weight * theirs[col == HD ? HD + 1 : col];
        }
        float* out = in_cluster ? block_result + head * (HD + 2)
                                : partial + ((size_t(b) * nq + kvh * REP + head) * splits + split) * (HD + 2);
        if (col == HD) {
            out[HD] = in_cluster ? m_all : m_all * kLn2;
            out[HD + 1] = total;
        } else {
            out[col] = total;
        }
    }
    if (!in_cluster) return;

    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every split's result is in its block's shared memory
    // Block r of the cluster finishes every splits-th (head, dim) pair.
    for (int item = split + splits * threadIdx.x; item < REP * HD; item += splits * kThreads) {
        const int head = item / HD, dcol = item % HD;
        float m_s[8], l_s[8], a_s[8];
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
            m_s[sp] = -INFINITY;
            l_s[sp] = a_s[sp] = 0.0f;
            if (sp < splits) {
                const float* theirs = cluster.map_shared_rank(block_result, sp) + head * (HD + 2);
                m_s[sp] = theirs[HD];
                l_s[sp] = theirs[HD + 1];
                a_s[sp] = theirs[dcol];
            }
        }
        float m_all = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) m_all = fmaxf(m_all, m_s[sp]);
        float l_all = 0.0f, a_all = 0.0f;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
            const float c = m_s[sp] == -INFINITY ? 0.0f : exp2f(m_s[sp] - m_all);
            l_all += l_s[sp] * c;
            a_all += a_s[sp] * c;
        }
        out_final[(size_t(b) * nq + kvh * REP + head) * HD + dcol] = uint16_t(bf16_pack(a_all / l_all, 0.0f) & 0xFFFF);
    }
    cluster.sync();  // nobody leaves while a peer may still read its shared memory
}

template <int HD>
__global__ void attention_merge_kernel(const float* partial, uint16_t* __restrict__ out,
                                       int splits) {
    pdl_launch_dependents();  // the next kernel may start its own prologue (a product: its weight fetch) at once
    pdl_wait();
    const size_t head = blockIdx.x;  // b * nq + query head
    const float* p = partial + head * splits * (HD + 2);
    float m_all = -INFINITY;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, ld_mutable(p + s * (HD + 2) + HD));
    for (int dcol = threadIdx.x; dcol < HD; dcol += blockDim.x) {
        float l_all = 0.0f, a_all = 0.0f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            const float ms = ld_mutable(p + s * (HD + 2) + HD);
            const float c = ms == -INFINITY ? 0.0f : __expf(ms - m_all);
            l_all += ld_mutable(p + s * (HD + 2) + HD + 1) * c;
            a_all += ld_mutable(p + s * (HD + 2) + dcol) * c;
        }
        out[head * HD + dcol] = uint16_t(bf16_pack(a_all / l_all, 0.0f) & 0xFFFF);
    }
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int64_t b200q_decode_attention_scratch_bytes(int64_t batch, int64_t nq, int64_t head_dim,
                                                        int64_t splits) {
    return batch * nq * splits * (head_dim + 2) * 4;
}

namespace b200q {
namespace {

int32_t launch_attention(const char* who, const void* q, const void* cache_k, const void* cache_v,
                         const int64_t* positions, void* out, void* scratch, int64_t batch, int64_t nq,
                         int64_t nkv, int64_t head_dim, int64_t max_seq, int64_t splits, void* stream,
                         bool in_cluster = false, const void* rope = nullptr) {
    B200Q_REQUIRE(batch >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0 && splits >= 1 && splits <= 65535,
                  "%s: bad shape", who);
    if (batch == 0) return B200Q_OK;
    const int rep = int(nq / nkv);
    B200Q_REQUIRE((head_dim == 128 || head_dim == 64) && (rep == 1 || rep == 2 || rep == 4 || rep == 8),
                  "%s: head_dim is 64 or 128 and heads / kv_heads is 1, 2, 4 or 8", who);
    B200Q_REQUIRE(q && cache_k && cache_v && positions && out && (scratch || in_cluster) && aligned(q, 16) &&
                      aligned(cache_k, 16) && aligned(cache_v, 16) && aligned(scratch, 16) && aligned(positions, 8),
                  "%s: tensors must be 16-byte aligned (positions: int64)", who);
    B200Q_REQUIRE(max_seq > 0 && max_seq < (int64_t(1) << 30), "%s: bad cache length", who);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid{unsigned(splits), unsigned(nkv), unsigned(batch)};
    const float scale_log2 = 1.4426950408889634f / sqrtf(float(head_dim));  // softmax in base 2
#define B200Q_ATTN_W(HD, REP, WARPS) do {                                                             \
    const int kSmem = kAttnStages * 2 * (16 * WARPS) * HD * 2;                                        \
    ensure_dynamic_smem(reinterpret_cast<const void*>(attention_partial_kernel<HD, REP, WARPS>), kSmem); \
    cudaLaunchConfig_t config = {};                                                                   \
    config.gridDim = grid;                                                                            \
    config.blockDim = dim3(32 * WARPS);                                                               \
    config.dynamicSmemBytes = kSmem;                                                                  \
    config.stream = s;                                                                                \
    cudaLaunchAttribute attr[2];                                                                      \
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                  \
    attr[0].val.programmaticStreamSerializationAllowed = 1;                                           \
    attr[1].id = cudaLaunchAttributeClusterDimension;                                                 \
    attr[1].val.clusterDim.x = unsigned(splits);                                                      \
    attr[1].val.clusterDim.y = 1;                                                                     \
    attr[1].val.clusterDim.z = 1;                                                                     \
    config.attrs = attr;                                                                              \
    config.numAttrs = in_cluster ? 2 : 1;                                                             \
    err = cudaLaunchKernelEx(&config, attention_partial_kernel<HD, REP, WARPS>,                       \
                      static_cast<const uint16_t*>(q),                                               \
                      static_cast<uint16_t*>(const_cast<void*>(cache_k)),                             \
                      static_cast<uint16_t*>(const_cast<void*>(cache_v)), positions,                  \
                      static_cast<const float2*>(rope), in_cluster ? static_cast<float*>(nullptr)     \
                                                                   : static_cast<float*>(scratch),    \
                      static_cast<uint16_t*>(out), int(nq), int(nkv), int(max_seq), int(splits),      \
                      kAttnStages, scale_log2, decoder_error_word()); } while (0)
#define B200Q_ATTN(HD, REP) do { if (few_blocks) B200Q_ATTN_W(HD, REP, 8); else B200Q_ATTN_W(HD, REP, 4); } while (0)
    cudaError_t err = cudaSuccess;
    const bool few_blocks = splits * nkv * batch <= sm_count();
    if (head_dim == 128) {
        if (rep == 1) B200Q_ATTN(128, 1); else if (rep == 2) B200Q_ATTN(128, 2);
        else if (rep == 4) B200Q_ATTN(128, 4); else B200Q_ATTN(128, 8);
        if (!in_cluster && err == cudaSuccess)
            err = launch_overlapped(attention_merge_kernel<128>, dim3(unsigned(batch * nq)), dim3(128), 0, s,
                              static_cast<const float*>(scratch), static_cast<uint16_t*>(out), int(splits));
    } else {
        if (rep == 1) B200Q_ATTN(64, 1); else if (rep == 2) B200Q_ATTN(64, 2);
        else if (rep == 4) B200Q_ATTN(64, 4); else B200Q_ATTN(64, 8);
        if (!in_cluster && err == cudaSuccess)
            err = launch_overlapped(attention_merge_kernel<64>, dim3(unsigned(batch * nq)), dim3(64), 0, s,
                              static_cast<const float*>(scratch), static_cast<uint16_t*>(out), int(splits));
    }
#undef B200Q_ATTN
#undef B200Q_ATTN_W
    return launch_status(who, err);
}

}  // namespace
}  // namespace b200q

extern "C" int32_t b200q_decode_attention(const void* q, const void* cache_k, const void* cache_v,
                                          const int64_t* positions, void* out, void* scratch,
                                          int64_t batch, int64_t nq, int64_t nkv, int64_t head_dim,
                                          int64_t max_seq, int64_t splits, void* stream) {
    return launch_attention("decode_attention", q, cache_k, cache_v, positions, out, scratch, batch, nq,
                            nkv, head_dim, max_seq, splits, stream);
}

// One launch and no scratch: the splits (at most 8) of a (row, kv head) run as one
// thread-block cluster and merge through distributed shared memory.
extern "C" int32_t b200q_decode_attention_cluster(const void* q, const void* cache_k, const void* cache_v,
                                                  const int64_t* positions, void* out, int64_t batch,
                                                  int64_t nq, int64_t nkv, int64_t head_dim, int64_t max_seq,
                                                  int64_t splits, void* stream) {
    B200Q_REQUIRE(splits >= 1 && splits <= 8, "decode_attention_cluster: 1 to 8 splits, not %lld", (long long)splits);
    return launch_attention("decode_attention_cluster", q, cache_k, cache_v, positions, out, nullptr, batch, nq,
                            nkv, head_dim, max_seq, splits, stream, true);
}

// Rotary embedding, cache write and attention in one launch: qkv is the fused projection of
// the step, `rope` the table of b200q_rope_table.
extern "C" int32_t b200q_rope_attention(const void* qkv, const int64_t* positions, const void* rope,
                                        void* cache_k, void* cache_v, void* out, int64_t batch, int64_t nq,
                                        int64_t nkv, int64_t head_dim, int64_t max_seq, int64_t splits,
                                        void* stream) {
    B200Q_REQUIRE(splits >= 1 && splits <= 8, "rope_attention: 1 to 8 splits, not %lld", (long long)splits);
    B200Q_REQUIRE(rope != nullptr && aligned(rope, 8), "rope_attention: no table of cosines and sines");
    return launch_attention("rope_attention", qkv, cache_k, cache_v, positions, out, nullptr, batch, nq, nkv,
                            head_dim, max_seq, splits, stream, true, rope);
}

namespace b200q {
namespace {
// table[pos][i] = (cos, sin)(pos * theta^(-i / half)), the arithmetic of rope_cache_kernel.
__global__ void rope_table_kernel(float2* __restrict__ table, int half, int64_t total, float theta) {
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += int64_t(gridDim.x) * blockDim.x) {
        const int64_t pos = e / half;
        const int i = int(e % half);
        const float freq = powf(theta, -float(i) / float(half));
        float s, c;
        sincosf(float(pos) * freq, &s, &c);
        table[e] = make_float2(c, s);
    }
}
}  // namespace
}  // namespace b200q

extern "C" int32_t b200q_rope_table(void* table, int64_t max_seq, int64_t head_dim, float theta, void* stream) {
    B200Q_REQUIRE(table && aligned(table, 8) && max_seq > 0 && head_dim > 0 && head_dim % 2 == 0,
                  "rope_table: bad arguments");
    const int64_t total = max_seq * (head_dim / 2);
    rope_table_kernel<<<unsigned((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256), 256, 0,
                        static_cast<cudaStream_t>(stream)>>>(static_cast<float2*>(table), int(head_dim / 2), total,
                                                            theta);
    return launched("rope_table");
}

// ---- the same attention for callers that cannot allocate device memory ----------------
// Some hosts of this library have no way to hand it scratch memory: a runtime that owns a
// fixed arena sized before the model is known, a plug-in loaded into a server whose
// allocator is off limits to it, code running while a stream is being captured (no
// cudaMalloc there).  For them the splits' partial results live in a fixed array inside
// the library image instead: 4 MiB that every GPU which loads the library keeps until
// the process exits.
constexpr int64_t kStaticScratchBytes = int64_t(4) << 20;
static __device__ __align__(256) unsigned char g_attention_scratch[kStaticScratchBytes];

namespace b200q {
namespace {

// In host code `g_attention_scratch` is only a handle for the runtime, not a device
// address; the address is asked for once per device, with that device current.
void* static_scratch_address() {
    static void* cached[64] = {nullptr};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (cached[device] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_attention_scratch) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cached[device] = p;
    }
    return cached[device];
}

}  // namespace
}  // namespace b200q

extern "C" int64_t b200q_decode_attention_static_scratch_limit(void) { return kStaticScratchBytes; }

extern "C" int32_t b200q_decode_attention_static(const void* q, const void* cache_k, const void* cache_v,
                                                 const int64_t* positions, void* out, int64_t batch,
                                                 int64_t nq, int64_t nkv, int64_t head_dim, int64_t max_seq,
                                                 int64_t splits, void* stream) {
    B200Q_REQUIRE(batch >= 0 && nq > 0 && head_dim > 0 && splits >= 1, "decode_attention_static: bad shape");
    const int64_t need = b200q_decode_attention_scratch_bytes(batch, nq, head_dim, splits);
    B200Q_REQUIRE(need <= kStaticScratchBytes,
                  "decode_attention_static: batch %lld x %lld heads x %lld splits needs %lld bytes of scratch, "
                  "the built-in array holds %lld; use fewer splits or b200q_decode_attention with your own scratch",
                  (long long)batch, (long long)nq, (long long)splits, (long long)need,
                  (long long)kStaticScratchBytes);
    void* scratch = static_scratch_address();
    B200Q_REQUIRE(scratch != nullptr, "decode_attention_static: cudaGetSymbolAddress failed on this device");
    return launch_attention("decode_attention_static", q, cache_k, cache_v, positions, out, scratch, batch, nq,
                            nkv, head_dim, max_seq, splits, stream);
}

