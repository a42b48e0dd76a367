// The tensor-parallel reduction + residual add + RMSNorm of tp_allreduce.cu with a different
// exchange between the ranks: rows pushed as plain bf16, then one flag per (source rank, row).
//
// Same contract as b200q_tp_allreduce_add_rmsnorm (the reference's all_reduce after a
// `Shards` layer, stdlib/nn/parallel.linnet:9-11, plus the add and norm that follow), same
// arithmetic (rows summed in rank order in f32, one rounding to bf16), bounded waits.  Every
// rank has a receive area per call site, [source rank][rows][hidden] bf16, and its decode
// kernel writes its own partial sums into its own slot of it.  One block per row pushes that
// row into its slot of every peer's area (16-byte stores over NVLink); a block barrier
// followed by the flag threads' st.release.sys orders the pushes before the row's flag on
// every peer; the block then waits for the peers' flags of the row and sums what arrived.
//
// Measured against the tagged-word exchange of tp_allreduce.cu (8B-shape decoder, batch 1,
// ms per step): 2 GPUs 1.60 against 1.54; 8 GPUs 1.32 against 1.46.  Half the bytes cross
// NVLink and seven threads poll instead of all of them, which wins once seven peers push at
// once; the extra ordering step loses on two GPUs.  The host side picks by group size.
#include "common.cuh"

namespace b200q {
uint64_t tp_wait_limit_ns();  // tp_allreduce.cu
namespace {

constexpr int kMaxRanks = 8;

struct Peers {
    uint16_t* recv[kMaxRanks];   // every rank's receive area of this site [world][max_rows][hidden] bf16
    uint32_t* flags[kMaxRanks];  // every rank's flag words of this site [world][max_rows]
    int world, rank;
};

__device__ __forceinline__ float lo16(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi16(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

// CPT: 16-byte pieces of a row each thread keeps in registers from the push to the scaling
// (0: any width, rows re-read from memory).
template <int CPT>
__global__ void __launch_bounds__(512)
allreduce_flags_kernel(const Peers p, size_t slot_elems, int max_rows, uint32_t* __restrict__ epoch,
                             uint32_t* __restrict__ done, int* __restrict__ error, uint16_t* x,
                             const uint16_t* __restrict__ weight, uint16_t* __restrict__ y, int hidden,
                             float eps, uint64_t wait_limit_ns) {
    __shared__ float partial_sums[16];
    __shared__ int gave_up;
    constexpr int kHeld = CPT > 0 ? CPT : 1;
    const int row = blockIdx.x, chunks = hidden / 8;
    const uint4* wr = reinterpret_cast<const uint4*>(weight);
    uint4 g[kHeld], own[kHeld], v[kHeld];
    if (CPT > 0) {  // the norm weights do not depend on the kernel before this one
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            g[u] = c < chunks ? __ldg(wr + c) : make_uint4(0, 0, 0, 0);
        }
    }
    pdl_launch_dependents();  // the next kernel may start its own prologue (a product: its weight fetch) at once
    pdl_wait();  // this rank's partial sums come from the kernel before this one
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(epoch) + 1;
    // After one wait has run out every later call returns at once instead of waiting again.
    if (threadIdx.x == 0) gave_up = *reinterpret_cast<volatile int*>(error) != 0;

    // 1. push this rank's row into its slot of every peer's area
    const size_t row_at = size_t(p.rank) * slot_elems + size_t(row) * hidden;
    const uint4* mine = reinterpret_cast<const uint4*>(p.recv[p.rank] + row_at);
    auto push = [&](int c, const uint4& piece) {
        for (int peer = 0; peer < p.world; ++peer)
            if (peer != p.rank) reinterpret_cast<uint4*>(p.recv[peer] + row_at)[c] = piece;
    };
    if (CPT > 0) {
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            own[u] = c < chunks ? ld_mutable(mine + c) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            if (c < chunks) push(c, own[u]);
        }
    } else {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) push(c, ld_mutable(mine + c));
    }
    // The flag stores below are releases at system scope by threads that the barrier has
    // synchronised with every pushing thread: that orders all of the block's pushes before
    // the flags without a system-wide fence in each of the 512 threads.
    __syncthreads();
    // 2. raise the row's flag on every peer, then wait for every peer's flag here
    if (int(threadIdx.x) < p.world && int(threadIdx.x) != p.rank) {
        uint32_t* theirs = p.flags[threadIdx.x] + size_t(p.rank) * max_rows + row;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(e) : "memory");
        if (!gave_up) {
            const uint32_t* here = p.flags[p.rank] + size_t(threadIdx.x) * max_rows + row;
            uint64_t start = 0;
            for (uint32_t spins = 0;; ++spins) {
                uint32_t seen;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(here) : "memory");
                if (int32_t(seen - e) >= 0) break;
                if ((spins & 255u) == 255u) {
                    uint64_t now;
                    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                    if (start == 0) start = now;
                    if (now - start > wait_limit_ns) {  // a peer never arrived: give up, stay usable
                        atomicCAS(error, 0, 100 + int(threadIdx.x));
                        gave_up = 1;
                        break;
                    }
                }
            }
        }
    }
    __syncthreads();

    // 3. rows of all ranks in rank order (f32), one rounding, residual add, sum of squares
    uint4* xr = reinterpret_cast<uint4*>(x + size_t(row) * hidden);
    float sum_sq = 0.0f;
    auto reduce_add_square = [&](int c, const uint4& own_piece) {
        float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        uint4 t = ld_mutable(xr + c);
        uint4 q[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            q[r] = make_uint4(0, 0, 0, 0);
            if (r < p.world && r != p.rank)
                q[r] = ld_mutable(reinterpret_cast<const uint4*>(p.recv[p.rank] + size_t(r) * slot_elems +
                                                                 size_t(row) * hidden) + c);
        }
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            if (r >= p.world) break;
            const uint4 qr = r == p.rank ? own_piece : q[r];
            s[0] += lo16(qr.x); s[1] += hi16(qr.x); s[2] += lo16(qr.y); s[3] += hi16(qr.y);
            s[4] += lo16(qr.z); s[5] += hi16(qr.z); s[6] += lo16(qr.w); s[7] += hi16(qr.w);
        }
        // the reduced tensor is bf16 (one rounding), then the residual add rounds again
        const uint32_t d0 = pack16(s[0], s[1]), d1 = pack16(s[2], s[3]), d2 = pack16(s[4], s[5]),
                       d3 = pack16(s[6], s[7]);
        t.x = pack16(lo16(t.x) + lo16(d0), hi16(t.x) + hi16(d0));
        t.y = pack16(lo16(t.y) + lo16(d1), hi16(t.y) + hi16(d1));
        t.z = pack16(lo16(t.z) + lo16(d2), hi16(t.z) + hi16(d2));
        t.w = pack16(lo16(t.w) + lo16(d3), hi16(t.w) + hi16(d3));
        xr[c] = t;
        const uint32_t w4[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) sum_sq += lo16(w4[i]) * lo16(w4[i]) + hi16(w4[i]) * hi16(w4[i]);
        return t;
    };
    if (CPT > 0) {
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            v[u] = make_uint4(0, 0, 0, 0);
            if (c < chunks) v[u] = gave_up ? ld_mutable(xr + c) : reduce_add_square(c, own[u]);
        }
    } else if (!gave_up) {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) reduce_add_square(c, ld_mutable(mine + c));
    }
    for (int d = 16; d >= 1; d >>= 1) sum_sq += __shfl_xor_sync(0xFFFFFFFFu, sum_sq, d);
    if (threadIdx.x % 32 == 0) partial_sums[threadIdx.x / 32] = sum_sq;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < int(blockDim.x) / 32; ++i) total += partial_sums[i];
    const float rstd = rsqrtf(total / float(hidden) + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + size_t(row) * hidden);
    auto scaled = [&](const uint4& t, const uint4& gw) {
        uint4 o;
        o.x = pack16(lo16(t.x) * rstd * lo16(gw.x), hi16(t.x) * rstd * hi16(gw.x));
        o.y = pack16(lo16(t.y) * rstd * lo16(gw.y), hi16(t.y) * rstd * hi16(gw.y));
        o.z = pack16(lo16(t.z) * rstd * lo16(gw.z), hi16(t.z) * rstd * hi16(gw.z));
        o.w = pack16(lo16(t.w) * rstd * lo16(gw.w), hi16(t.w) * rstd * hi16(gw.w));
        return o;
    };
    if (CPT > 0) {
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            if (c < chunks) yr[c] = scaled(v[u], g[u]);
        }
    } else {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) yr[c] = scaled(ld_mutable(xr + c), wr[c]);
    }
    // The last block to finish advances the site's epoch (every block has read it by then).
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *done = 0;
            *reinterpret_cast<volatile uint32_t*>(epoch) = e;
        }
    }
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_tp_allreduce_add_rmsnorm_flags(const int64_t* peer_areas, const int64_t* peer_flags,
                                                  int64_t slot_elems, int64_t max_rows, int32_t world,
                                                  int32_t rank, void* epoch, void* done, void* error, void* x,
                                                  const void* weight, void* y, int64_t rows, int64_t hidden,
                                                  float eps, void* stream) {
    B200Q_REQUIRE(world >= 2 && world <= kMaxRanks && rank >= 0 && rank < world,
                  "tp_allreduce_add_rmsnorm_flags: 2..8 ranks, got world=%d rank=%d", world, rank);
    B200Q_REQUIRE(rows >= 0 && hidden > 0 && hidden % 8 == 0, "tp_allreduce_add_rmsnorm_flags: hidden must be a multiple of 8");
    B200Q_REQUIRE(rows <= max_rows && slot_elems >= max_rows * hidden && slot_elems % 8 == 0,
                  "tp_allreduce_add_rmsnorm_flags: %lld rows do not fit slots of %lld rows", (long long)rows,
                  (long long)max_rows);
    if (rows == 0) return B200Q_OK;
    B200Q_REQUIRE(peer_areas && peer_flags && epoch && done && error && x && weight && y,
                  "tp_allreduce_add_rmsnorm_flags: null argument");
    Peers p{};
    p.world = world;
    p.rank = rank;
    for (int r = 0; r < world; ++r) {
        p.recv[r] = reinterpret_cast<uint16_t*>(peer_areas[r]);
        p.flags[r] = reinterpret_cast<uint32_t*>(peer_flags[r]);
        B200Q_REQUIRE(p.recv[r] && p.flags[r] && aligned(p.recv[r], 16), "tp_allreduce_add_rmsnorm_flags: bad peer pointer");
    }
    const int chunks = int(hidden / 8);
    int threads = ((chunks + 31) / 32) * 32;
    threads = threads > 512 ? 512 : threads;
    const int held = (chunks + threads - 1) / threads;
    const dim3 grid{unsigned(rows)}, block{unsigned(threads)};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200Q_TP_LAUNCH(CPT)                                                                              \
    launch_overlapped(allreduce_flags_kernel<CPT>, grid, block, 0, s, p, size_t(slot_elems),        \
                      int(max_rows), static_cast<uint32_t*>(epoch), static_cast<uint32_t*>(done),         \
                      static_cast<int*>(error), static_cast<uint16_t*>(x),                                \
                      static_cast<const uint16_t*>(weight), static_cast<uint16_t*>(y), int(hidden), eps,     \
                      tp_wait_limit_ns())
    const cudaError_t err = held <= 1 ? B200Q_TP_LAUNCH(1) : held <= 2 ? B200Q_TP_LAUNCH(2)
                          : held <= 4 ? B200Q_TP_LAUNCH(4) : B200Q_TP_LAUNCH(0);
#undef B200Q_TP_LAUNCH
    return launch_status("tp_allreduce_add_rmsnorm_flags", err);
}
