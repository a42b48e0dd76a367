// Tensor-parallel epilogue of a row-split layer in ONE kernel: all-reduce of the ranks'
// partial sums over NVLink peer memory + residual add + RMSNorm.
//
// The reference sums the partial results of a `Shards` card with
// `std.nn.parallel::all_reduce` (stdlib/nn/parallel.linnet:9-11), which its runtime runs
// as a one-shot Triton kernel over symmetric memory for messages up to 128 KiB and NCCL
// otherwise (python/linnet/src/linnet/torch/collectives.py:145-167; kernel at
// python/linnet/src/linnet/torch/kernels.py:1107-1156, which spins without a bound).  A
// batch-1 decode step has 64 such reductions of 8 KiB: their latency, not their bytes,
// is the cost, and each is followed by a residual add and a norm.  This kernel does the
// three in one launch with plain peer stores and local loads (no multimem, no TMA), and
// with no barrier, fence or separate flag between the ranks:
//   1. every rank has a receive area per call site, [source rank][rows][hidden / 2] words
//      of 8 bytes: two bf16 values and the site's 32-bit epoch.  One block per row reads
//      this rank's partial sums and stores them, word by word with the epoch attached,
//      into its slot of every peer's area.  A word is ONE 64-bit element of the store and of
//      the polling load (st/ld.relaxed.sys.v2.b64): the memory model makes each element of a
//      vector access single-copy atomic, so a word whose epoch matches carries this call's
//      values (with 32-bit elements an epoch could be seen before the value beside it);
//   2. the block then reads the words the peers stored into its own area, polling (with a
//      bound) each until its epoch matches, adds the rows in rank order (the same order on
//      every rank, so all ranks get the same bits), rounds the sum to bf16 as an all-reduce
//      of bf16 tensors returns it, adds it to the residual stream x in place and writes
//      y = rms_norm(x) * weight.
// Latency is one NVLink crossing: nobody waits for an acknowledgement, a release or a remote
// load.  (The versions before this one: pull the peers' rows after a flag barrier; push the
// rows, fence, then push a flag per row.  Each ordering step cost microseconds per call.)
// One area per call site: a rank can only write a site's slots again after every rank has
// passed the NEXT site, i.e. after it finished reading this one (the caller alternates at
// least two sites).  Epochs live in device memory and advance once per call (the last
// block to finish bumps the site's counter), so the kernel replays inside a CUDA graph.  A
// poll that runs out (a second unless b200q_set_wait_limit_ns says otherwise) records an error code and lets the kernel finish
// with whatever it has; the context stays usable, and later calls skip their polls until
// the host clears the code.
#include "common.cuh"

namespace b200q {
uint64_t tp_wait_limit_ns();
namespace {

constexpr int kMaxRanks = 8;

struct Peers {
    uint2* area[kMaxRanks];  // every rank's receive area of this site [world][slot_words] of (2 bf16, epoch)
    int world, rank;
};

__device__ __forceinline__ float lo16(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi16(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}
// Two words of (values, epoch), each one 64-bit element: values in the low half.
struct Words2 {
    uint64_t a, b;
};
__device__ __forceinline__ Words2 ld_words(const void* p) {
    Words2 v;
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0,%1}, [%2];" : "=l"(v.a), "=l"(v.b) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_words(void* p, uint64_t a, uint64_t b) {
    asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1,%2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ uint64_t tagged(uint32_t values, uint32_t epoch) {
    return uint64_t(values) | (uint64_t(epoch) << 32);
}

// One 16-byte piece (8 bf16) of a row per thread and step; CPT pieces are kept in registers
// from the push to the scaling (0: any width, rows re-read from memory).
template <int CPT>
__global__ void __launch_bounds__(512)
allreduce_add_rmsnorm_kernel(const Peers p, size_t slot_words, const uint16_t* partial,
                             uint32_t* __restrict__ epoch, uint32_t* __restrict__ done,
                             int* __restrict__ error, uint16_t* x, const uint16_t* __restrict__ weight,
                             uint16_t* __restrict__ y, int hidden, float eps, uint64_t wait_limit_ns) {
    __shared__ float partial_sums[16];
    constexpr int kHeld = CPT > 0 ? CPT : 1;
    const int row = blockIdx.x, chunks = hidden / 8;
    const uint4* wr = reinterpret_cast<const uint4*>(weight);
    uint4 g[kHeld], v[kHeld];
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
    // After one poll has run out every later call returns at once instead of waiting again.
    bool gave_up = *reinterpret_cast<volatile int*>(error) != 0;

    const uint4* mine = reinterpret_cast<const uint4*>(partial + size_t(row) * hidden);
    const size_t row_words = size_t(row) * (hidden / 2);  // this row inside a slot, in words
    uint4* xr = reinterpret_cast<uint4*>(x + size_t(row) * hidden);
    float sum_sq = 0.0f;

    // piece c: push it to every peer, collect the peers' pieces, reduce, add, square
    auto exchange = [&](int c) {
        const uint4 own = ld_mutable(mine + c);
        for (int peer = 0; peer < p.world; ++peer)
            if (peer != p.rank) {
                uint2* dst = p.area[peer] + size_t(p.rank) * slot_words + row_words + 4 * c;
                st_words(dst, tagged(own.x, e), tagged(own.y, e));
                st_words(dst + 2, tagged(own.z, e), tagged(own.w, e));
            }
        uint4 t = ld_mutable(xr + c);
        uint4 q[kMaxRanks];
        unsigned pending = 0;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            q[r] = make_uint4(0, 0, 0, 0);
            if (r < p.world && r != p.rank) pending |= 1u << r;
        }
        if (gave_up) pending = 0;
        uint64_t start = 0;
        for (uint32_t spins = 0; pending != 0; ++spins) {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (pending & (1u << r)) {
                    const uint2* src = p.area[p.rank] + size_t(r) * slot_words + row_words + 4 * c;
                    const Words2 lo = ld_words(src), hi = ld_words(src + 2);
                    if (uint32_t(lo.a >> 32) == e && uint32_t(lo.b >> 32) == e && uint32_t(hi.a >> 32) == e &&
                        uint32_t(hi.b >> 32) == e) {
                        q[r] = make_uint4(uint32_t(lo.a), uint32_t(lo.b), uint32_t(hi.a), uint32_t(hi.b));
                        pending &= ~(1u << r);
                    }
                }
            if (pending != 0 && (spins & 63u) == 63u) {
                uint64_t now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                if (start == 0) start = now;
                if (now - start > wait_limit_ns) {  // a peer never arrived: give up, stay usable
                    atomicCAS(error, 0, 100 + (__ffs(int(pending)) - 1));
                    gave_up = true;
                    pending = 0;
                }
            }
        }
        if (gave_up) return t;
        float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            if (r >= p.world) break;
            const uint4 qr = r == p.rank ? own : q[r];
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
            if (c < chunks) v[u] = exchange(c);
        }
    } else {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) exchange(c);
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

// The exchange alone: out[i] = round(sum over ranks of in_r[i]), summed in f32 in rank order.
// One 16-byte piece (8 values) per thread; bf16 or f16.
template <bool F16>
__global__ void __launch_bounds__(512)
allreduce_words_kernel(const Peers p, size_t slot_words, const uint16_t* in, uint32_t* __restrict__ epoch,
                       uint32_t* __restrict__ done, int* __restrict__ error, uint16_t* __restrict__ out, int pieces,
                       uint64_t wait_limit_ns) {
    pdl_launch_dependents();  // the next kernel may start its own prologue (a product: its weight fetch) at once
    pdl_wait();
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(epoch) + 1;
    bool gave_up = *reinterpret_cast<volatile int*>(error) != 0;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < pieces) {
        const uint4 own = ld_mutable(reinterpret_cast<const uint4*>(in) + c);
        for (int peer = 0; peer < p.world; ++peer)
            if (peer != p.rank) {
                uint2* dst = p.area[peer] + size_t(p.rank) * slot_words + size_t(4) * c;
                st_words(dst, tagged(own.x, e), tagged(own.y, e));
                st_words(dst + 2, tagged(own.z, e), tagged(own.w, e));
            }
        uint4 q[kMaxRanks];
        unsigned pending = 0;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            q[r] = make_uint4(0, 0, 0, 0);
            if (r < p.world && r != p.rank) pending |= 1u << r;
        }
        if (gave_up) pending = 0;
        uint64_t start = 0;
        for (uint32_t spins = 0; pending != 0; ++spins) {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (pending & (1u << r)) {
                    const uint2* src = p.area[p.rank] + size_t(r) * slot_words + size_t(4) * c;
                    const Words2 lo = ld_words(src), hi = ld_words(src + 2);
                    if (uint32_t(lo.a >> 32) == e && uint32_t(lo.b >> 32) == e && uint32_t(hi.a >> 32) == e &&
                        uint32_t(hi.b >> 32) == e) {
                        q[r] = make_uint4(uint32_t(lo.a), uint32_t(lo.b), uint32_t(hi.a), uint32_t(hi.b));
                        pending &= ~(1u << r);
                    }
                }
            if (pending != 0 && (spins & 63u) == 63u) {
                uint64_t now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                if (start == 0) start = now;
                if (now - start > wait_limit_ns) {  // a peer never arrived: give up, stay usable
                    atomicCAS(error, 0, 100 + (__ffs(int(pending)) - 1));
                    gave_up = true;
                    pending = 0;
                }
            }
        }
        if (!gave_up) {
            auto low = [](uint32_t v) { return F16 ? __half2float(__ushort_as_half(uint16_t(v & 0xFFFFu))) : lo16(v); };
            auto high = [](uint32_t v) { return F16 ? __half2float(__ushort_as_half(uint16_t(v >> 16))) : hi16(v); };
            float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r) {
                if (r >= p.world) break;
                const uint4 qr = r == p.rank ? own : q[r];
                s[0] += low(qr.x); s[1] += high(qr.x); s[2] += low(qr.y); s[3] += high(qr.y);
                s[4] += low(qr.z); s[5] += high(qr.z); s[6] += low(qr.w); s[7] += high(qr.w);
            }
            auto pack = [](float a, float b) {
                if (!F16) return pack16(a, b);
                __half2 h = __floats2half2_rn(a, b);
                return *reinterpret_cast<uint32_t*>(&h);
            };
            reinterpret_cast<uint4*>(out)[c] = make_uint4(pack(s[0], s[1]), pack(s[2], s[3]), pack(s[4], s[5]), pack(s[6], s[7]));
        }
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

// How long the tensor-parallel kernels wait for a peer before they give up (shared with
// tp_allreduce_flags.cu).
static uint64_t g_tp_wait_limit_ns = 1000000000ull;
uint64_t tp_wait_limit_ns() { return g_tp_wait_limit_ns; }

}  // namespace b200q

using namespace b200q;

extern "C" int32_t b200q_set_wait_limit_ns(int64_t nanoseconds) {
    B200Q_REQUIRE(nanoseconds > 0 && nanoseconds <= 60000000000ll, "set_wait_limit_ns: between 1 ns and 60 s");
    g_tp_wait_limit_ns = uint64_t(nanoseconds);
    return B200Q_OK;
}

extern "C" int32_t b200q_tp_allreduce_add_rmsnorm(const int64_t* peer_areas, int64_t slot_words,
                                                  const void* partial, int32_t world, int32_t rank,
                                                  void* epoch, void* done, void* error, void* x,
                                                  const void* weight, void* y, int64_t rows, int64_t hidden,
                                                  float eps, void* stream) {
    B200Q_REQUIRE(world >= 2 && world <= kMaxRanks && rank >= 0 && rank < world,
                  "tp_allreduce_add_rmsnorm: 2..8 ranks, got world=%d rank=%d", world, rank);
    B200Q_REQUIRE(rows >= 0 && hidden > 0 && hidden % 8 == 0, "tp_allreduce_add_rmsnorm: hidden must be a multiple of 8");
    B200Q_REQUIRE(slot_words >= rows * (hidden / 2) && slot_words % 2 == 0,
                  "tp_allreduce_add_rmsnorm: %lld rows of %lld do not fit slots of %lld words", (long long)rows,
                  (long long)hidden, (long long)slot_words);
    if (rows == 0) return B200Q_OK;
    B200Q_REQUIRE(peer_areas && partial && epoch && done && error && x && weight && y && aligned(partial, 16),
                  "tp_allreduce_add_rmsnorm: null or misaligned argument");
    Peers p{};
    p.world = world;
    p.rank = rank;
    for (int r = 0; r < world; ++r) {
        p.area[r] = reinterpret_cast<uint2*>(peer_areas[r]);
        B200Q_REQUIRE(p.area[r] && aligned(p.area[r], 16), "tp_allreduce_add_rmsnorm: bad peer pointer");
    }
    const int chunks = int(hidden / 8);
    int threads = ((chunks + 31) / 32) * 32;
    threads = threads > 512 ? 512 : threads;
    const int held = (chunks + threads - 1) / threads;
    const dim3 grid{unsigned(rows)}, block{unsigned(threads)};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200Q_TP_LAUNCH(CPT)                                                                              \
    launch_overlapped(allreduce_add_rmsnorm_kernel<CPT>, grid, block, 0, s, p, size_t(slot_words),        \
                      static_cast<const uint16_t*>(partial), static_cast<uint32_t*>(epoch),               \
                      static_cast<uint32_t*>(done), static_cast<int*>(error), static_cast<uint16_t*>(x),  \
                      static_cast<const uint16_t*>(weight), static_cast<uint16_t*>(y), int(hidden), eps,     \
                      tp_wait_limit_ns())
    const cudaError_t err = held <= 1 ? B200Q_TP_LAUNCH(1) : held <= 2 ? B200Q_TP_LAUNCH(2)
                          : held <= 4 ? B200Q_TP_LAUNCH(4) : B200Q_TP_LAUNCH(0);
#undef B200Q_TP_LAUNCH
    return launch_status("tp_allreduce_add_rmsnorm", err);
}

extern "C" int32_t b200q_tp_allreduce(const int64_t* peer_areas, int64_t slot_words, const void* in, int32_t world,
                                      int32_t rank, void* epoch, void* done, void* error, void* out, int64_t count,
                                      int32_t dtype, void* stream) {
    B200Q_REQUIRE(world >= 2 && world <= kMaxRanks && rank >= 0 && rank < world,
                  "tp_allreduce: 2..8 ranks, got world=%d rank=%d", world, rank);
    B200Q_REQUIRE(dtype == B200Q_BF16 || dtype == B200Q_F16, "tp_allreduce: bf16 or f16");
    B200Q_REQUIRE(count >= 0 && count % 8 == 0, "tp_allreduce: a multiple of 8 values, not %lld", (long long)count);
    B200Q_REQUIRE(slot_words >= count / 2 && slot_words % 2 == 0, "tp_allreduce: %lld values do not fit slots of %lld words",
                  (long long)count, (long long)slot_words);
    if (count == 0) return B200Q_OK;
    B200Q_REQUIRE(peer_areas && in && epoch && done && error && out && aligned(in, 16) && aligned(out, 16),
                  "tp_allreduce: null or misaligned argument");
    Peers p{};
    p.world = world;
    p.rank = rank;
    for (int r = 0; r < world; ++r) {
        p.area[r] = reinterpret_cast<uint2*>(peer_areas[r]);
        B200Q_REQUIRE(p.area[r] && aligned(p.area[r], 16), "tp_allreduce: bad peer pointer");
    }
    const int pieces = int(count / 8);
    const int threads = pieces < 256 ? ((pieces + 31) / 32) * 32 : 256;
    const dim3 grid{unsigned((pieces + threads - 1) / threads)}, block{unsigned(threads)};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t err =
        dtype == B200Q_F16
            ? launch_overlapped(allreduce_words_kernel<true>, grid, block, 0, s, p, size_t(slot_words),
                                static_cast<const uint16_t*>(in), static_cast<uint32_t*>(epoch), static_cast<uint32_t*>(done),
                                static_cast<int*>(error), static_cast<uint16_t*>(out), pieces, tp_wait_limit_ns())
            : launch_overlapped(allreduce_words_kernel<false>, grid, block, 0, s, p, size_t(slot_words),
                                static_cast<const uint16_t*>(in), static_cast<uint32_t*>(epoch), static_cast<uint32_t*>(done),
                                static_cast<int*>(error), static_cast<uint16_t*>(out), pieces, tp_wait_limit_ns());
    return launch_status("tp_allreduce", err);
}
