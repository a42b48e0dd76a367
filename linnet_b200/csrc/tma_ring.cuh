// Pieces shared by the decode kernels whose weights come through the TMA unit into a ring of
// shared-memory stages (int4_gemv_tma.cuh, int8_gemv_tma.cuh): shared-memory accesses by 32-bit
// address, the first MMA of a chain, one TMA box of 64-byte pieces, mbarrier waits with a bound.
#pragma once

#include <cuda.h>

#include "gemv_common.cuh"
#include "umma.cuh"

namespace b200q {

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
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
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

// One of the two 16-bit scales of a word, as f32.
template <typename T>
__device__ __forceinline__ float scale_of(uint32_t word, int odd);
template <>
__device__ __forceinline__ float scale_of<__nv_bfloat16>(uint32_t word, int odd) {
    return __uint_as_float(__byte_perm(word, 0, odd ? 0x3244 : 0x1044));
}
template <>
__device__ __forceinline__ float scale_of<__half>(uint32_t word, int odd) {
    return __half2float(__ushort_as_half(uint16_t(odd ? word >> 16 : word & 0xFFFFu)));
}

// One box of the weight map -> shared memory; the barrier receives the bytes.
__device__ __forceinline__ void tma_item(uint32_t dst, const CUtensorMap* map, int row, int kblock, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(map), "r"(0), "r"(row), "r"(kblock), "r"(bar)
        : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_test_wait(uint32_t bar, uint32_t parity) {  // does not suspend the thread
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false (and the status word set) after about a second, or as soon as another
// warp of the device has given up.  SPIN: poll without suspending (the producer, one thread,
// which should see a freed stage at once); otherwise the hardware may park the warp a while.
template <bool SPIN = false>
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
    if (SPIN ? bar_test_wait(bar, parity) : bar_try_wait(bar, parity)) return true;
    const uint64_t start = umma::global_timer_ns();
    for (uint32_t spins = 0;; ++spins) {
        if (SPIN ? bar_test_wait(bar, parity) : bar_try_wait(bar, parity)) return true;
        if ((spins & 1023u) == 1023u) {
            if (*reinterpret_cast<volatile int*>(status) != 0) return false;
            if (umma::global_timer_ns() - start > 1000000000ull) {
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

}  // namespace b200q
