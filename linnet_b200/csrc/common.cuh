// Shared helpers of the b200q kernels: error reporting, argument checks and a
// few PTX wrappers.  Device code here targets sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/b200q.h"

namespace b200q {

// Message of the last failure on this host thread (read by b200q_last_error).
char* error_buffer();
int32_t fail(const char* format, ...);
int32_t unavailable(const char* format, ...);

// After a launch: turns a launch error into a status + message.  Never
// synchronises (an asynchronous fault shows at the caller's next sync).
int32_t launched(const char* what);
// The same for a launch call that returned `err`.
int32_t launch_status(const char* what, cudaError_t err);

inline bool aligned(const void* p, size_t bytes) {
    return (reinterpret_cast<uintptr_t>(p) % bytes) == 0;
}

// Shared argument validation of the int4 linear entry points.
int32_t check_int4_args(const char* who, const void* x, const uint8_t* packed, const void* scale,
                        const uint8_t* zero, void* y, int64_t rows, int64_t in, int64_t out,
                        int64_t group, int32_t dtype);

// Multiprocessor count of the current device (cached per device).
int sm_count();

// Function attributes are set once per (kernel, device), not per launch.
// ensure_dynamic_smem: makes `bytes` of dynamic shared memory launchable for `kernel` on the
// current device (a runtime call only when the limit set so far is lower).
// first_use_on_device: true the first time `kernel` is seen on the current device.
cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes);
bool first_use_on_device(const void* kernel);

#define B200Q_REQUIRE(cond, ...)                 \
    do {                                         \
        if (!(cond)) return ::b200q::fail(__VA_ARGS__); \
    } while (0)

// Device-side status of the decode-step kernels: a kernel that finds a position outside its
// cache records 1 + the batch row in this word (on the current device) and leaves the caches
// alone; b200q_decoder_status() reports and clears it.  The word lives in decoder_glue.cu;
// kernels get its device address as an argument.  nullptr if the address cannot be had.
int* decoder_error_word();
// Device address of the word that kernels with shared-memory pipelines (the tensor-core GEMMs,
// the TMA decode kernel) set when one of their bounded waits expires; read and cleared by
// b200q_int4_gemm_status().  Null when the device cannot be asked.
int* gemm_error_word();
__device__ __forceinline__ void record_bad_position(int* word, int row) {
    if (word != nullptr) atomicCAS(word, 0, 1 + row);
}

// ---- programmatic dependent launch ------------------------------------------
// A kernel launched with launch_overlapped() may start while the kernel before it in
// the stream is still draining; it must call pdl_wait() before it reads anything an
// earlier kernel wrote and before it writes anything an earlier kernel may still read.
// Chains of such kernels hide most of the launch latency between them.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... Params, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, Params(args)...);
}

// ---- device helpers -------------------------------------------------------

// Data written by earlier kernels of the stream (activations, positions, partial results)
// and programmatic dependent launch.  A kernel launched that way starts while the kernels
// before it are still running, and inside a CUDA graph the read-only data cache is not
// invalidated between such kernels: a decode step that reuses an address for a new tensor
// (the allocator does all the time) was served the old tensor's lines through __ldg.  So
// such data is never read through the non-coherent path here (no __ldg, no ld.global.nc, no
// const __restrict__ pointer, which lets the compiler pick it), and only after pdl_wait():
//   * ld_mutable(): ld.global.cg, which neither allocates in L1 nor hits in it; used wherever
//     a value is read once (the small kernels, staging into shared memory);
//   * ordinary coherent loads (ld.global.ca) where L1 reuse pays (the decode product's
//     activation fragments), which griddepcontrol.wait orders after the producer's stores.
// Weights, scales, zero points, norm weights and tables never change: any path will do.
__device__ __forceinline__ uint4 ld_mutable(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_mutable(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ld_mutable(const uint16_t* p) {
    uint16_t v;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_mutable(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ int64_t ld_mutable(const int64_t* p) {
    int64_t v;
    asm volatile("ld.global.cg.s64 %0, [%1];" : "=l"(v) : "l"(p));
    return v;
}
// An ordinary coherent load (through L1) as an instruction the compiler may move like
// arithmetic; it stays below pdl_wait() because its address is derived from a pointer that
// went through below_pdl_wait() after the wait.
__device__ __forceinline__ uint4 ld_activation_free(const uint4* p) {
    uint4 v;
    asm("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
template <typename P>
__device__ __forceinline__ P* below_pdl_wait(P* p) {
    asm volatile("" : "+l"(p));  // volatile: stays after the wait; opaque: nothing derived from p moves above it
    return p;
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    // 128-bit read-only load that does not allocate in L1: weight bytes are
    // used exactly once.
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t bits) {
    // (a & mask) | bits in one LOP3.
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(bits));
    return r;
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}

// Two bf16 values packed in 32 bits <-> f32.
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t bf16_pack(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

}  // namespace b200q
