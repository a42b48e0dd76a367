// Error reporting and device queries shared by every b200q entry point.
#include "common.cuh"

#include <cstring>
#include <mutex>
#include <vector>

namespace b200q {

char* error_buffer() {
    static thread_local char buffer[512] = "";
    return buffer;
}

static int32_t report(int32_t status, const char* format, va_list args) {
    vsnprintf(error_buffer(), 512, format, args);
    return status;
}

int32_t fail(const char* format, ...) {
    va_list args;
    va_start(args, format);
    const int32_t status = report(B200Q_ERROR, format, args);
    va_end(args);
    return status;
}

int32_t unavailable(const char* format, ...) {
    va_list args;
    va_start(args, format);
    const int32_t status = report(B200Q_UNAVAILABLE, format, args);
    va_end(args);
    return status;
}

int32_t launched(const char* what) {
    const cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) return B200Q_OK;
    return fail("%s: launch failed: %s", what, cudaGetErrorString(err));
}

int32_t launch_status(const char* what, cudaError_t err) {
    if (err == cudaSuccess) return launched(what);
    cudaGetLastError();
    return fail("%s: launch failed: %s", what, cudaGetErrorString(err));
}

int sm_count() {
    // Indexed by device ordinal; written once per device (benign if two host
    // threads race: both write the same value).
    static int cached[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (cached[device] == 0) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            count <= 0)
            count = 148;
        cached[device] = count;
    }
    return cached[device];
}

namespace {
struct KernelState {
    const void* kernel;
    int device;
    size_t smem;  // dynamic shared memory limit set so far
};
std::mutex g_kernel_mutex;
std::vector<KernelState> g_kernel_states;

// The entry of (kernel, current device), created on first use; `fresh` tells which.
KernelState& kernel_state(const void* kernel, bool* fresh) {
    int device = 0;
    cudaGetDevice(&device);
    for (KernelState& s : g_kernel_states)
        if (s.kernel == kernel && s.device == device) {
            *fresh = false;
            return s;
        }
    g_kernel_states.push_back(KernelState{kernel, device, 48 * 1024});
    *fresh = true;
    return g_kernel_states.back();
}
}  // namespace

cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes) {
    std::lock_guard<std::mutex> lock(g_kernel_mutex);
    bool fresh = false;
    KernelState& s = kernel_state(kernel, &fresh);
    if (bytes <= s.smem) return cudaSuccess;
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
    if (err == cudaSuccess) s.smem = bytes;
    return err;
}

bool first_use_on_device(const void* kernel) {
    std::lock_guard<std::mutex> lock(g_kernel_mutex);
    bool fresh = false;
    kernel_state(kernel, &fresh);
    return fresh;
}

}  // namespace b200q

extern "C" int32_t b200q_abi_version(void) { return B200Q_ABI_VERSION; }

extern "C" const char* b200q_last_error(void) { return b200q::error_buffer(); }

extern "C" int32_t b200q_device_ok(void) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess)
        return b200q::unavailable("no CUDA device is current");
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (major != 10)
        return b200q::unavailable("device %d has compute capability %d.x; these kernels are sm_100a only",
                                  device, major);
    return B200Q_OK;
}
