// The tail shared by the few-row (decode) kernels: partial sums of the warps of a
// block, and of the blocks of a cluster when K is split over one, meet in
// (distributed) shared memory; the first block of the cluster writes y.  No global
// scratch memory and no atomics.
#pragma once

#include <cooperative_groups.h>

#include "mma.cuh"

namespace b200q {

namespace cg = cooperative_groups;

// total[nt][mb][i] holds this thread's m16n8 accumulator fragments: rows g (i=0,1)
// and g+8 (i=2,3) of 16-row tile nt, activation rows mb*8 + 2t and 2t+1.
// red: shared memory, W * NT*16 * MB*8 floats, at the same offset in every block
// of the cluster.
template <typename H, int MB, int NT, int W>
__device__ __forceinline__ void reduce_and_store(const float (&total)[NT][MB][4], float* red,
                                                 int ksplit, int tile_row, int M, int N,
                                                 uint16_t* y) {
    constexpr int kCols = MB * 8, kRows = NT * 16;
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int g = lane / 4, t = lane % 4;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            float* dst = red + (size_t(warp) * kRows + nt * 16 + g) * kCols + mb * 8 + 2 * t;
            dst[0] = total[nt][mb][0];
            dst[1] = total[nt][mb][1];
            dst[8 * kCols] = total[nt][mb][2];
            dst[8 * kCols + 1] = total[nt][mb][3];
        }
    __syncthreads();
    for (int e = threadIdx.x; e < kRows * kCols; e += W * 32) {
        float sum = red[e];
#pragma unroll
        for (int w = 1; w < W; ++w) sum += red[size_t(w) * kRows * kCols + e];
        red[e] = sum;  // element e is only ever touched by this thread
    }
    if (ksplit > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (cluster.block_rank() == 0) {
            for (int e = threadIdx.x; e < kRows * kCols; e += W * 32) {
                float sum = red[e];
                for (int r = 1; r < ksplit; ++r) sum += cluster.map_shared_rank(red, r)[e];
                red[e] = sum;
            }
        }
        cluster.sync();  // peers stay resident until rank 0 has read them
        if (cluster.block_rank() != 0) return;
    }
    __syncthreads();
    // red is [row][col]; y is [m][n]: walk rows fastest so stores coalesce.
    for (int e = threadIdx.x; e < kRows * kCols; e += W * 32) {
        const int m = e / kRows, r = e % kRows;
        const int n = tile_row + r;
        if (m < M && n < N) y[size_t(m) * N + n] = H::from_float(red[size_t(r) * kCols + m]);
    }
}

// Launches `kernel` on a (tiles, ksplit) grid whose y extent forms one cluster.
// `overlap`: launch with programmatic stream serialization (the kernel must call
// pdl_wait() before reading activations or writing outputs).
template <typename Kernel, typename Args>
int32_t launch_clustered(const char* who, Kernel kernel, const Args& args, int tiles, int ksplit,
                         int threads, size_t smem, cudaStream_t stream, bool overlap = false) {
    if (smem > 227 * 1024) return fail("%s: %zu bytes of shared memory needed", who, smem);
    ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(unsigned(tiles), unsigned(ksplit), 1);
    config.blockDim = dim3(unsigned(threads), 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = unsigned(ksplit);
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = overlap ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&config, kernel, args);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail("%s: launch failed: %s", who, cudaGetErrorString(err));
    }
    return B200Q_OK;
}

}  // namespace b200q
