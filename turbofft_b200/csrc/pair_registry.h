// Table of the fused two-launch kernels (pair_fft.cuh) and their launcher.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace tfft {

struct PairKernel {
    const void* fn = nullptr;
    int dtype = 0;
    int logm1 = 0, loge1 = 0, logc1 = 0;  // first launch: line length, points per thread, lines per tile (log2)
    int logm2 = 0, loge2 = 0, logc2 = 0;  // last launch
    int threads = 0;
    size_t smem = 0;
};

void register_pair_kernel(const PairKernel& k);
const PairKernel* find_pair_kernel(int dtype, int logm1, int loge1, int logc1, int logm2, int loge2, int logc2);
int registered_pair_kernel_count();

// Blocks of this kernel that can be resident on the current device at once (0 on error); sets
// the kernel's dynamic shared memory limit on the way.
int pair_kernel_resident_blocks(const PairKernel& k);
// Cooperative launch of `grid` blocks (grid <= pair_kernel_resident_blocks); args is a PairArgs<float|double>.
cudaError_t launch_pair_kernel(const PairKernel& k, void* args, int grid, cudaStream_t stream);

}  // namespace tfft
