// Instances of the fused two-launch kernels, their registry and launcher.
#include "pair_fft.cuh"

#include <map>
#include <tuple>

#include "pair_registry.h"

namespace tfft {

namespace {
typedef std::tuple<int, int, int, int, int, int, int> PKey;
std::map<PKey, PairKernel>& ptable() {
    static std::map<PKey, PairKernel> t;
    return t;
}
}  // namespace

void register_pair_kernel(const PairKernel& k) {
    ptable()[PKey(k.dtype, k.logm1, k.loge1, k.logc1, k.logm2, k.loge2, k.logc2)] = k;
}

const PairKernel* find_pair_kernel(int dtype, int logm1, int loge1, int logc1, int logm2, int loge2, int logc2) {
    auto it = ptable().find(PKey(dtype, logm1, loge1, logc1, logm2, loge2, logc2));
    return it == ptable().end() ? nullptr : &it->second;
}

int registered_pair_kernel_count() { return (int)ptable().size(); }

int pair_kernel_resident_blocks(const PairKernel& k) {
    if (k.smem > 40 * 1024 &&
        cudaFuncSetAttribute(k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k.smem) != cudaSuccess)
        return 0;
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k.fn, k.threads, k.smem) != cudaSuccess) return 0;
    return sms * per_sm;
}

cudaError_t launch_pair_kernel(const PairKernel& k, void* args, int grid, cudaStream_t stream) {
    void* params[] = {args};
    return cudaLaunchCooperativeKernel(k.fn, dim3((unsigned)grid), dim3((unsigned)k.threads), params, k.smem, stream);
}

}  // namespace tfft

#define TFFT_PAIR_CAT2(a, b) a##b
#define TFFT_PAIR_CAT(a, b) TFFT_PAIR_CAT2(a, b)
#define TFFT_PAIR_INST(T, DT, M1, E1, C1, M2, E2, C2)                                                       \
    template __global__ void tfft::fft_pair_kernel<T, M1, E1, C1, M2, E2, C2>(                              \
        const __grid_constant__ tfft::PairArgs<T>);                                                         \
    namespace {                                                                                             \
    struct TFFT_PAIR_CAT(TfftPairReg_, __LINE__) {                                                          \
        TFFT_PAIR_CAT(TfftPairReg_, __LINE__)() {                                                           \
            typedef tfft::PairCfg<T, M1, E1, C1, M2, E2, C2> P;                                             \
            tfft::PairKernel k;                                                                             \
            k.fn = (const void*)&tfft::fft_pair_kernel<T, M1, E1, C1, M2, E2, C2>;                          \
            k.dtype = DT;                                                                                   \
            k.logm1 = M1, k.loge1 = E1, k.logc1 = C1, k.logm2 = M2, k.loge2 = E2, k.logc2 = C2;             \
            k.threads = P::THREADS;                                                                         \
            k.smem = P::SMEM_BYTES;                                                                         \
            tfft::register_pair_kernel(k);                                                                  \
        }                                                                                                   \
    } TFFT_PAIR_CAT(tfft_pair_reg_, __LINE__);                                                              \
    }

// complex64: the launches of the built-in rows 15 and 16 (256 threads each)
TFFT_PAIR_INST(float, 0, 8, 4, 4, 7, 4, 5)
TFFT_PAIR_INST(float, 0, 8, 4, 4, 8, 4, 4)
// complex128: row 16
TFFT_PAIR_INST(double, 1, 8, 4, 4, 8, 4, 4)
