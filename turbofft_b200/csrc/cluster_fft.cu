// Instances of the single-pass cluster kernels, their registry, twiddle tables and launcher.
#include "cluster_fft.cuh"

#include <cmath>
#include <map>
#include <tuple>

#include "cluster_registry.h"

namespace tfft {

namespace {
typedef std::tuple<int, int, int, int> CKey;  // dtype, logn, logg, prefetch + 2 * variant
std::map<CKey, ClusterKernel>& ctable() {
    static std::map<CKey, ClusterKernel> t;
    return t;
}
std::map<std::pair<int, int>, int>& cdefault() {  // (dtype, logn) -> first registered logg
    static std::map<std::pair<int, int>, int> t;
    return t;
}
}  // namespace

void register_cluster_kernel(const ClusterKernel& k) {
    ctable()[CKey(k.dtype, k.logn, k.logg, k.prefetch + 2 * k.variant)] = k;
    if (!k.prefetch && !k.variant) cdefault().insert({{k.dtype, k.logn}, k.logg});
}

const ClusterKernel* find_cluster_kernel(int dtype, int logn, int logg, int flavour) {
    if (logg < 0) {
        auto d = cdefault().find({dtype, logn});
        if (d == cdefault().end()) return nullptr;
        logg = d->second;
    }
    auto it = ctable().find(CKey(dtype, logn, logg, flavour));
    return it == ctable().end() ? nullptr : &it->second;
}

int registered_cluster_kernel_count() { return (int)ctable().size(); }

template <typename T>
void cluster_twiddles(const ClusterKernel& k, std::vector<T>& tw0, std::vector<T> (&twp)[4]) {
    const long double two_pi = 6.283185307179586476925286766559005768L;
    const long long n = 1LL << k.logn, u = n >> 1;
    const int logt = k.logn - 1 - k.lr;
    tw0.clear();
    for (int j = 0; j < k.lr0; ++j)
        for (long long b = 0; b < (n >> k.lr0); ++b) {
            const long long idx = (b << j) & (n - 1);
            const long double ang = -two_pi * (long double)idx / (long double)n;
            tw0.push_back((T)cosl(ang));
            tw0.push_back((T)sinl(ang));
        }
    for (int t = 1; t < k.s2; ++t) {
        std::vector<T>& v = twp[t - 1];
        v.clear();
        const int lp = k.lr0 - 1 + k.lr * (t - 1);
        for (int j = 0; j < k.lr; ++j)
            for (long long q = 0; q < (1LL << (logt - lp)); ++q) {
                const long long idx = ((q << lp) << j) & (u - 1);
                const long double ang = -two_pi * (long double)idx / (long double)u;
                const T c = (T)cosl(ang), s = (T)sinl(ang);
                v.push_back(c);
                v.push_back(c);
                v.push_back(s);
                v.push_back(s);
            }
    }
}
template void cluster_twiddles<float>(const ClusterKernel&, std::vector<float>&, std::vector<float> (&)[4]);
template void cluster_twiddles<double>(const ClusterKernel&, std::vector<double>&, std::vector<double> (&)[4]);

static void fill_config(const ClusterKernel& k, long long n_clusters, cudaStream_t stream, cudaLaunchConfig_t& cfg,
                        cudaLaunchAttribute* attr) {
    cfg = cudaLaunchConfig_t();
    cfg.gridDim = dim3((unsigned)(n_clusters << k.logg));
    cfg.blockDim = dim3((unsigned)k.threads);
    cfg.dynamicSmemBytes = k.smem;
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1u << k.logg;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
}

cudaError_t launch_cluster_kernel(const ClusterKernel& k, void* args, long long n_clusters, cudaStream_t stream) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    fill_config(k, n_clusters, stream, cfg, attr);
    void* kargs[] = {args};
    return cudaLaunchKernelExC(&cfg, k.fn, kargs);
}

int cluster_kernel_fits(const ClusterKernel& k) {
    if (cudaFuncSetAttribute(k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k.smem) != cudaSuccess) return 0;
    if (k.logg > 3 && cudaFuncSetAttribute(k.fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    fill_config(k, 1, nullptr, cfg, attr);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, k.fn, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

}  // namespace tfft

#define TFFT_CLUSTER_INST_X(T, DT, LOGN, LR0, LOGG, PF, LRU)                                                   \
    template __global__ void tfft::cluster_fft_kernel<T, LOGN, LR0, LOGG, PF, LRU>(                            \
        const __grid_constant__ tfft::ClusterArgs<T>);                                                         \
    namespace {                                                                                                \
    struct TFFT_CAT(TfftClReg_, __LINE__) {                                                                    \
        TFFT_CAT(TfftClReg_, __LINE__)() {                                                                     \
            typedef tfft::ClusterCfg<T, LOGN, LR0, LOGG, LRU> K;                                               \
            tfft::ClusterKernel k;                                                                             \
            k.fn = (const void*)&tfft::cluster_fft_kernel<T, LOGN, LR0, LOGG, PF, LRU>;                        \
            k.dtype = DT;                                                                                      \
            k.logn = LOGN;                                                                                     \
            k.lr0 = LR0;                                                                                       \
            k.lr = K::LR;                                                                                      \
            k.logg = LOGG;                                                                                     \
            k.s2 = K::S2;                                                                                      \
            k.prefetch = PF ? 1 : 0;                                                                           \
            k.variant = (sizeof(T) == 4 && LRU == 3) ? 1 : 0;                                                  \
            k.threads = K::TH;                                                                                 \
            k.smem = PF ? K::SMEM_BYTES_PF : K::SMEM_BYTES;                                                    \
            tfft::register_cluster_kernel(k);                                                                  \
        }                                                                                                      \
    } TFFT_CAT(tfft_clreg_, __LINE__);                                                                         \
    }
#define TFFT_CLUSTER_INST_PF(T, DT, LOGN, LR0, LOGG, PF) TFFT_CLUSTER_INST_X(T, DT, LOGN, LR0, LOGG, PF, (sizeof(T) == 4 ? 4 : 3))
#define TFFT_CLUSTER_INST(T, DT, LOGN, LR0, LOGG) TFFT_CLUSTER_INST_PF(T, DT, LOGN, LR0, LOGG, false)
#define TFFT_CAT2(a, b) a##b
#define TFFT_CAT(a, b) TFFT_CAT2(a, b)

// complex64: N = R0 * 16^3.  The first instance of a size is its default cluster size (the
// fastest measured: CTAs of 128 threads, four per SM, overlap their phases best).
TFFT_CLUSTER_INST(float, 0, 13, 1, 0)
TFFT_CLUSTER_INST(float, 0, 13, 1, 1)
TFFT_CLUSTER_INST(float, 0, 14, 2, 1)
TFFT_CLUSTER_INST(float, 0, 14, 2, 2)
TFFT_CLUSTER_INST(float, 0, 14, 2, 0)
TFFT_CLUSTER_INST(float, 0, 15, 3, 3)
TFFT_CLUSTER_INST(float, 0, 15, 3, 2)
TFFT_CLUSTER_INST(float, 0, 15, 3, 1)
TFFT_CLUSTER_INST(float, 0, 16, 4, 4)
TFFT_CLUSTER_INST(float, 0, 16, 4, 3)
TFFT_CLUSTER_INST(float, 0, 16, 4, 2)
TFFT_CLUSTER_INST(float, 0, 17, 5, 4)
TFFT_CLUSTER_INST(float, 0, 17, 5, 3)
// complex128: N = R0 * 8^S2
TFFT_CLUSTER_INST(double, 1, 12, 3, 0)
TFFT_CLUSTER_INST(double, 1, 13, 4, 1)
TFFT_CLUSTER_INST(double, 1, 14, 2, 2)
TFFT_CLUSTER_INST(double, 1, 15, 3, 3)
TFFT_CLUSTER_INST(double, 1, 16, 4, 4)
TFFT_CLUSTER_INST(double, 1, 16, 4, 3)
// prefetching variants (CTAs of 128 threads: exchange and landing buffers of three CTAs fit one SM)
TFFT_CLUSTER_INST_PF(float, 0, 13, 1, 1, true)
TFFT_CLUSTER_INST_PF(float, 0, 14, 2, 2, true)
TFFT_CLUSTER_INST_PF(float, 0, 15, 3, 3, true)
TFFT_CLUSTER_INST_PF(float, 0, 16, 4, 4, true)
// complex64 with 8 units per thread (radix-8 unit stages): half the registers, twice the warps
TFFT_CLUSTER_INST_X(float, 0, 13, 4, 1, false, 3)
TFFT_CLUSTER_INST_X(float, 0, 14, 2, 2, false, 3)
TFFT_CLUSTER_INST_X(float, 0, 15, 3, 3, false, 3)
TFFT_CLUSTER_INST_X(float, 0, 16, 4, 4, false, 3)
TFFT_CLUSTER_INST_X(float, 0, 15, 3, 4, false, 3)
