// Table of the single-pass cluster kernels (cluster_fft.cuh) and the host helpers that build
// their twiddle tables and launch them.  No counterpart in the reference, whose plans for the
// same sizes are two launches (include/param/A100/param_float2.csv rows 13-17).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <vector>

#include "fft_kernels.cuh"

namespace tfft {

// Argument block of cluster_fft_kernel (cluster_fft.cuh).
template <typename T>
struct ClusterArgs {
    typedef typename Cplx<T>::type C;
    const C* in;
    C* out;
    const C* tw0;     // stage 0: [j < LR0][b < N / R0] = W_N^(b * 2^j)
    const T* twp[4];  // stage t = 1 .. S2-1: [j < LR][k < T >> LP't] = (wr, wr, wi, wi), w = W_U^((k << LP't) * 2^j)
    long long n_signals;
    int signals_per_cluster;
    int conj_in;    // conjugate while loading (inverse transform)
    int scale_out;  // scale while storing: y = (y.x * scale_x, y.y * scale_y)
    T scale_x, scale_y;
    int* status;  // prefetching variant: set to 1 if a wait for the landing buffer ever gave up
};

struct ClusterKernel {
    const void* fn = nullptr;
    int dtype = 0, logn = 0, lr0 = 0, lr = 0, logg = 0, s2 = 0;
    int variant = 0;   // complex64 only: 1 = 8 units per thread (radix-8 unit stages) instead of 16
    int prefetch = 0;  // 1: the next signal's input is fetched into shared memory by bulk copies while this one is transformed
    int threads = 0;
    size_t smem = 0;
};

void register_cluster_kernel(const ClusterKernel& k);
// logg < 0: the first registered cluster size for (dtype, logn)
// flavour = prefetch + 2 * variant
const ClusterKernel* find_cluster_kernel(int dtype, int logn, int logg, int flavour);
int registered_cluster_kernel_count();

// Host images of the kernel's twiddle tables (ClusterArgs::tw0 / twp), as raw element arrays of
// float or double: tw0 holds (re, im) pairs, twp[t] holds (wr, wr, wi, wi) quadruples.
template <typename T>
void cluster_twiddles(const ClusterKernel& k, std::vector<T>& tw0, std::vector<T> (&twp)[4]);

// One launch over `batch` signals; args is a ClusterArgs<float|double>.
cudaError_t launch_cluster_kernel(const ClusterKernel& k, void* args, long long n_clusters, cudaStream_t stream);
// > 0 if a cluster of this kernel can be resident on the current device
int cluster_kernel_fits(const ClusterKernel& k);

}  // namespace tfft
