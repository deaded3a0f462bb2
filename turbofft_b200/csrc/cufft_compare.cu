// COMPARISON ONLY -- never linked into libturbofft_b200.so.
// cuFFT timing wrapper with the shape of the reference's profiler::cufft::test_cufft()
// (include/cufft/cufft.h:13-92): cufftPlan1d(N, C2C|Z2Z, batch), forward, out of place.
// Used by `turbofft --if_bench 11/12`, by --if_verify (the reference verifies against
// cuFFT, main.cu:98-102) and by the benchmark's side-by-side column.
#include <cuda_runtime.h>
#include <cufft.h>

extern "C" {

// Runs the transform once (ntest == 0) or times ntest runs after one warm-up.
// in/out: device pointers.  Returns 0 or the failing cuFFT/CUDA code (negated).
int tfft_cmp_cufft(int logN, long long batch, int dtype, const void* in, void* out, int ntest, float* ms_per_run,
                   void* stream) {
    cufftHandle plan;
    cudaStream_t st = (cudaStream_t)stream;
    if (cufftCreate(&plan) != CUFFT_SUCCESS) return -1;
    long long n[1] = {1LL << logN};
    size_t work = 0;
    cufftResult r = cufftMakePlanMany64(plan, 1, n, nullptr, 1, 1LL << logN, nullptr, 1, 1LL << logN,
                                        dtype == 0 ? CUFFT_C2C : CUFFT_Z2Z, batch, &work);
    if (r != CUFFT_SUCCESS) {
        cufftDestroy(plan);
        return -(int)r - 100;
    }
    cufftSetStream(plan, st);
    auto run = [&]() -> cufftResult {
        return dtype == 0 ? cufftExecC2C(plan, (cufftComplex*)in, (cufftComplex*)out, CUFFT_FORWARD)
                          : cufftExecZ2Z(plan, (cufftDoubleComplex*)in, (cufftDoubleComplex*)out, CUFFT_FORWARD);
    };
    r = run();
    if (r == CUFFT_SUCCESS && ntest > 0) {
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, st);
        for (int i = 0; i < ntest && r == CUFFT_SUCCESS; ++i) r = run();
        cudaEventRecord(e1, st);
        cudaEventSynchronize(e1);
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms_per_run) *ms_per_run = ms / ntest;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    const cudaError_t ce = cudaStreamSynchronize(st);
    cufftDestroy(plan);
    if (r != CUFFT_SUCCESS) return -(int)r - 100;
    return ce == cudaSuccess ? 0 : -(int)ce;
}

// Plan once, execute many times: lets the benchmark run a whole cuFFT sweep back to back the
// same way it runs ours (same thermal and power state).
int tfft_cmp_cufft_plan_create(int logN, long long batch, int dtype, void* stream, int* handle_out) {
    cufftHandle plan;
    if (!handle_out || cufftCreate(&plan) != CUFFT_SUCCESS) return -1;
    long long n[1] = {1LL << logN};
    size_t work = 0;
    cufftResult r = cufftMakePlanMany64(plan, 1, n, nullptr, 1, 1LL << logN, nullptr, 1, 1LL << logN,
                                        dtype == 0 ? CUFFT_C2C : CUFFT_Z2Z, batch, &work);
    if (r != CUFFT_SUCCESS) {
        cufftDestroy(plan);
        return -(int)r - 100;
    }
    cufftSetStream(plan, (cudaStream_t)stream);
    *handle_out = (int)plan;
    return 0;
}
int tfft_cmp_cufft_plan_exec(int handle, int dtype, const void* in, void* out) {
    const cufftResult r = dtype == 0 ? cufftExecC2C((cufftHandle)handle, (cufftComplex*)in, (cufftComplex*)out, CUFFT_FORWARD)
                                     : cufftExecZ2Z((cufftHandle)handle, (cufftDoubleComplex*)in, (cufftDoubleComplex*)out, CUFFT_FORWARD);
    return r == CUFFT_SUCCESS ? 0 : -(int)r - 100;
}
int tfft_cmp_cufft_plan_destroy(int handle) { return cufftDestroy((cufftHandle)handle) == CUFFT_SUCCESS ? 0 : -1; }

// "Offline" ABFT around cuFFT, the shape of the reference's unused prototype
// (include/cufft/cufft_ft.h:19-156 with include/cufft/reduction.cuh:1-27): per-position sums
// over groups of 16 signals are appended to the batch, cuFFT transforms batch + batch/16
// signals, and the same sums of the outputs are compared with the transformed checksums.
// It is the FT-without-fusion comparison point: two extra passes over the data.
}  // extern "C"

namespace {

template <typename C>
__global__ void __launch_bounds__(256) group_sum_kernel(const C* __restrict__ a, C* __restrict__ sums, long long n, int m) {
    const long long chunks = (n + 255) / 256;
    const long long grp = blockIdx.x / chunks;
    const long long i = (blockIdx.x % chunks) * 256 + threadIdx.x;
    if (i >= n) return;
    const C* p = a + grp * m * n + i;
    C acc;
    acc.x = acc.y = 0;
    for (int k = 0; k < m; ++k) {
        const C v = p[(long long)k * n];
        acc.x += v.x;
        acc.y += v.y;
    }
    sums[grp * n + i] = acc;
}

template <typename C>
__global__ void __launch_bounds__(256) group_check_kernel(const C* __restrict__ y, const C* __restrict__ want, long long n, int m,
                                                          double tol, unsigned int* bad) {
    const long long chunks = (n + 255) / 256;
    const long long grp = blockIdx.x / chunks;
    const long long i = (blockIdx.x % chunks) * 256 + threadIdx.x;
    if (i >= n) return;
    const C* p = y + grp * m * n + i;
    double sx = 0, sy = 0, mag = 0;
    for (int k = 0; k < m; ++k) {
        const C v = p[(long long)k * n];
        sx += v.x;
        sy += v.y;
        mag += fabs((double)v.x) + fabs((double)v.y);
    }
    const C w = want[grp * n + i];
    if (fabs(sx - w.x) + fabs(sy - w.y) > tol * (1.0 + mag)) atomicAdd(bad, 1u);
}

}  // namespace

extern "C" {

// Times cuFFT with the offline checksums around it.  in/out hold `batch` signals; the
// checksum signals live in a scratch area this function allocates (comparison code, not the
// product).  batch must be a multiple of 16.  *n_bad receives the number of failed checks of
// the last run (0 on clean data).
int tfft_cmp_cufft_offline_abft(int logN, long long batch, int dtype, const void* in, void* out, int ntest,
                                float* ms_per_run, unsigned int* n_bad, void* stream) {
    if (batch % 16) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    const long long n = 1LL << logN, groups = batch / 16;
    const size_t es = dtype == 0 ? sizeof(cufftComplex) : sizeof(cufftDoubleComplex);
    void *sums_in = nullptr, *sums_out = nullptr;
    unsigned int* bad = nullptr;
    if (cudaMalloc(&sums_in, groups * n * es) != cudaSuccess || cudaMalloc(&sums_out, groups * n * es) != cudaSuccess ||
        cudaMalloc(&bad, sizeof(unsigned int)) != cudaSuccess)
        return -2;
    cufftHandle plan, plan_sums;
    long long nn[1] = {n};
    size_t work = 0;
    int rc = 0;
    if (cufftCreate(&plan) != CUFFT_SUCCESS || cufftCreate(&plan_sums) != CUFFT_SUCCESS) rc = -3;
    if (!rc && cufftMakePlanMany64(plan, 1, nn, nullptr, 1, n, nullptr, 1, n, dtype == 0 ? CUFFT_C2C : CUFFT_Z2Z, batch, &work) != CUFFT_SUCCESS) rc = -4;
    if (!rc && cufftMakePlanMany64(plan_sums, 1, nn, nullptr, 1, n, nullptr, 1, n, dtype == 0 ? CUFFT_C2C : CUFFT_Z2Z, groups, &work) != CUFFT_SUCCESS) rc = -4;
    if (!rc) {
        cufftSetStream(plan, st);
        cufftSetStream(plan_sums, st);
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        for (int it = 0; it <= ntest && !rc; ++it) {
            if (it == 1) cudaEventRecord(e0, st);
            cudaMemsetAsync(bad, 0, sizeof(unsigned int), st);
            // sums of the inputs, their transform (the expected sums of the outputs), the batch, the check
            if (dtype == 0) {
                group_sum_kernel<cufftComplex><<<dim3((unsigned)(((n + 255) / 256) * groups)), 256, 0, st>>>((const cufftComplex*)in, (cufftComplex*)sums_in, n, 16);
                if (cufftExecC2C(plan_sums, (cufftComplex*)sums_in, (cufftComplex*)sums_out, CUFFT_FORWARD) != CUFFT_SUCCESS) rc = -5;
                if (!rc && cufftExecC2C(plan, (cufftComplex*)in, (cufftComplex*)out, CUFFT_FORWARD) != CUFFT_SUCCESS) rc = -5;
                group_check_kernel<cufftComplex><<<dim3((unsigned)(((n + 255) / 256) * groups)), 256, 0, st>>>((const cufftComplex*)out, (const cufftComplex*)sums_out, n, 16, 1e-4, bad);
            } else {
                group_sum_kernel<cufftDoubleComplex><<<dim3((unsigned)(((n + 255) / 256) * groups)), 256, 0, st>>>((const cufftDoubleComplex*)in, (cufftDoubleComplex*)sums_in, n, 16);
                if (cufftExecZ2Z(plan_sums, (cufftDoubleComplex*)sums_in, (cufftDoubleComplex*)sums_out, CUFFT_FORWARD) != CUFFT_SUCCESS) rc = -5;
                if (!rc && cufftExecZ2Z(plan, (cufftDoubleComplex*)in, (cufftDoubleComplex*)out, CUFFT_FORWARD) != CUFFT_SUCCESS) rc = -5;
                group_check_kernel<cufftDoubleComplex><<<dim3((unsigned)(((n + 255) / 256) * groups)), 256, 0, st>>>((const cufftDoubleComplex*)out, (const cufftDoubleComplex*)sums_out, n, 16, 1e-11, bad);
            }
        }
        cudaEventRecord(e1, st);
        cudaEventSynchronize(e1);
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms_per_run && ntest > 0) *ms_per_run = ms / ntest;
        if (n_bad) cudaMemcpy(n_bad, bad, sizeof(unsigned int), cudaMemcpyDeviceToHost);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    cufftDestroy(plan);
    cufftDestroy(plan_sums);
    cudaFree(sums_in);
    cudaFree(sums_out);
    cudaFree(bad);
    if (cudaGetLastError() != cudaSuccess && !rc) rc = -6;
    return rc;
}

}  // extern "C"
