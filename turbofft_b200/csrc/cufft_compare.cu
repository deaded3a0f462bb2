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

}  // extern "C"
