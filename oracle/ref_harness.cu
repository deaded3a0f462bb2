// TEST INFRASTRUCTURE -- not part of the product, never linked into it.
//
// Builds the UNMODIFIED reference (main.cu and the generated kernels it includes,
// compiled where they lie) for sm_100a and exposes two C entry points:
//   ref_run : feeds caller-supplied signals through the reference's own launch
//             protocol test_turbofft() (main.cu:4-73) and returns its output --
//             the "reference's own kernels" leg of the parity tests;
//   ref_cli : the reference's main() (main.cu:137-169) under another name, for
//             running its stock benchmark modes on this GPU.
// The reference's main.cu is included textually with `main` renamed; nothing else of
// it is touched.  Build recipe: oracle/build_ref.sh (outputs only under oracle/_ref/).
#define main turbofft_reference_main
#include "main.cu"
#undef main

namespace {

template <typename T, int FT, int ERR>
int run_typed(int logN, long long bs, int thread_bs, const void* in_host, void* out_host, int ntest,
              const char* param_csv) {
    ProgramConfig config;
    // the constants parseCommandLine() sets for --gpu A100 (CommandLineParser.h:103-109)
    config.gpu = "A100";
    config.param_1 = 28;
    config.param_2 = 16;
    config.smem_size = 128;
    config.sm_cnt = 108;
    config.smem_capacity = 164;
    config.logN = logN;
    config.N = 1LL << logN;
    config.bs = bs;
    config.bs_end = bs;
    config.thread_bs = thread_bs;
    config.if_ft = FT;
    config.if_err = ERR;
    config.param_file_path = param_csv;
    std::vector<std::vector<long long int> > params = utils::load_parameters(config.param_file_path);
    if ((long long)params.size() <= logN) return -2;

    // ABFT table exactly as TurboFFT_main() builds it (main.cu:85-93)
    T *checksum_d, *checksum_h;
    if (cudaMalloc((void**)&checksum_d, sizeof(T) * 16384 * 2) != cudaSuccess) return -3;
    checksum_h = (T*)calloc(16384 * 2, sizeof(T));
    T* dest = checksum_h;
    for (int i = 2; i <= (1 << 13); i *= 2) {
        utils::getDFTMatrixChecksum(dest, i);
        dest += i;
    }
    cudaMemcpy((void*)checksum_d, (void*)checksum_h, sizeof(T) * 16384 * 2, cudaMemcpyHostToDevice);

    // buffers and twiddle table from the reference's own initializeData(), then the
    // caller's signals replace its srandom(10) input
    T *input, *output_turbofft, *output_cufft, *input_d, *output_d, *twiddle_d;
    utils::initializeData<T>(input, input_d, output_d, output_turbofft, output_cufft, twiddle_d, config.N, bs);
    const size_t bytes = sizeof(T) * (size_t)config.N * (size_t)bs;
    cudaMemcpy((void*)input_d, in_host, bytes, cudaMemcpyHostToDevice);
    cudaMemset((void*)output_d, 0, 2 * bytes);

    test_turbofft<T, FT, ERR, 80>(input_d, output_d, output_turbofft, twiddle_d, checksum_d, params[logN], bs,
                                  thread_bs, ntest, config);
    const cudaError_t e = cudaDeviceSynchronize();
    const cudaError_t e2 = cudaGetLastError();
    memcpy(out_host, output_turbofft, bytes);
    cudaFree(input_d);
    cudaFree(output_d);
    cudaFree(twiddle_d);
    cudaFree(checksum_d);
    free(input);
    free(output_cufft);
    free(output_turbofft);
    free(checksum_h);
    return (e == cudaSuccess && e2 == cudaSuccess) ? 0 : -3;
}

}  // namespace

extern "C" {

// dtype 0 = float2, 1 = double2; returns 0, -1 bad argument, -2 no parameter row, -3 CUDA error,
// -4 refused.  Refused: float2 with logN 2, 3 or 4.  The reference's checked-in kernels for
// those three sizes were generated from an older parameter table (logN 4: tiles of 8 signals,
// 32 threads -- generated/float2/fft_radix_2_logN_4_upload_0.cuh:67-77) than the one its
// launcher reads (param/A100/param_float2.csv row 4: 4 signals, 16 threads), so they index
// past the buffers the launcher sizes; on a B200 that is an illegal address.  They are never
// run.
int ref_run(int dtype, int if_ft, int if_err, int logN, long long bs, int thread_bs, const void* in_host,
            void* out_host, int ntest, const char* param_csv) {
    if (logN < 1 || logN > 25 || bs < 1 || !in_host || !out_host || !param_csv) return -1;
    if (dtype == 0 && logN >= 2 && logN <= 4) return -4;
    const int mode = if_err ? 2 : (if_ft ? 1 : 0);
    if (dtype == 0) {
        if (mode == 0) return run_typed<float2, 0, 0>(logN, bs, thread_bs, in_host, out_host, ntest, param_csv);
        if (mode == 1) return run_typed<float2, 1, 0>(logN, bs, thread_bs, in_host, out_host, ntest, param_csv);
        return run_typed<float2, 1, 1>(logN, bs, thread_bs, in_host, out_host, ntest, param_csv);
    }
    if (mode == 0) return run_typed<double2, 0, 0>(logN, bs, thread_bs, in_host, out_host, ntest, param_csv);
    if (mode == 1) return run_typed<double2, 1, 0>(logN, bs, thread_bs, in_host, out_host, ntest, param_csv);
    return run_typed<double2, 1, 1>(logN, bs, thread_bs, in_host, out_host, ntest, param_csv);
}

int ref_cli(int argc, char** argv) { return turbofft_reference_main(argc, argv); }

}  // extern "C"
