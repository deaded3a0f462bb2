// `turbofft` command-line driver for the B200 library.
//
// Same flags, modes and output lines as the reference driver (main.cu:75-169 with the
// parser of include/utils/CommandLineParser.h:26-110), built on the C ABI of
// include/turbofft_b200.h instead of the reference's template dispatch:
//   --logN --bs --bs_end --bs_gap --if_profile --if_verify --if_bench 0|1|2|11|12
//   --if_ft --if_err --datatype 0|1 --thread_bs --gpu
// Output: "turboFFT, logN, logBS, ms, GFLOPS, GB/s" per measurement (main.cu:70), "cuFFT, ..."
// for the cuFFT comparison rows (include/cufft/cufft.h:45).  Differences, all deliberate:
// every CUDA call and launch is checked; the timed loop has no per-launch
// cudaDeviceSynchronize (main.cu:58); --bs_end defaults to --bs; --gpu defaults to B200 and
// selects param/<gpu>/param_<datatype>.csv next to the executable (built-in table if absent).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/turbofft_b200.h"

extern "C" int tfft_cmp_cufft(int logN, long long batch, int dtype, const void* in, void* out, int ntest,
                              float* ms_per_run, void* stream);

namespace {

struct Config {
    long long logN = 0, bs = 0, bs_end = 0, bs_gap = 1;
    int if_profile = 0, if_verify = 0, if_bench = 1, if_ft = 0, if_err = 0, datatype = 0, thread_bs = 1;
    int max_log_total = 28;  // the reference's param_1 for its A100 spec (CommandLineParser.h:104)
    std::string gpu = "B200";
    std::string param_path;  // empty = built-in table
};

void help() {
    printf("Usage: turbofft [options]\n"
           "  --logN <v>        transform length 2^v\n"
           "  --bs <v>          batch size\n"
           "  --bs_end <v>      last batch size of an iterative test (default: --bs)\n"
           "  --bs_gap <v>      batch step of an iterative test\n"
           "  --if_profile <0|1>\n"
           "  --if_verify <0|1> compare against cuFFT with the reference's 1e-4 test\n"
           "  --if_bench <0|1|2|11|12>  1: all batches, 2: logBS + logN = 28, 11/12: the same with cuFFT\n"
           "  --if_ft <0|1>     fault tolerance\n"
           "  --if_err <0|1>    error injection + correction (implies --if_ft 1)\n"
           "  --datatype <0|1>  0 FP32 (float2), 1 FP64 (double2)\n"
           "  --thread_bs <v>   tiles per thread block\n"
           "  --gpu <str>       parameter table directory (default B200)\n");
}

bool parse(int argc, char** argv, Config& c) {
    for (int i = 1; i < argc; ++i)
        if (!strcmp(argv[i], "--help") || !strcmp(argv[i], "-h")) {
            help();
            exit(EXIT_FAILURE);
        }
    for (int i = 1; i < argc; i += 2) {
        if (i + 1 >= argc) return false;
        const char* k = argv[i];
        const char* v = argv[i + 1];
        if (!strcmp(k, "--logN")) c.logN = atol(v);
        else if (!strcmp(k, "--bs")) c.bs = atol(v);
        else if (!strcmp(k, "--bs_end")) c.bs_end = atol(v);
        else if (!strcmp(k, "--bs_gap")) c.bs_gap = atol(v);
        else if (!strcmp(k, "--if_profile")) c.if_profile = atoi(v);
        else if (!strcmp(k, "--if_verify")) c.if_verify = atoi(v);
        else if (!strcmp(k, "--if_ft")) c.if_ft = atoi(v);
        else if (!strcmp(k, "--if_err")) { c.if_err = atoi(v); if (c.if_err) c.if_ft = 1; }
        else if (!strcmp(k, "--if_bench")) c.if_bench = atoi(v);
        else if (!strcmp(k, "--datatype")) c.datatype = atoi(v);
        else if (!strcmp(k, "--thread_bs")) c.thread_bs = atoi(v);
        else if (!strcmp(k, "--gpu")) c.gpu = v;
        else return false;
    }
    if (c.bs_end < c.bs) c.bs_end = c.bs;
    if (c.bs_gap < 1) c.bs_gap = 1;
    return true;
}

std::string exe_dir(const char* argv0) {
    std::string s(argv0);
    const size_t p = s.find_last_of('/');
    return p == std::string::npos ? "." : s.substr(0, p);
}

size_t esize(int dt) { return dt == 0 ? sizeof(float2) : sizeof(double2); }

// The reference's test signal (include/utils/initializeData.h:6-7,25-26,65-66).
void fill_input(void* host, long long count, int dt) {
    srandom(10);
    if (dt == 0) {
        float2* p = (float2*)host;
        for (long long i = 0; i < count; ++i) {
            p[i].x = (float)((double)(random() % 100 - 50) / 100.0);
            p[i].y = (float)((double)(random() % 100 - 50) / 100.0);
        }
    } else {
        double2* p = (double2*)host;
        for (long long i = 0; i < count; ++i) {
            p[i].x = (double)(random() % 100 - 50) / 1000.0;
            p[i].y = (double)(random() % 100 - 50) / 1000.0;
        }
    }
}

// compareData() of the reference (include/utils/compareData.h:4-35): first offender only.
template <typename C>
bool compare(const C* res, const C* ref, long long n, double bound) {
    printf("Compare begin.\n");
    for (long long i = 0; i < n; ++i) {
        double e = fabs((res[i].x - ref[i].x) / (1 + fabs(ref[i].x)));
        if (e > bound || res[i].x != res[i].x) {
            printf("Error detected: res[%lld].x=%f, res_ref[%lld].x=%f, rel_error=%f\n", i, (double)res[i].x, i,
                   (double)ref[i].x, e);
            return false;
        }
        e = fabs((res[i].y - ref[i].y) / (1 + fabs(ref[i].y)));
        if (e > bound || res[i].y != res[i].y) {
            printf("Error detected: res[%lld].y=%f, res_ref[%lld].y=%f, rel_error=%f\n", i, (double)res[i].y, i,
                   (double)ref[i].y, e);
            return false;
        }
    }
    printf("Compare finished.\n");
    return true;
}

void print_line(const char* name, long long logN, long long bs, float ms, int dt) {
    const double N = (double)(1LL << logN);
    const double gflops = 5.0 * N * (double)logN * (double)bs / ms * 1000.0 / 1e9;      // main.cu:68
    const double gbs = N * (double)bs * (double)esize(dt) * 2.0 / ms * 1000.0 / 1e9;    // main.cu:69
    printf("%s, %d, %d, %8.3f, %8.3f, %8.3f\n", name, (int)logN, (int)log2((double)bs), ms, gflops, gbs);
}

// One timed measurement of the library, following test_turbofft() (main.cu:47-70).
int time_turbofft(const Config& c, long long logN, long long bs, const void* in_d, void* out_d, int ntest, float* ms_out) {
    tfft_plan plan = nullptr;
    int rc = tfft_plan_create(&plan, (int)logN, bs, c.datatype, c.if_ft, c.if_err, c.thread_bs,
                              c.param_path.empty() ? nullptr : c.param_path.c_str(), 0);
    if (rc != TFFT_OK) {
        printf("turboFFT, %d, %d, plan failed: %s\n", (int)logN, (int)log2((double)bs), tfft_status_string(rc));
        return rc;
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    rc = tfft_exec(plan, in_d, out_d, nullptr);  // warm-up
    cudaEventRecord(e0);
    for (int j = 0; j < ntest && rc == TFFT_OK; ++j) rc = tfft_exec(plan, in_d, out_d, nullptr);
    cudaEventRecord(e1);
    const cudaError_t ce = cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc != TFFT_OK || ce != cudaSuccess) {
        printf("turboFFT, %d, %d, launch failed: %s (CUDA %d)\n", (int)logN, (int)log2((double)bs),
               tfft_status_string(rc), ce != cudaSuccess ? (int)ce : tfft_last_cuda_error(plan));
        tfft_plan_destroy(plan);
        return rc != TFFT_OK ? rc : TFFT_ERR_CUDA;
    }
    ms /= ntest;
    if (ms_out) *ms_out = ms;
    print_line("turboFFT", logN, bs, ms, c.datatype);
    if (c.if_ft) {
        int nd = 0, nc = 0, nb = 0;
        tfft_ft_status(plan, &nd, &nc, -1, nullptr, 0, &nb);
        printf("turboFFT_ft, %d, %d, blocks=%d, detected=%d, corrected=%d\n", (int)logN, (int)log2((double)bs), nb, nd, nc);
    }
    tfft_plan_destroy(plan);
    return TFFT_OK;
}

int time_cufft(const Config& c, long long logN, long long bs, const void* in_d, void* out_d, int ntest) {
    float ms = 0;
    const int rc = tfft_cmp_cufft((int)logN, bs, c.datatype, in_d, out_d, ntest, &ms, nullptr);
    if (rc != 0) {
        printf("cuFFT, %d, %d, failed (%d)\n", (int)logN, (int)log2((double)bs), rc);
        return rc;
    }
    print_line("cuFFT", logN, bs, ms, c.datatype);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    Config c;
    if (!parse(argc, argv, c)) {
        fprintf(stderr, "Invalid or incomplete argument\n");
        return EXIT_FAILURE;
    }
    const std::string csv = exe_dir(argv[0]) + "/param/" + c.gpu + "/param_" + (c.datatype == 1 ? "double2" : "float2") + ".csv";
    if (FILE* f = fopen(csv.c_str(), "r")) {
        fclose(f);
        c.param_path = csv;
    }
    printf("N: %lld, bs: %lld, bs_end: %lld, bs_gap: %lld\n", c.logN ? (1LL << c.logN) : 0LL, c.bs, c.bs_end, c.bs_gap);
    printf("if_profile: %d, if_verify: %d, if_bench: %d\n", c.if_profile, c.if_verify, c.if_bench);
    printf("if_ft: %d, if_err: %d\n", c.if_ft, c.if_err);
    printf("datatype: %d, thread_bs: %d\n", c.datatype, c.thread_bs);
    printf("gpu: %s, param_file_path: %s\n", c.gpu.c_str(), c.param_path.empty() ? "(built-in B200 table)" : c.param_path.c_str());

    const int ntest = 10;  // main.cu:79
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        fprintf(stderr, "no CUDA device: turbofft has no CPU path\n");
        return EXIT_FAILURE;
    }
    const size_t es = esize(c.datatype);
    int failures = 0;

    if (!c.if_bench) {
        if (c.logN < 1 || c.bs < 1) {
            fprintf(stderr, "--logN and --bs are required when --if_bench 0\n");
            return EXIT_FAILURE;
        }
        const long long count = (1LL << c.logN) * c.bs_end;
        void* host = malloc(count * es);
        void *in_d = nullptr, *out_d = nullptr;
        if (!host || cudaMalloc(&in_d, count * es) != cudaSuccess || cudaMalloc(&out_d, count * es) != cudaSuccess) {
            fprintf(stderr, "allocation failed\n");
            return EXIT_FAILURE;
        }
        fill_input(host, count, c.datatype);
        cudaMemcpy(in_d, host, count * es, cudaMemcpyHostToDevice);
        if (c.if_verify) {  // main.cu:98-102
            const long long n = (1LL << c.logN) * c.bs;
            std::vector<char> ours(n * es), theirs(n * es);
            failures += time_turbofft(c, c.logN, c.bs, in_d, out_d, 1, nullptr) != 0;
            cudaMemcpy(ours.data(), out_d, n * es, cudaMemcpyDeviceToHost);
            failures += time_cufft(c, c.logN, c.bs, in_d, out_d, 1) != 0;
            cudaMemcpy(theirs.data(), out_d, n * es, cudaMemcpyDeviceToHost);
            const bool ok = c.datatype == 0 ? compare((const float2*)ours.data(), (const float2*)theirs.data(), n, 1e-4)
                                            : compare((const double2*)ours.data(), (const double2*)theirs.data(), n, 1e-4);
            failures += !ok;
        }
        if (c.if_profile) {  // main.cu:104-111
            for (long long bs = c.bs; bs <= c.bs_end; bs += c.bs_gap) failures += time_cufft(c, c.logN, bs, in_d, out_d, ntest) != 0;
            for (long long bs = c.bs; bs <= c.bs_end; bs += c.bs_gap)
                failures += time_turbofft(c, c.logN, bs, in_d, out_d, ntest, nullptr) != 0;
        }
        cudaFree(in_d);
        cudaFree(out_d);
        free(host);
    } else {  // main.cu:114-128
        const long long count = 1LL << c.max_log_total;
        void *in_d = nullptr, *out_d = nullptr;
        if (cudaMalloc(&in_d, count * es) != cudaSuccess || cudaMalloc(&out_d, count * es) != cudaSuccess) {
            fprintf(stderr, "allocation failed\n");
            return EXIT_FAILURE;
        }
        {   // seeded input, generated in slices to keep the host buffer small
            const long long slice = 1LL << 24;
            void* host = malloc(slice * es);
            fill_input(host, slice, c.datatype);
            for (long long off = 0; off < count; off += slice)
                cudaMemcpy((char*)in_d + off * es, host, slice * es, cudaMemcpyHostToDevice);
            free(host);
        }
        for (long long logN = 1; logN <= 25; ++logN) {
            long long bs = 1;
            if (c.if_bench % 10 == 2) bs <<= (c.max_log_total - logN);
            for (long long i = 0; i <= c.max_log_total - logN; ++i) {
                if (c.if_bench > 10) failures += time_cufft(c, logN, bs, in_d, out_d, ntest) != 0;
                else failures += time_turbofft(c, logN, bs, in_d, out_d, ntest, nullptr) != 0;
                bs *= 2;
                if (c.if_bench % 10 == 2) break;
            }
        }
        cudaFree(in_d);
        cudaFree(out_d);
    }
    return failures ? EXIT_FAILURE : 0;
}
