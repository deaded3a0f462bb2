// Host side of the C ABI declared in include/turbofft_b200.h: launch planner, table
// builders and the exec loop.  It stands where test_turbofft() / TurboFFT_main()
// stand in the reference (main.cu:4-73, 75-135) but owns its tables, checks every
// CUDA call and never synchronises inside exec.
#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <mutex>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#ifndef TFFT_NVTX
#define TFFT_NVTX 1  // NVTX ranges around plan creation and every exec (header-only NVTX v3; free without a tool attached)
#endif
#if TFFT_NVTX
#include <nvtx3/nvToolsExt.h>
#endif

#include "../../include/turbofft_b200.h"
#include "fft_kernels.cuh"
#include "generated/ft_defaults.h"
#include "params.h"
#include "registry.h"
#include "cluster_registry.h"
#include "pair_fft.cuh"
#include "pair_registry.h"

using namespace tfft;

namespace {

std::atomic<long long> g_launches{0};

// Device staging buffers of tfft_exec_host, one grow-only pair per device shared by all
// plans (a sweep over many plans would otherwise hold one pair per plan).  Calls are
// serialised by the mutex; each call synchronises before it returns.
struct StagePair {
    void* in = nullptr;
    void* out = nullptr;
    size_t bytes = 0;
};
std::mutex g_stage_mu;
std::map<int, StagePair> g_stage;

// The pipelined host path of a device: chunk-sized staging slots (3 in + 3 out), one stream each for
// copy-in, transform and copy-out, and the events that order the slots.  Shared by all plans of the
// device and kept until the library is unloaded, so that consecutive calls -- of one plan or of
// several -- keep the pipeline full: the copy-out tail of one call overlaps the copy-in head of the next.
constexpr size_t kPipeChunkBytes = 64u << 20;
struct PipeSlots {
    void* in[3] = {nullptr, nullptr, nullptr};
    void* out[3] = {nullptr, nullptr, nullptr};
    size_t bytes = 0;
    cudaStream_t stream[3] = {nullptr, nullptr, nullptr};  // copy-in, transform, copy-out
    cudaEvent_t ev_in[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t ev_fft[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t ev_out[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t ev_start = nullptr;
    unsigned long long seq = 0;  // chunks queued so far: chunk n uses slot n % 3
    bool ready = false;
};
std::map<int, PipeSlots> g_pipe;

struct LaunchDesc {
    int role = 0, logm = 0, loge = 0, logc = 0;
    const KernelEntry* k = nullptr;
    long long n_tiles = 0;
    long long n_lines = 0;
    unsigned grid = 0;
    int log_b = 0, log_n1 = 0, log_q = 0, tw_lo_bits = 0;
    void* tw_st = nullptr;
    void* tw_lo = nullptr;
    void* tw_hi = nullptr;
    void* cks = nullptr;
    int* ft_located = nullptr;
    void* ft_diag = nullptr;
};

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) ok = false;
        if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// Named range on the calling host thread, visible to profilers that listen to NVTX.
struct NvtxRange {
#if TFFT_NVTX
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
#else
    explicit NvtxRange(const char*) {}
#endif
};

}  // namespace

struct tfft_plan_s {
    int logn = 0;
    long long batch = 0;
    int dtype = 0, if_ft = 0, if_err = 0, thread_bs = 1, device = 0;
    int n_launch = 0;
    LaunchDesc L[3];
    // single-pass plan (one cluster kernel, no scratch): kernel, its tables, signals per cluster
    const ClusterKernel* ck = nullptr;
    void* ctw0 = nullptr;
    void* ctwp[4] = {nullptr, nullptr, nullptr, nullptr};
    unsigned cgrid_clusters = 0;
    int* cstatus = nullptr;  // prefetching single-pass kernels: device word, 1 = a bounded wait gave up
    // fused two-launch plan (one persistent kernel, intermediate in a ring that stays in L2)
    const PairKernel* pk = nullptr;
    void* ring = nullptr;
    unsigned int* pair_done = nullptr;  // the ticket counter (8 bytes), then [2 * pair_chunks] tile counters
    int* pair_status = nullptr;
    long long pair_chunks = 0;
    int pair_log_chunk = 0, pair_lag = 1, pair_ring_chunks = 4, pair_grid = 0;
    void* scratch = nullptr;
    void* scratch2 = nullptr;          // 3-launch plans that correct: the middle launch writes here, so that
                                       // its own input survives for the recompute of a located tile
    unsigned int* ft_count = nullptr;  // [3][2]
    unsigned long long* oob = nullptr;  // checked build: first out-of-range access of the last exec
    size_t owned_bytes = 0;
    double err_inj = TFFT_DEFAULT_ERR_INJ;
    double err_smoothing = TFFT_DEFAULT_ERR_SMOOTHING;
    double err_threshold = TFFT_DEFAULT_ERR_THRESHOLD;
    int inj_enable = 0, inj_launch = -1, inj_period = 1, inj_phase = 0;
    int diag = 0;
    int ft_accumulate = 0;  // 1: the FT counters add up over execs until tfft_ft_status reads (and clears) them
    int csum = 0;        // 1: repair from the running checksums (FT_CSUM kernels) where they exist
    int strided = 0;     // 1: one ROLE_FIRST launch on its own, lines strided by 2^L[0].log_b (tfft_plan_create_strided)
    int inverse = 0;     // 0: forward; 1: conjugate in, conjugate out (inverse transform)
    double scale = 1.0;  // applied with the conjugation of the last launch
    cudaStream_t last_stream = nullptr;
    int last_cuda_error = 0;
    std::vector<void*> allocs;
    std::string param_csv;            // empty = built-in table
    char nvtx_name[64] = "tfft_exec";  // range name of this plan's execs
    // host-buffer pipeline (tfft_exec_host): sub-plans for one chunk / the ragged last chunk,
    // three internal streams and per-slot events
    tfft_plan chunk_plan = nullptr;
    tfft_plan tail_plan = nullptr;
    long long chunk_batch = 0;
    bool pipe_ready = false;  // the sub-plans of the pipelined host path exist
    size_t esize() const { return dtype == TFFT_FLOAT2 ? sizeof(float2) : sizeof(double2); }
};

namespace {

bool cuda_ok(tfft_plan p, cudaError_t e) {
    if (e == cudaSuccess) return true;
    if (p) p->last_cuda_error = (int)e;
    return false;
}

void* dev_alloc(tfft_plan p, size_t bytes) {
    void* ptr = nullptr;
    if (!cuda_ok(p, cudaMalloc(&ptr, bytes ? bytes : 16))) return nullptr;
    p->allocs.push_back(ptr);
    p->owned_bytes += bytes;
    return ptr;
}

// exp(-2*pi*i*j/2^logp) in extended precision, then rounded once to T.
template <typename C>
void fill_twiddles(std::vector<C>& v, long long count, long long stride, int logp) {
    v.resize((size_t)count);
    const long double two_pi = 6.283185307179586476925286766559005768L;
    const long double pn = std::ldexp(1.0L, logp);
    for (long long j = 0; j < count; ++j) {
        const long long idx = (j * stride) & (((long long)1 << logp) - 1);
        const long double ang = -two_pi * (long double)idx / pn;
        v[(size_t)j].x = (decltype(v[0].x))cosl(ang);
        v[(size_t)j].y = (decltype(v[0].y))sinl(ang);
    }
}

// Stage twiddles of the in-block Stockham exchange, in the order the kernel reads them
// (fft_kernels.cuh, KernelArgs::tw_st): for stage t with radix R_t = 2^lr and already
// transformed extent P_t = 2^lp, entry (j, b) = W_M^{((b >> lp) << lp) * 2^j} for j < lr and
// butterfly b < M / R_t.
template <typename C>
void stage_twiddles(std::vector<C>& v, int logm, int loge, bool remlast) {
    v.clear();
    const int stages = (logm + loge - 1) / loge;
    const int logr0 = logm - (stages - 1) * loge;
    const long double two_pi = 6.283185307179586476925286766559005768L;
    const long long m = 1LL << logm;
    for (int t = 0; t + 1 < stages; ++t) {
        // same stage order as Cfg::stage_logr / stage_logp of the kernel
        const int lr = remlast ? loge : (t == 0 ? logr0 : loge);
        const int lp = remlast ? t * loge : (t == 0 ? 0 : logr0 + (t - 1) * loge);
        for (int j = 0; j < lr; ++j) {
            const long long q = 1LL << j;
            for (long long b = 0; b < (m >> lr); ++b) {
                const long long idx = (((b >> lp) * q) << lp) & (m - 1);
                const long double ang = -two_pi * (long double)idx / (long double)m;
                C w;
                w.x = (decltype(w.x))cosl(ang);
                w.y = (decltype(w.y))sinl(ang);
                v.push_back(w);
            }
        }
    }
    if (v.empty()) v.resize(1);  // single-stage launches read nothing
}

// c = W_M r with r_j = omega^(j mod 3): the ABFT encoding vector of
// getDFTMatrixChecksum() (include/utils/abft.h:21-61), evaluated as the FFT of r in
// extended precision instead of the reference's O(M^2) float-angle loop.
void checksum_vector(int logm, std::vector<long double>& re, std::vector<long double>& im) {
    const int m = 1 << logm;
    re.assign(m, 0);
    im.assign(m, 0);
    const long double h = 0.8660253882408142L;  // float32-rounded sqrt(3)/2, as in constants.h:2-7
    const long double rr[3] = {1.0L, -0.5L, -0.5L};
    const long double ri[3] = {0.0L, -h, h};
    // bit-reversed load, then iterative radix-2 DIT
    for (int j = 0; j < m; ++j) {
        int r = 0;
        for (int b = 0; b < logm; ++b) r |= ((j >> b) & 1) << (logm - 1 - b);
        re[r] = rr[j % 3];
        im[r] = ri[j % 3];
    }
    const long double two_pi = 6.283185307179586476925286766559005768L;
    for (int len = 2; len <= m; len <<= 1) {
        for (int k = 0; k < len / 2; ++k) {
            const long double ang = -two_pi * (long double)k / (long double)len;
            const long double wr = cosl(ang), wi = sinl(ang);
            for (int s = 0; s < m; s += len) {
                const int a = s + k, b = s + k + len / 2;
                const long double tr = re[b] * wr - im[b] * wi;
                const long double ti = re[b] * wi + im[b] * wr;
                re[b] = re[a] - tr;
                im[b] = im[a] - ti;
                re[a] += tr;
                im[a] += ti;
            }
        }
    }
}

template <typename C>
bool upload(tfft_plan p, const std::vector<C>& host, void** dev) {
    *dev = dev_alloc(p, host.size() * sizeof(C));
    if (!*dev) return false;
    return cuda_ok(p, cudaMemcpy(*dev, host.data(), host.size() * sizeof(C), cudaMemcpyHostToDevice));
}

template <typename T>
bool build_tables(tfft_plan p) {
    typedef typename Cplx<T>::type C;
    for (int i = 0; i < p->n_launch; ++i) {
        LaunchDesc& d = p->L[i];
        // reuse tables of an earlier launch with the same line length and radix plan; the stage
        // twiddles also depend on the stage order, the checksum vector only on the line length
        int same = -1, same_len = -1;
        for (int j = 0; j < i; ++j) {
            if (p->L[j].logm == d.logm) same_len = j;
            if (p->L[j].logm == d.logm && p->L[j].loge == d.loge && p->L[j].k->remlast == d.k->remlast) same = j;
        }
        if (same >= 0) {
            d.tw_st = p->L[same].tw_st;
            d.cks = p->L[same].cks;
        } else if (same_len >= 0 && p->L[same_len].cks) {
            std::vector<C> t;
            stage_twiddles(t, d.logm, d.loge, d.k->remlast != 0);
            if (!upload(p, t, &d.tw_st)) return false;
            d.cks = p->L[same_len].cks;
        } else {
            std::vector<C> t;
            stage_twiddles(t, d.logm, d.loge, d.k->remlast != 0);
            if (!upload(p, t, &d.tw_st)) return false;
            if (p->if_ft) {
                std::vector<long double> re, im;
                checksum_vector(d.logm, re, im);
                std::vector<C> c(re.size());
                for (size_t k = 0; k < re.size(); ++k) {
                    // stored as the two fold weights: fold(x * c) = x.x * (c.x + c.y) + x.y * (c.x - c.y)
                    c[k].x = (T)(re[k] + im[k]);
                    c[k].y = (T)(re[k] - im[k]);
                }
                if (!upload(p, c, &d.cks)) return false;
            }
        }
        if (d.role == ROLE_FIRST && !p->strided) {
            const int logp = d.logm + d.log_b;
            d.tw_lo_bits = (logp + 1) / 2;
            std::vector<C> lo, hi;
            fill_twiddles(lo, 1LL << d.tw_lo_bits, 1, logp);
            fill_twiddles(hi, 1LL << (logp - d.tw_lo_bits), 1LL << d.tw_lo_bits, logp);
            if (!upload(p, lo, &d.tw_lo) || !upload(p, hi, &d.tw_hi)) return false;
        }
    }
    return true;
}

template <typename T>
bool build_cluster_tables(tfft_plan p) {
    std::vector<T> tw0, twp[4];
    cluster_twiddles<T>(*p->ck, tw0, twp);
    if (!upload(p, tw0, &p->ctw0)) return false;
    for (int t = 0; t + 1 < p->ck->s2; ++t)
        if (!upload(p, twp[t], &p->ctwp[t])) return false;
    return true;
}

int ilog2_exact(long long x) {
    int l = 0;
    while ((1LL << l) < x) ++l;
    return ((1LL << l) == x) ? l : -1;
}

// a launch can repair from the running checksums if the kernel exists and its three tiles fit
bool csum_ok(const KernelEntry* k) { return k && k->fn[FT_CSUM] && k->smem_csum <= 227u * 1024u; }

template <typename T>
int launch_cluster(tfft_plan p, const void* in, void* out, cudaStream_t st) {
    typedef typename Cplx<T>::type C;
    // the kernel stores 16 bytes per lane
    if (((uintptr_t)out & 15u) || ((uintptr_t)in & (sizeof(C) - 1))) return TFFT_ERR_BAD_ARG;
    ClusterArgs<T> a;
    memset(&a, 0, sizeof(a));
    a.in = (const C*)in;
    a.out = (C*)out;
    a.tw0 = (const C*)p->ctw0;
    for (int t = 0; t < 4; ++t) a.twp[t] = (const T*)p->ctwp[t];
    a.n_signals = p->batch;
    a.signals_per_cluster = p->thread_bs;
    a.conj_in = p->inverse ? 1 : 0;
    a.scale_out = (p->inverse || p->scale != 1.0) ? 1 : 0;
    a.scale_x = (T)p->scale;
    a.scale_y = (T)(p->inverse ? -p->scale : p->scale);
    a.status = p->cstatus;
    if (!cuda_ok(p, launch_cluster_kernel(*p->ck, &a, p->cgrid_clusters, st))) return TFFT_ERR_CUDA;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return TFFT_OK;
}

template <typename T>
void fill_launch_args(tfft_plan p, int i, KernelArgs<T>& a) {
    typedef typename Cplx<T>::type C;
    const LaunchDesc& d = p->L[i];
    memset(&a, 0, sizeof(a));
    a.tw_st = (const C*)d.tw_st;
    a.tw_lo = (const C*)d.tw_lo;
    a.tw_hi = (const C*)d.tw_hi;
    a.cks = (const C*)d.cks;
    a.n_tiles = d.n_tiles;
    a.n_lines = d.n_lines;
    a.tiles_per_cta = p->thread_bs;
    a.log_n = p->logn;
    a.log_b = d.log_b;
    a.log_n1 = d.log_n1;
    a.log_q = d.log_q;
    a.tw_lo_bits = d.tw_lo_bits;
    a.no_twiddle = p->strided;
    a.conj_in = (p->inverse && i == 0) ? 1 : 0;
    a.scale_out = ((p->inverse || p->scale != 1.0) && i == p->n_launch - 1) ? 1 : 0;
    a.scale_x = (T)p->scale;
    a.scale_y = (T)(p->inverse ? -p->scale : p->scale);
    a.n_elems = p->batch << p->logn;
    a.oob = p->oob;
}

// Both launches of a two-launch plan as one persistent kernel (pair_fft.cuh)
template <typename T>
int launch_pair(tfft_plan p, const void* in, void* out, cudaStream_t st) {
    typedef typename Cplx<T>::type C;
    PairArgs<T> a;
    fill_launch_args<T>(p, 0, a.first);
    fill_launch_args<T>(p, 1, a.last);
    const long long ring_signals = (long long)p->pair_ring_chunks << p->pair_log_chunk;
    a.first.in = (const C*)in;
    a.first.out = (C*)p->ring;
    a.last.in = (const C*)p->ring;
    a.last.out = (C*)out;
    a.first.ring_clear = a.last.ring_clear = ~(ring_signals - 1);
    a.queue = (unsigned long long*)p->pair_done;
    a.done = p->pair_done + 2;
    a.status = p->pair_status;
    a.n_chunks = p->pair_chunks;
    a.tiles1 = (int)((p->L[0].n_tiles / p->batch) << p->pair_log_chunk);
    a.tiles2 = (int)((p->L[1].n_tiles / p->batch) << p->pair_log_chunk);
    a.lag = p->pair_lag;
    a.ring_chunks = p->pair_ring_chunks;
    if (!cuda_ok(p, cudaMemsetAsync(p->pair_done, 0, (size_t)(2 * p->pair_chunks + 2) * sizeof(unsigned int), st)))
        return TFFT_ERR_CUDA;
    if (!cuda_ok(p, launch_pair_kernel(*p->pk, &a, p->pair_grid, st))) return TFFT_ERR_CUDA;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return TFFT_OK;
}

template <typename T>
int launch_all(tfft_plan p, const void* in, void* out, cudaStream_t st, void* scratch) {
    typedef typename Cplx<T>::type C;
    if (p->ck) return launch_cluster<T>(p, in, out, st);
    if (p->pk) return launch_pair<T>(p, in, out, st);
    const int ftmode = p->if_ft ? (p->if_err ? FT_CORRECT : FT_DETECT) : FT_OFF;
    if (p->if_ft && !p->ft_accumulate) {
        if (!cuda_ok(p, cudaMemsetAsync(p->ft_count, 0, 6 * sizeof(unsigned int), st))) return TFFT_ERR_CUDA;
    }
    const int inj_launch = p->inj_launch < 0 ? p->n_launch - 1 : p->inj_launch;
    for (int i = 0; i < p->n_launch; ++i) {
        const LaunchDesc& d = p->L[i];
        KernelArgs<T> a;
        memset(&a, 0, sizeof(a));
        // Buffers.  Plain plans: launch 0 in -> scratch, a middle launch in place in scratch, last
        // launch scratch -> out.  A correcting plan recomputes a located tile from the launch's
        // input, so no launch may overwrite what it reads: its middle launch goes scratch ->
        // scratch2 (the reference alternates two buffers for every launch, main.cu:11-12).
        const bool pingpong = p->scratch2 != nullptr;
        a.in = (const C*)(i == 0 ? in : (i == 2 && pingpong ? p->scratch2 : scratch));
        a.out = (C*)(i == p->n_launch - 1 ? out : (i == 1 && pingpong ? p->scratch2 : scratch));
        a.tw_st = (const C*)d.tw_st;
        a.tw_lo = (const C*)d.tw_lo;
        a.tw_hi = (const C*)d.tw_hi;
        a.cks = (const C*)d.cks;
        a.n_tiles = d.n_tiles;
        a.n_lines = d.n_lines;
        a.tiles_per_cta = p->thread_bs;
        a.log_n = p->logn;
        a.log_b = d.log_b;
        a.log_n1 = d.log_n1;
        a.log_q = d.log_q;
        a.tw_lo_bits = d.tw_lo_bits;
        a.no_twiddle = p->strided;
        a.conj_in = (p->inverse && i == 0) ? 1 : 0;
        a.scale_out = ((p->inverse || p->scale != 1.0) && i == p->n_launch - 1) ? 1 : 0;
        a.scale_x = (T)p->scale;
        a.scale_y = (T)(p->inverse ? -p->scale : p->scale);
        a.inj_on = (p->if_err && p->inj_enable && i == inj_launch) ? 1 : 0;
        a.inj_period = p->inj_period;
        a.inj_phase = p->inj_phase;
        a.err_inj = (T)p->err_inj;
        a.err_smoothing = (T)p->err_smoothing;
        a.err_threshold = (T)p->err_threshold;
        a.n_elems = p->batch << p->logn;
        a.oob = p->oob;
        a.ft_located = d.ft_located;
        a.ft_count = p->ft_count ? p->ft_count + 2 * i : nullptr;
        a.ft_diag = p->diag ? (T*)d.ft_diag : nullptr;
        void* args[] = {&a};
        const bool use_csum = ftmode == FT_CORRECT && p->csum && csum_ok(d.k);
        const void* fn = use_csum ? d.k->fn[FT_CSUM] : d.k->fn[ftmode];
        const size_t smem = use_csum ? d.k->smem_csum : d.k->smem;
        if (!cuda_ok(p, cudaLaunchKernel(fn, dim3(d.grid), dim3(d.k->threads), args, smem, st)))
            return TFFT_ERR_CUDA;
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return TFFT_OK;
}

}  // namespace

extern "C" {

int tfft_plan_create(tfft_plan* plan, int logN, long long batch, int dtype, int if_ft, int if_err, int thread_bs,
                     const char* param_csv, int device) {
    if (!plan) return TFFT_ERR_BAD_ARG;
    *plan = nullptr;
    if (logN < 1 || logN > 30 || batch < 1 || (dtype != TFFT_FLOAT2 && dtype != TFFT_DOUBLE2) || thread_bs < 0 ||
        device < 0)
        return TFFT_ERR_BAD_ARG;
    NvtxRange range("tfft_plan_create");
    if (if_err) if_ft = 1;  // as the reference CLI does (CommandLineParser.h:62-64)
    const bool auto_thread_bs = thread_bs == 0;
    if (auto_thread_bs) thread_bs = builtin_thread_bs(dtype, logN, if_ft);  // the tuned value of this size
    std::vector<ParamRow> rows;
    std::string err;
    if (param_csv && param_csv[0]) {
        if (!load_param_file(param_csv, rows, err)) return TFFT_ERR_PARAM_FILE;
    } else {
        if (!parse_param_csv(builtin_param_csv(dtype), rows, err)) return TFFT_ERR_PARAM_FILE;
    }
    if ((int)rows.size() <= logN || rows[logN].launches == 0) return TFFT_ERR_UNSUPPORTED;
    const ParamRow& row = rows[logN];
    if (!validate_row(row, err)) return TFFT_ERR_PARAM_FILE;

    DeviceGuard guard(device);
    if (!guard.ok) return TFFT_ERR_CUDA;

    // Sizes the built-in single-pass table names run as ONE cluster kernel (no FT variant of it
    // exists, and a caller's own parameter file always means the launches that file describes).
    if (!if_ft && !(param_csv && param_csv[0])) {
        const int logg = builtin_single_pass_cluster(dtype, logN);
        if (logg >= 0) {
            const int rc = tfft_plan_create_single_pass(plan, logN, batch, dtype, logg, thread_bs, device);
            if (rc == TFFT_OK) return rc;
            *plan = nullptr;  // e.g. no room for a cluster on this device: fall back to the launches of the row
        }
    }

    tfft_plan p = new (std::nothrow) tfft_plan_s();
    if (!p) return TFFT_ERR_ALLOC;
    p->logn = logN;
    p->batch = batch;
    p->dtype = dtype;
    p->if_ft = if_ft ? 1 : 0;
    p->if_err = if_err ? 1 : 0;
    p->inj_enable = p->if_err;
    p->thread_bs = thread_bs;
    p->device = device;
    p->n_launch = row.launches;
    snprintf(p->nvtx_name, sizeof(p->nvtx_name), "tfft_exec logN=%d batch=%lld %s ft=%d", logN, batch,
             dtype == TFFT_FLOAT2 ? "c64" : "c128", p->if_ft + p->if_err);
    if (param_csv && param_csv[0]) p->param_csv = param_csv;
    const int ftmode = p->if_ft ? (p->if_err ? FT_CORRECT : FT_DETECT) : FT_OFF;

    int status = TFFT_OK;
    long long outer = batch;  // product of batch and the digits already transformed
    int log_rest = logN;      // log2 of the not yet transformed extent, including this launch
    for (int i = 0; i < row.launches && status == TFFT_OK; ++i) {
        LaunchDesc& d = p->L[i];
        d.logm = row.logni[i];
        d.logc = ilog2_exact(row.bs[i]);
        d.loge = ilog2_exact(row.n[i]);
        if (d.loge > d.logm) d.loge = d.logm;
        d.role = row.launches == 1 ? ROLE_SINGLE : (i == row.launches - 1 ? ROLE_LAST : ROLE_FIRST);
        log_rest -= d.logm;
        if (d.role == ROLE_SINGLE) {
            d.n_lines = batch;
            d.n_tiles = (batch + (1LL << d.logc) - 1) >> d.logc;
        } else if (d.role == ROLE_FIRST) {
            d.log_b = log_rest;
            if (d.log_b < d.logc) d.logc = d.log_b;  // fewer columns than a tile is wide
            d.n_tiles = outer << (d.log_b - d.logc);
        } else {
            d.log_n1 = row.logni[0];
            d.log_q = row.launches == 3 ? row.logni[1] : 0;
            if (d.log_n1 < d.logc) d.logc = d.log_n1;
            d.n_tiles = (batch << (logN - d.logm)) >> d.logc;
        }
        outer <<= d.logm;
        d.k = find_kernel(dtype, d.role, d.logm, d.loge, d.logc);
        if (!d.k || !d.k->fn[ftmode]) {
            status = TFFT_ERR_UNSUPPORTED;
            break;
        }
        const long long grid = (d.n_tiles + thread_bs - 1) / thread_bs;
        if (grid > 2147483647LL) {
            status = TFFT_ERR_TOO_LARGE;
            break;
        }
        d.grid = (unsigned)grid;
        if (d.k->smem > 40 * 1024) {  // FT kernels add a little static shared memory on top
            if (!cuda_ok(p, cudaFuncSetAttribute(d.k->fn[ftmode], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)d.k->smem)))
                status = TFFT_ERR_CUDA;
        }
    }
    if (status == TFFT_OK && auto_thread_bs && thread_bs > 1) {
        // The tuned value assumes a batch that fills the device many times over.  With fewer tiles it would leave
        // SMs without a block, so it is cut down until every launch has at least one block per resident slot.
        int sms = 0;
        long long cap = thread_bs;
        if (cuda_ok(p, cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device))) {
            for (int i = 0; i < p->n_launch; ++i) {
                int per_sm = 0;
                if (!cuda_ok(p, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, p->L[i].k->fn[ftmode],
                                                                               p->L[i].k->threads, p->L[i].k->smem)))
                    break;
                const long long slots = (long long)sms * (per_sm > 0 ? per_sm : 1);
                const long long fit = p->L[i].n_tiles / slots;
                if (fit < cap) cap = fit < 1 ? 1 : fit;
            }
        }
        p->last_cuda_error = 0;  // an occupancy query that failed only means no cap
        if (cap < thread_bs) {
            thread_bs = (int)cap;
            p->thread_bs = thread_bs;
            for (int i = 0; i < p->n_launch; ++i) p->L[i].grid = (unsigned)((p->L[i].n_tiles + thread_bs - 1) / thread_bs);
        }
    }
    if (status == TFFT_OK) {
        const bool ok = dtype == TFFT_FLOAT2 ? build_tables<float>(p) : build_tables<double>(p);
        if (!ok) status = p->last_cuda_error ? TFFT_ERR_CUDA : TFFT_ERR_ALLOC;
    }
    if (status == TFFT_OK && p->n_launch > 1) {
        p->scratch = dev_alloc(p, ((size_t)batch << logN) * p->esize());
        if (!p->scratch) status = TFFT_ERR_ALLOC;
        if (status == TFFT_OK && p->n_launch == 3 && p->if_err) {
            p->scratch2 = dev_alloc(p, ((size_t)batch << logN) * p->esize());
            if (!p->scratch2) status = TFFT_ERR_ALLOC;
        }
    }
#if TFFT_BOUNDS_CHECK
    if (status == TFFT_OK) {
        p->oob = (unsigned long long*)dev_alloc(p, sizeof(unsigned long long));
        if (!p->oob || !cuda_ok(p, cudaMemset(p->oob, 0, sizeof(unsigned long long)))) status = TFFT_ERR_ALLOC;
    }
#endif
    if (status == TFFT_OK && p->if_ft) {
        p->ft_count = (unsigned int*)dev_alloc(p, 6 * sizeof(unsigned int));
        // zeroed here as well as before every exec: in accumulating mode nothing else clears them
        if (!p->ft_count || !cuda_ok(p, cudaMemset(p->ft_count, 0, 6 * sizeof(unsigned int)))) status = TFFT_ERR_ALLOC;
        for (int i = 0; i < p->n_launch && status == TFFT_OK; ++i) {
            p->L[i].ft_located = (int*)dev_alloc(p, (size_t)p->L[i].grid * sizeof(int));
            p->L[i].ft_diag = dev_alloc(p, (size_t)p->L[i].grid * 3 * (p->esize() / 2));
            if (!p->L[i].ft_located || !p->L[i].ft_diag) status = TFFT_ERR_ALLOC;
        }
    }
    if (status != TFFT_OK) {
        for (void* q : p->allocs) cudaFree(q);
        delete p;
        return status;
    }
    *plan = p;
    return TFFT_OK;
}

int tfft_plan_create_single_pass(tfft_plan* plan, int logN, long long batch, int dtype, int log_cluster, int thread_bs,
                                 int device) {
    if (!plan) return TFFT_ERR_BAD_ARG;
    *plan = nullptr;
    if (logN < 1 || logN > 30 || batch < 1 || (dtype != TFFT_FLOAT2 && dtype != TFFT_DOUBLE2) || thread_bs < 1 || device < 0)
        return TFFT_ERR_BAD_ARG;
    int flavour = 0;
    if (log_cluster >= 0) {
        flavour = ((log_cluster & TFFT_SINGLE_PASS_PREFETCH) ? 1 : 0) + ((log_cluster & TFFT_SINGLE_PASS_RADIX8) ? 2 : 0);
        log_cluster &= ~(TFFT_SINGLE_PASS_PREFETCH | TFFT_SINGLE_PASS_RADIX8);
    }
    const ClusterKernel* ck = find_cluster_kernel(dtype, logN, log_cluster, flavour);
    if (!ck) return TFFT_ERR_UNSUPPORTED;
    DeviceGuard guard(device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    if (cluster_kernel_fits(*ck) < 1) return TFFT_ERR_UNSUPPORTED;
    const long long clusters = (batch + thread_bs - 1) / thread_bs;
    if ((clusters << ck->logg) > 2147483647LL) return TFFT_ERR_TOO_LARGE;
    tfft_plan p = new (std::nothrow) tfft_plan_s();
    if (!p) return TFFT_ERR_ALLOC;
    p->logn = logN;
    p->batch = batch;
    p->dtype = dtype;
    p->thread_bs = thread_bs;
    p->device = device;
    p->n_launch = 1;
    p->ck = ck;
    p->cgrid_clusters = (unsigned)clusters;
    snprintf(p->nvtx_name, sizeof(p->nvtx_name), "tfft_exec logN=%d batch=%lld %s single-pass", logN, batch,
             dtype == TFFT_FLOAT2 ? "c64" : "c128");
    bool ok = dtype == TFFT_FLOAT2 ? build_cluster_tables<float>(p) : build_cluster_tables<double>(p);
    if (ok && ck->prefetch) {
        p->cstatus = (int*)dev_alloc(p, sizeof(int));
        ok = p->cstatus && cuda_ok(p, cudaMemset(p->cstatus, 0, sizeof(int)));
    }
    if (!ok) {
        const int status = p->last_cuda_error ? TFFT_ERR_CUDA : TFFT_ERR_ALLOC;
        for (void* q : p->allocs) cudaFree(q);
        delete p;
        return status;
    }
    *plan = p;
    return TFFT_OK;
}

int tfft_plan_create_strided(tfft_plan* plan, int logN, long long inner, long long outer, int dtype, int device) {
    if (!plan) return TFFT_ERR_BAD_ARG;
    *plan = nullptr;
    const int log_b = ilog2_exact(inner);
    if (logN < 1 || logN > 30 || inner < 1 || log_b < 0 || outer < 1 || (dtype != TFFT_FLOAT2 && dtype != TFFT_DOUBLE2) || device < 0)
        return TFFT_ERR_BAD_ARG;
    // the widest compiled strided-line kernel for this length whose tile fits the inner extent
    const KernelEntry* k = nullptr;
    int logc = 0, loge = 0;
    for (int c = 5; c >= 0 && !k; --c) {
        if (c > log_b) continue;
        for (int e = 5; e >= 1 && !k; --e) {
            const KernelEntry* q = find_kernel(dtype, ROLE_FIRST, logN, e, c);
            if (q && q->fn[FT_OFF]) {
                k = q;
                logc = c;
                loge = e;
            }
        }
    }
    if (!k) return TFFT_ERR_UNSUPPORTED;
    const long long tiles = outer << (log_b - logc);
    if (tiles > 2147483647LL || (outer << log_b) > (1LL << (62 - logN))) return TFFT_ERR_TOO_LARGE;
    DeviceGuard guard(device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    tfft_plan p = new (std::nothrow) tfft_plan_s();
    if (!p) return TFFT_ERR_ALLOC;
    p->logn = logN;
    p->batch = outer << log_b;
    p->dtype = dtype;
    p->device = device;
    p->n_launch = 1;
    p->strided = 1;
    LaunchDesc& d = p->L[0];
    d.role = ROLE_FIRST;
    d.logm = logN;
    d.loge = loge;
    d.logc = logc;
    d.log_b = log_b;
    d.n_tiles = tiles;
    d.grid = (unsigned)tiles;
    d.k = k;
    snprintf(p->nvtx_name, sizeof(p->nvtx_name), "tfft_exec logN=%d strided inner=%lld outer=%lld", logN, inner, outer);
    int status = TFFT_OK;
    if (k->smem > 40 * 1024 &&
        !cuda_ok(p, cudaFuncSetAttribute(k->fn[FT_OFF], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k->smem)))
        status = TFFT_ERR_CUDA;
    if (status == TFFT_OK) {
        const bool okb = dtype == TFFT_FLOAT2 ? build_tables<float>(p) : build_tables<double>(p);
        if (!okb) status = p->last_cuda_error ? TFFT_ERR_CUDA : TFFT_ERR_ALLOC;
    }
#if TFFT_BOUNDS_CHECK
    if (status == TFFT_OK) {
        p->oob = (unsigned long long*)dev_alloc(p, sizeof(unsigned long long));
        if (!p->oob || !cuda_ok(p, cudaMemset(p->oob, 0, sizeof(unsigned long long)))) status = TFFT_ERR_ALLOC;
    }
#endif
    if (status != TFFT_OK) {
        for (void* q : p->allocs) cudaFree(q);
        delete p;
        return status;
    }
    *plan = p;
    return TFFT_OK;
}

int tfft_plan_device_status(tfft_plan p, int* status) {
    if (!p || !status) return TFFT_ERR_BAD_ARG;
    *status = 0;
    const int* word = p->cstatus ? p->cstatus : p->pair_status;
    if (!word) return TFFT_OK;
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    if (!cuda_ok(p, cudaMemcpy(status, word, sizeof(int), cudaMemcpyDeviceToHost))) return TFFT_ERR_CUDA;
    return TFFT_OK;
}

int tfft_plan_fuse_launches(tfft_plan p, int log_chunk_signals, int lag) {
    if (!p || log_chunk_signals < 0 || log_chunk_signals > 20 || lag < 0 || lag > 2) return TFFT_ERR_BAD_ARG;
    if (p->pk) return TFFT_OK;
    if (p->n_launch != 2 || p->if_ft || p->strided || p->ck) return TFFT_ERR_UNSUPPORTED;
    const LaunchDesc& a = p->L[0];
    const LaunchDesc& b = p->L[1];
    const PairKernel* pk = find_pair_kernel(p->dtype, a.logm, a.loge, a.logc, b.logm, b.loge, b.logc);
    if (!pk) return TFFT_ERR_UNSUPPORTED;
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    int coop = 0;
    if (!cuda_ok(p, cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, p->device))) return TFFT_ERR_CUDA;
    const int resident = coop ? pair_kernel_resident_blocks(*pk) : 0;
    if (resident < 1) return TFFT_ERR_UNSUPPORTED;
    const long long chunk = 1LL << log_chunk_signals;
    const long long chunks = (p->batch + chunk - 1) / chunk;
    const long long t1 = (a.n_tiles / p->batch) << log_chunk_signals, t2 = (b.n_tiles / p->batch) << log_chunk_signals;
    if (t1 > (1LL << 30) || t2 > (1LL << 30)) return TFFT_ERR_TOO_LARGE;
    const int ring_chunks = 4;  // a power of two above lag + 1
    void* ring = dev_alloc(p, ((size_t)(ring_chunks * chunk) << p->logn) * p->esize());
    unsigned int* done = (unsigned int*)dev_alloc(p, (size_t)(2 * chunks + 2) * sizeof(unsigned int));
    int* status = (int*)dev_alloc(p, sizeof(int));
    if (!ring || !done || !status) return TFFT_ERR_ALLOC;  // the plan keeps what was allocated until it is destroyed
    if (!cuda_ok(p, cudaMemset(status, 0, sizeof(int)))) return TFFT_ERR_CUDA;
    // the launches' whole-batch intermediate is not needed any more
    if (p->scratch) {
        for (size_t i = 0; i < p->allocs.size(); ++i)
            if (p->allocs[i] == p->scratch) {
                p->allocs.erase(p->allocs.begin() + (long)i);
                break;
            }
        cudaFree(p->scratch);
        p->owned_bytes -= ((size_t)p->batch << p->logn) * p->esize();
        p->scratch = nullptr;
    }
    p->ring = ring;
    p->pair_done = done;
    p->pair_status = status;
    p->pair_chunks = chunks;
    p->pair_log_chunk = log_chunk_signals;
    p->pair_lag = lag;
    p->pair_ring_chunks = ring_chunks;
    const long long items = (chunks + lag) * (t1 + t2);
    p->pair_grid = (int)(items < resident ? items : resident);
    p->pk = pk;
    return TFFT_OK;
}

int tfft_plan_cluster_size(tfft_plan p) { return p ? (p->ck ? (1 << p->ck->logg) : 0) : TFFT_ERR_BAD_ARG; }

int tfft_exec(tfft_plan p, const void* in, void* out, void* stream) {
    if (!p || !in || !out) return TFFT_ERR_BAD_ARG;
    if (in == out && p->n_launch == 1 && p->if_err && !(p->csum && csum_ok(p->L[0].k))) return TFFT_ERR_UNSUPPORTED;
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    p->last_stream = st;
    NvtxRange range(p->nvtx_name);
    return p->dtype == TFFT_FLOAT2 ? launch_all<float>(p, in, out, st, p->scratch) : launch_all<double>(p, in, out, st, p->scratch);
}

size_t tfft_scratch_bytes(tfft_plan p) {
    if (!p || p->n_launch < 2 || p->ck || p->pk) return 0;  // single-pass and fused plans carry what they need
    return ((size_t)p->batch << p->logn) * p->esize();
}

int tfft_exec_ws(tfft_plan p, const void* in, void* out, void* workspace, void* stream) {
    if (!p || !in || !out) return TFFT_ERR_BAD_ARG;
    if (p->if_ft || p->pk) return TFFT_ERR_UNSUPPORTED;  // FT status buffers / the fused kernel's ring and counters belong to the plan: one exec at a time
    if (tfft_scratch_bytes(p) && !workspace) return TFFT_ERR_BAD_ARG;
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    NvtxRange range(p->nvtx_name);
    return p->dtype == TFFT_FLOAT2 ? launch_all<float>(p, in, out, st, workspace) : launch_all<double>(p, in, out, st, workspace);
}

// Pipelined form of tfft_exec_host for plans without FT whose batch spans several chunks:
// the batch is cut into chunks of whole signals (about 64 MiB); chunk i is copied in on one
// stream, transformed on a second and copied out on a third, three slots deep, so the two
// PCIe directions and the kernels overlap.  Returns TFFT_ERR_UNSUPPORTED when the plan does
// not qualify (the caller then takes the plain path).
static int exec_host_pipelined(tfft_plan p, const void* in_host, void* out_host, cudaStream_t user, bool sync) {
    const size_t sig_bytes = ((size_t)1 << p->logn) * p->esize();
    long long cb = (long long)(kPipeChunkBytes / sig_bytes);
    // signals longer than a chunk travel one per chunk (up to 512 MiB each: six staging slots of that size)
    if (cb < 1 && sig_bytes <= ((size_t)512 << 20)) cb = 1;
    // chunk plans are ordinary launch plans over whole signals: strided-batch, single-pass and fused plans
    // (and FT plans, whose status is per plan) take the unchunked path with their own kernels
    if (p->if_ft || p->strided || p->ck || p->pk || cb < 1 || p->batch < 3 * cb) return TFFT_ERR_UNSUPPORTED;
    if (!p->pipe_ready) {
        // every resource is created only if it is still missing, so a call that failed half way
        // can be repeated; the plan's destructor releases whatever exists
        const char* csv = p->param_csv.empty() ? nullptr : p->param_csv.c_str();
        if (!p->chunk_plan) {
            const int rc = tfft_plan_create(&p->chunk_plan, p->logn, cb, p->dtype, 0, 0, p->thread_bs, csv, p->device);
            if (rc != TFFT_OK) return rc;
            p->chunk_batch = cb;
        }
        if (p->batch % p->chunk_batch && !p->tail_plan) {
            const int rc = tfft_plan_create(&p->tail_plan, p->logn, p->batch % p->chunk_batch, p->dtype, 0, 0,
                                            p->thread_bs, csv, p->device);
            if (rc != TFFT_OK) return rc;
        }
        tfft_set_direction(p, p->inverse, p->scale);  // hand the direction down to the sub-plans
        p->pipe_ready = true;
    }
    cb = p->chunk_batch;
    const size_t chunk_bytes = (size_t)cb * sig_bytes;
    std::lock_guard<std::mutex> lock(g_stage_mu);
    PipeSlots& ps = g_pipe[p->device];
    if (!ps.ready) {
        for (int i = 0; i < 3; ++i) {
            if (!ps.stream[i] && !cuda_ok(p, cudaStreamCreateWithFlags(&ps.stream[i], cudaStreamNonBlocking)))
                return TFFT_ERR_CUDA;
            if ((!ps.ev_in[i] && !cuda_ok(p, cudaEventCreateWithFlags(&ps.ev_in[i], cudaEventDisableTiming))) ||
                (!ps.ev_fft[i] && !cuda_ok(p, cudaEventCreateWithFlags(&ps.ev_fft[i], cudaEventDisableTiming))) ||
                (!ps.ev_out[i] && !cuda_ok(p, cudaEventCreateWithFlags(&ps.ev_out[i], cudaEventDisableTiming))))
                return TFFT_ERR_CUDA;
        }
        if (!ps.ev_start && !cuda_ok(p, cudaEventCreateWithFlags(&ps.ev_start, cudaEventDisableTiming)))
            return TFFT_ERR_CUDA;
        ps.ready = true;
    }
    cudaStream_t s_in = ps.stream[0], s_fft = ps.stream[1], s_out = ps.stream[2];
    if (ps.bytes < chunk_bytes) {
        // larger slots: whatever earlier calls queued on the old ones has to finish first
        for (int i = 0; i < 3; ++i)
            if (!cuda_ok(p, cudaStreamSynchronize(ps.stream[i]))) return TFFT_ERR_CUDA;
        for (int i = 0; i < 3; ++i) {
            if (ps.in[i]) cudaFree(ps.in[i]);
            if (ps.out[i]) cudaFree(ps.out[i]);
            ps.in[i] = ps.out[i] = nullptr;
        }
        ps.bytes = 0;
        ps.seq = 0;
        for (int i = 0; i < 3; ++i)
            if (!cuda_ok(p, cudaMalloc(&ps.in[i], chunk_bytes)) || !cuda_ok(p, cudaMalloc(&ps.out[i], chunk_bytes)))
                return TFFT_ERR_ALLOC;
        ps.bytes = chunk_bytes;
    }
    // everything queued on the caller's stream so far comes first
    if (!cuda_ok(p, cudaEventRecord(ps.ev_start, user))) return TFFT_ERR_CUDA;
    for (int i = 0; i < 3; ++i)
        if (!cuda_ok(p, cudaStreamWaitEvent(ps.stream[i], ps.ev_start, 0))) return TFFT_ERR_CUDA;
    const long long nchunk = (p->batch + cb - 1) / cb;
    for (long long c = 0; c < nchunk; ++c) {
        const int slot = (int)(ps.seq % 3);
        const long long this_b = (c == nchunk - 1 && p->batch % cb) ? p->batch % cb : cb;
        const size_t bytes = (size_t)this_b * sig_bytes;
        const char* src = (const char*)in_host + (size_t)c * chunk_bytes;
        char* dst = (char*)out_host + (size_t)c * chunk_bytes;
        if (ps.seq >= 3) {
            // slot reuse (by this call or an earlier one): its previous transform has consumed in[slot], its
            // previous copy-out has drained out[slot]
            if (!cuda_ok(p, cudaStreamWaitEvent(s_in, ps.ev_fft[slot], 0))) return TFFT_ERR_CUDA;
            if (!cuda_ok(p, cudaStreamWaitEvent(s_fft, ps.ev_out[slot], 0))) return TFFT_ERR_CUDA;
        }
        ++ps.seq;
        if (!cuda_ok(p, cudaMemcpyAsync(ps.in[slot], src, bytes, cudaMemcpyHostToDevice, s_in))) return TFFT_ERR_CUDA;
        if (!cuda_ok(p, cudaEventRecord(ps.ev_in[slot], s_in))) return TFFT_ERR_CUDA;
        if (!cuda_ok(p, cudaStreamWaitEvent(s_fft, ps.ev_in[slot], 0))) return TFFT_ERR_CUDA;
        const int rc = tfft_exec(this_b == cb ? p->chunk_plan : p->tail_plan, ps.in[slot], ps.out[slot], s_fft);
        if (rc != TFFT_OK) return rc;
        if (!cuda_ok(p, cudaEventRecord(ps.ev_fft[slot], s_fft))) return TFFT_ERR_CUDA;
        if (!cuda_ok(p, cudaStreamWaitEvent(s_out, ps.ev_fft[slot], 0))) return TFFT_ERR_CUDA;
        if (!cuda_ok(p, cudaMemcpyAsync(dst, ps.out[slot], bytes, cudaMemcpyDeviceToHost, s_out))) return TFFT_ERR_CUDA;
        if (!cuda_ok(p, cudaEventRecord(ps.ev_out[slot], s_out))) return TFFT_ERR_CUDA;
    }
    p->last_stream = s_fft;
    if (sync)
        for (int i = 0; i < 3; ++i)
            if (!cuda_ok(p, cudaStreamSynchronize(ps.stream[i]))) return TFFT_ERR_CUDA;
    return TFFT_OK;
}

// the unchunked form: whole batch in, transform, whole batch out on the caller's stream
static int exec_host_plain(tfft_plan p, const void* in_host, void* out_host, void* stream) {
    const size_t bytes = ((size_t)p->batch << p->logn) * p->esize();
    std::lock_guard<std::mutex> lock(g_stage_mu);
    StagePair& sp = g_stage[p->device];
    if (sp.bytes < bytes) {
        if (sp.in) cudaFree(sp.in);
        if (sp.out) cudaFree(sp.out);
        sp = StagePair();
        if (!cuda_ok(p, cudaMalloc(&sp.in, bytes)) || !cuda_ok(p, cudaMalloc(&sp.out, bytes))) {
            if (sp.in) cudaFree(sp.in);
            sp = StagePair();
            return TFFT_ERR_ALLOC;
        }
        sp.bytes = bytes;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (!cuda_ok(p, cudaMemcpyAsync(sp.in, in_host, bytes, cudaMemcpyHostToDevice, st))) return TFFT_ERR_CUDA;
    const int rc = tfft_exec(p, sp.in, sp.out, stream);
    if (rc != TFFT_OK) return rc;
    if (!cuda_ok(p, cudaMemcpyAsync(out_host, sp.out, bytes, cudaMemcpyDeviceToHost, st))) return TFFT_ERR_CUDA;
    if (!cuda_ok(p, cudaStreamSynchronize(st))) return TFFT_ERR_CUDA;
    return TFFT_OK;
}

int tfft_exec_host(tfft_plan p, const void* in_host, void* out_host, void* stream) {
    if (!p || !in_host || !out_host) return TFFT_ERR_BAD_ARG;
    NvtxRange range("tfft_exec_host");
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    const int rc = exec_host_pipelined(p, in_host, out_host, (cudaStream_t)stream, true);
    if (rc != TFFT_ERR_UNSUPPORTED) return rc;
    return exec_host_plain(p, in_host, out_host, stream);
}

int tfft_exec_host_async(tfft_plan p, const void* in_host, void* out_host, void* stream) {
    if (!p || !in_host || !out_host) return TFFT_ERR_BAD_ARG;
    NvtxRange range("tfft_exec_host_async");
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    const int rc = exec_host_pipelined(p, in_host, out_host, (cudaStream_t)stream, false);
    if (rc != TFFT_ERR_UNSUPPORTED) return rc;
    // plans the pipeline does not take run at once; what the pipeline still holds is unaffected
    return exec_host_plain(p, in_host, out_host, stream);
}

int tfft_host_sync(int device) {
    if (device < 0) return TFFT_ERR_BAD_ARG;
    DeviceGuard guard(device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_stage_mu);
    auto it = g_pipe.find(device);
    if (it == g_pipe.end()) return TFFT_OK;
    for (int i = 0; i < 3; ++i)
        if (it->second.stream[i] && cudaStreamSynchronize(it->second.stream[i]) != cudaSuccess) return TFFT_ERR_CUDA;
    return TFFT_OK;
}

size_t tfft_workspace_bytes(tfft_plan p) { return p ? p->owned_bytes : 0; }

int tfft_plan_info(tfft_plan p, int* info) {
    if (!p || !info) return TFFT_ERR_BAD_ARG;
    info[0] = p->n_launch;
    for (int i = 0; i < 3; ++i) {
        int* o = info + 1 + 6 * i;
        if (i == 0 && p->ck) {
            o[0] = p->logn;
            o[1] = 1;
            o[2] = 2 << p->ck->lr;
            o[3] = (int)(p->cgrid_clusters << p->ck->logg);
            o[4] = p->ck->threads;
            o[5] = (int)p->ck->smem;
        } else if (i < p->n_launch) {
            const LaunchDesc& d = p->L[i];
            o[0] = d.logm;
            o[1] = 1 << d.logc;
            o[2] = 1 << d.loge;
            o[3] = (int)d.grid;
            o[4] = d.k->threads;
            o[5] = (int)d.k->smem;
        } else {
            for (int j = 0; j < 6; ++j) o[j] = 0;
        }
    }
    return TFFT_OK;
}

int tfft_set_ft_params(tfft_plan p, double err_inj, double err_smoothing, double err_threshold) {
    if (!p) return TFFT_ERR_BAD_ARG;
    p->err_inj = err_inj;
    p->err_smoothing = err_smoothing;
    p->err_threshold = err_threshold;
    return TFFT_OK;
}

int tfft_set_correction(tfft_plan p, int from_checksums) {
    if (!p) return TFFT_ERR_BAD_ARG;
    if (from_checksums && !p->if_err) return TFFT_ERR_BAD_ARG;
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    if (from_checksums) {
        bool any = false;
        for (int i = 0; i < p->n_launch; ++i) {
            const KernelEntry* k = p->L[i].k;
            if (!csum_ok(k)) continue;  // this launch keeps recomputing
            any = true;
            if (k->smem_csum > 40 * 1024 &&
                !cuda_ok(p, cudaFuncSetAttribute(k->fn[FT_CSUM], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k->smem_csum)))
                return TFFT_ERR_CUDA;
        }
        if (!any) return TFFT_ERR_UNSUPPORTED;
    }
    p->csum = from_checksums ? 1 : 0;
    return TFFT_OK;
}

int tfft_set_direction(tfft_plan p, int inverse, double scale) {
    if (!p || !(scale == scale)) return TFFT_ERR_BAD_ARG;
    p->inverse = inverse ? 1 : 0;
    p->scale = scale;
    if (p->chunk_plan) tfft_set_direction(p->chunk_plan, inverse, scale);
    if (p->tail_plan) tfft_set_direction(p->tail_plan, inverse, scale);
    return TFFT_OK;
}

int tfft_set_injection(tfft_plan p, int enable, int launch, int period, int phase) {
    if (!p || period < 1 || phase < 0 || phase >= period || launch >= p->n_launch) return TFFT_ERR_BAD_ARG;
    p->inj_enable = enable ? 1 : 0;
    p->inj_launch = launch;
    p->inj_period = period;
    p->inj_phase = phase;
    return TFFT_OK;
}

int tfft_ft_status(tfft_plan p, int* n_detected, int* n_corrected, int launch, int* located, int cap, int* n_blocks) {
    if (!p) return TFFT_ERR_BAD_ARG;
    if (n_detected) *n_detected = 0;
    if (n_corrected) *n_corrected = 0;
    if (n_blocks) *n_blocks = 0;
    if (!p->if_ft) return TFFT_OK;
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    if (!cuda_ok(p, cudaStreamSynchronize(p->last_stream))) return TFFT_ERR_CUDA;
    unsigned int cnt[6];
    if (!cuda_ok(p, cudaMemcpy(cnt, p->ft_count, sizeof(cnt), cudaMemcpyDeviceToHost))) return TFFT_ERR_CUDA;
    if (p->ft_accumulate && !cuda_ok(p, cudaMemset(p->ft_count, 0, sizeof(cnt)))) return TFFT_ERR_CUDA;
    for (int i = 0; i < p->n_launch; ++i) {
        if (n_detected) *n_detected += (int)cnt[2 * i];
        if (n_corrected) *n_corrected += (int)cnt[2 * i + 1];
    }
    if (launch < 0) launch = p->n_launch - 1;
    if (launch >= p->n_launch) return TFFT_ERR_BAD_ARG;
    if (n_blocks) *n_blocks = (int)p->L[launch].grid;
    if (located && cap > 0) {
        const size_t n = (size_t)(cap < (int)p->L[launch].grid ? cap : (int)p->L[launch].grid);
        if (!cuda_ok(p, cudaMemcpy(located, p->L[launch].ft_located, n * sizeof(int), cudaMemcpyDeviceToHost)))
            return TFFT_ERR_CUDA;
    }
    return TFFT_OK;
}

int tfft_set_ft_accumulate(tfft_plan p, int enable) {
    if (!p) return TFFT_ERR_BAD_ARG;
    if (enable && !p->ft_accumulate && p->ft_count) {  // start the totals from zero
        DeviceGuard guard(p->device);
        if (!guard.ok) return TFFT_ERR_CUDA;
        if (!cuda_ok(p, cudaStreamSynchronize(p->last_stream)) || !cuda_ok(p, cudaMemset(p->ft_count, 0, 6 * sizeof(unsigned int))))
            return TFFT_ERR_CUDA;
    }
    p->ft_accumulate = enable ? 1 : 0;
    return TFFT_OK;
}

int tfft_bounds_status(tfft_plan p, long long* bad_index, int* site) {
    if (!p) return TFFT_ERR_BAD_ARG;
    if (bad_index) *bad_index = -1;
    if (site) *site = 0;
#if TFFT_BOUNDS_CHECK
    if (!p->oob) return TFFT_ERR_UNSUPPORTED;  // single-pass plans carry no checks
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    if (!cuda_ok(p, cudaStreamSynchronize(p->last_stream))) return TFFT_ERR_CUDA;
    unsigned long long w = 0;
    if (!cuda_ok(p, cudaMemcpy(&w, p->oob, sizeof(w), cudaMemcpyDeviceToHost))) return TFFT_ERR_CUDA;
    if (w >> 63) {
        long long idx = (long long)(w & ((1ULL << 56) - 1));
        if (idx & (1LL << 55)) idx |= ~((1LL << 56) - 1);  // sign of a negative index
        if (bad_index) *bad_index = idx;
        if (site) *site = (int)((w >> 56) & 0x7f);
        if (!cuda_ok(p, cudaMemset(p->oob, 0, sizeof(w)))) return TFFT_ERR_CUDA;
        return 1;
    }
    return TFFT_OK;
#else
    return TFFT_ERR_UNSUPPORTED;
#endif
}

int tfft_enable_ft_diag(tfft_plan p, int enable) {
    if (!p) return TFFT_ERR_BAD_ARG;
    p->diag = enable ? 1 : 0;
    return TFFT_OK;
}

int tfft_ft_diag(tfft_plan p, int launch, double* diag, int cap_blocks) {
    if (!p || !diag || !p->if_ft) return TFFT_ERR_BAD_ARG;
    if (launch < 0) launch = p->n_launch - 1;
    if (launch >= p->n_launch) return TFFT_ERR_BAD_ARG;
    DeviceGuard guard(p->device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    if (!cuda_ok(p, cudaStreamSynchronize(p->last_stream))) return TFFT_ERR_CUDA;
    const size_t n = 3 * (size_t)(cap_blocks < (int)p->L[launch].grid ? cap_blocks : (int)p->L[launch].grid);
    if (p->dtype == TFFT_FLOAT2) {
        std::vector<float> tmp(n);
        if (!cuda_ok(p, cudaMemcpy(tmp.data(), p->L[launch].ft_diag, n * sizeof(float), cudaMemcpyDeviceToHost)))
            return TFFT_ERR_CUDA;
        for (size_t i = 0; i < n; ++i) diag[i] = tmp[i];
    } else {
        if (!cuda_ok(p, cudaMemcpy(diag, p->L[launch].ft_diag, n * sizeof(double), cudaMemcpyDeviceToHost)))
            return TFFT_ERR_CUDA;
    }
    return TFFT_OK;
}

int tfft_plan_destroy(tfft_plan p) {
    if (!p) return TFFT_ERR_BAD_ARG;
    DeviceGuard guard(p->device);
    if (p->pipe_ready) tfft_host_sync(p->device);  // chunks this plan queued with tfft_exec_host_async still use its sub-plans
    if (p->chunk_plan) tfft_plan_destroy(p->chunk_plan);
    if (p->tail_plan) tfft_plan_destroy(p->tail_plan);
    for (void* q : p->allocs) cudaFree(q);
    delete p;
    return TFFT_OK;
}

int tfft_last_cuda_error(tfft_plan p) { return p ? p->last_cuda_error : 0; }

const char* tfft_status_string(int s) {
    switch (s) {
        case TFFT_OK: return "ok";
        case TFFT_ERR_BAD_ARG: return "bad argument";
        case TFFT_ERR_UNSUPPORTED: return "unsupported size or mode (no parameter row or no compiled kernel)";
        case TFFT_ERR_CUDA: return "CUDA error";
        case TFFT_ERR_PARAM_FILE: return "parameter CSV missing or malformed";
        case TFFT_ERR_ALLOC: return "allocation failed";
        case TFFT_ERR_TOO_LARGE: return "size beyond the supported maximum";
        default: return "unknown status";
    }
}

long long tfft_launch_count(void) { return g_launches.load(); }

}  // extern "C"

// ------------------------------------------------------------------------------------------
// tfft_exec_static: the multi-launch transform with NO allocation anywhere on the call path.
//
// Multi-launch plans keep their intermediate result in a scratch buffer that
// tfft_plan_create() obtains with cudaMalloc.  Some callers must not allocate at the time
// they call -- code running inside a memory-pool-managed region, inside a latency-critical
// loop that forbids driver allocation calls, or in a process whose device memory has been
// handed out completely.  For them the scratch buffer and the twiddle tables live in two
// file-scope __device__ arrays that every GPU loading this library holds from load to
// exit: 16 MiB of scratch and 512 KiB of tables.
//
// In host code the names of those arrays are host-side stand-ins, not device addresses, so
// the device address is looked up once per device with cudaGetSymbolAddress (with that
// device current) and passed to the kernels like any other pointer.
namespace {

constexpr size_t kStaticScratchBytes = 16u << 20;
constexpr size_t kStaticTableBytes = 512u << 10;
constexpr int kStaticMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) unsigned char g_static_tables[kStaticTableBytes];

struct StaticDeviceState {
    bool ready = false;
    void* scratch = nullptr;  // device address of g_static_scratch on this device
    void* tables = nullptr;   // device address of g_static_tables on this device
    int table_logn = -1;      // which (logN, dtype) the table region currently holds
    int table_dtype = -1;
    LaunchDesc L[3];
    int n_launch = 0;
};
std::mutex g_static_mu;
StaticDeviceState g_static_dev[kStaticMaxDevices];

// Geometry and kernels of the launches of one built-in parameter row (FT off); the same
// rules as tfft_plan_create(), without owning anything.
int static_geometry(const ParamRow& row, int logN, long long batch, int dtype, LaunchDesc* L) {
    long long outer = batch;
    int log_rest = logN;
    for (int i = 0; i < row.launches; ++i) {
        LaunchDesc& d = L[i];
        d = LaunchDesc();
        d.logm = row.logni[i];
        d.logc = ilog2_exact(row.bs[i]);
        d.loge = ilog2_exact(row.n[i]);
        if (d.loge > d.logm) d.loge = d.logm;
        d.role = i == row.launches - 1 ? ROLE_LAST : ROLE_FIRST;
        log_rest -= d.logm;
        if (d.role == ROLE_FIRST) {
            d.log_b = log_rest;
            if (d.log_b < d.logc) d.logc = d.log_b;
            d.n_tiles = outer << (d.log_b - d.logc);
        } else {
            d.log_n1 = row.logni[0];
            d.log_q = row.launches == 3 ? row.logni[1] : 0;
            if (d.log_n1 < d.logc) d.logc = d.log_n1;
            d.n_tiles = (batch << (logN - d.logm)) >> d.logc;
        }
        outer <<= d.logm;
        d.k = find_kernel(dtype, d.role, d.logm, d.loge, d.logc);
        if (!d.k || !d.k->fn[FT_OFF]) return TFFT_ERR_UNSUPPORTED;
        if (d.n_tiles > 2147483647LL) return TFFT_ERR_TOO_LARGE;
        d.grid = (unsigned)d.n_tiles;
    }
    return TFFT_OK;
}

// Number of entries of stage_twiddles(logm, loge, *): sum over all stages but the last of
// log2(R_t) * M / R_t; the set of radices does not depend on the stage order.
size_t stage_twiddle_count(int logm, int loge) {
    const int stages = (logm + loge - 1) / loge;
    const int logr0 = logm - (stages - 1) * loge;
    if (stages == 1) return 1;
    // remainder radix first: stages 0..S-2 = logr0, loge, ...; remainder last: loge x (S-1).
    // The kernel reads the table in its own order, so both cases are sized for the larger one.
    size_t first = (size_t)logr0 << (logm - logr0), last = 0;
    for (int t = 1; t + 1 < stages; ++t) first += (size_t)loge << (logm - loge);
    for (int t = 0; t + 1 < stages; ++t) last += (size_t)loge << (logm - loge);
    return first > last ? first : last;
}

// Lays the twiddle tables of the launches out in the static table region and, if `fill`,
// builds them on the host and copies them there (stream ordered).  The layout depends only
// on (logN, dtype), so a call that finds its own tables already resident passes fill = false
// and only gets the pointers.  No allocation on the device.
template <typename T>
int static_place_tables(StaticDeviceState& st, bool fill, cudaStream_t stream) {
    typedef typename Cplx<T>::type C;
    size_t off = 0;
    auto reserve = [&](size_t count, void** dev) -> int {
        const size_t bytes = count * sizeof(C);
        if (off + bytes > kStaticTableBytes) return TFFT_ERR_TOO_LARGE;
        *dev = (unsigned char*)st.tables + off;
        off += (bytes + 255) & ~(size_t)255;
        return TFFT_OK;
    };
    auto copy = [&](const std::vector<C>& host, void* dev) -> int {
        // pageable source: cudaMemcpyAsync returns once the data is staged, so `host` may go away
        return cudaMemcpyAsync(dev, host.data(), host.size() * sizeof(C), cudaMemcpyHostToDevice, stream) == cudaSuccess
                   ? TFFT_OK
                   : TFFT_ERR_CUDA;
    };
    for (int i = 0; i < st.n_launch; ++i) {
        LaunchDesc& d = st.L[i];
        int rc = reserve(stage_twiddle_count(d.logm, d.loge), &d.tw_st);
        if (rc != TFFT_OK) return rc;
        if (fill) {
            std::vector<C> t;
            stage_twiddles(t, d.logm, d.loge, d.k->remlast != 0);
            if ((rc = copy(t, d.tw_st)) != TFFT_OK) return rc;
        }
        if (d.role == ROLE_FIRST) {
            const int logp = d.logm + d.log_b;
            d.tw_lo_bits = (logp + 1) / 2;
            if ((rc = reserve((size_t)1 << d.tw_lo_bits, &d.tw_lo)) != TFFT_OK) return rc;
            if ((rc = reserve((size_t)1 << (logp - d.tw_lo_bits), &d.tw_hi)) != TFFT_OK) return rc;
            if (fill) {
                std::vector<C> lo, hi;
                fill_twiddles(lo, 1LL << d.tw_lo_bits, 1, logp);
                fill_twiddles(hi, 1LL << (logp - d.tw_lo_bits), 1LL << d.tw_lo_bits, logp);
                if ((rc = copy(lo, d.tw_lo)) != TFFT_OK) return rc;
                if ((rc = copy(hi, d.tw_hi)) != TFFT_OK) return rc;
            }
        }
    }
    return TFFT_OK;
}

template <typename T>
int static_launch(const StaticDeviceState& st, int logN, const void* in, void* out, cudaStream_t stream) {
    typedef typename Cplx<T>::type C;
    for (int i = 0; i < st.n_launch; ++i) {
        const LaunchDesc& d = st.L[i];
        KernelArgs<T> a;
        memset(&a, 0, sizeof(a));
        a.in = (const C*)(i == 0 ? in : st.scratch);
        a.out = (C*)(i == st.n_launch - 1 ? out : st.scratch);
        a.tw_st = (const C*)d.tw_st;
        a.tw_lo = (const C*)d.tw_lo;
        a.tw_hi = (const C*)d.tw_hi;
        a.n_tiles = d.n_tiles;
        a.tiles_per_cta = 1;
        a.log_n = logN;
        a.log_b = d.log_b;
        a.log_n1 = d.log_n1;
        a.log_q = d.log_q;
        a.tw_lo_bits = d.tw_lo_bits;
        a.inj_period = 1;
        void* args[] = {&a};
        if (cudaLaunchKernel(d.k->fn[FT_OFF], dim3(d.grid), dim3(d.k->threads), args, d.k->smem, stream) != cudaSuccess)
            return TFFT_ERR_CUDA;
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return TFFT_OK;
}

}  // namespace

extern "C" int tfft_exec_static(int logN, long long batch, int dtype, const void* in, void* out, int device,
                                void* stream) {
    if (!in || !out || batch < 1 || logN < 1 || logN > 24 || (dtype != TFFT_FLOAT2 && dtype != TFFT_DOUBLE2) ||
        device < 0 || device >= kStaticMaxDevices)
        return TFFT_ERR_BAD_ARG;
    const size_t esize = dtype == TFFT_FLOAT2 ? sizeof(float2) : sizeof(double2);
    // the whole intermediate result must fit in the static scratch array
    if ((unsigned long long)batch > ((kStaticScratchBytes / esize) >> logN)) return TFFT_ERR_TOO_LARGE;
    std::vector<ParamRow> rows;
    std::string err;
    if (!parse_param_csv(builtin_param_csv(dtype), rows, err)) return TFFT_ERR_PARAM_FILE;
    if ((int)rows.size() <= logN || rows[logN].launches < 2) return TFFT_ERR_UNSUPPORTED;  // 1-launch sizes use no scratch
    if (!validate_row(rows[logN], err)) return TFFT_ERR_PARAM_FILE;

    DeviceGuard guard(device);
    if (!guard.ok) return TFFT_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticDeviceState& st = g_static_dev[device];
    if (!st.ready) {
        // once per device, with that device current: device addresses of the two arrays
        if (cudaGetSymbolAddress(&st.scratch, g_static_scratch) != cudaSuccess) return TFFT_ERR_CUDA;
        if (cudaGetSymbolAddress(&st.tables, g_static_tables) != cudaSuccess) return TFFT_ERR_CUDA;
        st.ready = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    st.n_launch = rows[logN].launches;
    int rc = static_geometry(rows[logN], logN, batch, dtype, st.L);
    if (rc != TFFT_OK) return rc;
    for (int i = 0; i < st.n_launch; ++i)
        if (st.L[i].k->smem > 40 * 1024 &&
            cudaFuncSetAttribute(st.L[i].k->fn[FT_OFF], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st.L[i].k->smem) !=
                cudaSuccess)
            return TFFT_ERR_CUDA;
    // The table region keeps the previous call's tables: a call with the same (logN, dtype)
    // finds them in place and only recomputes the pointers -- no host table building and no
    // host-to-device copy, which is what a call inside a stream capture needs.  A change of
    // size rebuilds them on the host and uploads them on the caller's stream, behind the
    // previous call's kernels.
    const bool fill = !(st.table_logn == logN && st.table_dtype == dtype);
    if (fill) st.table_logn = st.table_dtype = -1;  // nothing valid if the upload fails half way
    rc = dtype == TFFT_FLOAT2 ? static_place_tables<float>(st, fill, s) : static_place_tables<double>(st, fill, s);
    if (rc != TFFT_OK) return rc;
    st.table_logn = logN;
    st.table_dtype = dtype;
    return dtype == TFFT_FLOAT2 ? static_launch<float>(st, logN, in, out, s) : static_launch<double>(st, logN, in, out, s);
}

namespace tfft {
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace tfft
