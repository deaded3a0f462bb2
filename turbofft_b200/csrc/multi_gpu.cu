// One transform too long for a GPU, driven from ONE process over several devices with peer
// access (the tfft_mg_* entries of include/turbofft_b200.h).  No counterpart in the reference,
// which is single-GPU.  Same four-step algorithm and the same kernels as the multi-process form
// (turbofft_b200/multi_gpu.py): N = N1 * N2 seen as an N1 x N2 row-major matrix whose rows are
// block-distributed over the ranks;
//   exchange 1  every rank transposes its rows and stores them straight into all ranks' receive
//               buffers over NVLink (tfft_scatter_transpose_part), giving each rank N2/P columns
//               with all N1 rows as contiguous lines;
//   transform 1 local FFTs of length N1 (an ordinary plan, FT if asked);
//   exchange 2  the same kernel with the twiddle W_N^(n2 k1) folded in, back to rows;
//   transform 2 local FFTs of length N2 -> X[k1 + N1 k2] at rank(k1), [k1_local][k2];
//   (natural order: a third exchange leaves each rank its contiguous slab of X).
// Nothing on a device ever waits for a peer: the order between ranks is made of CUDA events
// recorded on one device's stream and waited for on another's, all enqueued by the calling host
// thread.  Each exchange is cut into `pipeline` pieces on a low-priority stream; the transform
// of the lines piece g completed runs on a high-priority stream while piece g + 1 is in flight.
#include <cuda_runtime.h>

#include <new>
#include <vector>

#include "../../include/turbofft_b200.h"

struct tfft_mg_plan_s {
    int logn = 0, dtype = 0, if_ft = 0, P = 0, natural = 0, G = 1;
    int l1 = 0, l2 = 0;
    long long n1 = 0, n2 = 0, n1l = 0, n2l = 0;
    size_t esize = 8;
    int max_blocks = 0;
    std::vector<int> dev;
    std::vector<cudaStream_t> side, fast;
    std::vector<void*> buf0, buf1, tmp;
    std::vector<tfft_plan> plan1, plan2;
    std::vector<std::vector<cudaEvent_t>> ev_x1, ev_x2;  // [rank][piece]: that piece of the exchange has been issued and has completed
    std::vector<cudaEvent_t> ev_f1, ev_f2, ev_x3, ev_done, ev_user;
    int last_cuda_error = 0;
    bool ran = false;
};

namespace {

struct Dev {
    int prev = -1;
    explicit Dev(int d) {
        cudaGetDevice(&prev);
        cudaSetDevice(d);
    }
    ~Dev() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

bool ok(tfft_mg_plan p, cudaError_t e) {
    if (e == cudaSuccess) return true;
    p->last_cuda_error = (int)e;
    return false;
}

void release(tfft_mg_plan p) {
    for (int r = 0; r < p->P; ++r) {
        Dev d(p->dev[r]);
        if (r < (int)p->plan1.size() && p->plan1[r]) tfft_plan_destroy(p->plan1[r]);
        if (r < (int)p->plan2.size() && p->plan2[r]) tfft_plan_destroy(p->plan2[r]);
        for (auto* v : {&p->buf0, &p->buf1, &p->tmp})
            if (r < (int)v->size() && (*v)[r]) cudaFree((*v)[r]);
        for (auto* v : {&p->side, &p->fast})
            if (r < (int)v->size() && (*v)[r]) cudaStreamDestroy((*v)[r]);
        for (auto* v : {&p->ev_f1, &p->ev_f2, &p->ev_x3, &p->ev_done, &p->ev_user})
            if (r < (int)v->size() && (*v)[r]) cudaEventDestroy((*v)[r]);
        for (auto* v : {&p->ev_x1, &p->ev_x2})
            if (r < (int)v->size())
                for (cudaEvent_t e : (*v)[r])
                    if (e) cudaEventDestroy(e);
    }
    delete p;
}

// One exchange in G pieces plus the transforms behind it.  src[r]: rank r's [rows][cols] matrix;
// every rank's receive buffer buf[r] gets [cols / P] lines of pitch ld with rank r's rows at r * rows.
int exchange_and_transform(tfft_mg_plan p, const std::vector<const void*>& src, const std::vector<void*>& buf,
                           long long rows, long long cols, long long ld, int twiddle, std::vector<tfft_plan>& plans,
                           int line_log, const std::vector<void*>& out, std::vector<std::vector<cudaEvent_t>>& ev_x,
                           std::vector<cudaEvent_t>& ev_f) {
    const int P = p->P, G = p->G;
    const long long piece = (cols / P) / G;  // lines of a receiver completed by one piece
    const size_t step = (size_t)piece * ((size_t)1 << line_log) * p->esize;
    for (int g = 0; g < G; ++g)
        for (int r = 0; r < P; ++r) {
            Dev d(p->dev[r]);
            const int rc = tfft_scatter_transpose_part(src[r], buf.data(), P, rows, cols, ld, (long long)r * rows, twiddle,
                                                       p->logn, g * piece, piece, p->max_blocks, p->dtype, p->side[r]);
            if (rc != TFFT_OK) return rc;
            if (!ok(p, cudaEventRecord(ev_x[r][g], p->side[r]))) return TFFT_ERR_CUDA;
        }
    for (int g = 0; g < G; ++g)
        for (int r = 0; r < P; ++r) {
            Dev d(p->dev[r]);
            for (int q = 0; q < P; ++q)  // every sender's piece g has landed
                if (!ok(p, cudaStreamWaitEvent(p->fast[r], ev_x[q][g], 0))) return TFFT_ERR_CUDA;
            const int rc = tfft_exec(plans[r], (const char*)buf[r] + g * step, (char*)out[r] + g * step, p->fast[r]);
            if (rc != TFFT_OK) return rc;
        }
    for (int r = 0; r < P; ++r) {
        Dev d(p->dev[r]);
        if (!ok(p, cudaEventRecord(ev_f[r], p->fast[r]))) return TFFT_ERR_CUDA;
    }
    return TFFT_OK;
}

}  // namespace

extern "C" {

int tfft_mg_plan_create(tfft_mg_plan* plan, int logN, int dtype, int if_ft, int n_devices, const int* devices,
                        int natural_order, int pipeline) {
    if (!plan) return TFFT_ERR_BAD_ARG;
    *plan = nullptr;
    if (!devices || n_devices < 1 || n_devices > 16 || (n_devices & (n_devices - 1)) || logN < 12 || logN > 40 ||
        (dtype != TFFT_FLOAT2 && dtype != TFFT_DOUBLE2) || pipeline < 1)
        return TFFT_ERR_BAD_ARG;
    tfft_mg_plan p = new (std::nothrow) tfft_mg_plan_s();
    if (!p) return TFFT_ERR_ALLOC;
    p->logn = logN;
    p->dtype = dtype;
    p->if_ft = if_ft ? 1 : 0;
    p->P = n_devices;
    p->natural = natural_order ? 1 : 0;
    p->G = pipeline;
    p->l1 = (logN + 1) / 2;
    p->l2 = logN - p->l1;
    p->n1 = 1LL << p->l1;
    p->n2 = 1LL << p->l2;
    p->n1l = p->n1 / n_devices;
    p->n2l = p->n2 / n_devices;
    p->esize = dtype == TFFT_FLOAT2 ? 8 : 16;
    p->dev.assign(devices, devices + n_devices);
    // each rank's share of both factors must split into `pipeline` pieces of whole 32-line tiles
    if (p->n1l < 32LL * pipeline || p->n2l < 32LL * pipeline || p->n1l % (32LL * pipeline) || p->n2l % (32LL * pipeline)) {
        delete p;
        return TFFT_ERR_UNSUPPORTED;
    }
    const int P = n_devices;
    int status = TFFT_OK;
    // peer access between every pair of distinct devices
    for (int a = 0; a < P && status == TFFT_OK; ++a) {
        Dev d(p->dev[a]);
        for (int b = 0; b < P && status == TFFT_OK; ++b) {
            if (p->dev[a] == p->dev[b]) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, p->dev[a], p->dev[b]) != cudaSuccess || !can) {
                status = TFFT_ERR_UNSUPPORTED;
                break;
            }
            const cudaError_t e = cudaDeviceEnablePeerAccess(p->dev[b], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (e != cudaSuccess) {
                p->last_cuda_error = (int)e;
                status = TFFT_ERR_CUDA;
            }
        }
    }
    p->side.assign(P, nullptr);
    p->fast.assign(P, nullptr);
    p->buf0.assign(P, nullptr);
    p->buf1.assign(P, nullptr);
    p->tmp.assign(P, nullptr);
    p->plan1.assign(P, nullptr);
    p->plan2.assign(P, nullptr);
    p->ev_f1.assign(P, nullptr);
    p->ev_f2.assign(P, nullptr);
    p->ev_x3.assign(P, nullptr);
    p->ev_done.assign(P, nullptr);
    p->ev_user.assign(P, nullptr);
    p->ev_x1.assign(P, std::vector<cudaEvent_t>(pipeline, nullptr));
    p->ev_x2.assign(P, std::vector<cudaEvent_t>(pipeline, nullptr));
    const size_t slab = (size_t)((1ULL << logN) / P) * p->esize;
    for (int r = 0; r < P && status == TFFT_OK; ++r) {
        Dev d(p->dev[r]);
        int lo = 0, hi = 0, sms = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);  // lo = least urgent
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->dev[r]);
        // the exchange is NVLink bound: a few resident blocks per SM saturate the links and the
        // transforms it overlaps with get the rest
        if (pipeline > 1 && P > 1) p->max_blocks = 4 * sms;
        bool good = ok(p, cudaStreamCreateWithPriority(&p->side[r], cudaStreamNonBlocking, lo)) &&
                    ok(p, cudaStreamCreateWithPriority(&p->fast[r], cudaStreamNonBlocking, hi)) &&
                    ok(p, cudaMalloc(&p->buf0[r], slab)) && ok(p, cudaMalloc(&p->buf1[r], slab)) &&
                    ok(p, cudaMalloc(&p->tmp[r], slab));
        for (cudaEvent_t* e : {&p->ev_f1[r], &p->ev_f2[r], &p->ev_x3[r], &p->ev_done[r], &p->ev_user[r]})
            good = good && ok(p, cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        for (int g = 0; g < pipeline; ++g)
            good = good && ok(p, cudaEventCreateWithFlags(&p->ev_x1[r][g], cudaEventDisableTiming)) &&
                   ok(p, cudaEventCreateWithFlags(&p->ev_x2[r][g], cudaEventDisableTiming));
        if (!good) {
            status = TFFT_ERR_CUDA;
            break;
        }
        status = tfft_plan_create(&p->plan1[r], p->l1, p->n2l / pipeline, dtype, if_ft, 0, 1, nullptr, p->dev[r]);
        if (status == TFFT_OK)
            status = tfft_plan_create(&p->plan2[r], p->l2, p->n1l / pipeline, dtype, if_ft, 0, 1, nullptr, p->dev[r]);
        if (status == TFFT_OK && if_ft) {
            tfft_set_ft_accumulate(p->plan1[r], 1);
            tfft_set_ft_accumulate(p->plan2[r], 1);
        }
    }
    if (status != TFFT_OK) {
        release(p);
        return status;
    }
    *plan = p;
    return TFFT_OK;
}

int tfft_mg_exec(tfft_mg_plan p, const void* const* in, void* const* out, void* const* streams) {
    if (!p || !in || !out) return TFFT_ERR_BAD_ARG;
    const int P = p->P;
    for (int r = 0; r < P; ++r)
        if (!in[r] || !out[r]) return TFFT_ERR_BAD_ARG;
    // order against the caller's streams and against the previous call (whose last readers of the
    // receive buffers must be done before any rank stores into them again)
    for (int r = 0; r < P; ++r) {
        Dev d(p->dev[r]);
        if (streams) {
            if (!ok(p, cudaEventRecord(p->ev_user[r], (cudaStream_t)streams[r]))) return TFFT_ERR_CUDA;
            if (!ok(p, cudaStreamWaitEvent(p->side[r], p->ev_user[r], 0))) return TFFT_ERR_CUDA;
        }
        if (p->ran)
            for (int q = 0; q < P; ++q)
                if (!ok(p, cudaStreamWaitEvent(p->side[r], p->ev_done[q], 0))) return TFFT_ERR_CUDA;
    }
    std::vector<const void*> src(in, in + P);
    int rc = exchange_and_transform(p, src, p->buf0, p->n1l, p->n2, p->n1, 0, p->plan1, p->l1, p->tmp, p->ev_x1, p->ev_f1);
    if (rc != TFFT_OK) return rc;
    for (int r = 0; r < P; ++r) {  // exchange 2 reads what transform 1 wrote
        Dev d(p->dev[r]);
        if (!ok(p, cudaStreamWaitEvent(p->side[r], p->ev_f1[r], 0))) return TFFT_ERR_CUDA;
        src[r] = p->tmp[r];
    }
    std::vector<void*> outs(out, out + P);
    rc = exchange_and_transform(p, src, p->buf1, p->n2l, p->n1, p->n2, 1, p->plan2, p->l2, outs, p->ev_x2, p->ev_f2);
    if (rc != TFFT_OK) return rc;
    if (p->natural) {
        // X[k1 + N1 k2]: one more transposing exchange, then each rank copies its slab out of buffer 0
        for (int r = 0; r < P; ++r) {
            Dev d(p->dev[r]);
            if (!ok(p, cudaStreamWaitEvent(p->side[r], p->ev_f2[r], 0))) return TFFT_ERR_CUDA;
            rc = tfft_scatter_transpose_part(out[r], p->buf0.data(), P, p->n1l, p->n2, p->n1, (long long)r * p->n1l, 0, p->logn, 0,
                                             p->n2l, 0, p->dtype, p->side[r]);
            if (rc != TFFT_OK) return rc;
            if (!ok(p, cudaEventRecord(p->ev_x3[r], p->side[r]))) return TFFT_ERR_CUDA;
        }
        const size_t slab = (size_t)((1ULL << p->logn) / P) * p->esize;
        for (int r = 0; r < P; ++r) {
            Dev d(p->dev[r]);
            for (int q = 0; q < P; ++q)
                if (!ok(p, cudaStreamWaitEvent(p->fast[r], p->ev_x3[q], 0))) return TFFT_ERR_CUDA;
            if (!ok(p, cudaMemcpyAsync(out[r], p->buf0[r], slab, cudaMemcpyDeviceToDevice, p->fast[r]))) return TFFT_ERR_CUDA;
        }
    }
    for (int r = 0; r < P; ++r) {
        Dev d(p->dev[r]);
        if (!ok(p, cudaEventRecord(p->ev_done[r], p->fast[r]))) return TFFT_ERR_CUDA;
        if (streams && !ok(p, cudaStreamWaitEvent((cudaStream_t)streams[r], p->ev_done[r], 0))) return TFFT_ERR_CUDA;
    }
    p->ran = true;
    return TFFT_OK;
}

int tfft_mg_sync(tfft_mg_plan p) {
    if (!p) return TFFT_ERR_BAD_ARG;
    for (int r = 0; r < p->P; ++r) {
        Dev d(p->dev[r]);
        if (!ok(p, cudaStreamSynchronize(p->side[r])) || !ok(p, cudaStreamSynchronize(p->fast[r]))) return TFFT_ERR_CUDA;
    }
    return TFFT_OK;
}

int tfft_mg_ft_status(tfft_mg_plan p, int* n_detected, int* n_corrected) {
    if (!p) return TFFT_ERR_BAD_ARG;
    int nd = 0, nc = 0;
    if (p->if_ft) {
        const int rc = tfft_mg_sync(p);
        if (rc != TFFT_OK) return rc;
        for (int r = 0; r < p->P; ++r)
            for (tfft_plan q : {p->plan1[r], p->plan2[r]}) {
                int d = 0, c = 0;
                const int s = tfft_ft_status(q, &d, &c, -1, nullptr, 0, nullptr);
                if (s != TFFT_OK) return s;
                nd += d;
                nc += c;
            }
    }
    if (n_detected) *n_detected = nd;
    if (n_corrected) *n_corrected = nc;
    return TFFT_OK;
}

int tfft_mg_last_cuda_error(tfft_mg_plan p) { return p ? p->last_cuda_error : 0; }

int tfft_mg_destroy(tfft_mg_plan p) {
    if (!p) return TFFT_ERR_BAD_ARG;
    tfft_mg_sync(p);
    release(p);
    return TFFT_OK;
}

}  // extern "C"
