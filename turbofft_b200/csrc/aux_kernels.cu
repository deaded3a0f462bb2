// Helper kernels behind the C ABI that are not FFT launches: the STREAM-style copy
// that measures the HBM peak every roofline fraction is quoted against, and the
// (twiddled) transposes the multi-GPU four-step transform is assembled from.
#include <cuda_runtime.h>

#include <cstring>

#include "../../include/turbofft_b200.h"
#include "registry.h"

namespace {

// Each block copies one contiguous chunk of 2 x 256 x 16 bytes and exits; on B200 a
// full grid of short blocks measured higher than a persistent grid-stride loop.
__global__ void __launch_bounds__(256) stream_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                          size_t n) {
    const size_t i0 = (size_t)blockIdx.x * 512 + threadIdx.x;
    const size_t i1 = i0 + 256;
    uint4 a, b;
    if (i0 < n) a = __ldcs(src + i0);
    if (i1 < n) b = __ldcs(src + i1);
    if (i0 < n) __stcs(dst + i0, a);
    if (i1 < n) __stcs(dst + i1, b);
}

template <typename C> struct RealOf;
template <> struct RealOf<float2> { typedef float type; };
template <> struct RealOf<double2> { typedef double type; };

// exp(-2*pi*i*ph / 2^log_total).  Single precision splits the phase into two exactly
// representable angles (high and low 15 bits) and multiplies the two unit vectors, which keeps
// float accuracy for totals up to 2^30 without double-precision arithmetic.
__device__ __forceinline__ float2 unit_twiddle(unsigned long long ph, int log_total, float) {
    const int lo_bits = log_total > 15 ? log_total - 15 : 0;
    const unsigned long long hi = ph >> lo_bits, lo = ph & ((1ULL << lo_bits) - 1);
    float s1, c1, s2, c2;
    sincospif(-2.0f * (float)hi / (float)(1ULL << (log_total - lo_bits)), &s1, &c1);
    sincospif(-2.0f * (float)lo / (float)(1ULL << log_total), &s2, &c2);
    return make_float2(c1 * c2 - s1 * s2, s1 * c2 + c1 * s2);
}
__device__ __forceinline__ double2 unit_twiddle(unsigned long long ph, int log_total, double) {
    double sn, cs;
    sincospi(-2.0 * (double)ph / (double)(1ULL << log_total), &sn, &cs);
    return make_double2(cs, sn);
}

// 32x32 tile transpose through padded shared memory; TW multiplies by
// exp(-2*pi*i*(row0+r)*(col0+c)/2^log_total); the integer phase (r*c mod 2^log_total) is
// reduced exactly before the angle is formed.
template <typename C, bool TW>
__global__ void __launch_bounds__(256) transpose_kernel(const C* __restrict__ src, C* __restrict__ dst, long long rows,
                                                        long long cols, long long row0, long long col0, int log_total) {
    __shared__ C tile[32][33];
    const long long tiles_c = (cols + 31) / 32;
    const long long tr = blockIdx.x / tiles_c, tc = blockIdx.x % tiles_c;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const long long r = tr * 32 + ty + 8 * k, c = tc * 32 + tx;
        if (r < rows && c < cols) {
            C v = src[r * cols + c];
            if (TW) {
                typedef typename RealOf<C>::type T;
                const unsigned long long mask = (1ULL << log_total) - 1;
                const unsigned long long ph = ((unsigned long long)(row0 + r) * (unsigned long long)(col0 + c)) & mask;
                const C u = unit_twiddle(ph, log_total, T(0));
                C w;
                w.x = v.x * u.x - v.y * u.y;
                w.y = v.x * u.y + v.y * u.x;
                v = w;
            }
            tile[ty + 8 * k][tx] = v;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const long long c = tc * 32 + ty + 8 * k, r = tr * 32 + tx;
        if (r < rows && c < cols) dst[c * rows + r] = tile[tx][ty + 8 * k];
    }
}

// dst[b][a][0..run) = src[a][b][0..run): swaps the two outer axes of an [A][B][run] array
// whose innermost runs are contiguous; run is counted in 16-byte words.
__global__ void __launch_bounds__(256) permute102_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                         long long A, long long B, long long run) {
    const long long total = A * B * run;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long w = i % run;
        const long long ab = i / run;
        const long long a = ab % A, b = ab / A;  // i enumerates the destination [b][a][w]
        dst[i] = __ldcs(src + (a * B + b) * run + w);
    }
}

// Fused "transpose + all-to-all + unpack" of the multi-GPU four-step transform: element
// (i, c) of the local row-major matrix src[rows][cols] goes to rank j = c / cb, into that
// rank's buffer dst[j] at [(c % cb) * ld + row0 + i] -- the transposed position in the
// receiver's layout -- optionally multiplied by exp(-2*pi*i*(row0 + i)*c / 2^log_total).
// dst[j] are device pointers (this GPU's own buffer for j == rank, peer mappings otherwise);
// the stores are plain coalesced st.global over NVLink, 32 consecutive elements per row of a
// tile.  Completion on the receivers is established by the caller (a stream-ordered barrier
// after the kernel); this kernel never waits on a peer.
constexpr int kMaxPeers = 16;
template <typename C>
struct PeerPtrs {
    C* p[kMaxPeers];
    long long ld[kMaxPeers];    // line pitch of receiver j's buffer, in elements
    long long roff[kMaxPeers];  // where this sender's rows start inside a line of receiver j
};


template <typename C, bool TW>
__global__ void __launch_bounds__(256) scatter_transpose_kernel(const C* __restrict__ src, PeerPtrs<C> dst, long long rows,
                                                                long long cols, long long cb, long long row0,
                                                                int log_total, int n_peers, long long sub_off, long long sub_len) {
    __shared__ C tile[32][33];
    // the launch covers, for every receiver j, the columns j*cb + sub_off + [0, sub_len)
    const long long ts = sub_len / 32;
    const long long n_tiles = (rows / 32) * ts * n_peers;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    // grid-stride over the tiles: a caller that overlaps this kernel with transforms gives it a
    // small grid so that it keeps a few slots per SM and leaves the rest to them
    for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const long long tr = t / (ts * n_peers);
        const long long rem = t % (ts * n_peers);
        const long long c0 = (rem / ts) * cb + sub_off + (rem % ts) * 32;
        const long long c = c0 + tx;
        // a thread's four rows are 8 apart: w_k = w_0 * (W^(8c))^k, two evaluations instead of four
        C w, step;
        if (TW) {
            typedef typename RealOf<C>::type T;
            const unsigned long long mask = (1ULL << log_total) - 1;
            w = unit_twiddle(((unsigned long long)(row0 + tr * 32 + ty) * (unsigned long long)c) & mask, log_total, T(0));
            step = unit_twiddle((8ULL * (unsigned long long)c) & mask, log_total, T(0));
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const long long r = tr * 32 + ty + 8 * k;
            C v = __ldcs(src + r * cols + c);
            if (TW) {
                C u;
                u.x = v.x * w.x - v.y * w.y;
                u.y = v.x * w.y + v.y * w.x;
                v = u;
                if (k < 3) {
                    C n;
                    n.x = w.x * step.x - w.y * step.y;
                    n.y = w.x * step.y + w.y * step.x;
                    w = n;
                }
            }
            tile[ty + 8 * k][tx] = v;
        }
        __syncthreads();
        const int j = (int)(c0 / cb);  // a tile never straddles two receivers: cb, sub_off are multiples of 32
        C* base = dst.p[j] + dst.roff[j] + tr * 32 + tx;
        const long long ld = dst.ld[j];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const long long c = c0 + ty + 8 * k;
            base[(c % cb) * ld] = tile[tx][ty + 8 * k];
        }
        __syncthreads();  // the tile buffer is reused by the next iteration
    }
}

// The same exchange for complex64 with 16-byte stores: tiles of 64 rows x 32 columns, a lane
// writes two consecutive rows of one receiver column as one float4, so a warp's store covers a
// 512-byte run of the receiver's line (the 32-row form above writes 256-byte runs of 8-byte
// elements, which the NVLink path moves at a lower rate).  Needs rows % 64 == 0 and receiver
// lines that start on 16-byte boundaries.
template <bool TW>
__global__ void __launch_bounds__(256) scatter_transpose_wide_kernel(const float2* __restrict__ src, PeerPtrs<float2> dst,
                                                                     long long rows, long long cols, long long cb,
                                                                     long long row0, int log_total, int n_peers,
                                                                     long long sub_off, long long sub_len) {
    __shared__ __align__(16) float2 tile[32][66];  // [column][row]; pitch 66 keeps every tile row 16-byte aligned
    const long long ts = sub_len / 32;
    const long long n_tiles = (rows / 64) * ts * n_peers;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const long long tr = t / (ts * n_peers);
        const long long rem = t % (ts * n_peers);
        const long long c0 = (rem / ts) * cb + sub_off + (rem % ts) * 32;
        const long long c = c0 + tx;
        float2 w, step;
        if (TW) {
            const unsigned long long mask = (1ULL << log_total) - 1;
            w = unit_twiddle(((unsigned long long)(row0 + tr * 64 + ty) * (unsigned long long)c) & mask, log_total, 0.0f);
            step = unit_twiddle((8ULL * (unsigned long long)c) & mask, log_total, 0.0f);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const long long r = tr * 64 + ty + 8 * k;
            float2 v = __ldcs(src + r * cols + c);
            if (TW) {
                const float2 u = make_float2(v.x * w.x - v.y * w.y, v.x * w.y + v.y * w.x);
                v = u;
                if (k < 7) w = make_float2(w.x * step.x - w.y * step.y, w.x * step.y + w.y * step.x);
            }
            tile[tx][ty + 8 * k] = v;
        }
        __syncthreads();
        const int j = (int)(c0 / cb);
        float2* base = dst.p[j] + dst.roff[j] + tr * 64;
        const long long ld = dst.ld[j];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const long long cc = c0 + ty + 8 * k;
            const float4 v = *reinterpret_cast<const float4*>(&tile[ty + 8 * k][2 * tx]);
            reinterpret_cast<float4*>(base + (cc % cb) * ld)[tx] = v;
        }
        __syncthreads();
    }
}

template <bool TW>
int launch_transpose(const void* src, void* dst, long long rows, long long cols, long long row0, long long col0,
                     int log_total, int dtype, void* stream) {
    if (!src || !dst || rows < 1 || cols < 1 || (dtype != TFFT_FLOAT2 && dtype != TFFT_DOUBLE2)) return TFFT_ERR_BAD_ARG;
    if (TW && (log_total < 1 || log_total > 62 || (dtype == TFFT_FLOAT2 && log_total > 39))) return TFFT_ERR_BAD_ARG;
    const long long blocks = ((rows + 31) / 32) * ((cols + 31) / 32);
    if (blocks > 2147483647LL) return TFFT_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == TFFT_FLOAT2)
        transpose_kernel<float2, TW><<<(unsigned)blocks, 256, 0, st>>>((const float2*)src, (float2*)dst, rows, cols, row0,
                                                                      col0, log_total);
    else
        transpose_kernel<double2, TW><<<(unsigned)blocks, 256, 0, st>>>((const double2*)src, (double2*)dst, rows, cols,
                                                                        row0, col0, log_total);
    tfft::note_launch();
    return cudaGetLastError() == cudaSuccess ? TFFT_OK : TFFT_ERR_CUDA;
}

}  // namespace

extern "C" {

int tfft_stream_copy(const void* src, void* dst, size_t bytes, void* stream) {
    if (!src || !dst || (bytes & 15) || (((size_t)src | (size_t)dst) & 15)) return TFFT_ERR_BAD_ARG;
    const size_t n = bytes / 16;
    if (n == 0) return TFFT_OK;
    const size_t blocks = (n + 511) / 512;
    if (blocks > 2147483647ULL) return TFFT_ERR_TOO_LARGE;
    stream_copy_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, n);
    tfft::note_launch();
    return cudaGetLastError() == cudaSuccess ? TFFT_OK : TFFT_ERR_CUDA;
}

int tfft_permute102(const void* src, void* dst, long long A, long long B, long long run_elems, int dtype,
                    void* stream) {
    if (!src || !dst || A < 1 || B < 1 || run_elems < 1 || (dtype != TFFT_FLOAT2 && dtype != TFFT_DOUBLE2))
        return TFFT_ERR_BAD_ARG;
    const long long bytes = run_elems * (dtype == TFFT_FLOAT2 ? 8 : 16);
    if ((bytes & 15) || (((size_t)src | (size_t)dst) & 15)) return TFFT_ERR_BAD_ARG;
    const long long run = bytes / 16;
    const long long total = A * B * run;
    long long blocks = (total + 255) / 256;
    if (blocks > 148LL * 64) blocks = 148LL * 64;
    permute102_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, A, B, run);
    tfft::note_launch();
    return cudaGetLastError() == cudaSuccess ? TFFT_OK : TFFT_ERR_CUDA;
}

int tfft_scatter_transpose_ex(const void* src, void* const* dst, const long long* dst_ld, const long long* dst_row0,
                              int n_peers, long long rows, long long cols, long long tw_row0, int twiddle, int log_total,
                              long long sub_off, long long sub_len, int max_blocks, int dtype, void* stream) {
    if (!src || !dst || !dst_ld || !dst_row0 || n_peers < 1 || n_peers > kMaxPeers || rows < 32 || cols < 32 ||
        (rows & 31) || (cols & 31) || cols % n_peers || ((cols / n_peers) & 31) ||
        (dtype != TFFT_FLOAT2 && dtype != TFFT_DOUBLE2))
        return TFFT_ERR_BAD_ARG;
    if (twiddle && (log_total < 1 || log_total > 62 || (dtype == TFFT_FLOAT2 && log_total > 39))) return TFFT_ERR_BAD_ARG;
    const long long cb = cols / n_peers;
    if (sub_off < 0 || sub_len < 32 || (sub_off & 31) || (sub_len & 31) || sub_off + sub_len > cb) return TFFT_ERR_BAD_ARG;
    for (int i = 0; i < n_peers; ++i)
        if (!dst[i] || dst_ld[i] < rows || dst_row0[i] < 0 || dst_row0[i] + rows > dst_ld[i]) return TFFT_ERR_BAD_ARG;
    long long blocks = (rows / 32) * (sub_len / 32) * n_peers;
    if (max_blocks > 0 && blocks > max_blocks) blocks = max_blocks;
    if (blocks > 2147483647LL) blocks = 2147483647LL;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == TFFT_FLOAT2) {
        PeerPtrs<float2> pp;
        bool wide = (rows & 63) == 0;
        for (int i = 0; i < kMaxPeers; ++i) {
            pp.p[i] = (float2*)(i < n_peers ? dst[i] : nullptr);
            pp.ld[i] = i < n_peers ? dst_ld[i] : 0;
            pp.roff[i] = i < n_peers ? dst_row0[i] : 0;
            if (i < n_peers && (((size_t)dst[i] & 15) || (dst_ld[i] & 1) || (dst_row0[i] & 1))) wide = false;
        }
        if (wide) {
            long long wblocks = (rows / 64) * (sub_len / 32) * n_peers;
            if (max_blocks > 0 && wblocks > max_blocks) wblocks = max_blocks;
            if (wblocks > 2147483647LL) wblocks = 2147483647LL;
            if (twiddle)
                scatter_transpose_wide_kernel<true><<<(unsigned)wblocks, 256, 0, st>>>((const float2*)src, pp, rows, cols, cb, tw_row0, log_total, n_peers, sub_off, sub_len);
            else
                scatter_transpose_wide_kernel<false><<<(unsigned)wblocks, 256, 0, st>>>((const float2*)src, pp, rows, cols, cb, tw_row0, log_total, n_peers, sub_off, sub_len);
        } else if (twiddle)
            scatter_transpose_kernel<float2, true><<<(unsigned)blocks, 256, 0, st>>>((const float2*)src, pp, rows, cols, cb, tw_row0, log_total, n_peers, sub_off, sub_len);
        else
            scatter_transpose_kernel<float2, false><<<(unsigned)blocks, 256, 0, st>>>((const float2*)src, pp, rows, cols, cb, tw_row0, log_total, n_peers, sub_off, sub_len);
    } else {
        PeerPtrs<double2> pp;
        for (int i = 0; i < kMaxPeers; ++i) {
            pp.p[i] = (double2*)(i < n_peers ? dst[i] : nullptr);
            pp.ld[i] = i < n_peers ? dst_ld[i] : 0;
            pp.roff[i] = i < n_peers ? dst_row0[i] : 0;
        }
        if (twiddle)
            scatter_transpose_kernel<double2, true><<<(unsigned)blocks, 256, 0, st>>>((const double2*)src, pp, rows, cols, cb, tw_row0, log_total, n_peers, sub_off, sub_len);
        else
            scatter_transpose_kernel<double2, false><<<(unsigned)blocks, 256, 0, st>>>((const double2*)src, pp, rows, cols, cb, tw_row0, log_total, n_peers, sub_off, sub_len);
    }
    tfft::note_launch();
    return cudaGetLastError() == cudaSuccess ? TFFT_OK : TFFT_ERR_CUDA;
}

int tfft_scatter_transpose_part(const void* src, void* const* peer_dst, int n_peers, long long rows, long long cols,
                                long long ld_dst, long long row0, int twiddle, int log_total, long long sub_off,
                                long long sub_len, int max_blocks, int dtype, void* stream) {
    if (n_peers < 1 || n_peers > kMaxPeers) return TFFT_ERR_BAD_ARG;
    long long ld[kMaxPeers], r0[kMaxPeers];
    for (int i = 0; i < n_peers; ++i) {
        ld[i] = ld_dst;
        r0[i] = row0;
    }
    return tfft_scatter_transpose_ex(src, peer_dst, ld, r0, n_peers, rows, cols, row0, twiddle, log_total, sub_off, sub_len,
                                     max_blocks, dtype, stream);
}

int tfft_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width, size_t height,
                 void* stream) {
    if (!dst || !src || !width || !height || dst_pitch < width || src_pitch < width) return TFFT_ERR_BAD_ARG;
    return cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, height, cudaMemcpyDefault, (cudaStream_t)stream) ==
                   cudaSuccess
               ? TFFT_OK
               : TFFT_ERR_CUDA;
}

int tfft_scatter_transpose(const void* src, void* const* peer_dst, int n_peers, long long rows, long long cols,
                           long long ld_dst, long long row0, int twiddle, int log_total, int dtype, void* stream) {
    if (n_peers < 1 || cols % n_peers) return TFFT_ERR_BAD_ARG;
    return tfft_scatter_transpose_part(src, peer_dst, n_peers, rows, cols, ld_dst, row0, twiddle, log_total, 0,
                                       cols / n_peers, 0, dtype, stream);
}

// Peer-visible device buffers for the fused exchange: plain cudaMalloc so that the IPC
// handle refers to the start of the buffer.
int tfft_peer_alloc(size_t bytes, void** ptr) {
    if (!ptr || !bytes) return TFFT_ERR_BAD_ARG;
    return cudaMalloc(ptr, bytes) == cudaSuccess ? TFFT_OK : TFFT_ERR_ALLOC;
}
int tfft_peer_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? TFFT_OK : TFFT_ERR_CUDA; }
int tfft_peer_export(const void* ptr, void* handle64) {
    if (!ptr || !handle64) return TFFT_ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    return cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle64, (void*)ptr) == cudaSuccess ? TFFT_OK : TFFT_ERR_CUDA;
}
int tfft_peer_open(const void* handle64, void** ptr) {
    if (!ptr || !handle64) return TFFT_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? TFFT_OK : TFFT_ERR_CUDA;
}
int tfft_peer_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? TFFT_OK : TFFT_ERR_CUDA; }

int tfft_transpose(const void* src, void* dst, long long rows, long long cols, int dtype, void* stream) {
    return launch_transpose<false>(src, dst, rows, cols, 0, 0, 1, dtype, stream);
}

int tfft_twiddle_transpose(const void* src, void* dst, long long rows, long long cols, long long row0, long long col0,
                           int log_total, int dtype, void* stream) {
    return launch_transpose<true>(src, dst, rows, cols, row0, col0, log_total, dtype, stream);
}

}  // extern "C"
