/* turbofft_b200 -- C ABI of the B200 (sm_100a) batched power-of-two C2C FFT with
 * fused two-sided ABFT checksums.
 *
 * The reference (shixun404/TurboFFT) has no library API: its "operator" is the
 * kernel-pointer table TurboFFT_Kernel_Entry<T, if_ft, if_err, gpu>::turboFFTArr
 * (include/TurboFFT.h:22-25), driven by the launch protocol of test_turbofft()
 * (main.cu:4-73).  Each entry point below names the piece of that protocol it
 * replaces.  All pointers are plain device or host addresses; no C++ or torch
 * types cross this boundary.  Every function returns 0 on success or a negative
 * tfft_status; nothing calls exit().
 *
 * Conventions: forward transform, unnormalised, exp(-2*pi*i*n*k/N)
 * (include/utils/initializeData.h:31-37); input and output are [batch][N]
 * interleaved complex (float2 or double2) in natural order; the input buffer is
 * never written unless in == out.
 */
#ifndef TURBOFFT_B200_H
#define TURBOFFT_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tfft_plan_s* tfft_plan;

typedef enum {
    TFFT_OK = 0,
    TFFT_ERR_BAD_ARG = -1,      /* null pointer, logN out of range, batch < 1, ... */
    TFFT_ERR_UNSUPPORTED = -2,  /* no parameter row / no compiled kernel for this size */
    TFFT_ERR_CUDA = -3,         /* a CUDA call failed; see tfft_last_cuda_error() */
    TFFT_ERR_PARAM_FILE = -4,   /* parameter CSV missing or malformed */
    TFFT_ERR_ALLOC = -5,        /* device or host allocation failed */
    TFFT_ERR_TOO_LARGE = -6     /* size beyond a stated maximum */
} tfft_status;

/* dtype codes follow the reference CLI: --datatype 0 = float2, 1 = double2
 * (include/utils/CommandLineParser.h:67-69). */
enum { TFFT_FLOAT2 = 0, TFFT_DOUBLE2 = 1 };

/* Replaces: load_parameters() + the geometry loop of test_turbofft()
 * (include/utils/readCSV.h:13-33, main.cu:8-41) and the table set-up of
 * TurboFFT_main()/initializeData() (main.cu:85-93, initializeData.h:31-37).
 * param_csv: path of an 11-column parameter file (logN, launches, logN1..3,
 * BS1..3, n1..3; readme.md:46-60) or NULL for the built-in B200 table.
 * if_ft / if_err / thread_bs: the reference CLI flags of the same names; thread_bs = 0 picks
 * the value the tuner recorded for this size (param/B200/thread_bs_<dtype>.csv, else 1), cut down
 * for small batches until every launch still has a block for every resident slot of the device.
 * Allocates the twiddle and checksum tables, the scratch buffer of multi-launch
 * plans and the FT status buffers on `device`. */
int tfft_plan_create(tfft_plan* plan, int logN, long long batch, int dtype, int if_ft, int if_err,
                     int thread_bs, const char* param_csv, int device);

/* No counterpart in the reference, whose plans for 2^13..2^17 points are two launches
 * through a scratch buffer (include/param/A100/param_float2.csv rows 13-17).  Single-pass
 * plan: the whole signal is held in the shared memory of a thread-block cluster of
 * 2^log_cluster CTAs (distributed shared memory for the one exchange that crosses CTAs), so
 * HBM is read once and written once and the plan owns no scratch buffer.  log_cluster = -1
 * picks the default cluster size of the size.  FT off only; thread_bs = signals per cluster.
 * TFFT_ERR_UNSUPPORTED if no such kernel exists for (logN, dtype, log_cluster) or the device
 * cannot hold one cluster of it.  tfft_plan_create() makes this kind of plan by itself for
 * the sizes of the built-in single-pass table (param/B200/single_pass_<dtype>.csv) when
 * if_ft == 0 and param_csv == NULL.  `in` must be aligned to the element size and `out` to
 * 16 bytes; in == out is allowed. */
int tfft_plan_create_single_pass(tfft_plan* plan, int logN, long long batch, int dtype, int log_cluster,
                                 int thread_bs, int device);
/* OR-ed into log_cluster: the variant whose CTAs fetch their share of the NEXT signal into a
 * second shared-memory buffer with bulk asynchronous copies completing on an mbarrier while the
 * current signal is transformed (thread_bs > 1 gives it something to fetch ahead).  Its wait for
 * that buffer is bounded; tfft_plan_device_status reports 1 if a wait ever gave up (the output
 * of that exec is then invalid), 0 otherwise (synchronises with the device). */
#define TFFT_SINGLE_PASS_PREFETCH 16
/* OR-ed into log_cluster (complex64): the variant whose threads hold 16 points instead of 32
 * (radix-8 stages), with half the registers per thread and twice the resident warps. */
#define TFFT_SINGLE_PASS_RADIX8 32
int tfft_plan_device_status(tfft_plan plan, int* status);
/* Strided batch: the array is [outer][N][inner] (row-major, contiguous) and the transform runs
 * along the middle axis -- lines of N = 2^logN points strided by `inner` (a power of two),
 * outer * inner of them: the batch as an extra dimension, as the reference's small-N kernels
 * treat it (fft_codegen.py:756-762), and what a 2-D transform needs for its column pass.  One
 * launch of the strided-line kernel a multi-launch plan uses for its first launch, without the
 * inter-launch twiddle; tiles are adjacent columns, so rows are read and written in runs of up
 * to 32 elements.  Lengths: those with a compiled strided-line kernel (2^1..2^12 in the shipped
 * build), else TFFT_ERR_UNSUPPORTED.  FT off.  in == out is allowed.  tfft_set_direction
 * applies. */
int tfft_plan_create_strided(tfft_plan* plan, int logN, long long inner, long long outer, int dtype, int device);
/* Turns a two-launch plan (FT off) into ONE persistent, cooperatively launched kernel that runs
 * both launches chunk by chunk: 2^log_chunk_signals signals per chunk, the last launch `lag`
 * (0..2) chunks behind the first, the intermediate in a ring of 4 chunks that is small enough to
 * stay in L2 -- the whole-batch intermediate of the two launches (2 * batch * N elements of HBM
 * traffic) disappears and its buffer is freed.  Blocks order their accesses to the ring through
 * per-chunk counters with bounded waits; tfft_plan_device_status reports 1 if a wait ever gave
 * up (the output of that exec is then invalid).  TFFT_ERR_UNSUPPORTED if the plan is not two
 * FT-off launches, no fused kernel is compiled for its two launch shapes, or the device cannot
 * launch cooperatively.  The ring and the counters belong to the plan: one exec at a time
 * (tfft_exec_ws refuses such a plan).  The reference has no counterpart (its plans are separate launches,
 * TurboFFT.h:120-140). */
int tfft_plan_fuse_launches(tfft_plan plan, int log_chunk_signals, int lag);
/* CTAs per cluster of a single-pass plan, 0 for a plan made of ordinary launches. */
int tfft_plan_cluster_size(tfft_plan plan);

/* Replaces: the launch loop of test_turbofft() (main.cu:53-62) without its
 * per-launch cudaDeviceSynchronize().  `in` and `out` are device pointers to
 * batch*N complex elements; the result is always at `out` (the reference leaves
 * it in a launch-count dependent half of a 2x buffer, main.cu:11-12,72).
 * in == out is allowed except for 1-launch plans with if_err (the located tile
 * is recomputed from the input; see tfft_set_correction for the way around).  `stream` is a cudaStream_t (NULL = default).
 * Stream ordered; returns without synchronising. */
int tfft_exec(tfft_plan plan, const void* in, void* out, void* stream);

/* The same launches with the intermediate buffer supplied by the caller, so that ONE plan can be
 * executed from several host threads on several streams at the same time (tfft_exec keeps the
 * intermediate result of multi-launch plans in a buffer the plan owns, which two overlapping
 * execs would share).  workspace: tfft_scratch_bytes(plan) bytes of device memory, 256-byte
 * aligned, private to this exec until it has completed (NULL when that is 0: one-launch and
 * single-pass plans).  Plans without FT only (the FT status buffers are per plan), and not
 * fused plans (tfft_plan_fuse_launches): TFFT_ERR_UNSUPPORTED otherwise.  The reference's launcher is single-threaded and
 * synchronises after every launch (main.cu:58); it has nothing to share. */
size_t tfft_scratch_bytes(tfft_plan plan);
int tfft_exec_ws(tfft_plan plan, const void* in, void* out, void* workspace, void* stream);

/* Same transform with HOST buffers: copies batch*N elements to the device, runs
 * tfft_exec and copies the result back, then synchronises.  Replaces the
 * cudaMemcpy pair around the launches in initializeData()/test_turbofft()
 * (initializeData.h:39, main.cu:72).  Plans without FT whose batch spans at least
 * three chunks (64 MiB of whole signals, or one signal of up to 512 MiB) are pipelined: chunks of whole signals are copied in,
 * transformed and copied out on three internal streams so both PCIe directions
 * overlap the kernels (use pinned host buffers).  Device staging buffers, the
 * three streams and their events are per device, grow-only, shared by all plans
 * and kept until the library is unloaded; calls are serialised. */
int tfft_exec_host(tfft_plan plan, const void* in_host, void* out_host, void* stream);
/* The same call without the final synchronisation, for a sequence of transforms (of one plan or
 * of several): the chunks of consecutive calls share the device's three pipeline streams, so the
 * copy-out of one call's last chunks overlaps the copy-in of the next call's first ones instead
 * of each call filling and draining the pipeline alone (about 6 % of a 2 GiB call).  The host
 * buffers must stay valid and untouched until tfft_host_sync(device) has returned; results are
 * complete only then.  Work queued on `stream` before the call is waited for; nothing is queued
 * on `stream` behind it.  Plans the pipeline does not take (FT, strided, single-pass, fused,
 * batches under three chunks) run and complete inside the call as tfft_exec_host does.  A plan
 * may be destroyed while its chunks are in flight: tfft_plan_destroy waits for them. */
int tfft_exec_host_async(tfft_plan plan, const void* in_host, void* out_host, void* stream);
int tfft_host_sync(int device);

/* Bytes of device memory the plan owns (tables + scratch + status). */
size_t tfft_workspace_bytes(tfft_plan plan);

/* Number of launches and, per launch i < 3: log2 of the sub-transform, lines
 * per tile, points per thread, grid size, threads per block, dynamic shared
 * memory bytes -- the quantities test_turbofft() derives at main.cu:22-32.
 * info must hold 1 + 3*6 ints. */
int tfft_plan_info(tfft_plan plan, int* info);

/* The three literals fft_codegen.py bakes into the generated source
 * (--err_inj, --err_smoothing, --err_threshold; fft_codegen.py:414,495,714-719)
 * as run-time values.  Defaults: 100, 1000, 1e-3. */
int tfft_set_ft_params(tfft_plan plan, double err_inj, double err_smoothing, double err_threshold);

/* How a located tile is repaired (plans created with if_err).  0 (default): recompute it
 * from its input, what the reference's generated kernels do (fft_codegen.py:149-193).
 * 1: subtract sum(y) - F(sum(x)) taken over the block's tiles, the correction the reference
 * prepares (it accumulates both sums, fft_codegen.py:356-357,422-423) but leaves commented
 * out (:370,:403,:427-429; test.ipynb cell 0).  It does not read the input again, so a
 * 1-launch plan may then run in place; it costs two more tiles of shared memory per block.
 * Available for single and last launches; first and middle launches keep recomputing, and
 * no launch of a correcting plan overwrites what it reads (a three-launch plan created with
 * if_err owns a second scratch buffer for its middle launch, as the reference alternates
 * two buffers, main.cu:11-12).  TFFT_ERR_UNSUPPORTED if no launch of the plan has it.
 * The repaired outputs equal the fault-free ones up to rounding, not bit for bit. */
int tfft_set_correction(tfft_plan plan, int from_checksums);

/* Direction and normalisation (no counterpart in the reference, which is forward and
 * unnormalised only).  inverse != 0 computes scale * conj(F(conj(x))), i.e. the inverse DFT
 * for scale = 1/N; inverse == 0 computes scale * F(x).  The conjugations and the scaling
 * ride on the first launch's loads and the last launch's stores; FT checksums are taken on
 * the conjugated data and are unaffected.  Default: forward, scale 1. */
int tfft_set_direction(tfft_plan plan, int inverse, double scale);

/* Fault site selection.  The reference injects into every block of the last
 * launch (fft_codegen.py:412-415): that is launch = -1, period = 1, phase = 0
 * and is the default when the plan was created with if_err.  period > 1 hits
 * only blocks b with b % period == phase (sparse faults); launch selects which
 * launch of a multi-launch plan is hit; enable = 0 turns injection off while
 * keeping correction on. */
int tfft_set_injection(tfft_plan plan, int enable, int launch, int period, int phase);

/* FT outcome of the most recent tfft_exec (synchronises the plan's last
 * stream).  n_detected / n_corrected: blocks whose checksum test fired / tiles
 * recomputed, summed over launches.  located (may be NULL): for launch
 * `launch`, the per-block located tile iteration, 1-based, -1 = nothing
 * detected -- the register `k` of the reference kernels
 * (fft_codegen.py:47,495), which the reference never exports.  At most cap
 * entries are written; *n_blocks receives the launch's grid size. */
int tfft_ft_status(tfft_plan plan, int* n_detected, int* n_corrected, int launch, int* located, int cap,
                   int* n_blocks);

/* Counter mode (no counterpart in the reference, whose kernels keep no counters).  0
 * (default): n_detected / n_corrected describe the most recent tfft_exec.  1: they add up
 * over every tfft_exec until tfft_ft_status reads them, which also clears them -- for
 * callers that run one plan many times per job (the pieces of a pipelined multi-GPU
 * transform) and want the job's totals.  The per-block `located` array is always the last
 * exec's. */
int tfft_set_ft_accumulate(tfft_plan plan, int enable);

/* Per-block checksum residuals of launch `launch` from the most recent exec:
 * delta, S, delta_w as doubles, 3 per block (fft_codegen.py:432-495 keeps them
 * in registers).  Only recorded after tfft_enable_ft_diag(plan, 1). */
int tfft_enable_ft_diag(tfft_plan plan, int enable);
int tfft_ft_diag(tfft_plan plan, int launch, double* diag, int cap_blocks);

int tfft_plan_destroy(tfft_plan plan);

/* Checked build only (the library compiled with -DTFFT_BOUNDS_CHECK=1,
 * libturbofft_b200_check.so): every global load and store of the data buffers compares its
 * element index with the plan's batch * N; an access outside is skipped and the first one
 * is recorded.  Returns 0 if the most recent execs stayed inside, 1 if not (*bad_index = the
 * element index, *site = 1/2 load, 3/4 store; the record is cleared), TFFT_ERR_UNSUPPORTED
 * in the normal build.  The reference has no such check, and its stale generated kernels
 * for float2 logN 2..4 index out of bounds
 * (include/code_gen/generated/float2/fft_radix_2_logN_4_upload_0.cuh:67-77). */
int tfft_bounds_status(tfft_plan plan, long long* bad_index, int* site);

/* No counterpart in the reference.  One-shot transform for callers that cannot allocate
 * device memory when they call (no cudaMalloc allowed: pool-managed regions, allocation-free
 * service loops, devices whose memory is fully handed out).  Runs the built-in multi-launch
 * plan for (logN, dtype), FT off, with the intermediate buffer and the twiddle tables in
 * static device arrays of the library (16 MiB + 512 KiB per GPU that uses it).
 * Limits: the size must be a multi-launch one of the built-in table (tfft_plan_info tells;
 * at most logN 24) and batch * 2^logN * sizeof(element) <= 16 MiB, else
 * TFFT_ERR_UNSUPPORTED / TFFT_ERR_TOO_LARGE.  Calls no cudaMalloc/cudaFree.
 * Set-up: the first call on a device looks up the arrays' device addresses.  With CUDA's
 * lazy module loading (the default) that look-up, and the first launch of each kernel, is
 * also the moment the driver reserves the arrays and loads the code, so make one warm-up
 * call per device and size BEFORE entering the region that must not allocate and before
 * any stream capture (or run with CUDA_MODULE_LOADING=EAGER).
 * Tables: the twiddle tables of the last (logN, dtype) stay in the static table array.  A
 * call with the same (logN, dtype) reuses them and issues kernels only; a call with another
 * size rebuilds them on the host and uploads them on the caller's stream from pageable
 * memory, which a stream capture cannot record -- so only repeat sizes inside a capture.
 * Sharing: all calls share the arrays, which keep the previous call's contents (every
 * element that is read is written first, so nothing needs clearing); two calls whose
 * kernels overlap on the GPU race -- issue them on one stream or synchronise in between. */
int tfft_exec_static(int logN, long long batch, int dtype, const void* in, void* out, int device, void* stream);

/* Last CUDA error code seen by any call on this plan (0 = none). */
int tfft_last_cuda_error(tfft_plan plan);
const char* tfft_status_string(int status);

/* Number of kernels this library launched since it was loaded (all plans). */
long long tfft_launch_count(void);

/* STREAM-style device copy with 128-bit loads and stores, used as the measured
 * HBM peak every roofline fraction is quoted against. bytes must be a multiple
 * of 16.  Stream ordered. */
int tfft_stream_copy(const void* src, void* dst, size_t bytes, void* stream);

/* One transform too long for one GPU, over several devices driven by ONE process (no counterpart
 * in the reference, which is single-GPU; its device/default_fft.h:14 only notes the wish).
 * N = 2^logN = N1 * N2 with N1 = 2^ceil(logN/2); rank r (= position in `devices`) holds
 * elements [r * N / P, (r + 1) * N / P) of the signal in in[r] on devices[r].  Four-step:
 * transposing exchange, N2/P local transforms of length N1, twiddled transposing exchange,
 * N1/P local transforms of length N2.  The exchanges are kernels that store straight into the
 * other devices' receive buffers over NVLink (peer access is enabled between all pairs; a
 * device may appear more than once, which runs several ranks on one GPU); ranks are ordered
 * by CUDA events only, nothing on a device waits for a peer.  pipeline = G >= 1 cuts every
 * exchange into G pieces and overlaps piece g + 1 with the transforms of piece g (each rank's
 * N1/P and N2/P must be multiples of 32 * G, else TFFT_ERR_UNSUPPORTED).
 * Output: natural_order == 0: X[k1 + N1 * k2] at rank k1 / (N1 / P), out[rank][(k1 % (N1/P)) * N2 + k2]
 * ("transposed out"); natural_order != 0: out[r] = X[r * N / P ...], one more exchange.
 * if_ft: every local transform carries the fused two-sided checksums (detect only).
 * The plan owns three buffers of N / P elements per device plus the local plans. */
typedef struct tfft_mg_plan_s* tfft_mg_plan;
int tfft_mg_plan_create(tfft_mg_plan* plan, int logN, int dtype, int if_ft, int n_devices, const int* devices,
                        int natural_order, int pipeline);
/* in, out: n_devices device pointers (in[r] may equal out[r]).  streams: n_devices cudaStream_t
 * or NULL; if given, the work on devices[r] starts behind what streams[r] holds and streams[r]
 * continues behind it.  Returns without synchronising; tfft_mg_sync waits for every device. */
int tfft_mg_exec(tfft_mg_plan plan, const void* const* in, void* const* out, void* const* streams);
int tfft_mg_sync(tfft_mg_plan plan);
/* Blocks whose checksum test fired / tiles repaired, summed over all local transforms of all
 * ranks since the last call of this function (synchronises). */
int tfft_mg_ft_status(tfft_mg_plan plan, int* n_detected, int* n_corrected);
int tfft_mg_last_cuda_error(tfft_mg_plan plan);
int tfft_mg_destroy(tfft_mg_plan plan);

/* Building blocks of the multi-GPU four-step transform (no counterpart in the
 * reference, which is single-GPU).  They work on local complex arrays in device
 * memory.
 * tfft_transpose:         [rows][cols] -> dst[c][r] = src[r][c]
 * tfft_twiddle_transpose: dst[c][r] = src[r][c] * exp(-2*pi*i * (row0 + r) * (col0 + c) / 2^log_total)
 * tfft_permute102:        [A][B][run] -> dst[b][a][:] = src[a][b][:]  (pack / unpack of the
 *                         all-to-all exchanges; run * sizeof(element) must be a multiple of 16)
 */
int tfft_permute102(const void* src, void* dst, long long A, long long B, long long run_elems, int dtype,
                    void* stream);

/* Fused exchange of the four-step transform: transpose (+ optional twiddle) of the local
 * [rows][cols] matrix written straight into the receivers' buffers.  Element (i, c) goes to
 * rank j = c / (cols / n_peers) at peer_dst[j][(c % (cols / n_peers)) * ld_dst + row0 + i],
 * times exp(-2*pi*i*(row0 + i)*c / 2^log_total) if twiddle != 0.  peer_dst: host array of
 * n_peers (<= 16) device pointers, the caller's own buffer at its own rank and peer
 * mappings (tfft_peer_open) elsewhere.  rows, cols and cols / n_peers must be multiples of
 * 32.  The stores are ordinary global stores over NVLink; the kernel does not wait for
 * anybody -- order it against the receivers' next kernel with a stream-ordered barrier. */
int tfft_scatter_transpose(const void* src, void* const* peer_dst, int n_peers, long long rows, long long cols,
                           long long ld_dst, long long row0, int twiddle, int log_total, int dtype, void* stream);

/* The same for a slice of every receiver's block: only the columns j * (cols / n_peers) +
 * sub_off + [0, sub_len) of each receiver j (multiples of 32).  Lets a caller cut one
 * exchange into pieces and overlap piece g + 1 with the transform of piece g; max_blocks > 0
 * bounds the grid (the kernel strides over its tiles) so that the NVLink-bound copy holds only
 * a few slots per SM and the transforms get the rest. */
int tfft_scatter_transpose_part(const void* src, void* const* peer_dst, int n_peers, long long rows, long long cols,
                                long long ld_dst, long long row0, int twiddle, int log_total, long long sub_off,
                                long long sub_len, int max_blocks, int dtype, void* stream);

/* General form: receiver j's buffer has its own line pitch dst_ld[j] and this sender's rows
 * start at dst_row0[j] inside a line; the twiddle uses the global row index tw_row0 + i.  With
 * local staging buffers as "receivers" (pitch = rows, offset 0) the kernel becomes the pack
 * step of a copy-engine exchange: the packed block of receiver j is then moved by
 * tfft_copy_2d.  complex64 twiddles support log_total <= 39.  No counterpart in the
 * reference (single GPU). */
int tfft_scatter_transpose_ex(const void* src, void* const* dst, const long long* dst_ld, const long long* dst_row0,
                              int n_peers, long long rows, long long cols, long long tw_row0, int twiddle, int log_total,
                              long long sub_off, long long sub_len, int max_blocks, int dtype, void* stream);

/* Stream-ordered 2-D copy between any two device buffers this process can address (its own
 * or peer mappings): height rows of width bytes, pitches in bytes.  Runs on the copy engines,
 * so it takes no SM from the transforms it overlaps with. */
int tfft_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width, size_t height,
                 void* stream);

/* Receive buffers other processes can map: cudaMalloc + CUDA IPC handle (64 bytes). */
int tfft_peer_alloc(size_t bytes, void** ptr);
int tfft_peer_free(void* ptr);
int tfft_peer_export(const void* ptr, void* handle64);
int tfft_peer_open(const void* handle64, void** ptr);
int tfft_peer_close(void* ptr);
int tfft_transpose(const void* src, void* dst, long long rows, long long cols, int dtype, void* stream);
int tfft_twiddle_transpose(const void* src, void* dst, long long rows, long long cols, long long row0,
                           long long col0, int log_total, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TURBOFFT_B200_H */
