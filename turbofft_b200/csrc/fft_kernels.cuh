// Batched power-of-two complex FFT kernels for sm_100a (B200).
//
// One kernel template covers every launch of a 1-, 2- or 3-launch split of a
// 2^logN transform.  It plays the part of the reference's generated
// fft_radix_2<T, logN, launch, if_ft, if_err> family
// (include/TurboFFT_radix_2_template.h:1-3, emitted by
// include/code_gen/scripts/fft_codegen.py:198-504) but shares no structure with
// it: butterflies are radix-2^LOGE (up to 32) on registers, the in-block data
// exchange is a Stockham autosort through shared memory, twiddles come from
// correctly rounded tables, and all index arithmetic is 64-bit.
//
// A launch transforms "lines" of length M = 2^LOGM.  A tile is C = 2^LOGC lines
// that are adjacent in memory in the way the role needs:
//   ROLE_SINGLE  whole signals, contiguous in and out (1-launch plans)
//   ROLE_FIRST   lines strided by B = 2^log_b, the C lines of a tile are C
//                adjacent columns; result goes back to the same positions and is
//                multiplied by the inter-launch twiddle W_{M*B}^{col*k}
//                (first and middle launches; fft_codegen.py:385-400)
//   ROLE_LAST    contiguous lines in, digit-reversed (transposed) store so that
//                the final order is natural (fft_codegen.py:143-148); the C
//                lines of a tile are C consecutive values of the slowest digit,
//                which makes the strided store run over C adjacent addresses.
//
// Fault tolerance (FT_DETECT / FT_CORRECT) folds the two-sided checksum of the
// reference into the same pass (fft_codegen.py:359-384, 432-503, 149-193):
// left side  sum_p fold(x_p * c_p) with c = W_M r taken while loading,
// right side sum_k fold(y_k * r_{k mod 3}) taken before the store,
// and a copy weighted by the 1-based tile counter that locates the tile.
// FT_CORRECT repairs the located tile by recomputing it from its input (what the reference
// ships, fft_codegen.py:149-193); FT_CSUM repairs it from the per-position sums of the
// block's inputs and outputs, y_bad -= sum(y) - F(sum(x)) -- the correction the reference
// accumulates rPtr_3 / rPtr_4 for but leaves commented out (fft_codegen.py:356-357,
// 422-429; test.ipynb cell 0) -- which does not need the input again.
#pragma once
#include <cuda_runtime.h>

#ifndef TFFT_F32X2
#define TFFT_F32X2 1  // complex64 butterflies add and subtract with the packed f32x2 instructions of sm_100
#endif
#ifndef TFFT_FT_PREFETCH
#define TFFT_FT_PREFETCH 0  // 1: the FT kernels (eight tiles per block) prefetch as well; measured 3 % slower over the sweep
#endif
#ifndef TFFT_L2_PREFETCH
#define TFFT_L2_PREFETCH 1  // blocks that loop over tiles ask L2 for the next tile while they transform this one
#endif
#ifndef TFFT_BOUNDS_CHECK
#define TFFT_BOUNDS_CHECK 0  // 1: every global load/store index of the data buffers is checked (see KernelArgs::oob)
#endif
#ifndef TFFT_FT_LEAN
#define TFFT_FT_LEAN 1  // 1: the FT kernels keep less state in registers (see FtRegs) and fit the plain kernels' 64
#endif
#ifndef TFFT_FT_OCC
#define TFFT_FT_OCC 4  // quarters of the plain kernels' resident-thread target that the FT variants aim for
#endif

namespace tfft {

enum { ROLE_SINGLE = 0, ROLE_FIRST = 1, ROLE_LAST = 2 };
enum { FT_OFF = 0, FT_DETECT = 1, FT_CORRECT = 2, FT_CSUM = 3 };

template <typename T> struct Cplx;
template <> struct Cplx<float> { typedef float2 type; };
template <> struct Cplx<double> { typedef double2 type; };

template <typename T>
struct KernelArgs {
    typedef typename Cplx<T>::type C;
    const C* in;
    C* out;
    const C* tw_st;  // in-block stage twiddles, laid out so that a warp reads them coalesced:
                     // stage t, j < log2 R_t, butterfly b -> w^(2^j) with w = W_M^{(b >> logP_t) << logP_t}
                     // at stage_offset(t) + j * (M / R_t) + b; the other powers are products of these
    const C* tw_lo;  // W_P^j, j < 2^tw_lo_bits (inter-launch twiddle, low part)
    const C* tw_hi;  // W_P^(j << tw_lo_bits)   (high part), P = M * B
    const C* cks;    // FT only, M entries: fold weights of c = W_M r as (c.x + c.y, c.x - c.y)
    long long n_tiles;
    long long n_lines;  // ROLE_SINGLE: number of signals (ragged last tile)
    int tiles_per_cta;  // the reference's thread_bs
    int log_n;          // log2 of the whole transform
    int log_b;          // ROLE_FIRST: log2 of the line stride
    int log_n1;         // ROLE_LAST: log2 of the slowest digit's extent
    int log_q;          // ROLE_LAST: log2 of the middle digit's extent (0 for 2 launches)
    int tw_lo_bits;
    int inj_on;         // add err_inj to one element of one tile per selected block
    int inj_period;     // blocks b with b % inj_period == inj_phase are hit
    int inj_phase;
    int no_twiddle;     // ROLE_FIRST used on its own (strided batch): no inter-launch twiddle
    int conj_in;        // conjugate while loading (first launch of an inverse transform)
    int scale_out;      // scale while storing (last launch): y = (y.x * scale_x, y.y * scale_y);
    T scale_x;          // inverse transform: (s, -s) conjugates and scales; forward with a norm: (s, s)
    T scale_y;
    T err_inj;
    T err_smoothing;
    T err_threshold;
    // Checked build (TFFT_BOUNDS_CHECK): extent of `in` / `out` in elements and a status word that
    // receives the first out-of-range access (bit 63 set, bits 56..62 the access site, bits 0..55
    // the element index); the offending access is skipped.  Unused in the normal build.
    long long n_elems;
    unsigned long long* oob;
    // Fused two-launch kernel (pair_fft.cuh): bits of the signal index that are cleared when the
    // intermediate is addressed, so that it lives in a ring of a few signals; 0 = whole buffer
    long long ring_clear;
    int* ft_located;          // per block: located tile iteration (1-based) or -1
    unsigned int* ft_count;   // [0] blocks that detected, [1] tiles recomputed
    T* ft_diag;               // per block: delta, S, delta_w (may be null)
};

// ---------------------------------------------------------------- complex helpers
template <typename C> __device__ __forceinline__ C cadd(C a, C b) { C r; r.x = a.x + b.x; r.y = a.y + b.y; return r; }
template <typename C> __device__ __forceinline__ C csub(C a, C b) { C r; r.x = a.x - b.x; r.y = a.y - b.y; return r; }
#if TFFT_F32X2
// sm_100 packed single precision: one instruction adds (subtracts) both components of a
// complex value held in an aligned register pair.  a - b is formed as fma(b, -1, a), which
// rounds exactly like the subtraction, so results are bit-identical to the scalar form.
template <> __device__ __forceinline__ float2 cadd<float2>(float2 a, float2 b) { return __fadd2_rn(a, b); }
template <> __device__ __forceinline__ float2 csub<float2>(float2 a, float2 b) {
    return __ffma2_rn(b, make_float2(-1.0f, -1.0f), a);
}
#endif
template <typename C> __device__ __forceinline__ C cmul(C a, C b) {
    C r;
    r.x = a.x * b.x - a.y * b.y;
    r.y = a.x * b.y + a.y * b.x;
    return r;
}

// Per-thread checksum accumulator: acc += v.x * w.x + v.y * w.y.  complex64 keeps the two
// products in the halves of one packed register pair (one f32x2 fma per element instead of two
// scalar ones) and adds the halves when the tile is done; complex128 accumulates in a scalar.
template <typename T> struct FtAcc { typedef T type; };
template <typename T> __device__ __forceinline__ void acc_fma(T& acc, typename Cplx<T>::type v, typename Cplx<T>::type w) {
    acc = fma(v.x, w.x, acc);
    acc = fma(v.y, w.y, acc);
}
template <typename T> __device__ __forceinline__ T acc_sum(T acc) { return acc; }
template <typename A> __device__ __forceinline__ A acc_zero() { return A(0); }
#if TFFT_F32X2
template <> struct FtAcc<float> { typedef float2 type; };
__device__ __forceinline__ void acc_fma(float2& acc, float2 v, float2 w) { acc = __ffma2_rn(v, w, acc); }
__device__ __forceinline__ float acc_sum(float2 acc) { return acc.x + acc.y; }
template <> __device__ __forceinline__ float2 acc_zero<float2>() { return make_float2(0.0f, 0.0f); }
#endif

// cos(2*pi*k/32), k = 0..8
template <typename T> __device__ __forceinline__ constexpr T cos32_tab(int k) {
    return k == 0 ? T(1.0)
         : k == 1 ? T(0.98078528040323044912618223613424)
         : k == 2 ? T(0.92387953251128675612818318939679)
         : k == 3 ? T(0.83146961230254523707878837761791)
         : k == 4 ? T(0.70710678118654752440084436210485)
         : k == 5 ? T(0.55557023301960222474283081394853)
         : k == 6 ? T(0.38268343236508977172845998403040)
         : k == 7 ? T(0.19509032201612826784828486847702)
                  : T(0.0);
}
// cos and sin of 2*pi*k/32 for 0 <= k <= 16
template <typename T> __device__ __forceinline__ constexpr T cos32(int k) { return k <= 8 ? cos32_tab<T>(k) : -cos32_tab<T>(16 - k); }
template <typename T> __device__ __forceinline__ constexpr T sin32(int k) { return k <= 8 ? cos32_tab<T>(8 - k) : cos32_tab<T>(k - 8); }

template <int LR> __device__ __forceinline__ constexpr int brev(int q) {
    int r = 0;
    for (int i = 0; i < LR; ++i) r |= ((q >> i) & 1) << (LR - 1 - i);
    return r;
}

__device__ __forceinline__ constexpr int ilog2(int x) {
    int l = 0;
    while (x > 1) {
        x >>= 1;
        ++l;
    }
    return l;
}

// In-register radix-R decimation-in-frequency FFT over v[u + j*STR], j < R.
// X[q] is left at v[u + brev(q)*STR].  Every index is a compile-time constant
// once the loops are unrolled, so v stays in registers.
template <int LR, int LH, int STR, typename T, typename C, int E>
__device__ __forceinline__ void dif_level(C (&v)[E], const int u) {
    constexpr int R = 1 << LR;
    constexpr int half = 1 << LH;
#pragma unroll
    for (int t = 0; t < R / 2; ++t) {
        const int j = t & (half - 1);
        const int blk = (t >> LH) << (LH + 1);
        const int ia = u + (blk + j) * STR;
        const int ib = ia + half * STR;
        const C a = v[ia];
        const C b = v[ib];
        v[ia] = cadd(a, b);
        const C d = csub(a, b);
        // multiply by W_{2*half}^j = exp(-2*pi*i*j/(2*half)); angle index in 32nds of a turn
        const int k32 = j * (16 >> LH);
        C w;
        if (k32 == 0) {
            w = d;
        } else if (k32 == 8) {  // -i
            w.x = d.y;
            w.y = -d.x;
        } else if (k32 == 4) {  // (1 - i)/sqrt2
            const T h = cos32_tab<T>(4);
            w.x = (d.x + d.y) * h;
            w.y = (d.y - d.x) * h;
        } else if (k32 == 12) {  // (-1 - i)/sqrt2
            const T h = cos32_tab<T>(4);
            w.x = (d.y - d.x) * h;
            w.y = -(d.x + d.y) * h;
        } else {
            const T wr = cos32<T>(k32);
            const T wi = -sin32<T>(k32);
            w.x = d.x * wr - d.y * wi;
            w.y = d.x * wi + d.y * wr;
        }
        v[ib] = w;
    }
    if constexpr (LH > 0) dif_level<LR, LH - 1, STR, T>(v, u);
}

template <int LR, int STR, typename T, typename C, int E>
__device__ __forceinline__ void dif_butterfly(C (&v)[E], const int u) {
    if constexpr (LR > 0) dif_level<LR, LR - 1, STR, T>(v, u);
}

// ---------------------------------------------------------------- shared-memory layout
// pad(a) = a + (a >> PADSHIFT); rows layout (ROLE_SINGLE, ROLE_LAST): line pitch =
// pad(M - 1) + 1 + EXTRA; cols layout (ROLE_FIRST): position pad(a) * C + c.  REMLAST moves the
// remainder radix (line length not a power of the per-thread radix) from the first register
// stage to the last one; the generator picks it wherever that order is at least as free of
// bank conflicts (for a few instances it is the only conflict-free one).  The primary
// template is a reasonable default; generated/smem_layouts.h specialises it per instance
// with the conflict-free choice found by codegen/smem_layout.py.
template <typename T, int LOGM, int LOGE, int LOGC, int ROLE>
struct SmemLayout {
    static constexpr int M = 1 << LOGM;
    static constexpr int TPL = 1 << (LOGM - LOGE);
    static constexpr int BANKW = 128 / (2 * (int)sizeof(T));
    static constexpr int PADSHIFT = ROLE == ROLE_FIRST ? 31 : (sizeof(T) == 4 ? 4 : 3);
    static constexpr int MPAD = (M - 1) + ((M - 1) >> PADSHIFT) + 1;
    static constexpr int EXTRA = ROLE == ROLE_FIRST ? 0
                                 : ROLE == ROLE_LAST ? ((MPAD | 1) - MPAD)
                                 : (TPL >= BANKW ? 0 : ((MPAD + BANKW - 1) / BANKW) * BANKW + TPL - MPAD);
    static constexpr int REMLAST = 0;
};
#include "generated/smem_layouts.h"

// ---------------------------------------------------------------- configuration
template <typename T, int LOGM, int LOGE, int LOGC, int ROLE>
struct Cfg {
    static_assert(LOGE >= 1 && LOGE <= 5, "elements per thread: 2..32");
    static_assert(LOGE <= LOGM, "a thread cannot hold more than a line");
    static constexpr int M = 1 << LOGM;
    static constexpr int E = 1 << LOGE;
    static constexpr int C = 1 << LOGC;
    static constexpr int LOGTPL = LOGM - LOGE;  // threads per line
    static constexpr int TPL = 1 << LOGTPL;
    static constexpr int THREADS = TPL * C;
    static constexpr int S = (LOGM + LOGE - 1) / LOGE;  // register stages
    static constexpr int LOGR0 = LOGM - (S - 1) * LOGE; // the remainder radix: first stage, or last with REMLAST
    static_assert(ROLE != ROLE_LAST || S >= 2, "transposed store needs one exchange");
    static constexpr bool CFAST_IN = (ROLE == ROLE_FIRST);
    static constexpr bool CFAST_OUT = (ROLE != ROLE_SINGLE);
    static constexpr bool LAYOUT_COLS = (ROLE == ROLE_FIRST);
    typedef SmemLayout<T, LOGM, LOGE, LOGC, ROLE> L;
    static constexpr bool REMLAST = L::REMLAST != 0 && S > 1;
    // log2 radix of register stage t and log2 of the product of the radices before it
    static __host__ __device__ constexpr int stage_logr(int t) { return REMLAST ? (t == S - 1 ? LOGR0 : LOGE) : (t == 0 ? LOGR0 : LOGE); }
    static __host__ __device__ constexpr int stage_logp(int t) { return REMLAST ? t * LOGE : (t == 0 ? 0 : LOGR0 + (t - 1) * LOGE); }
    static constexpr int PADSHIFT = L::PADSHIFT;
    static constexpr int MPAD = (M - 1) + ((M - 1) >> PADSHIFT) + 1;
    static constexpr int PITCH = MPAD + L::EXTRA;
    // One thread per line (M == E, whole signals): lines are too short to be read coalesced
    // by their owner, so the tile -- contiguous in memory -- is staged through shared memory:
    // cooperative coalesced copy in, each thread picks up its line (pitch M + 1), and back.
    static constexpr bool STAGED_IO = (ROLE == ROLE_SINGLE && S == 1 && TPL == 1 && LOGM >= 2);
    static constexpr int SMEM_ELEMS = STAGED_IO ? (M + 1) * C : (S > 1 ? (LAYOUT_COLS ? MPAD * C : PITCH * C) : 0);
    static constexpr size_t SMEM_BYTES = (size_t)SMEM_ELEMS * 2 * sizeof(T);
    // FT_CSUM keeps two more tiles in shared memory: the running sums of inputs and outputs
    static constexpr size_t smem_bytes(int ft) { return SMEM_BYTES + (ft == FT_CSUM ? (size_t)2 * M * C * 2 * sizeof(T) : 0); }
    // Occupancy target handed to the compiler as the register cap: enough blocks for
    // 1024 (fp32) / 512 (fp64) resident threads per SM unless shared memory allows fewer.
    // The FT variants carry the checksum state on top and get a quarter more registers;
    // 32 points per thread need twice the registers, so half the threads.
    static constexpr int SMEM_BLOCKS = SMEM_BYTES ? (int)((220 * 1024) / SMEM_BYTES) : 32;
    // ft: the FT mode (0 = off).  The complex64 detect / recompute kernels fit the plain kernels' register
    // budget (TFFT_FT_OCC = 4 quarters); the running-checksum variant and complex128 spill there and keep 3.
    static constexpr int min_blocks(int ft) {
        const int quarters = ft == 0 ? 4 : ((sizeof(T) == 4 && ft != 3) ? TFFT_FT_OCC : 3);
        const int target = (sizeof(T) == 4 ? 1024 : 512) * quarters / 4 / (LOGE == 5 ? 2 : 1);
        const int tb = (target + THREADS - 1) / THREADS;
        const int b = SMEM_BLOCKS < tb ? SMEM_BLOCKS : tb;
        return b < 1 ? 1 : b;
    }
};

template <typename T, int LOGM, int LOGE, int LOGC, int ROLE, int FT>
struct Fft {
    typedef Cfg<T, LOGM, LOGE, LOGC, ROLE> K;
    typedef typename Cplx<T>::type C;
    static constexpr int E = K::E;
    static constexpr int TPL = K::TPL;

    struct Geom {
        long long in_base, out_base, in_rs, in_cs, out_rs, out_cs, col0;
        int ncols;
    };

    // per-thread FT state that lives across the tiles of a block.  The left-checksum
    // weights are NOT kept here: 2E registers per thread cost more (spills or occupancy)
    // than re-reading them per tile from the L1-resident table.
    struct FtRegs {
#if TFFT_FT_LEAN
        int s3;   // s mod 3: which of the three fold weights the thread's first output takes
#else
        C ab[3];  // fold weights (alpha, beta) of the right checksum, rotated by s mod 3
#endif
    };
    typedef typename FtAcc<T>::type A;  // checksum accumulator of one tile

    // Checked build only: is element index idx inside the data buffers?  Records the first offender.
    static __device__ __forceinline__ bool in_range(const KernelArgs<T>& a, long long idx, int site) {
#if TFFT_BOUNDS_CHECK
        if (idx < 0 || idx >= a.n_elems) {
            if (a.oob)
                atomicCAS(a.oob, 0ULL,
                          (1ULL << 63) | ((unsigned long long)site << 56) | ((unsigned long long)idx & ((1ULL << 56) - 1)));
            return false;
        }
#endif
        return true;
    }

    template <int ST> static __device__ __forceinline__ constexpr int logR() { return K::stage_logr(ST); }
    template <int ST> static __device__ __forceinline__ constexpr int logP() { return K::stage_logp(ST); }
    // first entry of stage ST in the stage-twiddle table: sum over earlier stages of log2(R) * M / R
    template <int ST> static __device__ __forceinline__ constexpr int twOff() {
        int off = 0;
        for (int t = 0; t < ST; ++t) {
            const int lr = K::stage_logr(t);
            off += lr << (LOGM - lr);
        }
        return off;
    }

    template <bool CF> static __device__ __forceinline__ void map_thread(int& s, int& c) {
        const int tid = threadIdx.x;
        if (CF) {
            c = tid & (K::C - 1);
            s = tid >> LOGC;
        } else {
            s = tid & (TPL - 1);
            c = tid >> K::LOGTPL;
        }
    }

    // Shared-memory position of Stockham address a of line c.  Row layout pads one
    // element per 2^PADSHIFT.  soff(x + y, c) == soff(x, c) + sdelta(y) whenever x and y
    // occupy disjoint bit fields, which lets every unrolled access use a constant offset
    // from one per-thread base.
    static __device__ __forceinline__ int soff(int a, int c) {
        if (K::LAYOUT_COLS) return (a + (a >> K::PADSHIFT)) * K::C + c;
        return c * K::PITCH + a + (a >> K::PADSHIFT);
    }
    static __device__ __forceinline__ constexpr int sdelta(int y) {
        return K::LAYOUT_COLS ? (y + (y >> K::PADSHIFT)) * K::C : y + (y >> K::PADSHIFT);
    }

    static __device__ __forceinline__ Geom decode(const KernelArgs<T>& a, long long tile) {
        Geom g;
        if (ROLE == ROLE_SINGLE) {
            const long long line0 = tile << LOGC;
            g.in_base = g.out_base = line0 << LOGM;
            g.in_rs = g.out_rs = 1;
            g.in_cs = g.out_cs = K::M;
            const long long left = a.n_lines - line0;
            g.ncols = left < K::C ? (int)left : K::C;
            g.col0 = 0;
        } else if (ROLE == ROLE_FIRST) {
            const int ltpo = a.log_b - LOGC;  // log2 tiles per outer index
            const long long o = tile >> ltpo;
            const long long b0 = (tile & ((1LL << ltpo) - 1)) << LOGC;
            g.in_base = (o << (LOGM + a.log_b)) + b0;
            g.out_base = ((o & ~a.ring_clear) << (LOGM + a.log_b)) + b0;
            g.in_rs = g.out_rs = 1LL << a.log_b;
            g.in_cs = g.out_cs = 1;
            g.ncols = K::C;
            g.col0 = b0;
        } else {
            const int lk = a.log_n1 - LOGC;
            const long long batch = tile >> (lk + a.log_q);
            const long long t = tile & ((1LL << (lk + a.log_q)) - 1);
            const long long k10 = (t & ((1LL << lk) - 1)) << LOGC;
            const long long k2 = t >> lk;
            g.in_base = ((batch & ~a.ring_clear) << a.log_n) + (((k10 << a.log_q) + k2) << LOGM);
            g.in_rs = 1;
            g.in_cs = 1LL << (a.log_q + LOGM);
            g.out_base = (batch << a.log_n) + k10 + (k2 << a.log_n1);
            g.out_rs = 1LL << (a.log_n1 + a.log_q);
            g.out_cs = 1;
            g.ncols = K::C;
            g.col0 = 0;
        }
        return g;
    }

    // Final stage: natural-order outputs, right checksum, inter-launch twiddle, store.
    // CS: 0 plain, 1 add the outputs to the block's running sum, 2 correction pass (v holds
    // F(sum of inputs); the located tile's stored outputs get sum(y) - F(sum(x)) subtracted)
    template <int LR, bool DO_FT, int CS>
    static __device__ __forceinline__ void finish(C (&v)[E], C* sm, const KernelArgs<T>& a, const Geom& g, int s, int c,
                                                  const FtRegs& f, A& tout) {
        constexpr int R = 1 << LR, NB = E / R;
        C y[E];
#pragma unroll
        for (int u = 0; u < NB; ++u)
#pragma unroll
            for (int q = 0; q < R; ++q) y[u + q * NB] = v[u + brev<LR>(q) * NB];
        if (DO_FT) {
            constexpr int t3 = (K::LOGTPL & 1) ? 2 : 1;  // TPL mod 3
#if TFFT_FT_LEAN
            // the outputs of each residue class are summed first (adds only), then the three sums are
            // folded with the weights (1, 1), (a1, a2), (a2, a1), a1/a2 = -1/2 -/+ h, picked by s mod 3
            C cls[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) cls[k].x = cls[k].y = T(0);
#pragma unroll
            for (int i = 0; i < E; ++i) cls[(i * t3) % 3] = cadd(cls[(i * t3) % 3], y[i]);
            const T h = T(0.8660253882408142);
            C w0, w1, w2;
            w0.x = w0.y = T(1);
            w1.x = T(-0.5) - h, w1.y = T(-0.5) + h;
            w2.x = T(-0.5) + h, w2.y = T(-0.5) - h;
            const int s3 = f.s3;  // class k carries weight (s3 + k) mod 3
            const C c0 = s3 == 0 ? cls[0] : (s3 == 1 ? cls[2] : cls[1]);
            const C c1 = s3 == 0 ? cls[1] : (s3 == 1 ? cls[0] : cls[2]);
            const C c2 = s3 == 0 ? cls[2] : (s3 == 1 ? cls[1] : cls[0]);
            acc_fma(tout, c0, w0);
            acc_fma(tout, c1, w1);
            acc_fma(tout, c2, w2);
#else
#pragma unroll
            for (int i = 0; i < E; ++i) acc_fma(tout, y[i], f.ab[(i * t3) % 3]);
#endif
        }
        if constexpr (CS != 0) {
            C* sy = sm + K::SMEM_ELEMS + E * K::THREADS + threadIdx.x;
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const C acc = sy[i * K::THREADS];
                if (CS == 1) sy[i * K::THREADS] = cadd(acc, y[i]);
                else y[i] = csub(acc, y[i]);  // the error this block's outputs carry at this position
            }
        }
        if (ROLE == ROLE_FIRST && !a.no_twiddle) {
            // y_k *= W_P^{col*k}, k = s + i*TPL, i.e. base * step^i
            const unsigned long long col = (unsigned long long)(g.col0 + c);
            const unsigned long long pmask = (1ULL << (LOGM + a.log_b)) - 1;
            const unsigned long long lomask = (1ULL << a.tw_lo_bits) - 1;
            const unsigned long long jb = (col * (unsigned long long)s) & pmask;
            const unsigned long long js = (col * (unsigned long long)TPL) & pmask;
            // w_i = base * step^i is formed as A[i >> LL] * B[i & (2^LL - 1)] with
            // A[a] = base * step^(a << LL), B[b] = step^b: about sqrt(E) live values instead of E,
            // every w_i at most ~log2(E)+1 products deep.
            constexpr int LL = LOGE / 2, LH = LOGE - LL, NLO = 1 << LL, NHI = 1 << LH;
            C A[NHI], B[NLO];
            A[0] = cmul(__ldg(a.tw_lo + (jb & lomask)), __ldg(a.tw_hi + (jb >> a.tw_lo_bits)));
            B[0].x = T(1);
            B[0].y = T(0);
            const C step = cmul(__ldg(a.tw_lo + (js & lomask)), __ldg(a.tw_hi + (js >> a.tw_lo_bits)));
            C big = step;  // becomes step^(2^LL)
            if constexpr (NLO > 1) {
                B[1] = step;
#pragma unroll
                for (int b = 2; b < NLO; ++b) B[b] = (b & 1) ? cmul(B[b - 1], B[1]) : cmul(B[b / 2], B[b / 2]);
                big = cmul(B[NLO / 2], B[NLO / 2]);
            }
#pragma unroll
            for (int h = 1; h < NHI; ++h) A[h] = cmul(A[h - 1], big);
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const C w = (i & (NLO - 1)) ? cmul(A[i >> LL], B[i & (NLO - 1)]) : A[i >> LL];
                y[i] = cmul(y[i], w);
            }
        }
        if (a.scale_out) {
#pragma unroll
            for (int i = 0; i < E; ++i) {
                y[i].x *= a.scale_x;
                y[i].y *= a.scale_y;
            }
        }
        if constexpr (K::STAGED_IO) {
            // every thread only touches its own line here, so no barrier is needed before
#pragma unroll
            for (int i = 0; i < E; ++i) sm[c * (K::M + 1) + i] = y[i];
            __syncthreads();
            const long long valid = (long long)g.ncols << LOGM;
            C* dst = a.out + g.out_base;
#pragma unroll
            for (int k = 0; k < K::M; ++k) {
                const int fl = k * K::C + (int)threadIdx.x;
                if (fl < valid && in_range(a, g.out_base + fl, 3)) dst[fl] = sm[(fl >> LOGM) * (K::M + 1) + (fl & (K::M - 1))];
            }
        } else if (c < g.ncols) {
            const long long o0 = g.out_base + (long long)c * g.out_cs + (long long)s * g.out_rs;
            C* dst = a.out + o0;
#pragma unroll
            for (int i = 0; i < E; ++i) {
                if (!in_range(a, o0 + (long long)i * TPL * g.out_rs, 4)) continue;
                if (CS == 2) dst[(long long)i * TPL * g.out_rs] = csub(dst[(long long)i * TPL * g.out_rs], y[i]);
                else dst[(long long)i * TPL * g.out_rs] = y[i];
            }
        }
    }

    template <int ST, bool DO_FT, int CS>
    static __device__ __forceinline__ void stage(C (&v)[E], C* sm, const KernelArgs<T>& a, const Geom& g,
                                                 const FtRegs& f, A& tout) {
        constexpr int LR = logR<ST>(), R = 1 << LR, LP = logP<ST>(), P = 1 << LP, NB = E / R;
        constexpr bool LASTST = (ST == K::S - 1);
        constexpr bool CF = LASTST ? K::CFAST_OUT : K::CFAST_IN;
        int s, c;
        map_thread<CF>(s, c);
        if (ST > 0) {
            {
                const C* rd = sm + soff(s, c);  // s < TPL and i * TPL share no bits
#pragma unroll
                for (int i = 0; i < E; ++i) v[i] = rd[sdelta(i * TPL)];
            }
            __syncthreads();  // everybody has read before anybody overwrites
        }
#pragma unroll
        for (int u = 0; u < NB; ++u) dif_butterfly<LR, NB, T>(v, u);
        if constexpr (!LASTST) {
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                const int b = s + u * TPL;
                const int p = b & (P - 1);
                const int nlo = b >> LP;
                // p, q << LP and nlo << (LP + LR) are disjoint bit fields of the address
                C* wr = sm + soff(p + (nlo << (LP + LR)), c);
                // w^q for q < R: the log2(R) powers w^(2^j) come from the table, every other
                // power is one product of two already known ones (at most log2(R) table
                // entries deep, so the rounding of a table entry is never amplified)
                const C* tw = a.tw_st + twOff<ST>() + b;
                C w[R];
#pragma unroll
                for (int j = 0; j < LR; ++j) w[1 << j] = __ldg(tw + j * (K::M / R));
#pragma unroll
                for (int q = 3; q < R; ++q)
                    if (q & (q - 1)) w[q] = cmul(w[q - (1 << ilog2(q))], w[1 << ilog2(q)]);
#pragma unroll
                for (int q = 0; q < R; ++q) {
                    C val = v[u + brev<LR>(q) * NB];
                    if (q > 0) val = cmul(val, w[q]);
                    wr[sdelta(q << LP)] = val;
                }
            }
            __syncthreads();
            stage<ST + 1, DO_FT, CS>(v, sm, a, g, f, tout);
        } else {
            finish<LR, DO_FT, CS>(v, sm, a, g, s, c, f, tout);
        }
    }

    // Asks L2 for the input of a tile this block will load next (prefetch.global.L2, no register,
    // no shared memory): the HBM read of tile t + 1 then overlaps the transform of tile t, which a
    // block that fills its SM alone cannot get from a neighbour.  One request per 128-byte line.
    static __device__ __forceinline__ void prefetch_tile(const KernelArgs<T>& a, long long tile_id) {
#if TFFT_L2_PREFETCH
        // only where a block fills its SM alone (whole signals of 128 KB and more): with several
        // blocks per SM the neighbours already overlap their phases and the extra requests measured
        // slower (2^12, 2^13 and every strided-line launch)
        if constexpr ((ROLE == ROLE_SINGLE && !K::STAGED_IO && K::SMEM_BYTES >= 120 * 1024) ||
                      (TFFT_FT_PREFETCH && FT != FT_OFF && !K::STAGED_IO)) {
            const Geom g = decode(a, tile_id);
            int s, c;
            map_thread<K::CFAST_IN>(s, c);
            constexpr int PER_LINE = 128 / (2 * (int)sizeof(T));  // elements per 128-byte line
            // the index that runs over adjacent addresses: the column for strided lines, the row otherwise
            const int fast = K::CFAST_IN ? c : s;
            if ((fast & (PER_LINE - 1)) == 0 && c < g.ncols) {
                const C* src = a.in + g.in_base + (long long)c * g.in_cs + (long long)s * g.in_rs;
#pragma unroll
                for (int i = 0; i < E; ++i)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(src + (long long)i * TPL * g.in_rs));
            }
        }
#endif
    }

    // One tile: load, all stages, store.  tin/tout receive this thread's share of the
    // tile's left and right checksums.
    // L2ONLY: the input is read past L1 (it was written by other blocks of the SAME launch)
    // after_loads: called once the tile's global loads have been issued (pair_fft.cuh hangs a deferred signal there)
    struct NoHook {
        __device__ __forceinline__ void operator()() const {}
    };
    template <bool DO_FT, bool DO_INJ, int CS = 0, bool L2ONLY = false, typename Hook = NoHook>
    static __device__ __forceinline__ void tile(const KernelArgs<T>& a, C* sm, long long tile_id, bool inject,
                                                const FtRegs& f, A& tin, A& tout, Hook after_loads = Hook()) {
        static_assert(CS == 0 || (!K::STAGED_IO && ROLE != ROLE_FIRST), "checksum correction: single and last launches only");
        const Geom g = decode(a, tile_id);
        int s, c;
        map_thread<K::CFAST_IN>(s, c);
        C v[E];
        if constexpr (CS == 2) {
            // the "signal" of the correction pass is the sum of the block's inputs
            const C* sx = sm + K::SMEM_ELEMS + threadIdx.x;
#pragma unroll
            for (int i = 0; i < E; ++i) v[i] = sx[i * K::THREADS];
        } else if constexpr (K::STAGED_IO) {
            // flat element f of the tile = line f / M, row f % M; consecutive threads, consecutive f
            const long long valid = (long long)g.ncols << LOGM;
            const C* src = a.in + g.in_base;
            __syncthreads();  // previous tile's copy-out has finished reading shared memory
#pragma unroll
            for (int k = 0; k < K::M; ++k) {
                const int fl = k * K::C + (int)threadIdx.x;
                C t;
                t.x = t.y = T(0);
                if (fl < valid && in_range(a, g.in_base + fl, 1)) t = src[fl];
                sm[(fl >> LOGM) * (K::M + 1) + (fl & (K::M - 1))] = t;
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < E; ++i) v[i] = sm[c * (K::M + 1) + i];
        } else if (c < g.ncols) {
            const long long i0 = g.in_base + (long long)c * g.in_cs + (long long)s * g.in_rs;
            const C* src = a.in + i0;
#pragma unroll
            for (int i = 0; i < E; ++i) {
                if (in_range(a, i0 + (long long)i * TPL * g.in_rs, 2))
                    v[i] = L2ONLY ? __ldcg(src + (long long)i * TPL * g.in_rs) : src[(long long)i * TPL * g.in_rs];
                else v[i].x = v[i].y = T(0);
            }
        } else {
#pragma unroll
            for (int i = 0; i < E; ++i) v[i].x = v[i].y = T(0);
        }
        after_loads();
        if (CS != 2 && a.conj_in) {  // inverse transform: F^-1(x) = conj(F(conj(x))) / N
#pragma unroll
            for (int i = 0; i < E; ++i) v[i].y = -v[i].y;
        }
        if constexpr (CS == 1) {  // before the fault is injected, as the reference sums rPtr_3
            C* sx = sm + K::SMEM_ELEMS + threadIdx.x;
#pragma unroll
            for (int i = 0; i < E; ++i) sx[i * K::THREADS] = cadd(sx[i * K::THREADS], v[i]);
        }
        if (DO_FT) {
            // fold(x * c) = x.x * (c.x + c.y) + x.y * (c.x - c.y); rows s + i*TPL, coalesced over s
            const C* wt = a.cks + s;
#pragma unroll
            for (int i = 0; i < E; ++i) acc_fma(tin, v[i], __ldg(wt + i * TPL));
        }
        if (DO_INJ) {
            if (inject && threadIdx.x == 0) v[0].x += a.err_inj;
        }
        stage<0, DO_FT, CS>(v, sm, a, g, f, tout);
    }

    static __device__ __forceinline__ T warp_sum(T x) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
        return x;
    }

    static __device__ __forceinline__ void run(const KernelArgs<T>& a, C* sm) {
        const long long grid = gridDim.x;
        if (FT == FT_OFF) {
            FtRegs f;
            A tin = acc_zero<A>(), tout = acc_zero<A>();
            for (int it = 0; it < a.tiles_per_cta; ++it) {
                const long long t = blockIdx.x + it * grid;
                if (t >= a.n_tiles) break;
                if (it + 1 < a.tiles_per_cta && t + grid < a.n_tiles) prefetch_tile(a, t + grid);
                tile<false, false>(a, sm, t, false, f, tin, tout);
            }
            return;
        }
        // ---- FT: checksum weights
        FtRegs f;
        {
            int s, c;
            map_thread<K::CFAST_OUT>(s, c);
            // r_j = omega^j with the float32-rounded imaginary part of the reference
            // (include/turbofft/constants.h:2-7)
            const T h = T(0.8660253882408142);
            const T alpha[3] = {T(1), T(-0.5) - h, T(-0.5) + h};
            const T beta[3] = {T(1), T(-0.5) + h, T(-0.5) - h};
            const int s3 = s % 3;
#if TFFT_FT_LEAN
            f.s3 = s3;
            (void)alpha;
            (void)beta;
#else
#pragma unroll
            for (int t = 0; t < 3; ++t) {
                const int j = (s3 + t) % 3;
                f.ab[t].x = j == 0 ? alpha[0] : (j == 1 ? alpha[1] : alpha[2]);
                f.ab[t].y = j == 0 ? beta[0] : (j == 1 ? beta[1] : beta[2]);
            }
#endif
        }
        const bool hit = a.inj_on && ((int)(blockIdx.x % (unsigned)a.inj_period) == a.inj_phase);
        const int inj_it = (int)((blockIdx.x / (unsigned)a.inj_period) % (unsigned)a.tiles_per_cta);
        T acc_in = 0, acc_out = 0, acc_w = 0;
        int done = 0;
        constexpr int CSACC = (FT == FT_CSUM) ? 1 : 0;
        if constexpr (FT == FT_CSUM) {
            // running sums live in shared memory, one slot per (thread, register): nobody else touches them
            C* sums = sm + K::SMEM_ELEMS + threadIdx.x;
#pragma unroll
            for (int i = 0; i < 2 * E; ++i) sums[i * K::THREADS].x = sums[i * K::THREADS].y = T(0);
        }
        for (int it = 0; it < a.tiles_per_cta; ++it) {
            const long long t = blockIdx.x + it * grid;
            if (t >= a.n_tiles) break;
            A tin2 = acc_zero<A>(), tout2 = acc_zero<A>();
            if (it + 1 < a.tiles_per_cta && t + grid < a.n_tiles) prefetch_tile(a, t + grid);
            tile<true, !(TFFT_FT_LEAN && FT == FT_DETECT), CSACC>(a, sm, t, hit && it == inj_it, f, tin2, tout2);
            const T tin = acc_sum(tin2), tout = acc_sum(tout2);
            acc_in += tin;
            acc_out += tout;
            acc_w = fma(T(it + 1), tin - tout, acc_w);
            ++done;
        }
        // ---- block decision (fft_codegen.py:432-503)
        __shared__ T red[3][32];
        __shared__ int s_k;
        T delta = warp_sum(acc_in - acc_out);
        T mag = warp_sum(fabs(acc_in) + fabs(acc_out));
        T dw = warp_sum(acc_w);
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
        constexpr int NW = (K::THREADS + 31) / 32;
        if (lane == 0) {
            red[0][wid] = delta;
            red[1][wid] = mag;
            red[2][wid] = dw;
        }
        __syncthreads();
        if (wid == 0) {
            delta = lane < NW ? red[0][lane] : T(0);
            mag = lane < NW ? red[1][lane] : T(0);
            dw = lane < NW ? red[2][lane] : T(0);
            delta = warp_sum(delta);
            mag = warp_sum(mag);
            dw = warp_sum(dw);
            if (lane == 0) {
                int k = -1;
                if (fabs(delta) / (a.err_smoothing + fabs(mag)) > a.err_threshold) k = (int)round(fabs(dw) / fabs(delta));
                s_k = k;
                a.ft_located[blockIdx.x] = k;
                if (k != -1) atomicAdd(a.ft_count, 1u);
                if (a.ft_diag) {
                    a.ft_diag[3 * (long long)blockIdx.x + 0] = delta;
                    a.ft_diag[3 * (long long)blockIdx.x + 1] = mag;
                    a.ft_diag[3 * (long long)blockIdx.x + 2] = dw;
                }
            }
        }
        __syncthreads();
        if constexpr (FT == FT_CORRECT) {
            // recompute the located tile from the untouched input (fft_codegen.py:149-193)
            const int k = s_k;
            if (k >= 1 && k <= done) {
                A tin = acc_zero<A>(), tout = acc_zero<A>();
                tile<false, false>(a, sm, blockIdx.x + (long long)(k - 1) * grid, false, f, tin, tout);
                if (threadIdx.x == 0) atomicAdd(a.ft_count + 1, 1u);
            }
        }
        if constexpr (FT == FT_CSUM) {
            // transform the summed inputs and take sum(y) - F(sum(x)) off the located tile's outputs
            const int k = s_k;
            if (k >= 1 && k <= done) {
                A tin = acc_zero<A>(), tout = acc_zero<A>();
                tile<false, false, 2>(a, sm, blockIdx.x + (long long)(k - 1) * grid, false, f, tin, tout);
                if (threadIdx.x == 0) atomicAdd(a.ft_count + 1, 1u);
            }
        }
    }
};

template <typename T, int LOGM, int LOGE, int LOGC, int ROLE, int FT>
__global__ void __launch_bounds__((Cfg<T, LOGM, LOGE, LOGC, ROLE>::THREADS),
                                  (Cfg<T, LOGM, LOGE, LOGC, ROLE>::min_blocks(FT)))
fft_kernel(const __grid_constant__ KernelArgs<T> a) {
    extern __shared__ __align__(16) unsigned char tfft_smem_raw[];
    typedef typename Cplx<T>::type C;
    Fft<T, LOGM, LOGE, LOGC, ROLE, FT>::run(a, reinterpret_cast<C*>(tfft_smem_raw));
}

}  // namespace tfft
