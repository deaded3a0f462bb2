// Single-pass FFT of one whole signal of 2^13 .. 2^17 points held in the shared memory of a
// thread-block cluster (sm_100a): one read and one write of HBM where the multi-launch plans of
// the same sizes (the reference's too: include/param/A100/param_float2.csv rows 13-17, launch
// loop main.cu:53-62) make two round trips through a scratch buffer.
//
// Algorithm.  Stockham autosort over the whole signal, every thread of the cluster holding 2R
// complex points in registers.
//   stage 0     radix R0 = N / R^S2 on interleaved (re, im) data straight from global memory;
//               results leave as "units": two adjacent complex values stored planar,
//               (re0, re1, im0, im1) = 16 bytes.
//   stages >= 1 radix R on units.  After stage 0 the data is R0 interleaved independent
//               sub-transforms, and the two halves of a unit belong to two of them that share
//               every twiddle factor, so both are transformed by the same instruction stream:
//               for complex64 with the packed f32x2 arithmetic of sm_100 (one instruction per
//               two lanes), for complex128 with ordinary scalar instructions.
// Exchanges between stages go through shared memory.  The thread-to-CTA assignment changes from
// stage to stage (a different bit field of the thread's global index selects the CTA) such that
// exactly ONE exchange crosses CTAs -- the one after stage 1, written with st.shared::cluster
// into the owning CTA's memory and fenced by barrier.cluster -- and all others stay inside the
// CTA.  Global loads and stores are coalesced runs of at least 128 bytes per CTA.
//
// Variants of the one template: units per thread (16 at 128 registers; 8 -- radix-8 stages, one
// stage more -- at 64 registers and twice the resident warps), cluster size (1 .. 16 CTAs), and a
// prefetching form whose CTAs fetch their share of the next signal into a second shared-memory
// buffer with cp.async.bulk copies completing on an mbarrier (bounded wait, status word) while the
// current signal is transformed.
//
// Unit m of the Stockham array of a stage is read by global thread s = m mod T as its j-th
// input, j = m / T (T = threads in the cluster); it lives in CTA rank(s) at local index
// j * TH + lid(s), padded by pad(L) = L + (L >> 3) + (L >> 6) against bank conflicts.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "cluster_registry.h"
#include "fft_kernels.cuh"

namespace tfft {

// ---------------------------------------------------------------- two-lane arithmetic
// P2<T>: one value per lane.  complex64: a packed register pair and the f32x2 instructions;
// complex128: two doubles and scalar instructions.
__device__ __forceinline__ float2 p_add(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 p_mul(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 p_fma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 p_sub(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.0f, -1.0f), a); }
__device__ __forceinline__ float2 p_neg(float2 a) { return __fmul2_rn(a, make_float2(-1.0f, -1.0f)); }
__device__ __forceinline__ float2 p_set(float x) { return make_float2(x, x); }
__device__ __forceinline__ double2 p_add(double2 a, double2 b) { return make_double2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ double2 p_mul(double2 a, double2 b) { return make_double2(a.x * b.x, a.y * b.y); }
__device__ __forceinline__ double2 p_fma(double2 a, double2 b, double2 c) { return make_double2(fma(a.x, b.x, c.x), fma(a.y, b.y, c.y)); }
__device__ __forceinline__ double2 p_sub(double2 a, double2 b) { return make_double2(a.x - b.x, a.y - b.y); }
__device__ __forceinline__ double2 p_neg(double2 a) { return make_double2(-a.x, -a.y); }
__device__ __forceinline__ double2 p_set(double x) { return make_double2(x, x); }

template <typename T>
struct Unit {  // two complex values, planar: lane 0 = (re.x, im.x), lane 1 = (re.y, im.y)
    typename Cplx<T>::type re, im;
};

// Radix-2^LR decimation-in-frequency butterflies on units; X[q] is left at v[brev(q)].
template <int LR, int LH, typename T, int R>
__device__ __forceinline__ void dif_level_u(Unit<T> (&v)[R]) {
    constexpr int half = 1 << LH;
#pragma unroll
    for (int t = 0; t < R / 2; ++t) {
        const int j = t & (half - 1);
        const int ia = ((t >> LH) << (LH + 1)) + j;
        const int ib = ia + half;
        const Unit<T> a = v[ia], b = v[ib];
        v[ia].re = p_add(a.re, b.re);
        v[ia].im = p_add(a.im, b.im);
        const int k32 = j * (16 >> LH);  // twiddle exp(-2*pi*i*k32/32)
        if (k32 == 0) {
            v[ib].re = p_sub(a.re, b.re);
            v[ib].im = p_sub(a.im, b.im);
        } else if (k32 == 8) {  // -i * (a - b)
            v[ib].re = p_sub(a.im, b.im);
            v[ib].im = p_sub(b.re, a.re);
        } else {
            const auto dr = p_sub(a.re, b.re), di = p_sub(a.im, b.im);
            if (k32 == 4) {  // (1 - i) / sqrt2
                const auto h = p_set(cos32_tab<T>(4));
                v[ib].re = p_mul(p_add(dr, di), h);
                v[ib].im = p_mul(p_sub(di, dr), h);
            } else if (k32 == 12) {  // (-1 - i) / sqrt2
                v[ib].re = p_mul(p_sub(di, dr), p_set(cos32_tab<T>(4)));
                v[ib].im = p_mul(p_add(dr, di), p_set(-cos32_tab<T>(4)));
            } else {
                const T wr = cos32<T>(k32), wi = -sin32<T>(k32);
                v[ib].re = p_fma(dr, p_set(wr), p_mul(di, p_set(-wi)));
                v[ib].im = p_fma(dr, p_set(wi), p_mul(di, p_set(wr)));
            }
        }
    }
    if constexpr (LH > 0) dif_level_u<LR, LH - 1, T, R>(v);
}

// ---------------------------------------------------------------- geometry
// LRU: log2 radix of the unit stages (a thread holds 2R complex points): 4 for complex64 at 128
// registers per thread, 3 for complex128 -- and for the complex64 variant with half the registers
// and twice the resident warps.
template <typename T, int LOGN, int LR0, int LOGG, int LRU = (sizeof(T) == 4 ? 4 : 3)>
struct ClusterCfg {
    static constexpr int LR = LRU;
    static constexpr int R = 1 << LR, R0 = 1 << LR0;
    static constexpr int E = 2 * R;  // complex points per thread
    static constexpr int S2 = (LOGN - LR0) / LR;
    static_assert(LR0 + LR * S2 == LOGN && LR0 >= 1 && LR0 <= LR + 1, "N = R0 * R^S2 with 2 <= R0 <= 2R");
    static_assert(S2 >= 2 && S2 <= 5, "two to five unit stages");
    static constexpr int LOGT = LOGN - 1 - LR;  // log2 threads per cluster
    static constexpr int T_ = 1 << LOGT;
    static constexpr int G = 1 << LOGG;
    static constexpr int LOGTH = LOGT - LOGG;
    static constexpr int TH = 1 << LOGTH;  // threads per CTA
    static constexpr int NB0 = E / R0;     // stage-0 butterflies per thread
    static constexpr int N = 1 << LOGN;
    // bit position of the CTA rank inside the global thread index, per stage
    static __host__ __device__ constexpr int rank_pos(int t) {
        return t == 0 ? LOGT - LR0 + 1 - LOGG : (t == 1 ? LOGT - LOGG : LR0 - 1 + LR - LOGG);
    }
    static_assert(LOGT - LR0 + 1 - LOGG >= 0 && LR0 - 1 + LR - LOGG >= 0, "cluster too large for this size");
    // log2 of the sub-transform count P' (in units) seen by unit stage t >= 1
    static __host__ __device__ constexpr int logp(int t) { return LR0 - 1 + LR * (t - 1); }
    static __host__ __device__ constexpr int pad(int l) { return l + (l >> 3) + (l >> 6); }
    static constexpr int UNITS = pad(R * TH - 1) + 1;
    static constexpr size_t SMEM_BYTES = (size_t)UNITS * 4 * sizeof(T);
    // prefetching variant: behind the exchange buffer, a landing buffer for the CTA's share of the
    // next signal (E * TH complex values) and the mbarrier its bulk copies complete on
    static constexpr size_t SMEM_BYTES_PF = SMEM_BYTES + (size_t)E * TH * 2 * sizeof(T) + 16;
    // entries of the twiddle tables
    static constexpr size_t tw0_count() { return (size_t)LR0 << (LOGN - LR0); }
    static __host__ __device__ constexpr size_t twp_count(int t) { return ((size_t)LR << (LOGT - logp(t))) * 4; }  // in T
};

template <typename T, int LOGN, int LR0, int LOGG, bool PF = false, int LRU = (sizeof(T) == 4 ? 4 : 3)>
struct ClusterFft {
    typedef ClusterCfg<T, LOGN, LR0, LOGG, LRU> K;
    typedef typename Cplx<T>::type C;  // one complex value, or one value per lane
    typedef Unit<T> U;
    static constexpr int R = K::R, LR = K::LR, E = K::E, TH = K::TH, LOGT = K::LOGT;

    // global thread index of (rank, lid) at stage t
    static __device__ __forceinline__ int join(int t, int rank, int lid) {
        const int rp = K::rank_pos(t);
        return ((lid >> rp) << (rp + LOGG)) | (rank << rp) | (lid & ((1 << rp) - 1));
    }
    // Where unit m of the array read by stage t lives: padded local index and CTA rank.  Both are
    // sums (ORs) of the contributions of m's bits, so for m = x + y with disjoint bit fields
    // place(x + y) = place(x) + place(y): per-thread base plus compile-time offsets.
    static __host__ __device__ constexpr int local_index(int t, int m) {
        const int rp = K::rank_pos(t);
        const int s = m & (K::T_ - 1), j = m >> LOGT;
        const int lid = ((s >> (rp + LOGG)) << rp) | (s & ((1 << rp) - 1));
        return K::pad(j * TH + lid);
    }
    static __host__ __device__ constexpr int owner_rank(int t, int m) {
        return ((m & (K::T_ - 1)) >> K::rank_pos(t)) & (K::G - 1);
    }

    static __device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
    static __device__ __forceinline__ void cluster_arrive() {
        if constexpr (LOGG > 0) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    }
    // Arrival that publishes nothing: it only tells the peers that this thread no longer needs
    // what it read from its own shared memory.  The caller places it behind instructions that
    // consumed every loaded value, so the loads have completed.
    static __device__ __forceinline__ void cluster_arrive_relaxed() {
        if constexpr (LOGG > 0) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    }
    static __device__ __forceinline__ void cluster_wait() {
        if constexpr (LOGG > 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    static __device__ __forceinline__ int cluster_rank() {
        if constexpr (LOGG == 0) return 0;
        uint32_t r;
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
        return (int)r;
    }
    static __device__ __forceinline__ void store_unit(T* sm, int idx, const U& u) {
        if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(sm + 4 * (size_t)idx) = make_float4(u.re.x, u.re.y, u.im.x, u.im.y);
        } else {
            double2* p = reinterpret_cast<double2*>(sm + 4 * (size_t)idx);
            p[0] = u.re;
            p[1] = u.im;
        }
    }
    static __device__ __forceinline__ U load_unit(const T* sm, int idx) {
        U u;
        if constexpr (sizeof(T) == 4) {
            const float4 f = *reinterpret_cast<const float4*>(sm + 4 * (size_t)idx);
            u.re = make_float2(f.x, f.y);
            u.im = make_float2(f.z, f.w);
        } else {
            const double2* p = reinterpret_cast<const double2*>(sm + 4 * (size_t)idx);
            u.re = p[0];
            u.im = p[1];
        }
        return u;
    }
    // the same store into the shared memory of CTA `rank` of the cluster
    static __device__ __forceinline__ void store_unit_remote(T* sm, int idx, int rank, const U& u) {
        const uint32_t local = smem_u32(sm + 4 * (size_t)idx);
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
        if constexpr (sizeof(T) == 4) {
            asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(u.re.x), "f"(u.re.y), "f"(u.im.x),
                         "f"(u.im.y)
                         : "memory");
        } else {
            asm volatile("st.shared::cluster.v2.f64 [%0], {%1, %2};" ::"r"(remote), "d"(u.re.x), "d"(u.re.y) : "memory");
            asm volatile("st.shared::cluster.v2.f64 [%0], {%1, %2};" ::"r"(remote + 16), "d"(u.im.x), "d"(u.im.y) : "memory");
        }
    }

    // ---- stage 0: registers <- global (or the landing buffer) ...
    static __device__ __forceinline__ void stage0_load(const ClusterArgs<T>& a, C (&v)[E], const C* src, int first, int stride) {
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] = src[first + i * stride];
        if (a.conj_in) {
#pragma unroll
            for (int i = 0; i < E; ++i) v[i].y = -v[i].y;
        }
    }
    // ... -> radix R0 -> twiddle -> units in local shared memory
    static __device__ __forceinline__ void stage0_compute(const ClusterArgs<T>& a, T* sm, C (&v)[E], int s0) {
        constexpr int R0 = K::R0, NB0 = K::NB0;
#pragma unroll
        for (int u = 0; u < NB0; ++u) dif_butterfly<LR0, NB0, T>(v, u);
        // unit m = (q >> 1) + (R0 / 2) * b with b = s0 + u * T: thread part, u part, q part
        const int base = local_index(1, (R0 / 2) * s0);
#pragma unroll
        for (int u = 0; u < NB0; ++u) {
            const int b = s0 + u * K::T_;
            const C* tw = a.tw0 + b;
            C w[R0];
#pragma unroll
            for (int j = 0; j < LR0; ++j) w[1 << j] = __ldg(tw + j * (K::N / R0));
#pragma unroll
            for (int q = 3; q < R0; ++q)
                if (q & (q - 1)) w[q] = cmul(w[q - (1 << ilog2(q))], w[1 << ilog2(q)]);
#pragma unroll
            for (int q = 0; q < R0; q += 2) {
                C y0 = v[u + brev<LR0>(q) * NB0];
                C y1 = cmul(v[u + brev<LR0>(q + 1) * NB0], w[q + 1]);
                if (q > 0) y0 = cmul(y0, w[q]);
                U un;
                un.re.x = y0.x;
                un.re.y = y1.x;
                un.im.x = y0.y;
                un.im.y = y1.y;
                store_unit(sm, base + local_index(1, (q >> 1) + (R0 / 2) * u * K::T_), un);
            }
        }
    }

    // ---- prefetch of a signal's share into the landing buffer: bulk copies completing on an mbarrier
    static __device__ __forceinline__ void bar_init(uint64_t* bar) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)) : "memory");
    }
    static __device__ __forceinline__ void prefetch(const ClusterArgs<T>& a, C* land, uint64_t* bar, const C* src, int rank) {
        constexpr int RP0 = K::rank_pos(0);
        constexpr int RUN = 1 << RP0;                  // contiguous elements of this CTA per (i, run) in global memory
        constexpr int RUNS_PER_I = TH >> RP0;
        constexpr int NRUN = E * RUNS_PER_I;
        constexpr uint32_t RUN_BYTES = RUN * (uint32_t)sizeof(C);
        static_assert(RUN_BYTES % 16 == 0, "bulk copies move multiples of 16 bytes");
        const uint32_t bar_s = smem_u32(bar);
        if (threadIdx.x == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_s), "r"((uint32_t)(E * TH * sizeof(C)))
                         : "memory");
        for (int r = threadIdx.x; r < NRUN; r += TH) {
            const int i = r / RUNS_PER_I, lh = r % RUNS_PER_I;
            const C* g = src + join(0, rank, lh << RP0) + (size_t)i * K::T_;
            const uint32_t dst = smem_u32(land + i * TH + (lh << RP0));
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                         "l"(g), "r"(RUN_BYTES), "r"(bar_s)
                         : "memory");
        }
    }
    // Bounded wait for the landing buffer: gives up after a long time, records it and goes on (the
    // result is then wrong, the host sees the status word; the kernel never hangs).
    static __device__ __forceinline__ void bar_wait(const ClusterArgs<T>& a, uint64_t* bar, uint32_t parity) {
        const uint32_t bar_s = smem_u32(bar);
        for (int spin = 0; spin < (1 << 22); ++spin) {
            uint32_t done;
            asm volatile(
                "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(bar_s), "r"(parity)
                : "memory");
            if (done) return;
        }
        if (a.status) atomicExch(a.status, 1);
    }

    // ---- unit stage ST (1 .. S2): read R units, butterflies, then twiddle + exchange or store
    template <int ST>
    static __device__ __forceinline__ void unit_stage(const ClusterArgs<T>& a, T* sm, C* dst, int rank, int lid) {
        constexpr bool LAST = (ST == K::S2);
        constexpr bool REMOTE = (ST == 1 && LOGG > 0);  // the exchange behind this stage crosses CTAs
        const int s = join(ST, rank, lid);
        U v[R];
        {
            const int rd = K::pad(lid);
#pragma unroll
            for (int j = 0; j < R; ++j) v[j] = load_unit(sm, rd + K::pad(j * TH));
        }
        // everybody has read its inputs before anybody overwrites them
        if constexpr (!REMOTE) __syncthreads();
        dif_level_u<LR, LR - 1, T, R>(v);
        if constexpr (REMOTE) cluster_arrive_relaxed();  // the butterflies used every input: all reads are done
        if constexpr (LAST) {
            // natural order: unit m = s + q * T holds the complex outputs 2m, 2m + 1
            C* o = dst + 2 * (size_t)s;
#pragma unroll
            for (int q = 0; q < R; ++q) {
                U y = v[brev<LR>(q)];
                if (a.scale_out) {
                    y.re = p_mul(y.re, p_set(a.scale_x));
                    y.im = p_mul(y.im, p_set(a.scale_y));
                }
                if constexpr (sizeof(T) == 4) {
                    *reinterpret_cast<float4*>(o + 2 * (size_t)q * K::T_) = make_float4(y.re.x, y.im.x, y.re.y, y.im.y);
                } else {
                    o[2 * (size_t)q * K::T_] = make_double2(y.re.x, y.im.x);
                    o[2 * (size_t)q * K::T_ + 1] = make_double2(y.re.y, y.im.y);
                }
            }
        } else {
            constexpr int LP = K::logp(ST);
            const int pp = s & ((1 << LP) - 1), nlo = s >> LP;
            // w^(2^j) from the table, both lanes share it: (wr, wr, wi, wi)
            C wr[LR], wi[LR];
            {
                const T* tw = a.twp[ST - 1] + 4 * (size_t)nlo;
#pragma unroll
                for (int j = 0; j < LR; ++j) {
                    if constexpr (sizeof(T) == 4) {
                        const float4 f = __ldg(reinterpret_cast<const float4*>(tw + 4 * (size_t)j * (K::T_ >> LP)));
                        wr[j] = make_float2(f.x, f.y);
                        wi[j] = make_float2(f.z, f.w);
                    } else {
                        const double2* p = reinterpret_cast<const double2*>(tw + 4 * (size_t)j * (K::T_ >> LP));
                        wr[j] = __ldg(p);
                        wi[j] = __ldg(p + 1);
                    }
                }
            }
            // low powers w^1..w^(2^LL - 1) and high powers w^(h << LL): every w^q is one product of the two
            constexpr int LL = LR / 2, NLO = 1 << LL, NHI = 1 << (LR - LL);
            C lo_r[NLO], lo_i[NLO], hi_r[NHI], hi_i[NHI];
#pragma unroll
            for (int x = 1; x < NLO; ++x) {
                if ((x & (x - 1)) == 0) {
                    lo_r[x] = wr[ilog2(x)];
                    lo_i[x] = wi[ilog2(x)];
                } else {
                    const int hb = 1 << ilog2(x);
                    lo_r[x] = p_fma(lo_r[x - hb], lo_r[hb], p_neg(p_mul(lo_i[x - hb], lo_i[hb])));
                    lo_i[x] = p_fma(lo_r[x - hb], lo_i[hb], p_mul(lo_i[x - hb], lo_r[hb]));
                }
            }
#pragma unroll
            for (int x = 1; x < NHI; ++x) {
                if ((x & (x - 1)) == 0) {
                    hi_r[x] = wr[LL + ilog2(x)];
                    hi_i[x] = wi[LL + ilog2(x)];
                } else {
                    const int hb = 1 << ilog2(x);
                    hi_r[x] = p_fma(hi_r[x - hb], hi_r[hb], p_neg(p_mul(hi_i[x - hb], hi_i[hb])));
                    hi_i[x] = p_fma(hi_r[x - hb], hi_i[hb], p_mul(hi_i[x - hb], hi_r[hb]));
                }
            }
            if constexpr (REMOTE) cluster_wait();  // every CTA of the cluster has read its inputs
            // unit m = pp + q * P' + nlo * P' * R
            const int base = local_index(ST + 1, pp + (nlo << (LP + LR)));
            // receiving CTA of the crossing exchange: the top bits of q, plus bits of pp when the
            // cluster has more CTAs than the radix has outputs
            const int rank_base = REMOTE ? owner_rank(ST + 1, pp + (nlo << (LP + LR))) : 0;
#pragma unroll
            for (int q = 0; q < R; ++q) {
                U y = v[brev<LR>(q)];
                if (q > 0) {
                    C qr, qi;
                    const int l = q & (NLO - 1), h = q >> LL;
                    if (h == 0) {
                        qr = lo_r[l];
                        qi = lo_i[l];
                    } else if (l == 0) {
                        qr = hi_r[h];
                        qi = hi_i[h];
                    } else {
                        qr = p_fma(hi_r[h], lo_r[l], p_neg(p_mul(hi_i[h], lo_i[l])));
                        qi = p_fma(hi_r[h], lo_i[l], p_mul(hi_i[h], lo_r[l]));
                    }
                    const C re = p_fma(y.re, qr, p_neg(p_mul(y.im, qi)));
                    const C im = p_fma(y.re, qi, p_mul(y.im, qr));
                    y.re = re;
                    y.im = im;
                }
                const int idx = base + local_index(ST + 1, q << LP);
                if constexpr (REMOTE) store_unit_remote(sm, idx, rank_base | owner_rank(ST + 1, q << LP), y);
                else store_unit(sm, idx, y);
            }
            if constexpr (REMOTE) {
                cluster_arrive();
                cluster_wait();
            } else {
                __syncthreads();
            }
        }
    }

    template <int ST>
    static __device__ __forceinline__ void unit_stages(const ClusterArgs<T>& a, T* sm, C* dst, int rank, int lid) {
        unit_stage<ST>(a, sm, dst, rank, lid);
        if constexpr (ST < K::S2) unit_stages<ST + 1>(a, sm, dst, rank, lid);
    }

    static __device__ __forceinline__ void run(const ClusterArgs<T>& a, T* sm) {
        const int rank = cluster_rank();
        const int lid = threadIdx.x;
        const long long cluster_id = blockIdx.x >> LOGG, n_clusters = gridDim.x >> LOGG;
        const int s0 = join(0, rank, lid);
        C* land = reinterpret_cast<C*>(sm + 4 * (size_t)K::UNITS);
        uint64_t* bar = reinterpret_cast<uint64_t*>(land + E * TH);
        uint32_t parity = 0;
        if constexpr (PF) {
            if (threadIdx.x == 0) bar_init(bar);
            __syncthreads();
            if (cluster_id < a.n_signals && a.signals_per_cluster > 0) prefetch(a, land, bar, a.in + (cluster_id << LOGN), rank);
        }
        for (int it = 0; it < a.signals_per_cluster; ++it) {
            const long long sig = cluster_id + it * n_clusters;
            if (sig >= a.n_signals) break;  // the same decision in every CTA of the cluster
            C v[E];
            if constexpr (PF) {
                bar_wait(a, bar, parity);
                parity ^= 1u;
                stage0_load(a, v, land, lid, TH);
                __syncthreads();  // everybody has its values: the landing buffer is free for the next signal
                const long long next = sig + n_clusters;
                if (it + 1 < a.signals_per_cluster && next < a.n_signals) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    prefetch(a, land, bar, a.in + (next << LOGN), rank);
                }
            } else {
                stage0_load(a, v, a.in + (sig << LOGN), s0, K::T_);
            }
            stage0_compute(a, sm, v, s0);
            __syncthreads();
            // (the last stage ends with a barrier behind its reads, so the next signal's stage 0
            // may overwrite shared memory at once)
            unit_stages<1>(a, sm, a.out + (sig << LOGN), rank, lid);
        }
    }
};

// resident threads per SM the register cap aims at: 512 at 128 registers (384 with the landing
// buffer of the prefetching variant), 1024 for the complex64 variant with 8 units per thread
template <typename T, bool PF, int LRU>
constexpr int cluster_resident_threads() { return (sizeof(T) == 4 && LRU == 3) ? 1024 : (PF ? 384 : 512); }

template <typename T, int LOGN, int LR0, int LOGG, bool PF, int LRU>
__global__ void __launch_bounds__((ClusterCfg<T, LOGN, LR0, LOGG, LRU>::TH),
                                  (cluster_resident_threads<T, PF, LRU>() / ClusterCfg<T, LOGN, LR0, LOGG, LRU>::TH))
cluster_fft_kernel(const __grid_constant__ ClusterArgs<T> a) {
    extern __shared__ __align__(16) unsigned char tfft_cluster_smem[];
    ClusterFft<T, LOGN, LR0, LOGG, PF, LRU>::run(a, reinterpret_cast<T*>(tfft_cluster_smem));
}

}  // namespace tfft
