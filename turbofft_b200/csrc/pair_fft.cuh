// Both launches of a two-launch plan as ONE persistent kernel whose intermediate stays in L2.
//
// A two-launch plan writes the whole intermediate (batch * N elements) to HBM and reads it back.
// Here the batch is cut into chunks of a few signals.  The grid is persistent and co-resident
// (cooperative launch); its blocks walk one global list of work items in order,
//
//     super-step j:  [ first-launch tiles of chunk j ][ last-launch tiles of chunk j - lag ]
//
// and the intermediate of chunk c lives in slot c mod R of a ring of R chunks, small enough to
// stay in L2 between the store of the first launch's tile and the load of the last launch's.
// Two counters per chunk order the accesses:
//   * a last-launch tile of chunk c waits until every first-launch tile of chunk c has finished,
//   * a first-launch tile of chunk c waits until every last-launch tile of chunk c - R has
//     finished (the slot it overwrites has been read).
// Both dependencies point at items EARLIER in the list, every block takes its items in
// increasing order and all blocks are resident, so the earliest unfinished item can always
// run: the waits cannot deadlock.  They are bounded all the same: a wait that gives up sets the
// status word and the block returns.
//
// The reference has no counterpart: its plans of the same sizes are separate launches
// (include/param/A100/param_float2.csv rows 13-22, TurboFFT.h:120-140).
#pragma once
#include "fft_kernels.cuh"

namespace tfft {

template <typename T>
struct PairArgs {
    KernelArgs<T> first;  // out = the ring, ring_clear set
    KernelArgs<T> last;   // in = the ring, ring_clear set
    unsigned int* done;   // [2 * n_chunks], zero at launch: finished tiles per chunk, first launch then last
    int* status;          // set to 1 if a wait gave up
    long long n_chunks;
    int tiles1;       // first-launch tiles per chunk
    int tiles2;       // last-launch tiles per chunk
    int lag;          // super-steps between a chunk's first-launch and last-launch tiles
    int ring_chunks;  // R
};

constexpr int PAIR_WAIT_POLLS = 1 << 20;

__device__ __forceinline__ unsigned int pair_ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T, int M1, int E1, int C1, int M2, int E2, int C2>
struct PairCfg {
    typedef Cfg<T, M1, E1, C1, ROLE_FIRST> K1;
    typedef Cfg<T, M2, E2, C2, ROLE_LAST> K2;
    static_assert(K1::THREADS == K2::THREADS, "both launches must use the same block size");
    static constexpr int THREADS = K1::THREADS;
    static constexpr size_t SMEM_BYTES = K1::SMEM_BYTES > K2::SMEM_BYTES ? K1::SMEM_BYTES : K2::SMEM_BYTES;
    static constexpr int MIN_BLOCKS = K1::min_blocks(FT_OFF) < K2::min_blocks(FT_OFF) ? K1::min_blocks(FT_OFF) : K2::min_blocks(FT_OFF);
};

// Publishes a finished tile: every store of the block that a barrier ordered before this call
// becomes visible device-wide, then the chunk's counter moves.
__device__ __forceinline__ void pair_signal(unsigned int* counter) {
    __threadfence();
    atomicAdd(counter, 1u);
}

// Run by thread 0 inside the NEXT tile, after that tile's loads have been issued: the fence of
// the previous tile's signal then waits for stores that have been in flight for a load latency
// already, instead of stalling the block right behind them.
struct PairDeferredSignal {
    unsigned int* counter;
    __device__ __forceinline__ void operator()() const {
        if (threadIdx.x == 0 && counter) pair_signal(counter);
    }
};

template <typename T, int M1, int E1, int C1, int M2, int E2, int C2>
__global__ void __launch_bounds__((PairCfg<T, M1, E1, C1, M2, E2, C2>::THREADS), (PairCfg<T, M1, E1, C1, M2, E2, C2>::MIN_BLOCKS))
fft_pair_kernel(const __grid_constant__ PairArgs<T> p) {
    typedef Fft<T, M1, E1, C1, ROLE_FIRST, FT_OFF> F1;
    typedef Fft<T, M2, E2, C2, ROLE_LAST, FT_OFF> F2;
    typedef typename Cplx<T>::type C;
    extern __shared__ __align__(16) unsigned char tfft_pair_smem_raw[];
    C* sm = reinterpret_cast<C*>(tfft_pair_smem_raw);
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = 0;

    const long long per = (long long)p.tiles1 + p.tiles2;
    const long long n_items = (p.n_chunks + p.lag) * per;
    unsigned int* pending = nullptr;  // thread 0: counter of the tile this block finished last, not yet published
    for (long long i = blockIdx.x; i < n_items; i += gridDim.x) {
        const long long j = i / per;
        const int slot = (int)(i - j * per);
        const bool is_first = slot < p.tiles1;
        const long long chunk = is_first ? j : j - p.lag;
        if (chunk < 0 || chunk >= p.n_chunks) continue;
        const long long tile = is_first ? chunk * p.tiles1 + slot : chunk * p.tiles2 + (slot - p.tiles1);
        if (tile >= (is_first ? p.first.n_tiles : p.last.n_tiles)) continue;

        // what this item waits for: a counter and the number of tiles of that chunk (the last chunk may be ragged)
        const unsigned int* flag = nullptr;
        long long need = 0;
        if (is_first) {
            if (chunk >= p.ring_chunks) {
                const long long dep = chunk - p.ring_chunks;
                flag = p.done + p.n_chunks + dep;
                need = p.last.n_tiles - dep * p.tiles2;
                if (need > p.tiles2) need = p.tiles2;
            }
        } else {
            flag = p.done + chunk;
            need = p.first.n_tiles - chunk * p.tiles1;
            if (need > p.tiles1) need = p.tiles1;
        }
        int must_wait = 0;
        if (flag && threadIdx.x == 0) must_wait = pair_ld_acquire(flag) < (unsigned int)need;
        // one barrier in the common case: the previous tile has finished with shared memory and has
        // issued its stores, and everybody learns whether the dependency is already met
        if (__syncthreads_or(must_wait)) {
            if (threadIdx.x == 0) {
                // a block that waits holds no unpublished tile (or two blocks could wait for each other)
                if (pending) pair_signal(pending);
                pending = nullptr;
                int polls = 0;
                while (pair_ld_acquire(flag) < (unsigned int)need) {
                    if (++polls > PAIR_WAIT_POLLS || *(volatile int*)p.status) {
                        *(volatile int*)p.status = 1;
                        s_abort = 1;
                        break;
                    }
                    __nanosleep(100);
                }
            }
            __syncthreads();
        }
        if (s_abort) return;

        typename F1::FtRegs f1;
        typename F2::FtRegs f2;
        typename FtAcc<T>::type tin = acc_zero<typename FtAcc<T>::type>(), tout = tin;
        PairDeferredSignal hook;
        hook.counter = pending;
        if (is_first) F1::template tile<false, false, 0, false>(p.first, sm, tile, false, f1, tin, tout, hook);
        else F2::template tile<false, false, 0, true>(p.last, sm, tile, false, f2, tin, tout, hook);
        pending = p.done + (is_first ? chunk : p.n_chunks + chunk);
    }
    __syncthreads();
    if (threadIdx.x == 0 && pending) pair_signal(pending);
}

}  // namespace tfft
