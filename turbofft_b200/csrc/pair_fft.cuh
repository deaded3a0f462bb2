// Both launches of a two-launch plan as ONE persistent kernel whose intermediate stays in L2.
//
// A two-launch plan writes the whole intermediate (batch * N elements) to HBM and reads it back.
// Here the batch is cut into chunks of a few signals.  The grid is persistent and co-resident
// (cooperative launch); its blocks draw tickets from one global list of work items,
//
//     super-step j:  [ first-launch tiles of chunk j ][ last-launch tiles of chunk j - lag ]
//
// (an atomic counter: the block that is free takes the next item, as the hardware's block
// scheduler would -- work assigned statically, item i to block i mod grid, measured 5-8 % slower),
// and the intermediate of chunk c lives in slot c mod R of a ring of R chunks, small enough to
// stay in L2 between the store of the first launch's tile and the load of the last launch's.
// Two counters per chunk order the accesses:
//   * a last-launch tile of chunk c waits until every first-launch tile of chunk c has finished,
//   * a first-launch tile of chunk c waits until every last-launch tile of chunk c - R has
//     finished (the slot it overwrites has been read).
// Both dependencies point at items EARLIER in the list, every block draws its tickets in
// increasing order (it holds at most the one it works on and the next one) and all blocks are
// resident, so the earliest unfinished item is always some block's current item and can run:
// the waits cannot deadlock.  They are bounded all the same: a wait that gives up sets the
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
    unsigned long long* queue;  // zero at launch: the next ticket
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
// It also draws the block's next ticket there, so that the atomic's round trip hides behind the tile.
struct PairDeferredSignal {
    unsigned int* counter;
    unsigned long long* queue;
    unsigned long long* next_ticket;  // shared memory
    __device__ __forceinline__ void operator()() const {
        if (threadIdx.x == 0) {
            if (counter) pair_signal(counter);
            *next_ticket = atomicAdd(queue, 1ULL);
        }
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
    __shared__ unsigned long long s_ticket[2];  // by iteration parity: thread 0 writes the next one while others may still read this one
    if (threadIdx.x == 0) s_abort = 0;

    const long long per = (long long)p.tiles1 + p.tiles2;
    const long long n_items = (p.n_chunks + p.lag) * per;

    // item i of the list: which launch, chunk and tile, and what it waits for (a counter and the number
    // of tiles of that chunk, whose last one may be ragged); tile < 0 for the empty slots of the first
    // and last super-steps and of a ragged last chunk
    struct Item {
        bool is_first;
        long long chunk, tile, need;
        const unsigned int* flag;
    };
    auto decode = [&](long long i) {
        Item it;
        const long long j = i / per;
        const int slot = (int)(i - j * per);
        it.is_first = slot < p.tiles1;
        it.chunk = it.is_first ? j : j - p.lag;
        it.tile = it.is_first ? it.chunk * p.tiles1 + slot : it.chunk * p.tiles2 + (slot - p.tiles1);
        it.flag = nullptr;
        it.need = 0;
        if (it.chunk < 0 || it.chunk >= p.n_chunks || it.tile >= (it.is_first ? p.first.n_tiles : p.last.n_tiles)) {
            it.tile = -1;
        } else if (it.is_first) {
            if (it.chunk >= p.ring_chunks) {
                const long long dep = it.chunk - p.ring_chunks;
                it.flag = p.done + p.n_chunks + dep;
                it.need = p.last.n_tiles - dep * p.tiles2;
                if (it.need > p.tiles2) it.need = p.tiles2;
            }
        } else {
            it.flag = p.done + it.chunk;
            it.need = p.first.n_tiles - it.chunk * p.tiles1;
            if (it.need > p.tiles1) it.need = p.tiles1;
        }
        return it;
    };

    unsigned int* pending = nullptr;  // thread 0: counter of the tile this block finished last, not yet published
    // s_ticket[parity] is the item of this iteration; thread 0 draws the next one into the other slot
    // while the tile runs (nobody reads that slot before the next iteration's barrier)
    if (threadIdx.x == 0) s_ticket[0] = atomicAdd(p.queue, 1ULL);
    for (int parity = 0;; parity ^= 1) {
        int must_wait = 0;
        if (threadIdx.x == 0) {
            const unsigned long long ticket = s_ticket[parity];
            if ((long long)ticket < n_items) {
                const Item mine = decode((long long)ticket);
                if (mine.tile >= 0 && mine.flag) must_wait = pair_ld_acquire(mine.flag) < (unsigned int)mine.need;
            }
        }
        // one barrier in the common case: the previous tile has finished with shared memory and has issued
        // its stores, everybody learns the ticket and whether its dependency is already met
        const int waiting = __syncthreads_or(must_wait);
        const long long i = (long long)s_ticket[parity];
        if (i >= n_items) break;
        const Item item = decode(i);
        if (item.tile < 0) {
            if (threadIdx.x == 0) s_ticket[parity ^ 1] = atomicAdd(p.queue, 1ULL);
            continue;
        }
        const bool is_first = item.is_first;
        const long long chunk = item.chunk, tile = item.tile;
        if (waiting) {
            if (threadIdx.x == 0) {
                // a block that waits holds no unpublished tile (or two blocks could wait for each other)
                if (pending) pair_signal(pending);
                pending = nullptr;
                int polls = 0;
                while (pair_ld_acquire(item.flag) < (unsigned int)item.need) {
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
        hook.queue = p.queue;
        hook.next_ticket = &s_ticket[parity ^ 1];
        if (is_first) F1::template tile<false, false, 0, false>(p.first, sm, tile, false, f1, tin, tout, hook);
        else F2::template tile<false, false, 0, true>(p.last, sm, tile, false, f2, tin, tout, hook);
        pending = p.done + (is_first ? chunk : p.n_chunks + chunk);
    }
    __syncthreads();
    if (threadIdx.x == 0 && pending) pair_signal(pending);
}

}  // namespace tfft
