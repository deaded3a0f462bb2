// Kernel table: the B200 counterpart of TurboFFT_Kernel_Entry<...>::turboFFTArr[26][3]
// (include/TurboFFT.h:22-25).  Instead of one pointer per (logN, launch) the table is
// keyed by what a launch does -- (dtype, role, log2 line length, log2 points per thread,
// log2 lines per tile, FT mode) -- so that any parameter row whose launches are compiled
// can be planned at run time.
#pragma once
#include <cstddef>

namespace tfft {

struct KernelEntry {
    const void* fn[4];  // FT_OFF, FT_DETECT, FT_CORRECT, FT_CSUM (null = not compiled)
    int threads;
    size_t smem;        // dynamic shared memory of the first three modes
    size_t smem_csum;   // FT_CSUM adds two tiles of running sums
    int remlast;        // 1: the remainder radix sits in the last register stage (stage-twiddle table order)
};

void register_kernel(int dtype, int role, int logm, int loge, int logc, int ft, const void* fn, int threads,
                     size_t smem, int remlast);
const KernelEntry* find_kernel(int dtype, int role, int logm, int loge, int logc);
int registered_kernel_count();
// counts one kernel launch of this library (see tfft_launch_count)
void note_launch();

}  // namespace tfft
