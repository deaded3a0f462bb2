// Instantiation + registration macro used by the generated instance lists
// (generated/<dtype>/inst_ft<mode>_<part>.cu, written by codegen/fft_codegen.py).
#pragma once
#include "fft_kernels.cuh"
#include "registry.h"

#define TFFT_CAT2(a, b) a##b
#define TFFT_CAT(a, b) TFFT_CAT2(a, b)

// T: float|double, DT: 0|1, ROLE: 0 single, 1 first/middle, 2 last, FT: 0 off, 1 detect, 2 correct (recompute),
// 3 correct from the running checksums (single and last launches only)
#define TFFT_INST(T, DT, LOGM, LOGE, LOGC, ROLE, FT)                                                        \
    template __global__ void tfft::fft_kernel<T, LOGM, LOGE, LOGC, ROLE, FT>(                               \
        const __grid_constant__ tfft::KernelArgs<T>);                                                       \
    namespace {                                                                                             \
    struct TFFT_CAT(TfftReg_, __LINE__) {                                                                   \
        TFFT_CAT(TfftReg_, __LINE__)() {                                                                    \
            typedef tfft::Cfg<T, LOGM, LOGE, LOGC, ROLE> K;                                                 \
            tfft::register_kernel(DT, ROLE, LOGM, LOGE, LOGC, FT,                                           \
                                  (const void*)&tfft::fft_kernel<T, LOGM, LOGE, LOGC, ROLE, FT>, K::THREADS, \
                                  K::smem_bytes(FT), K::REMLAST ? 1 : 0);                                  \
        }                                                                                                   \
    } TFFT_CAT(tfft_reg_, __LINE__);                                                                        \
    }
