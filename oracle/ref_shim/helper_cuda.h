/* TEST INFRASTRUCTURE.  Minimal stand-in for the cuda-samples header the reference
 * includes (include/utils/utils.h:4) but does not ship: only checkCudaErrors is used. */
#pragma once
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <vector>
#include <string>
#include <sstream>
#include <fstream>
#include <iostream>
#define checkCudaErrors(call)                                                              \
    do {                                                                                   \
        const int tfft_shim_err_ = (int)(call);                                            \
        if (tfft_shim_err_ != 0) {                                                         \
            fprintf(stderr, "CUDA/cuFFT error %d at %s:%d\n", tfft_shim_err_, __FILE__, __LINE__); \
            exit(EXIT_FAILURE);                                                            \
        }                                                                                  \
    } while (0)
