// CUDA_CHECK with the behaviour of the reference's include/grpo/cuda_utils.cuh:8-16: a failed
// runtime call prints the error with its location and ends the process.
#pragma once

#include <cstdio>
#include <cstdlib>

#include <cuda_runtime.h>

#define CUDA_CHECK(call)                                                                         \
    do {                                                                                         \
        const cudaError_t grpo_status_ = (call);                                                 \
        if (grpo_status_ != cudaSuccess) {                                                       \
            std::fprintf(stderr, "CUDA error: %s at %s:%d\n", cudaGetErrorString(grpo_status_), \
                         __FILE__, __LINE__);                                                    \
            std::exit(1);                                                                        \
        }                                                                                        \
    } while (0)
