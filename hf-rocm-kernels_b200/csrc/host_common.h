// Host-side helpers shared by the translation units of libhfrk_b200.so: the per-thread error
// text behind hfrk_last_error() and the CUDA-call check that turns a failure into a status code
// (the library reports by return value, like the reference's launcher:
// csrc/op_src/skinny_gemm/skinny_gemm_caller.cu:9-17).
#pragma once

#include <cuda_runtime.h>

#include "../../include/hfrk_b200.h"

namespace hfrk {

void set_last_error(const char* text);
void set_last_error_at(const char* text, const char* call);

// 1 unless the environment switches programmatic dependent launch off for the plain entry points
// (HFRK_PDL=0). With it the weight stream of a call starts while the previous kernel on the stream
// drains, which is only correct when that kernel does not write W: true for inference, where
// weights are static.
int default_use_pdl();

}  // namespace hfrk

// On failure hfrk_last_error() reads "<CUDA's message>: <the call that failed>".
#define HFRK_CUDA_TRY(expr)                                                    \
    do {                                                                       \
        cudaError_t hfrk_err_ = (expr);                                        \
        if (hfrk_err_ != cudaSuccess) {                                        \
            ::hfrk::set_last_error_at(cudaGetErrorString(hfrk_err_), #expr);   \
            (void)cudaGetLastError();                                          \
            return HFRK_CUDA_ERROR;                                            \
        }                                                                      \
    } while (0)
