// Pieces shared by the element-wise kernels of the decode path (swiglu, residual + RMS norm):
// 16-bit <-> fp32 conversions, the e4m3 encoder, the grid-wide zero fill of the buffer the next
// GEMM accumulates into, and the launch with the programmatic-dependent-launch attribute.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "host_common.h"

namespace hfrk {

constexpr int kSmCount = 148;

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) {
    return __half2float(v);
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}

// Two fp32 -> two e4m3fn bytes, round to nearest even, saturating at +-448.
__device__ __forceinline__ uint32_t pack_e4m3x2(float lo, float hi) {
    return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

// e4m3fnuz has no negative zero (0x80 is its NaN): bytes equal to 0x80 become 0x00, as
// utils/fp8.py:26-30 of the reference does.
__device__ __forceinline__ uint32_t clear_negative_zero_bytes(uint32_t word) {
    return word & ~__vcmpeq4(word, 0x80808080u);
}

// Zeroes `bytes` bytes (a multiple of 2) starting at `base` (2-byte aligned) with the whole grid.
__device__ __forceinline__ void zero_range(uint8_t* base, size_t bytes) {
    if (bytes == 0) return;
    const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t head = (16 - (reinterpret_cast<uintptr_t>(base) & 15u)) & 15u;
    const size_t head_bytes = head < bytes ? head : bytes;
    for (size_t i = tid * 2; i < head_bytes; i += nthreads * 2) *reinterpret_cast<uint16_t*>(base + i) = 0;
    uint8_t* body = base + head_bytes;
    const size_t body_vecs = (bytes - head_bytes) / 16;
    for (size_t i = tid; i < body_vecs; i += nthreads) reinterpret_cast<uint4*>(body)[i] = make_uint4(0, 0, 0, 0);
    uint8_t* tail = body + body_vecs * 16;
    const size_t tail_bytes = bytes - head_bytes - body_vecs * 16;
    for (size_t i = tid * 2; i < tail_bytes; i += nthreads * 2) *reinterpret_cast<uint16_t*>(tail + i) = 0;
}

template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Launches `kernel` on `stream`, as a programmatic dependent of the kernel before it unless
// HFRK_PDL=0. The kernels launched this way call griddepcontrol.wait before their first load.
template <typename Kernel, typename... Args>
int launch_elementwise(Kernel kernel, unsigned grid, unsigned block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1];
    unsigned num_attrs = 0;
    if (default_use_pdl()) {
        attrs[num_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[num_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++num_attrs;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = num_attrs;
    HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, args...));
    return HFRK_SUCCESS;
}


}  // namespace hfrk
