// SwiGLU fused with the fp8 quantisation of the down projection's input and with the zeroing of
// the buffer that projection accumulates into.
//
//   out[r, c] = e4m3( silu(gate_up[r, c]) * gate_up[r, hidden + c] * (1 / scale) ),   next_buffer <- 0
//
// Replaces the reference's launcher and kernels csrc/op_src/swiglu/swiglu_dispatch.cu:8-42,
// swiglu_vectorized.cu and swiglu_scalar.cu:24-66 (fp16 in, e4m3fnuz out, one 16-byte load of gate
// and one of up per thread and 8 outputs). The arithmetic keeps the reference's order: silu in
// fp32, times up, times the reciprocal of the scale, then one rounding to fp8.
//
// The kernel is bound by HBM: 4 bytes read and 1 written per output element. Every thread owns
// 8 consecutive outputs of one row (two 16-byte loads, one 8-byte store) and the grid strides
// over the whole matrix, so rows of any length keep all SMs loading. It is launched as a
// programmatic dependent of the GEMM before it and releases the GEMM after it at once: that
// GEMM's weight prefetch overlaps this kernel entirely.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/hfrk_b200.h"
#include "host_common.h"
#include "elementwise_common.cuh"
#include "ptx_sm100.cuh"

namespace hfrk {
namespace {

constexpr int kSwigluThreads = 256;
constexpr int kSwigluCtasPerSm = 8;

// x / (1 + e^-x) with the accurate expf and an IEEE division: the same expression torch evaluates
// for silu on fp32 (reference: operators/swiglu/reference.py:18-21).
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

template <typename T, bool kFnuz>
__device__ __forceinline__ uint2 swiglu_8(const uint4& gate_raw, const uint4& up_raw, float inv_scale) {
    const T* g = reinterpret_cast<const T*>(&gate_raw);
    const T* u = reinterpret_cast<const T*>(&up_raw);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float t = silu_f32(to_f32<T>(g[j]));
        t *= to_f32<T>(u[j]);
        t *= inv_scale;
        // An e4m3fnuz byte is worth half of the same byte read as e4m3fn: encode twice the value.
        v[j] = kFnuz ? t * 2.0f : t;
    }
    uint2 packed;
    packed.x = pack_e4m3x2(v[0], v[1]) | (pack_e4m3x2(v[2], v[3]) << 16);
    packed.y = pack_e4m3x2(v[4], v[5]) | (pack_e4m3x2(v[6], v[7]) << 16);
    if (kFnuz) {
        packed.x = clear_negative_zero_bytes(packed.x);
        packed.y = clear_negative_zero_bytes(packed.y);
    }
    return packed;
}

// Vector path: hidden % 8 == 0, gate_up 16-byte aligned, out 8-byte aligned.
template <typename T, bool kFnuz>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_fp8_vec8_kernel(const T* __restrict__ gate_up, const float* __restrict__ scale_dev, uint8_t* __restrict__ out,
                       uint8_t* __restrict__ next_buffer, size_t buffer_bytes, int rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const float inv_scale = 1.0f / __ldg(scale_dev);
    const int vecs_per_row = hidden >> 3;
    const size_t total = static_cast<size_t>(rows) * vecs_per_row;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t v = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // Two independent vectors per iteration: four 16-byte loads in flight per thread.
    for (; v + stride < total; v += 2 * stride) {
        const size_t v2 = v + stride;
        const size_t r1 = v / vecs_per_row, c1 = v - r1 * vecs_per_row;
        const size_t r2 = v2 / vecs_per_row, c2 = v2 - r2 * vecs_per_row;
        const uint4* row1 = reinterpret_cast<const uint4*>(gate_up + r1 * 2 * hidden);
        const uint4* row2 = reinterpret_cast<const uint4*>(gate_up + r2 * 2 * hidden);
        const uint4 g1 = __ldcs(row1 + c1), u1 = __ldcs(row1 + vecs_per_row + c1);
        const uint4 g2 = __ldcs(row2 + c2), u2 = __ldcs(row2 + vecs_per_row + c2);
        reinterpret_cast<uint2*>(out + r1 * hidden)[c1] = swiglu_8<T, kFnuz>(g1, u1, inv_scale);
        reinterpret_cast<uint2*>(out + r2 * hidden)[c2] = swiglu_8<T, kFnuz>(g2, u2, inv_scale);
    }
    if (v < total) {
        const size_t r1 = v / vecs_per_row, c1 = v - r1 * vecs_per_row;
        const uint4* row1 = reinterpret_cast<const uint4*>(gate_up + r1 * 2 * hidden);
        const uint4 g1 = __ldcs(row1 + c1), u1 = __ldcs(row1 + vecs_per_row + c1);
        reinterpret_cast<uint2*>(out + r1 * hidden)[c1] = swiglu_8<T, kFnuz>(g1, u1, inv_scale);
    }
    zero_range(next_buffer, buffer_bytes);
}

// Scalar path: any hidden, any alignment.
template <typename T, bool kFnuz>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_fp8_scalar_kernel(const T* __restrict__ gate_up, const float* __restrict__ scale_dev,
                         uint8_t* __restrict__ out, uint8_t* __restrict__ next_buffer, size_t buffer_bytes, int rows,
                         int hidden) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const float inv_scale = 1.0f / __ldg(scale_dev);
    const size_t total = static_cast<size_t>(rows) * hidden;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r = i / hidden, c = i - r * hidden;
        const T* row = gate_up + r * 2 * hidden;
        float t = silu_f32(to_f32<T>(row[c]));
        t *= to_f32<T>(row[hidden + c]);
        t *= inv_scale;
        if (kFnuz) t *= 2.0f;
        uint8_t byte = static_cast<uint8_t>(pack_e4m3x2(t, 0.0f) & 0xffu);
        if (kFnuz && byte == 0x80u) byte = 0;
        out[i] = byte;
    }
    zero_range(next_buffer, buffer_bytes);
}

template <typename T>
int launch_swiglu(const void* gate_up, const float* scale_dev, void* out, void* next_buffer, int rows, int hidden,
                  size_t buffer_bytes, bool fnuz, bool vec, cudaStream_t stream) {
    const size_t items = static_cast<size_t>(rows) * (vec ? hidden / 8 : hidden);
    // Enough threads for one item each (two on the vector path), capped at a full machine: the
    // kernels stride over what is left.
    size_t want = (items + kSwigluThreads - 1) / kSwigluThreads;
    const size_t zero_want = (buffer_bytes / 16 + kSwigluThreads - 1) / kSwigluThreads;
    if (zero_want > want) want = zero_want;
    const size_t cap = static_cast<size_t>(kSmCount) * kSwigluCtasPerSm;
    const unsigned grid = static_cast<unsigned>(want < 1 ? 1 : (want > cap ? cap : want));
    const T* in = static_cast<const T*>(gate_up);
    uint8_t* o = static_cast<uint8_t*>(out);
    uint8_t* nb = static_cast<uint8_t*>(next_buffer);
    if (vec) {
        return fnuz ? launch_elementwise(swiglu_fp8_vec8_kernel<T, true>, grid, kSwigluThreads, stream, in,
                                         scale_dev, o, nb, buffer_bytes, rows, hidden)
                    : launch_elementwise(swiglu_fp8_vec8_kernel<T, false>, grid, kSwigluThreads, stream, in,
                                         scale_dev, o, nb, buffer_bytes, rows, hidden);
    }
    return fnuz ? launch_elementwise(swiglu_fp8_scalar_kernel<T, true>, grid, kSwigluThreads, stream, in, scale_dev,
                                     o, nb, buffer_bytes, rows, hidden)
                : launch_elementwise(swiglu_fp8_scalar_kernel<T, false>, grid, kSwigluThreads, stream, in, scale_dev,
                                     o, nb, buffer_bytes, rows, hidden);
}

}  // namespace
}  // namespace hfrk

extern "C" int hfrk_swiglu_fp8(const void* gate_up, const float* scale_dev, void* out, void* next_buffer, int rows,
                               int hidden, int64_t buffer_cols, int in_dtype, int out_kind, int force_scalar,
                               void* stream) {
    using namespace hfrk;
    if (rows < 0 || hidden < 0 || buffer_cols < 0) {
        set_last_error("swiglu: negative extent");
        return HFRK_INVALID_CONFIG;
    }
    if (in_dtype != HFRK_F16 && in_dtype != HFRK_BF16) {
        set_last_error("swiglu: gate_up must be fp16 or bf16");
        return HFRK_BAD_DTYPE;
    }
    if (out_kind != HFRK_E4M3FN && out_kind != HFRK_E4M3FNUZ) {
        set_last_error("swiglu: output must be e4m3fn or e4m3fnuz");
        return HFRK_BAD_DTYPE;
    }
    const size_t buffer_bytes = static_cast<size_t>(rows) * static_cast<size_t>(buffer_cols) * 2;
    if (static_cast<size_t>(rows) * hidden == 0 && buffer_bytes == 0) return HFRK_SUCCESS;
    if (scale_dev == nullptr || (static_cast<size_t>(rows) * hidden != 0 && (gate_up == nullptr || out == nullptr)) ||
        (buffer_bytes != 0 && next_buffer == nullptr)) {
        set_last_error("swiglu: null pointer");
        return HFRK_INVALID_CONFIG;
    }
    if ((reinterpret_cast<uintptr_t>(gate_up) & 1u) || (reinterpret_cast<uintptr_t>(next_buffer) & 1u)) {
        set_last_error("swiglu: 16-bit tensors must be 2-byte aligned");
        return HFRK_BAD_ALIGNMENT;
    }
    const bool vec = !force_scalar && hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(gate_up) & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(out) & 7u) == 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool fnuz = out_kind == HFRK_E4M3FNUZ;
    if (in_dtype == HFRK_F16)
        return launch_swiglu<__half>(gate_up, scale_dev, out, next_buffer, rows, hidden, buffer_bytes, fnuz, vec, s);
    return launch_swiglu<__nv_bfloat16>(gate_up, scale_dev, out, next_buffer, rows, hidden, buffer_bytes, fnuz, vec,
                                        s);
}
