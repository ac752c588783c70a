// Residual add + RMS norm, fused with the fp8 quantisation of the next projection's input and with
// the zeroing of the buffer that projection accumulates into.
//
//   residual <- input + residual                       (rounded to the 16-bit type, in place)
//   y        = residual * rsqrt(mean(residual^2) + eps) * weight
//   output   = e4m3(y / scale)   or   y in the 16-bit type when no scale is given
//
// Replaces the reference's launcher and kernels csrc/op_src/residual_rms/residual_rms_dispatch.cu:8-63,
// residual_rms_vectorized.cu:13-175 and residual_rms_scalar.cu:11-74, and keeps the arithmetic of
// the vectorised kernel, which is what the reference runs on aligned tensors:
//   * the sum is formed in the 16-bit type, squares are accumulated in fp32;
//   * fp8 output: float(residual) * float(weight) * (normaliser / scale), one rounding to fp8
//     (residual_rms_vectorized.cu:124-135);
//   * 16-bit output: round(float(residual) * normaliser) to 16 bits, then a 16-bit multiply by the
//     weight (residual_rms_vectorized.cu:138-146), which is also what the torch reference does
//     (operators/residual_rms/reference.py:21-29).
//
// One CTA per row. Every thread keeps the sums it formed in registers (up to kRegChunks vectors
// of 8), so each element is read once and written once; longer rows re-read their own stores,
// which are still in L1/L2. At decode sizes (16 rows of 4096) the kernel is latency bound: it is
// launched as a programmatic dependent, so its prologue overlaps the tail of the GEMM before it,
// and it releases the GEMM after it at once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hfrk_b200.h"
#include "elementwise_common.cuh"
#include "host_common.h"
#include "ptx_sm100.cuh"

namespace hfrk {
namespace {

constexpr int kRegChunks = 2;
constexpr int kOutSame = 0;   // output in the input's 16-bit type
constexpr int kOutFn = 1;     // e4m3fn bytes
constexpr int kOutFnuz = 2;   // e4m3fnuz bytes

__device__ __forceinline__ __half add16(__half a, __half b) { return __hadd(a, b); }
__device__ __forceinline__ __nv_bfloat16 add16(__nv_bfloat16 a, __nv_bfloat16 b) { return __hadd(a, b); }
__device__ __forceinline__ __half mul16(__half a, __half b) { return __hmul(a, b); }
__device__ __forceinline__ __nv_bfloat16 mul16(__nv_bfloat16 a, __nv_bfloat16 b) { return __hmul(a, b); }

// Sum over the CTA, result in every thread. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        float w = lane < warps ? scratch[lane] : 0.0f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) w += __shfl_xor_sync(0xffffffffu, w, off);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

template <typename T, int kOut>
__device__ __forceinline__ void normalise_store_8(const uint4& sum_raw, const uint4& weight_raw, float normaliser,
                                                  float quant_factor, void* out_row, int chunk) {
    const T* s = reinterpret_cast<const T*>(&sum_raw);
    const T* w = reinterpret_cast<const T*>(&weight_raw);
    if (kOut == kOutSame) {
        uint4 packed;
        T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = mul16(from_f32<T>(to_f32<T>(s[j]) * normaliser), w[j]);
        reinterpret_cast<uint4*>(out_row)[chunk] = packed;
    } else {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (to_f32<T>(s[j]) * to_f32<T>(w[j])) * quant_factor;
        uint2 packed;
        packed.x = pack_e4m3x2(v[0], v[1]) | (pack_e4m3x2(v[2], v[3]) << 16);
        packed.y = pack_e4m3x2(v[4], v[5]) | (pack_e4m3x2(v[6], v[7]) << 16);
        if (kOut == kOutFnuz) {
            packed.x = clear_negative_zero_bytes(packed.x);
            packed.y = clear_negative_zero_bytes(packed.y);
        }
        reinterpret_cast<uint2*>(out_row)[chunk] = packed;
    }
}

// Vector path: cols % 8 == 0, input/residual/weight 16-byte aligned, output aligned to its vector.
template <typename T, int kOut>
__global__ void __launch_bounds__(1024)
residual_rms_vec8_kernel(const T* __restrict__ input, T* __restrict__ residual, const T* __restrict__ weight,
                         const float* __restrict__ scale_dev, float epsilon, void* __restrict__ output,
                         uint8_t* __restrict__ next_buffer, size_t buffer_bytes, int cols) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int chunks = cols >> 3;
    const size_t row = blockIdx.x;
    // The weight does not depend on the kernel before this one: fetch it ahead of the wait.
    uint4 w_regs[kRegChunks];
#pragma unroll
    for (int i = 0; i < kRegChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) w_regs[i] = __ldg(reinterpret_cast<const uint4*>(weight) + c);
    }
    pdl_wait_prior_grids();

    const uint4* in_row = reinterpret_cast<const uint4*>(input + row * cols);
    uint4* res_row = reinterpret_cast<uint4*>(residual + row * cols);
    uint4 sums[kRegChunks];
    float sq = 0.0f;
    // All loads of the register-resident part are issued before the first add.
    uint4 a_regs[kRegChunks], b_regs[kRegChunks];
#pragma unroll
    for (int i = 0; i < kRegChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            a_regs[i] = __ldcs(in_row + c);
            b_regs[i] = res_row[c];
        }
    }
#pragma unroll
    for (int i = 0; i < kRegChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            const T* a = reinterpret_cast<const T*>(&a_regs[i]);
            const T* b = reinterpret_cast<const T*>(&b_regs[i]);
            T* s = reinterpret_cast<T*>(&sums[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[j] = add16(b[j], a[j]);
                const float x = to_f32<T>(s[j]);
                sq = fmaf(x, x, sq);
            }
            res_row[c] = sums[i];
        }
    }
    for (int c = threadIdx.x + kRegChunks * blockDim.x; c < chunks; c += blockDim.x) {
        const uint4 av = __ldcs(in_row + c), bv = res_row[c];
        uint4 sv;
        const T* a = reinterpret_cast<const T*>(&av);
        const T* b = reinterpret_cast<const T*>(&bv);
        T* s = reinterpret_cast<T*>(&sv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j] = add16(b[j], a[j]);
            const float x = to_f32<T>(s[j]);
            sq = fmaf(x, x, sq);
        }
        res_row[c] = sv;
    }

    const float variance = block_sum(sq, scratch) / static_cast<float>(cols);
    const float normaliser = 1.0f / sqrtf(variance + epsilon);
    float quant_factor = 1.0f;
    if (kOut != kOutSame) {
        quant_factor = normaliser / __ldg(scale_dev);
        // An e4m3fnuz byte is worth half of the same byte read as e4m3fn: encode twice the value.
        if (kOut == kOutFnuz) quant_factor *= 2.0f;
    }

    void* out_row = kOut == kOutSame ? static_cast<void*>(static_cast<T*>(output) + row * cols)
                                     : static_cast<void*>(static_cast<uint8_t*>(output) + row * cols);
#pragma unroll
    for (int i = 0; i < kRegChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) normalise_store_8<T, kOut>(sums[i], w_regs[i], normaliser, quant_factor, out_row, c);
    }
    for (int c = threadIdx.x + kRegChunks * blockDim.x; c < chunks; c += blockDim.x) {
        // This thread wrote res_row[c] itself a moment ago.
        const uint4 sv = res_row[c];
        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(weight) + c);
        normalise_store_8<T, kOut>(sv, wv, normaliser, quant_factor, out_row, c);
    }
    // only with fp8 output, as in the reference (residual_rms_dispatch.cu:33-43 passes no buffer otherwise):
    // a 16-bit output does not feed a GEMM that accumulates into next_buffer
    if (kOut != kOutSame) zero_range(next_buffer, buffer_bytes);
}

// Scalar path: any cols, any alignment.
template <typename T, int kOut>
__global__ void __launch_bounds__(1024)
residual_rms_scalar_kernel(const T* __restrict__ input, T* __restrict__ residual, const T* __restrict__ weight,
                           const float* __restrict__ scale_dev, float epsilon, void* __restrict__ output,
                           uint8_t* __restrict__ next_buffer, size_t buffer_bytes, int cols) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const size_t row = blockIdx.x;
    const T* in_row = input + row * cols;
    T* res_row = residual + row * cols;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const T s = add16(res_row[c], in_row[c]);
        const float x = to_f32<T>(s);
        sq = fmaf(x, x, sq);
        res_row[c] = s;
    }
    const float variance = block_sum(sq, scratch) / static_cast<float>(cols);
    const float normaliser = 1.0f / sqrtf(variance + epsilon);
    float quant_factor = 1.0f;
    if (kOut != kOutSame) {
        quant_factor = normaliser / __ldg(scale_dev);
        if (kOut == kOutFnuz) quant_factor *= 2.0f;
    }
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const T s = res_row[c];  // written by this thread above
        if (kOut == kOutSame) {
            static_cast<T*>(output)[row * cols + c] = mul16(from_f32<T>(to_f32<T>(s) * normaliser), weight[c]);
        } else {
            const float v = (to_f32<T>(s) * to_f32<T>(weight[c])) * quant_factor;
            uint8_t byte = static_cast<uint8_t>(pack_e4m3x2(v, 0.0f) & 0xffu);
            if (kOut == kOutFnuz && byte == 0x80u) byte = 0;
            static_cast<uint8_t*>(output)[row * cols + c] = byte;
        }
    }
    // only with fp8 output, as in the reference (residual_rms_dispatch.cu:33-43 passes no buffer otherwise):
    // a 16-bit output does not feed a GEMM that accumulates into next_buffer
    if (kOut != kOutSame) zero_range(next_buffer, buffer_bytes);
}

// CTA size. A hint that is a multiple of 32 is taken as it is. Otherwise one work item (a 16-byte
// vector, or an element on the scalar path) per thread: the shortest critical path, which is what
// the few rows of a decode step need. With more rows than the machine holds CTAs at once, two items
// per thread: smaller CTAs, more of them per SM, so one CTA's reduction overlaps another's loads.
int choose_threads(int work_items, int rows, int hint) {
    if (hint >= 32 && hint <= 1024 && hint % 32 == 0) return hint;
    if (rows > 2 * kSmCount) work_items = (work_items + 1) / 2;
    int threads = ((work_items + 31) / 32) * 32;
    if (threads < 64) threads = 64;
    if (threads > 1024) threads = 1024;
    return threads;
}

template <typename T, int kOut>
int launch_residual_rms(const void* input, void* residual, const void* weight, const float* scale_dev, float epsilon,
                        void* output, void* next_buffer, size_t buffer_bytes, int rows, int cols, bool vec,
                        int num_threads, cudaStream_t stream) {
    const T* in = static_cast<const T*>(input);
    T* res = static_cast<T*>(residual);
    const T* w = static_cast<const T*>(weight);
    uint8_t* nb = static_cast<uint8_t*>(next_buffer);
    const unsigned grid = static_cast<unsigned>(rows);
    if (vec) {
        const unsigned block = static_cast<unsigned>(choose_threads(cols / 8, rows, num_threads));
        return launch_elementwise(residual_rms_vec8_kernel<T, kOut>, grid, block, stream, in, res, w, scale_dev,
                                  epsilon, output, nb, buffer_bytes, cols);
    }
    const unsigned block = static_cast<unsigned>(choose_threads(cols, rows, num_threads));
    return launch_elementwise(residual_rms_scalar_kernel<T, kOut>, grid, block, stream, in, res, w, scale_dev,
                              epsilon, output, nb, buffer_bytes, cols);
}

template <typename T>
int dispatch_out(int out_mode, const void* input, void* residual, const void* weight, const float* scale_dev,
                 float epsilon, void* output, void* next_buffer, size_t buffer_bytes, int rows, int cols, bool vec,
                 int num_threads, cudaStream_t stream) {
    switch (out_mode) {
        case kOutSame:
            return launch_residual_rms<T, kOutSame>(input, residual, weight, scale_dev, epsilon, output, next_buffer,
                                                    buffer_bytes, rows, cols, vec, num_threads, stream);
        case kOutFn:
            return launch_residual_rms<T, kOutFn>(input, residual, weight, scale_dev, epsilon, output, next_buffer,
                                                  buffer_bytes, rows, cols, vec, num_threads, stream);
        default:
            return launch_residual_rms<T, kOutFnuz>(input, residual, weight, scale_dev, epsilon, output, next_buffer,
                                                    buffer_bytes, rows, cols, vec, num_threads, stream);
    }
}

}  // namespace
}  // namespace hfrk

extern "C" int hfrk_residual_rms(const void* input, void* residual, const void* weight, const float* scale_dev,
                                 float epsilon, void* output, void* next_buffer, int rows, int cols,
                                 int64_t buffer_cols, int dtype, int out_kind, int num_threads, int force_scalar,
                                 void* stream) {
    using namespace hfrk;
    if (rows < 0 || cols < 0 || buffer_cols < 0) {
        set_last_error("residual_rms: negative extent");
        return HFRK_INVALID_CONFIG;
    }
    if (dtype != HFRK_F16 && dtype != HFRK_BF16) {
        set_last_error("residual_rms: input, residual and weight must be fp16 or bf16");
        return HFRK_BAD_DTYPE;
    }
    if (out_kind != HFRK_OUT_SAME && out_kind != HFRK_OUT_E4M3FN && out_kind != HFRK_OUT_E4M3FNUZ) {
        set_last_error("residual_rms: unknown output kind");
        return HFRK_BAD_DTYPE;
    }
    if (!(epsilon > 0.0f)) {
        set_last_error("residual_rms: epsilon must be positive");
        return HFRK_INVALID_CONFIG;
    }
    if (rows == 0) return HFRK_SUCCESS;
    if (cols == 0) {
        set_last_error("residual_rms: rows without columns have no mean");
        return HFRK_INVALID_CONFIG;
    }
    const size_t buffer_bytes = static_cast<size_t>(rows) * static_cast<size_t>(buffer_cols) * 2;
    if (input == nullptr || residual == nullptr || weight == nullptr || output == nullptr ||
        (out_kind != HFRK_OUT_SAME && scale_dev == nullptr) || (buffer_bytes != 0 && next_buffer == nullptr)) {
        set_last_error("residual_rms: null pointer");
        return HFRK_INVALID_CONFIG;
    }
    const uintptr_t all16 = reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(residual) |
                            reinterpret_cast<uintptr_t>(weight);
    if ((all16 & 1u) || (reinterpret_cast<uintptr_t>(next_buffer) & 1u) ||
        (out_kind == HFRK_OUT_SAME && (reinterpret_cast<uintptr_t>(output) & 1u))) {
        set_last_error("residual_rms: 16-bit tensors must be 2-byte aligned");
        return HFRK_BAD_ALIGNMENT;
    }
    const uintptr_t out_mask = out_kind == HFRK_OUT_SAME ? 15u : 7u;
    const bool vec = !force_scalar && cols % 8 == 0 && (all16 & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(output) & out_mask) == 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int out_mode = out_kind == HFRK_OUT_SAME ? kOutSame : (out_kind == HFRK_OUT_E4M3FN ? kOutFn : kOutFnuz);
    if (dtype == HFRK_F16)
        return dispatch_out<__half>(out_mode, input, residual, weight, scale_dev, epsilon, output, next_buffer,
                                    buffer_bytes, rows, cols, vec, num_threads, s);
    return dispatch_out<__nv_bfloat16>(out_mode, input, residual, weight, scale_dev, epsilon, output, next_buffer,
                                       buffer_bytes, rows, cols, vec, num_threads, s);
}
