// Plain SIMT kernel for D <- D_in + scale * A * W^T with fp8 e4m3 operands: one warp per output
// column n, lanes stride over K in 16-byte pieces, fp32 FMAs, a warp-shuffle reduction. No TMA,
// no tensor cores, no shared memory. It is a diagnostic: it lets a wrong result of the tcgen05
// kernel be bisected (pipeline vs descriptors vs epilogue) and cross-checks full-size shapes on
// the device. hfrk_skinny_gemm_fp8 never dispatches to it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hfrk_b200.h"
#include "host_common.h"

namespace hfrk {
namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t packed) {
    const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(packed), __NV_E4M3);
    return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

__device__ __forceinline__ void unpack16(const uint4& raw, float (&out)[16]) {
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 lo = e4m3x2_to_float2(static_cast<uint16_t>(words[i] & 0xffffu));
        const float2 hi = e4m3x2_to_float2(static_cast<uint16_t>(words[i] >> 16));
        out[4 * i + 0] = lo.x;
        out[4 * i + 1] = lo.y;
        out[4 * i + 2] = hi.x;
        out[4 * i + 3] = hi.y;
    }
}

template <int MT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
skinny_gemm_fp8_simt_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ W, void* D,
                            const float* __restrict__ scale_dev, float kind_factor, int m, int n, int k,
                            int64_t w_row_stride, int d_dtype, int accumulate) {
    const int lane = threadIdx.x & 31;
    const int col = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (col >= n) return;
    const uint8_t* w_row = W + static_cast<size_t>(col) * w_row_stride;
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.0f;

    for (int kk = lane * 16; kk < k; kk += 32 * 16) {
        float wv[16];
        unpack16(*reinterpret_cast<const uint4*>(w_row + kk), wv);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            if (i < m) {
                float av[16];
                unpack16(__ldg(reinterpret_cast<const uint4*>(A + static_cast<size_t>(i) * k + kk)), av);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[i] = fmaf(av[j], wv[j], acc[i]);
            }
        }
    }
    const float scale = __ldg(scale_dev) * kind_factor;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        float v = acc[i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0 && i < m) {
            const size_t idx = static_cast<size_t>(i) * n + col;
            float d_in = 0.0f;
            if (accumulate) {
                d_in = d_dtype == HFRK_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(D)[idx])
                                            : __half2float(static_cast<const __half*>(D)[idx]);
            }
            const float out = fmaf(v, scale, d_in);
            if (d_dtype == HFRK_BF16) {
                static_cast<__nv_bfloat16*>(D)[idx] = __float2bfloat16_rn(out);
            } else {
                static_cast<__half*>(D)[idx] = __float2half_rn(out);
            }
        }
    }
}

}  // namespace
}  // namespace hfrk

extern "C" int hfrk_skinny_gemm_fp8_simt(const void* A, const void* W, void* D, const float* scale_dev, int m,
                                         int n, int k, int64_t w_row_stride, int a_kind, int w_kind, int d_dtype,
                                         int accumulate, void* stream) {
    using namespace hfrk;
    if (A == nullptr || W == nullptr || D == nullptr || scale_dev == nullptr || m <= 0 || n <= 0 || k <= 0)
        return HFRK_INVALID_CONFIG;
    if ((a_kind != HFRK_E4M3FN && a_kind != HFRK_E4M3FNUZ) || (w_kind != HFRK_E4M3FN && w_kind != HFRK_E4M3FNUZ) ||
        (d_dtype != HFRK_F16 && d_dtype != HFRK_BF16))
        return HFRK_BAD_DTYPE;  // the diagnostic kernel has no fp32 output
    if (k % 16 != 0) return HFRK_K_NOT_DIVISIBLE;
    if (w_row_stride < k || w_row_stride % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15u) ||
        (reinterpret_cast<uintptr_t>(W) & 15u))
        return HFRK_BAD_ALIGNMENT;
    const float kind_factor = (a_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f) * (w_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid(static_cast<unsigned>((n + kWarpsPerBlock - 1) / kWarpsPerBlock));
    const dim3 block(kWarpsPerBlock * 32);
    constexpr int kChunk = 8;
    for (int m0 = 0; m0 < m; m0 += kChunk) {
        const int mc = m - m0 < kChunk ? m - m0 : kChunk;
        const uint8_t* a_chunk = static_cast<const uint8_t*>(A) + static_cast<size_t>(m0) * k;
        uint8_t* d_chunk = static_cast<uint8_t*>(D) + static_cast<size_t>(m0) * n * 2;
        if (mc == 1) {
            skinny_gemm_fp8_simt_kernel<1><<<grid, block, 0, s>>>(a_chunk, static_cast<const uint8_t*>(W), d_chunk,
                                                                 scale_dev, kind_factor, mc, n, k, w_row_stride,
                                                                 d_dtype, accumulate);
        } else {
            skinny_gemm_fp8_simt_kernel<kChunk><<<grid, block, 0, s>>>(a_chunk, static_cast<const uint8_t*>(W),
                                                                      d_chunk, scale_dev, kind_factor, mc, n, k,
                                                                      w_row_stride, d_dtype, accumulate);
        }
        HFRK_CUDA_TRY(cudaGetLastError());
    }
    return HFRK_SUCCESS;
}
