// Constants and small device helpers shared by the two kernels of the FP8 skinny GEMM (the
// cluster split-K kernel and the stream-K kernel): tile geometry, the bounded mbarrier wait, the
// device status word and the fp16/bf16 output accessors.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/hfrk_b200.h"
#include "ptx_sm100.cuh"

namespace hfrk {

constexpr int kTileN = 128;                        // W rows per CTA  (tcgen05.mma M)
constexpr int kBlockK = 128;                       // fp8 elements per stage row = one swizzle atom
constexpr int kUmmaK = 32;                         // K of one tcgen05.mma for 8-bit operands
constexpr int kWStageBytes = kTileN * kBlockK;     // 16 KiB of W per stage
constexpr int kMaxStages = 12;
constexpr int kThreads = 192;                      // 4 epilogue warps + producer warp + MMA warp
constexpr int kEpilogueThreads = 128;
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kMaxMPad = 64;                       // tokens per launch (larger M loops on the host)
constexpr int kMaxSplit = 16;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kNumSms = 148;
constexpr int kCtrlBytes = 256;                     // shared-memory control block after the ring
constexpr long long kWaitLimitCycles = 4000000000LL;  // about two seconds of SM clock

enum Role : int { kRoleProducer = 1, kRoleMma = 2, kRoleEpilogue = 3, kRolePeer = 4 };

// Device-side status of this library on the current device. Written only when a bounded wait
// runs out; read and cleared by hfrk_device_status().
__device__ unsigned int g_device_status = 0;

__device__ __forceinline__ void record_timeout(int role) {
    const unsigned int word = (static_cast<unsigned int>(HFRK_DEVICE_TIMEOUT) << 24) |
                              (static_cast<unsigned int>(role) << 16) | (blockIdx.x & 0xffffu);
    atomicCAS(&g_device_status, 0u, word);
}

__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                            int role) {
    const long long start = clock64();
    for (;;) {
        for (int i = 0; i < 32; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (*abort_flag) return false;
        if (clock64() - start > kWaitLimitCycles) {
            *abort_flag = 1u;
            record_timeout(role);
            return false;
        }
    }
}

// Waits for the phase with the given parity to complete; false if the wait ran out or another
// role of this CTA already gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  int role) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, role);
}

__device__ __forceinline__ float load_out(const void* d, size_t idx, int dtype) {
    if (dtype == HFRK_F32) return static_cast<const float*>(d)[idx];
    return dtype == HFRK_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(d)[idx])
                              : __half2float(static_cast<const __half*>(d)[idx]);
}

__device__ __forceinline__ void store_out(void* d, size_t idx, int dtype, float v) {
    if (dtype == HFRK_F32) {
        static_cast<float*>(d)[idx] = v;
    } else if (dtype == HFRK_BF16) {
        static_cast<__nv_bfloat16*>(d)[idx] = __float2bfloat16_rn(v);
    } else {
        static_cast<__half*>(d)[idx] = __float2half_rn(v);
    }
}

}  // namespace hfrk
