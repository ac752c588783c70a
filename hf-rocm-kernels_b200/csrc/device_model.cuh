// What the launch planner needs to know about the GPU it plans for: the number of SMs and how many
// thread-block clusters of a given size the chip holds AT ONCE. The second figure is measured, not
// looked up: a cluster lives inside one GPC, the 148 SMs of a B200 are spread unevenly over its
// GPCs, the spread differs from chip to chip, and a grid whose clusters are not all resident at the
// same moment falls off a cliff (the late clusters start when the others leave and stream alone).
// The reference hard-codes its CU count (csrc/op_src/skinny_gemm/core.cu:24); here the device is asked.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "host_common.h"
#include "skinny_gemm_common.cuh"

namespace hfrk {

constexpr int kModelMaxSplit = 16;
constexpr int kModelMaxPerSm = 3;        // the GEMM kernel's registers allow three CTAs per SM
constexpr int kSmemPerSm = 228 * 1024;        // shared memory of one SM
constexpr int kSmemCtaReserve = 1024;         // taken by the system per resident CTA

struct DeviceModel {
    int sms = kNumSms;
    // capacity[split][per_sm]: clusters of `split` CTAs resident at once when `per_sm` CTAs fit on an SM
    int capacity[kModelMaxSplit + 1][kModelMaxPerSm + 1] = {};
    bool measured = false;
};

// Counter and failure flag of the residency probe.
__device__ unsigned int g_probe_words[2];

// Every CTA announces itself and then waits, for a bounded time, until all CTAs of the grid have
// done so. If the whole grid is resident at once the count completes within microseconds; if some
// clusters only start after others have left, the early ones run out of time and say so.
__global__ void __launch_bounds__(kThreads) residency_probe_kernel(unsigned int total, long long limit_cycles) {
    extern __shared__ uint8_t probe_smem[];
    if (threadIdx.x == 0) {
        probe_smem[0] = 0;   // the dynamic shared memory is what sets the CTAs per SM
        atomicAdd(&g_probe_words[0], 1u);
        const long long start = clock64();
        while (*reinterpret_cast<volatile unsigned int*>(&g_probe_words[0]) < total) {
            if (clock64() - start > limit_cycles) {
                atomicExch(&g_probe_words[1], 1u);
                break;
            }
        }
    }
}

namespace model_detail {

inline std::mutex& mutex() {
    static std::mutex m;
    return m;
}
inline DeviceModel* per_device() {
    static DeviceModel models[64];
    return models;
}
inline DeviceModel& override_model() {
    static DeviceModel m;
    return m;
}
inline bool& override_on() {
    static bool on = false;
    return on;
}

// True if `clusters` clusters of `split` CTAs, `per_sm` CTAs to an SM, are resident at once.
inline int probe_fits(int split, int per_sm, int clusters, cudaStream_t stream, bool* fits) {
    const unsigned int zeros[2] = {0u, 0u};
    HFRK_CUDA_TRY(cudaMemcpyToSymbolAsync(g_probe_words, zeros, sizeof(zeros), 0, cudaMemcpyHostToDevice, stream));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(clusters), static_cast<unsigned>(split), 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    // exactly per_sm CTAs of this footprint fit on an SM
    cfg.dynamicSmemBytes = static_cast<size_t>(kSmemPerSm / per_sm - kSmemCtaReserve) & ~static_cast<size_t>(127);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1;
    attr.val.clusterDim.y = static_cast<unsigned>(split);
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = split > 1 ? 1 : 0;
    const unsigned int total = static_cast<unsigned int>(clusters) * split;
    const long long limit = 100000;   // about 50 microseconds
    HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, residency_probe_kernel, total, limit));
    unsigned int words[2] = {0u, 0u};
    HFRK_CUDA_TRY(cudaMemcpyFromSymbolAsync(words, g_probe_words, sizeof(words), 0, cudaMemcpyDeviceToHost, stream));
    HFRK_CUDA_TRY(cudaStreamSynchronize(stream));
    *fits = words[1] == 0u && words[0] == total;
    return HFRK_SUCCESS;
}

inline int measure(DeviceModel* model) {
    int dev = 0;
    HFRK_CUDA_TRY(cudaGetDevice(&dev));
    HFRK_CUDA_TRY(cudaDeviceGetAttribute(&model->sms, cudaDevAttrMultiProcessorCount, dev));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(residency_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(residency_probe_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    cudaStream_t stream = nullptr;
    HFRK_CUDA_TRY(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    int rc = HFRK_SUCCESS;
    for (int per_sm = 1; per_sm <= kModelMaxPerSm && rc == HFRK_SUCCESS; ++per_sm) {
        model->capacity[1][per_sm] = model->sms * per_sm;   // no cluster, nothing to pack
        for (int split = 2; split <= kModelMaxSplit && rc == HFRK_SUCCESS; ++split) {
            // largest resident cluster count by bisection; the paper bound is all CTA slots
            int lo = 0, hi = model->sms * per_sm / split;
            while (lo < hi && rc == HFRK_SUCCESS) {
                const int mid = (lo + hi + 1) / 2;
                bool fits = false;
                rc = probe_fits(split, per_sm, mid, stream, &fits);
                if (fits) {
                    lo = mid;
                } else {
                    hi = mid - 1;
                }
            }
            model->capacity[split][per_sm] = lo;
        }
    }
    (void)cudaStreamDestroy(stream);
    model->measured = rc == HFRK_SUCCESS;
    return rc;
}

// Used while nothing could be measured (no device, or the first call came inside a stream capture,
// where nothing may be launched and waited for): what the measurements on B200 came to, rounded down.
inline void fill_estimate(DeviceModel* model) {
    for (int per_sm = 1; per_sm <= kModelMaxPerSm; ++per_sm) {
        for (int split = 1; split <= kModelMaxSplit; ++split) {
            const int slots = model->sms * per_sm / split;
            model->capacity[split][per_sm] = split == 1 ? slots : (split <= 6 ? slots * 85 / 100 : slots * 70 / 100);
        }
    }
}

}  // namespace model_detail

// The model of the current device (or the injected one). `stream` is the stream of the call that
// asks: while it is being captured into a graph nothing is measured and an estimate is returned,
// uncached, so that the next call outside a capture measures.
inline DeviceModel device_model(cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(model_detail::mutex());
    if (model_detail::override_on()) return model_detail::override_model();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        DeviceModel fallback;
        model_detail::fill_estimate(&fallback);
        return fallback;
    }
    DeviceModel& model = model_detail::per_device()[dev];
    if (model.measured) return model;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) (void)cudaGetLastError();
    DeviceModel out;
    if (capturing == cudaStreamCaptureStatusNone) {
        // other threads may be capturing in the global mode: this thread's launches and waits are its own business
        cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
        (void)cudaThreadExchangeStreamCaptureMode(&mode);
        const int rc = model_detail::measure(&model);
        (void)cudaThreadExchangeStreamCaptureMode(&mode);
        if (rc == HFRK_SUCCESS) return model;
        (void)cudaGetLastError();
    }
    (void)cudaDeviceGetAttribute(&out.sms, cudaDevAttrMultiProcessorCount, dev);
    model_detail::fill_estimate(&out);
    return out;
}

}  // namespace hfrk
