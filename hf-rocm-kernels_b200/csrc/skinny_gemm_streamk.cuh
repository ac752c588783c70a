// Stream-K form of the FP8 skinny GEMM for B200 (sm_100a).
//
// Measurements that shaped it (B200, 148 SMs, one 128-row x 128-byte TMA box per K block):
//   * one CTA per SM cannot pull more than ~40 GB/s of weights, and HBM only saturates when every
//     SM streams, two CTAs each. A grid of (N/128 tiles) x (cluster split) CTAs leaves SMs idle
//     for most projection shapes.
//   * one thread can issue a tcgen05.mma (M=128, K=32) every ~64 cycles and a tcgen05.commit costs
//     ~110 more, so a stage carries two K blocks (eight MMAs) per commit.
// Hence: the (tile, K block) work items of the whole problem are laid out in one line and cut into
// equal contiguous ranges, one per CTA, with the grid sized to the SM count. A CTA's range may
// start and end inside a tile; such partial tiles are written as fp32 partials to a scratch buffer
// and the LAST contributor to arrive (an atomic counter per tile) adds them in CTA order, applies
// the scale and D_in and writes D. No CTA ever waits for another one, the sum order is fixed, and
// the counters reset themselves, so the result is deterministic and the scratch needs no memset
// between calls.
//
// Pipeline per CTA: warp 4 lane 0 = TMA producer (W boxes with an evict-first L2 policy, A boxes
// evict-last), warp 5 lane 0 = MMA issuer into one of two TMEM accumulators, warps 0-3 = epilogue
// (tcgen05.ld, direct store or partial + fix-up). All mbarrier waits are bounded.
// Programmatic dependent launch: W loads start before griddepcontrol.wait; A, D, the scratch and
// the counters are only touched after it.
//
// In the reference's terms this replaces csrc/op_src/skinny_gemm/skinny_gemm_kernel.cu:34-58 (the
// persistent tile loop with its split_k decomposition), producers/*.cu, consumers/*.cu and the
// atomic fp16 epilogue (consumers/mfma_16x16x32_consumer.cu:113-168).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "skinny_gemm_common.cuh"

namespace hfrk {

constexpr int kSkMaxStages = 12;
constexpr int kSkEpilogueBarrier = 1;   // named barrier id of the four epilogue warps

struct SkCtrl {
    uint64_t full[kSkMaxStages];
    uint64_t empty[kSkMaxStages];
    uint64_t acc_full[2];     // MMA -> epilogue : accumulator buffer complete
    uint64_t acc_empty[2];    // epilogue -> MMA : accumulator buffer drained (4 arrivals, one per warp)
    uint32_t tmem_base;
    volatile uint32_t abort;
    volatile uint32_t fix_old; // counter value seen by this CTA's arrival on the current tile
};
static_assert(sizeof(SkCtrl) <= kCtrlBytes, "control block grew");

struct SkParams {
    void* d;
    const float* scale;
    float kind_factor;
    int m, n;
    int m_pad;
    int nkb;             // K blocks per tile
    int total_units;     // tiles * nkb
    int stages;
    int d_dtype;
    int accumulate;
    float* partials;         // [2 * grid][m_pad][128] fp32
    unsigned int* counters;  // [tiles], zero between launches
    unsigned long long* stamps;
};

__device__ __forceinline__ void sk_stamp(const SkParams& p, int slot) {
    if (p.stamps != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.stamps[static_cast<size_t>(blockIdx.x) * 8 + slot] = t;
    }
}

// First unit of CTA g when `total` units are cut into `grid` contiguous ranges.
__device__ __forceinline__ int sk_range_begin(int g, int total, int grid) {
    return static_cast<int>(static_cast<long long>(g) * total / grid);
}

// The CTA whose range holds unit u.
__device__ __forceinline__ int sk_owner(int u, int total, int grid) {
    return static_cast<int>((static_cast<long long>(u + 1) * grid - 1) / total);
}

__device__ __forceinline__ bool sk_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, int role) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) {
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

// AND of a predicate over the 128 epilogue threads (named barrier with reduction).
__device__ __forceinline__ bool epilogue_all(bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t"
        ".reg .pred pin, pout;\n\t"
        "setp.ne.u32 pin, %1, 0;\n\t"
        "barrier.cta.red.and.pred pout, %2, %3, pin;\n\t"
        "selp.u32 %0, 1, 0, pout;\n\t"
        "}\n"
        : "=r"(out)
        : "r"(pred ? 1u : 0u), "r"(kSkEpilogueBarrier), "r"(kEpilogueThreads)
        : "memory");
    return out != 0;
}

// UPS = K blocks (128 bytes of K each) per pipeline stage: 2 halves the number of commits and
// barrier round trips of the single MMA-issuing thread, 1 keeps more, smaller stages in flight.
template <int UPS>
__global__ void __launch_bounds__(kThreads)
skinny_gemm_fp8_streamk_kernel(const __grid_constant__ CUtensorMap tmap_w,
                               const __grid_constant__ CUtensorMap tmap_a, const SkParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t ring_addr = (raw_addr + 1023u) & ~1023u;
    uint8_t* const ring_ptr = smem_raw + (ring_addr - raw_addr);
    const uint32_t a_bytes = static_cast<uint32_t>(p.m_pad) * kBlockK;
    const uint32_t unit_bytes = kWStageBytes + a_bytes;
    const uint32_t stage_bytes = UPS * unit_bytes;
    const uint32_t a_offset = UPS * kWStageBytes;  // A boxes follow the W boxes of a stage
    SkCtrl* const ctrl = reinterpret_cast<SkCtrl*>(ring_ptr + static_cast<size_t>(p.stages) * stage_bytes);
    const uint32_t full_bar = smem_u32(&ctrl->full[0]);
    const uint32_t empty_bar = smem_u32(&ctrl->empty[0]);
    const uint32_t acc_full_bar = smem_u32(&ctrl->acc_full[0]);
    const uint32_t acc_empty_bar = smem_u32(&ctrl->acc_empty[0]);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int grid = static_cast<int>(gridDim.x);
    const int g = static_cast<int>(blockIdx.x);
    const int u_begin = sk_range_begin(g, p.total_units, grid);
    const int u_end = sk_range_begin(g + 1, p.total_units, grid);
    const int my_units = u_end - u_begin;
    const int my_stages = (my_units + UPS - 1) / UPS;
    const uint32_t tmem_cols = p.m_pad <= 16 ? 32u : (p.m_pad <= 32 ? 64u : 128u);
    if (threadIdx.x == 0) sk_stamp(p, 0);

    // ---- set-up: the producer initialises the barriers and starts streaming at once; the other
    // warps meet it on a named barrier it only arrives at (it never blocks there).
    if (warp == kProducerWarp) {
        if (lane == 0) {
            ctrl->abort = 0u;
            for (int s = 0; s < p.stages; ++s) {
                mbar_init(full_bar + 8u * s, 1);
                mbar_init(empty_bar + 8u * s, 1);
            }
            for (int b = 0; b < 2; ++b) {
                mbar_init(acc_full_bar + 8u * b, 1);
                mbar_init(acc_empty_bar + 8u * b, kEpilogueThreads / 32);
            }
            mbar_init_fence();
        }
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"r"(kThreads) : "memory");
    } else {
        if (warp == kMmaWarp) {
            tmem_alloc(smem_u32(&ctrl->tmem_base), tmem_cols);
            tmem_relinquish_alloc_permit();
            tcgen05_fence_before_sync();
        }
        asm volatile("bar.sync 2, %0;" ::"r"(kThreads) : "memory");
        tcgen05_fence_after_sync();
    }
    pdl_launch_dependents();

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && my_units > 0) {
            prefetch_tensormap(&tmap_w);
            prefetch_tensormap(&tmap_a);
            const uint64_t pol_w = l2_policy_evict_first();
            const uint64_t pol_a = l2_policy_evict_last();
            const int prologue = my_stages < p.stages ? my_stages : p.stages;
            // Weights first: they do not depend on the previous kernel of the stream.
            for (int i = 0; i < prologue; ++i) {
                const int u0 = u_begin + i * UPS;
                const int cnt = u_end - u0 < UPS ? u_end - u0 : UPS;
                mbar_arrive_expect_tx(full_bar + 8u * i, cnt * unit_bytes);
                for (int j = 0; j < cnt; ++j) {
                    const int tile = (u0 + j) / p.nkb;
                    const int kb = (u0 + j) - tile * p.nkb;
                    tma_load_2d(ring_addr + i * stage_bytes + j * kWStageBytes, &tmap_w, full_bar + 8u * i,
                                kb * kBlockK, tile * kTileN, pol_w);
                }
            }
            pdl_wait_prior_grids();
            for (int i = 0; i < prologue; ++i) {
                const int u0 = u_begin + i * UPS;
                const int cnt = u_end - u0 < UPS ? u_end - u0 : UPS;
                for (int j = 0; j < cnt; ++j) {
                    const int kb = (u0 + j) % p.nkb;
                    tma_load_2d(ring_addr + i * stage_bytes + a_offset + j * a_bytes, &tmap_a, full_bar + 8u * i,
                                kb * kBlockK, 0, pol_a);
                }
            }
            sk_stamp(p, 2);
            int issued = prologue;
            for (int i = prologue; i < my_stages; ++i) {
                const int s = i % p.stages;
                const uint32_t round = static_cast<uint32_t>(i / p.stages);
                if (!sk_wait(empty_bar + 8u * s, (round - 1u) & 1u, &ctrl->abort, kRoleProducer)) break;
                const int u0 = u_begin + i * UPS;
                const int cnt = u_end - u0 < UPS ? u_end - u0 : UPS;
                mbar_arrive_expect_tx(full_bar + 8u * s, cnt * unit_bytes);
                for (int j = 0; j < cnt; ++j) {
                    const int tile = (u0 + j) / p.nkb;
                    const int kb = (u0 + j) - tile * p.nkb;
                    tma_load_2d(ring_addr + s * stage_bytes + j * kWStageBytes, &tmap_w, full_bar + 8u * s,
                                kb * kBlockK, tile * kTileN, pol_w);
                    tma_load_2d(ring_addr + s * stage_bytes + a_offset + j * a_bytes, &tmap_a, full_bar + 8u * s,
                                kb * kBlockK, 0, pol_a);
                }
                issued = i + 1;
            }
            if (ctrl->abort) {
                // Give copies already in flight a bounded chance to land before the CTA exits.
                for (int s = 0; s < p.stages && s < issued; ++s) {
                    const int last = ((issued - 1 - s) / p.stages) * p.stages + s;
                    const uint32_t parity = static_cast<uint32_t>(last / p.stages) & 1u;
                    const long long start = clock64();
                    while (!mbar_try_wait(full_bar + 8u * s, parity)) {
                        if (clock64() - start > kWaitLimitCycles / 8) break;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && my_units > 0) {
            const uint32_t tmem_acc = ctrl->tmem_base;
            const uint32_t idesc = umma_idesc_e4m3_f32(kTileN, p.m_pad);
            int u = u_begin;
            int seg = 0;
            bool alive = true;
            while (u < u_end && alive) {
                const int tile = u / p.nkb;
                const int kb0 = u - tile * p.nkb;
                const int cnt = (u_end - u) < (p.nkb - kb0) ? (u_end - u) : (p.nkb - kb0);
                const uint32_t buf = static_cast<uint32_t>(seg & 1);
                if (seg >= 2) {
                    const uint32_t use = static_cast<uint32_t>(seg >> 1);
                    if (!sk_wait(acc_empty_bar + 8u * buf, (use - 1u) & 1u, &ctrl->abort, kRoleMma)) break;
                    tcgen05_fence_after_sync();
                }
                const uint32_t d_tmem = tmem_acc + buf * static_cast<uint32_t>(p.m_pad);
                for (int c = 0; c < cnt; ++c) {
                    const int q = (u + c) - u_begin;
                    const int i = q / UPS;
                    const int j = q - i * UPS;
                    const int s = i % p.stages;
                    if (j == 0 || c == 0) {
                        // first touch of this stage by this segment; a stage shared by two segments is
                        // waited for twice, the second wait returns at once
                        const uint32_t round = static_cast<uint32_t>(i / p.stages);
                        if (!sk_wait(full_bar + 8u * s, round & 1u, &ctrl->abort, kRoleMma)) {
                            alive = false;
                            break;
                        }
                        tcgen05_fence_after_sync();
                        if (q == 0) sk_stamp(p, 3);
                    }
                    const uint64_t w_desc = umma_desc_kmajor_sw128(ring_addr + s * stage_bytes + j * kWStageBytes);
                    const uint64_t a_desc = umma_desc_kmajor_sw128(ring_addr + s * stage_bytes + a_offset + j * a_bytes);
#pragma unroll
                    for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                        umma_f8f6f4(d_tmem, w_desc + 2u * kk, a_desc + 2u * kk, idesc, (c | kk) != 0 ? 1u : 0u);
                    }
                    if (j == UPS - 1 || q == my_units - 1) umma_commit(empty_bar + 8u * s);
                }
                if (!alive) break;
                umma_commit(acc_full_bar + 8u * buf);
                u += cnt;
                ++seg;
            }
            sk_stamp(p, 4);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 0..3)
        if (my_units > 0) {
            pdl_wait_prior_grids();
            const uint32_t tmem_acc = ctrl->tmem_base;
            const int nl = static_cast<int>(threadIdx.x);  // TMEM lane = W row inside the tile
            const float scale = __ldg(p.scale) * p.kind_factor;
            const size_t slot_floats = static_cast<size_t>(p.m_pad) * kTileN;
            int u = u_begin;
            int seg = 0;
            while (u < u_end) {
                const int tile = u / p.nkb;
                const int kb0 = u - tile * p.nkb;
                const int cnt = (u_end - u) < (p.nkb - kb0) ? (u_end - u) : (p.nkb - kb0);
                const uint32_t buf = static_cast<uint32_t>(seg & 1);
                const uint32_t use = static_cast<uint32_t>(seg >> 1);
                const bool whole = cnt == p.nkb;
                const int n = tile * kTileN + nl;
                // partial tiles: slot 0 of this CTA for a tile it begins in, slot 1 for the tile it ends in
                float* const slot = p.partials + (static_cast<size_t>(g) * 2 + (seg == 0 ? 0 : 1)) * slot_floats;

                // The four warps must agree on giving up, or one would leave the others at a barrier.
                const bool landed = sk_wait(acc_full_bar + 8u * buf, use & 1u, &ctrl->abort, kRoleEpilogue);
                if (!epilogue_all(landed)) break;
                tcgen05_fence_after_sync();
                const uint32_t lane_taddr = tmem_acc + buf * static_cast<uint32_t>(p.m_pad) +
                                            (static_cast<uint32_t>(warp * 32) << 16);
                for (int c = 0; c < p.m_pad / 16; ++c) {
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(lane_taddr + static_cast<uint32_t>(c * 16), v);
                    tmem_ld_wait();
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = c * 16 + j;
                            if (m < p.m && n < p.n) {
                                const size_t idx = static_cast<size_t>(m) * p.n + n;
                                const float d_in = p.accumulate ? load_out(p.d, idx, p.d_dtype) : 0.0f;
                                store_out(p.d, idx, p.d_dtype, fmaf(__uint_as_float(v[j]), scale, d_in));
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = c * 16 + j;
                            if (m < p.m) slot[static_cast<size_t>(m) * kTileN + nl] = __uint_as_float(v[j]);
                        }
                    }
                }
                // The accumulator buffer is free again as soon as the loads above have completed.
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty_bar + 8u * buf) : "memory");
                }

                const bool final_seg = u + cnt == u_end;
                if (final_seg && threadIdx.x == 0) sk_stamp(p, 1);
                if (!whole) {
                    // Fix-up: publish the partial, count the arrival, and let the last arriver reduce.
                    const int g_lo = sk_owner(tile * p.nkb, p.total_units, grid);
                    const int g_hi = sk_owner(tile * p.nkb + p.nkb - 1, p.total_units, grid);
                    __threadfence();
                    asm volatile("bar.sync %0, %1;" ::"r"(kSkEpilogueBarrier), "r"(kEpilogueThreads) : "memory");
                    if (threadIdx.x == 0) ctrl->fix_old = atomicAdd(&p.counters[tile], 1u);
                    asm volatile("bar.sync %0, %1;" ::"r"(kSkEpilogueBarrier), "r"(kEpilogueThreads) : "memory");
                    const bool last = ctrl->fix_old == static_cast<uint32_t>(g_hi - g_lo);
                    if (final_seg && threadIdx.x == 0) sk_stamp(p, 5);
                    if (last) {
                        __threadfence();
                        if (n < p.n) {
                            // Sum the contributors in CTA order. Loads are issued in batches (16 tokens x
                            // up to 4 contributors) before they are consumed, so a tile costs a few L2
                            // round trips instead of one per value.
                            for (int m0 = 0; m0 < p.m; m0 += 16) {
                                float d_in[16];
                                float sum[16];
#pragma unroll
                                for (int j = 0; j < 16; ++j) {
                                    sum[j] = 0.0f;
                                    d_in[j] = (p.accumulate && m0 + j < p.m)
                                                  ? load_out(p.d, static_cast<size_t>(m0 + j) * p.n + n, p.d_dtype)
                                                  : 0.0f;
                                }
                                for (int c0 = g_lo; c0 <= g_hi; c0 += 4) {
                                    float v[4][16];
#pragma unroll
                                    for (int b = 0; b < 4; ++b) {
                                        const int c2 = c0 + b;
                                        const int first_tile = sk_range_begin(c2, p.total_units, grid) / p.nkb;
                                        const float* src = p.partials +
                                                           (static_cast<size_t>(c2) * 2 + (first_tile == tile ? 0 : 1)) *
                                                               slot_floats +
                                                           static_cast<size_t>(m0) * kTileN + nl;
#pragma unroll
                                        for (int j = 0; j < 16; ++j) {
                                            v[b][j] = (c2 <= g_hi && m0 + j < p.m) ? __ldcg(src + j * kTileN) : 0.0f;
                                        }
                                    }
#pragma unroll
                                    for (int b = 0; b < 4; ++b) {
#pragma unroll
                                        for (int j = 0; j < 16; ++j) sum[j] += v[b][j];
                                    }
                                }
#pragma unroll
                                for (int j = 0; j < 16; ++j) {
                                    if (m0 + j < p.m) {
                                        store_out(p.d, static_cast<size_t>(m0 + j) * p.n + n, p.d_dtype,
                                                  fmaf(sum[j], scale, d_in[j]));
                                    }
                                }
                            }
                        }
                        if (threadIdx.x == 0) p.counters[tile] = 0u;  // ready for the next launch
                    }
                    // keep fix_old stable until every thread has read it
                    asm volatile("bar.sync %0, %1;" ::"r"(kSkEpilogueBarrier), "r"(kEpilogueThreads) : "memory");
                }
                u += cnt;
                ++seg;
            }
            if (threadIdx.x == 0) sk_stamp(p, 6);
        }
    }

    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) tmem_dealloc(ctrl->tmem_base, tmem_cols);
    if (threadIdx.x == 0) sk_stamp(p, 7);
}

}  // namespace hfrk
