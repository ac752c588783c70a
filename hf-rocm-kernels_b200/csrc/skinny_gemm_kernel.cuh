// Device side of the FP8 skinny GEMM for B200 (sm_100a): the kernel template
// skinny_gemm_fp8_sm100_kernel<kMode> with its three instantiations (plain, row-parallel with the
// all-reduce in the epilogue, gate/up projection with swiglu in the epilogue), the parameter blocks
// it takes and the cross-GPU exchange it uses. Included by skinny_gemm_sm100.cu, which holds the
// launch planning and the C ABI. The design is described at the top of that file.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hfrk_b200.h"
#include "elementwise_common.cuh"
#include "ptx_sm100.cuh"
#include "skinny_gemm_common.cuh"

namespace hfrk {

struct Ctrl {
    uint64_t full[kMaxStages];    // TMA -> MMA : stage holds data
    uint64_t empty[kMaxStages];   // MMA -> TMA : stage may be overwritten
    uint64_t accum;               // MMA -> epilogue : accumulator complete
    uint64_t recv;                // peers -> this CTA : split-K partials landed (byte count)
    uint32_t tmem_base;
    volatile uint32_t abort;      // set by the first role whose wait ran out
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block grew");

// Row-parallel (K split over GPUs) exchange state, as seen by the kernel of ONE rank. Every rank
// owns an exchange buffer that its peers write into over NVLink:
//   cells : {fp32 value, epoch} [2 parities][world + 1 sources][elems_per_src], 8 bytes each
// A cell is written with ONE 8-byte store, so its reader sees value and epoch together: a cell
// whose epoch equals the current call's is valid. No flag, no fence and no barrier is needed
// between writer and reader. cells[p] is the base of rank p's buffer (p == rank: the local one).
// Sources 0..world-1 hold the partial sums of those ranks; source `world` holds finished sums
// sent back by the element's owner in the two-shot exchange.
constexpr int kMaxWorld = 8;
constexpr unsigned long long kTwoShotFromBytes = 1ull << 20;
struct RowparDev {
    int rank, world;
    int two_shot;               // set per launch: 0 = every rank sends its partials to every peer
    long long wait_cycles;      // how long a thread polls for a peer's cells before it gives up
    unsigned int elems_per_src;
    uint2* cells[kMaxWorld];
    unsigned int* call_index;   // local: number of completed calls on this communicator
    unsigned int* done_ctas;    // local: CTAs of the running call that have finished
};

struct GemmParams {
    void* d;
    const float* scale;
    float kind_factor;   // 0.5 per e4m3fnuz operand
    int m, n, k;
    int m_pad;           // MMA N: m rounded up to 16
    int tile_rows;       // W rows per CTA, <= 128: the MMA always covers 128 lanes, the rest is ignored
    int num_kblocks;     // ceil(k / 128)
    int split;           // CTAs per cluster along K
    int stages;
    int d_dtype;
    int accumulate;
    unsigned long long* stamps;  // optional [cta][8] globaltimer samples (diagnostic entry point only)
    RowparDev rp;                // used by the row-parallel instantiation only
    // used by the SwiGLU instantiation only: W holds act_cols gate rows followed by act_cols up rows
    uint8_t* act_out;            // [m, act_cols] fp8
    const float* act_scale;      // the activation is divided by this before the conversion to fp8
    int act_cols;
    int act_fnuz;                // 1 = write e4m3fnuz bytes, 0 = e4m3fn
    uint8_t* zero_ptr;           // buffer the next GEMM accumulates into, zeroed by this grid
    unsigned long long zero_bytes;
};

static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block grew");

__device__ __forceinline__ void stamp(const GemmParams& p, int slot) {
    if (p.stamps != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.stamps[(static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 8 + slot] = t;
    }
}


// ---------------------------------------------------------------- cross-GPU exchange (row-parallel)
__device__ __forceinline__ void st_relaxed_sys_v2(uint2* ptr, uint32_t x, uint32_t y) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(ptr), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const uint2* ptr) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr) : "memory");
    return v;
}

// All-reduce of the values this thread owns, fused into the GEMM epilogue. `val` holds CNT partial
// sums, `slot[i]` the element's index in the exchange buffer (0xffffffff = unused). All ranks run
// the same launch shape, so "this thread's element i" names the same output element on every rank.
//
// One-shot (rp.two_shot == 0): the thread writes {value, epoch} cells into every peer's buffer
// (plain 8-byte stores to peer memory: NVLink), then polls the matching cells of its own buffer
// until each carries this call's epoch, and adds the `world` contributions in rank order. One
// NVLink crossing of latency; every rank sends (world - 1) copies of its partial tile.
//
// Two-shot (rp.two_shot != 0): each CTA position has an owner rank. The other ranks send their
// partials to the owner only; the owner adds them in rank order and sends the finished sum to
// every peer. Two crossings of latency, but 1/world of the one-shot's traffic for the partials
// plus one copy of the result: the better trade once the partial tiles reach megabytes.
//
// Either way all ranks end with bit-identical sums. Nothing here synchronises the CTA; every wait
// is bounded. Returns false if a peer did not deliver in time (the status word is set).
template <int CNT>
__device__ __forceinline__ bool rowpar_exchange(const RowparDev& rp, unsigned int epoch, const uint32_t (&slot)[CNT],
                                                float (&val)[CNT], volatile uint32_t* abort_flag) {
    const unsigned int parity = epoch & 1u;
    const size_t sources = static_cast<size_t>(rp.world) + 1;
    const int owner = rp.two_shot ? static_cast<int>((blockIdx.x + blockIdx.y) % static_cast<unsigned>(rp.world)) : -1;
    const bool gather = !rp.two_shot || owner == rp.rank;   // this thread adds up the ranks' partials
    const size_t my_src = parity * sources + static_cast<size_t>(rp.rank);
    for (int peer = 0; peer < rp.world; ++peer) {
        if (peer == rp.rank || (rp.two_shot && peer != owner)) continue;
        uint2* dst = rp.cells[peer] + my_src * rp.elems_per_src;
#pragma unroll
        for (int i = 0; i < CNT; ++i) {
            if (slot[i] != 0xffffffffu) st_relaxed_sys_v2(dst + slot[i], __float_as_uint(val[i]), epoch);
        }
    }
    // Cells are fetched a batch at a time (4 elements x up to 7 peers in flight per thread) and the
    // batch is re-read until every cell shows the epoch; batches of unused elements are skipped,
    // which is the common case: a thread usually owns two or three elements of the tile.
    constexpr int kBatch = 4;
    bool ok = true;
    const long long start = clock64();
    const uint2* const mine = rp.cells[rp.rank] + parity * sources * rp.elems_per_src;
#pragma unroll
    for (int i0 = 0; i0 < CNT; i0 += kBatch) {
        bool any = false;
#pragma unroll
        for (int b = 0; b < kBatch; ++b) any |= slot[i0 + b] != 0xffffffffu;
        if (!any || !ok) continue;
        if (gather) {
            uint32_t got[kBatch][kMaxWorld];
            for (;;) {
                bool ready = true;
#pragma unroll
                for (int b = 0; b < kBatch; ++b) {
#pragma unroll
                    for (int src = 0; src < kMaxWorld; ++src) {
                        got[b][src] = 0u;
                        if (src < rp.world && src != rp.rank && slot[i0 + b] != 0xffffffffu) {
                            const uint2 cell =
                                ld_relaxed_sys_v2(mine + static_cast<size_t>(src) * rp.elems_per_src + slot[i0 + b]);
                            got[b][src] = cell.x;
                            ready &= cell.y == epoch;
                        }
                    }
                }
                if (ready) break;
                if (*abort_flag || clock64() - start > rp.wait_cycles) {
                    *abort_flag = 1u;
                    record_timeout(kRolePeer);
                    ok = false;
                    break;
                }
            }
            if (!ok) continue;
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                float sum = 0.0f;
#pragma unroll
                for (int src = 0; src < kMaxWorld; ++src) {
                    if (src < rp.world) sum += (src == rp.rank) ? val[i0 + b] : __uint_as_float(got[b][src]);
                }
                val[i0 + b] = sum;
            }
            if (rp.two_shot) {
                // the owner hands the finished sums to everyone else
                const size_t fin = (parity * sources + static_cast<size_t>(rp.world)) * rp.elems_per_src;
                for (int peer = 0; peer < rp.world; ++peer) {
                    if (peer == rp.rank) continue;
#pragma unroll
                    for (int b = 0; b < kBatch; ++b) {
                        if (slot[i0 + b] != 0xffffffffu)
                            st_relaxed_sys_v2(rp.cells[peer] + fin + slot[i0 + b], __float_as_uint(val[i0 + b]), epoch);
                    }
                }
            }
        } else {
            // not the owner: wait for the finished sums
            const uint2* const fin = mine + static_cast<size_t>(rp.world) * rp.elems_per_src;
            uint32_t got[kBatch];
            for (;;) {
                bool ready = true;
#pragma unroll
                for (int b = 0; b < kBatch; ++b) {
                    got[b] = 0u;
                    if (slot[i0 + b] != 0xffffffffu) {
                        const uint2 cell = ld_relaxed_sys_v2(fin + slot[i0 + b]);
                        got[b] = cell.x;
                        ready &= cell.y == epoch;
                    }
                }
                if (ready) break;
                if (*abort_flag || clock64() - start > rp.wait_cycles) {
                    *abort_flag = 1u;
                    record_timeout(kRolePeer);
                    ok = false;
                    break;
                }
            }
            if (!ok) continue;
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                if (slot[i0 + b] != 0xffffffffu) val[i0 + b] = __uint_as_float(got[b]);
            }
        }
    }
    return ok;
}

// Instantiations of the kernel.
//   kModePlain  : D <- D_in + scale * A.W^T
//   kModeRowPar : the epilogue all-reduces the tile over the ranks of a row-parallel group before D is written
//   kModeSwiglu : W is a gate/up projection; a CTA's tile is 64 gate rows plus the matching 64 up rows,
//                 and the epilogue writes fp8(silu(gate) * up / act_scale) instead of the projection
//                 (m <= 16: the host guarantees it; with a K split every CTA of the cluster ends up
//                 with whole token rows of the tile, so the two halves of a column still meet)
constexpr int kModePlain = 0;
constexpr int kModeRowPar = 1;
constexpr int kModeSwiglu = 2;
constexpr int kHalfTile = kTileN / 2;
constexpr int kAutoTileRowsOff = -1;   // make_plan: keep 128-row tiles (callers whose layout depends on them)

__device__ __forceinline__ float round_trip_16(float x, int dtype) {
    return dtype == HFRK_BF16 ? __bfloat162float(__float2bfloat16_rn(x)) : __half2float(__float2half_rn(x));
}

template <int kMode>
__global__ void __launch_bounds__(kThreads, 2)
skinny_gemm_fp8_sm100_kernel(const __grid_constant__ CUtensorMap tmap_w,
                             const __grid_constant__ CUtensorMap tmap_a, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // The swizzled operand tiles need 1024-byte alignment; dynamic shared memory only promises 16.
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t ring_addr = (raw_addr + 1023u) & ~1023u;
    uint8_t* const ring_ptr = smem_raw + (ring_addr - raw_addr);
    const uint32_t a_bytes = static_cast<uint32_t>(p.m_pad) * kBlockK;
    const uint32_t stage_bytes = kWStageBytes + a_bytes;
    // Bytes that land per stage: a W box of tile_rows rows (rows beyond it keep stale shared memory;
    // their accumulator lanes are never stored) and the activations.
    const uint32_t stage_tx = static_cast<uint32_t>(p.tile_rows) * kBlockK + a_bytes;
    Ctrl* const ctrl = reinterpret_cast<Ctrl*>(ring_ptr + static_cast<size_t>(p.stages) * stage_bytes);
    const uint32_t full_bar = smem_u32(&ctrl->full[0]);
    const uint32_t empty_bar = smem_u32(&ctrl->empty[0]);
    const uint32_t accum_bar = smem_u32(&ctrl->accum);
    const uint32_t recv_bar = smem_u32(&ctrl->recv);
    // Split-K reduction geometry: the m x 128 tile is cut into `split` element ranges of `chunk`
    // floats (a multiple of 4, so that every range is a 16-byte-aligned bulk copy).
    const int total = p.m * kTileN;
    // SwiGLU: a range is whole token rows of the tile (ceil(m / split) of them), so that the gate
    // half and the up half of a column always meet in the same CTA.
    const uint32_t chunk = kMode == kModeSwiglu
                               ? static_cast<uint32_t>(kTileN) * ((static_cast<uint32_t>(p.m) + p.split - 1) / p.split)
                               : ((static_cast<uint32_t>(total) + p.split - 1) / p.split + 3u) & ~3u;

    constexpr bool kRowPar = kMode == kModeRowPar;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * p.tile_rows;
    if (threadIdx.x == 0) stamp(p, 0);
    // One stage of W: a 128-row box, or (SwiGLU) the CTA's 64 gate rows and its 64 up rows, which
    // land one after the other in the same 16 KiB and look like one 128-row tile to the MMA.
    auto load_w = [&](uint32_t dst, uint32_t bar, int k_coord, uint64_t policy) {
        if (kMode == kModeSwiglu) {
            const int g0 = static_cast<int>(blockIdx.x) * kHalfTile;
            tma_load_2d(dst, &tmap_w, bar, k_coord, g0, policy);
            tma_load_2d(dst + kWStageBytes / 2, &tmap_w, bar, k_coord, p.act_cols + g0, policy);
        } else {
            tma_load_2d(dst, &tmap_w, bar, k_coord, n0, policy);
        }
    };

    // K blocks of this CTA: a contiguous range, the remainder spread over the first ranks.
    const int rank = p.split > 1 ? static_cast<int>(cluster_cta_rank()) : 0;
    const int kb_base = p.num_kblocks / p.split;
    const int kb_rem = p.num_kblocks % p.split;
    const int kb_count = kb_base + (rank < kb_rem ? 1 : 0);
    const int kb_start = rank * kb_base + (rank < kb_rem ? rank : kb_rem);
    const int prologue = kb_count < p.stages ? kb_count : p.stages;

    const uint32_t tmem_cols = p.m_pad <= 32 ? 32u : 64u;
    uint64_t pol_w = 0, pol_a = 0;

    // Set-up: the producer initialises the barriers, signals the other warps through a named
    // barrier it only arrives at, and goes straight on to the first loads.
    if (warp == kProducerWarp) {
        if (lane == 0) {
            ctrl->abort = 0u;
            for (int s = 0; s < p.stages; ++s) {
                mbar_init(full_bar + 8u * s, 1);
                mbar_init(empty_bar + 8u * s, 1);
            }
            mbar_init(accum_bar, 1);
            mbar_init(recv_bar, 1);
            mbar_init_fence();
            if (p.split > 1) mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>(p.split) * chunk * 4u);
        }
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"r"(kThreads) : "memory");
        if (lane == 0) {
            prefetch_tensormap(&tmap_w);
            prefetch_tensormap(&tmap_a);
            pol_w = l2_policy_evict_first();
            pol_a = l2_policy_evict_last();
            // Start the weight stream before anything else in the CTA is ready: W does not depend
            // on the previous kernel, A does.
            for (int i = 0; i < prologue; ++i) {
                mbar_arrive_expect_tx(full_bar + 8u * i, stage_tx);
                load_w(ring_addr + i * stage_bytes, full_bar + 8u * i, (kb_start + i) * kBlockK, pol_w);
            }
            pdl_wait_prior_grids();
            for (int i = 0; i < prologue; ++i) {
                tma_load_2d(ring_addr + i * stage_bytes + kWStageBytes, &tmap_a, full_bar + 8u * i,
                            (kb_start + i) * kBlockK, 0, pol_a);
            }
            stamp(p, 2);
        }
        __syncwarp();
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
    // Every CTA of the cluster has initialised its barriers once this cluster barrier completes;
    // it is only waited for much later, right before partials are pushed to the peers.
    if (p.split > 1) cluster_arrive_release();
    const uint32_t tmem_acc = ctrl->tmem_base;
    if (threadIdx.x == 0) stamp(p, 1);

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int issued = prologue;
            for (int i = prologue; i < kb_count; ++i) {
                const int s = i % p.stages;
                const uint32_t round = static_cast<uint32_t>(i / p.stages);
                if (!mbar_wait_bounded(empty_bar + 8u * s, (round - 1u) & 1u, &ctrl->abort, kRoleProducer)) break;
                mbar_arrive_expect_tx(full_bar + 8u * s, stage_tx);
                load_w(ring_addr + s * stage_bytes, full_bar + 8u * s, (kb_start + i) * kBlockK, pol_w);
                tma_load_2d(ring_addr + s * stage_bytes + kWStageBytes, &tmap_a, full_bar + 8u * s,
                            (kb_start + i) * kBlockK, 0, pol_a);
                issued = i + 1;
            }
            if (ctrl->abort) {
                // Give the copies already in flight a bounded chance to land before the CTA exits.
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
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_e4m3_f32(kTileN, p.m_pad);
            for (int i = 0; i < kb_count; ++i) {
                const int s = i % p.stages;
                const uint32_t round = static_cast<uint32_t>(i / p.stages);
                if (!mbar_wait_bounded(full_bar + 8u * s, round & 1u, &ctrl->abort, kRoleMma)) break;
                if (i == 0) stamp(p, 3);
                tcgen05_fence_after_sync();
                const uint64_t w_desc = umma_desc_kmajor_sw128(ring_addr + s * stage_bytes);
                const uint64_t a_desc = umma_desc_kmajor_sw128(ring_addr + s * stage_bytes + kWStageBytes);
#pragma unroll
                for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                    // +32 bytes along K inside the swizzle atom = +2 in the (address >> 4) field.
                    umma_f8f6f4(tmem_acc, w_desc + 2u * kk, a_desc + 2u * kk, idesc, (i | kk) != 0 ? 1u : 0u);
                }
                umma_commit(empty_bar + 8u * s);
            }
            umma_commit(accum_bar);
            stamp(p, 4);
        }
        __syncwarp();
    }

    // ---------------------------------------------------------------------- epilogue (warps 0..3)
    // split == 1: each thread owns one W row (= output column) and writes D straight from TMEM.
    // split  > 1: every CTA of the cluster owns one `chunk` of the tile. A CTA stages its partial
    // tile in its own shared memory and sends range q to CTA q with one bulk shared-to-shared copy
    // that counts bytes on q's `recv` barrier; an owner waits (bounded) until all `split` ranges
    // have landed, adds them in rank order out of its own memory and writes D. No cluster-wide
    // barrier sits on this path; the one issued at start-up only proves the peers' barriers exist.
    constexpr int kOwned = 8;  // owned elements per thread kept in registers (covers m <= 16)
    const bool epilogue_warp = warp < kEpilogueThreads / 32;
    const uint32_t recv_addr = smem_u32(ctrl) + kCtrlBytes;  // float recv[split][chunk]
    if (p.split > 1 && !epilogue_warp) cluster_wait_acquire();
    if (epilogue_warp) {
        pdl_wait_prior_grids();
        const int nl = threadIdx.x;  // TMEM lane = W row inside the tile
        const int n = n0 + nl;
        const bool lane_valid = nl < p.tile_rows && n < p.n;
        const bool direct = p.split == 1;
        const float scale = __ldg(p.scale) * p.kind_factor;
        const uint32_t lane_taddr = tmem_acc + (static_cast<uint32_t>(warp * 32) << 16);
        // Row-parallel: the call's epoch (completed calls + 1) and this tile's place in the exchange buffer.
        unsigned int epoch = 0;
        if (kRowPar) epoch = *reinterpret_cast<volatile unsigned int*>(p.rp.call_index) + 1u;
        const uint32_t tile_slot0 = blockIdx.x * static_cast<uint32_t>(total);

        // D_in is requested long before it is needed.
        float din[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            din[j] = (direct && p.accumulate && j < p.m && lane_valid)
                         ? load_out(p.d, static_cast<size_t>(j) * p.n + n, p.d_dtype)
                         : 0.0f;
        }
        float d_own[kOwned];
#pragma unroll
        for (int it = 0; it < kOwned; ++it) {
            const uint32_t off = threadIdx.x + it * kEpilogueThreads;
            const int e = static_cast<int>(rank * chunk + off);
            const int col = n0 + (e % kTileN);
            d_own[it] = (!direct && p.accumulate && off < chunk && e < total && (e % kTileN) < p.tile_rows && col < p.n)
                            ? load_out(p.d, static_cast<size_t>(e / kTileN) * p.n + col, p.d_dtype)
                            : 0.0f;
        }

        bool ok = mbar_wait_bounded(accum_bar, 0u, &ctrl->abort, kRoleEpilogue);
        ok = __all_sync(0xffffffffu, ok) && ctrl->abort == 0u;
        ok = __all_sync(0xffffffffu, ok);
        if (threadIdx.x == 0) stamp(p, 5);
        tcgen05_fence_after_sync();
        float* const partial = reinterpret_cast<float*>(ring_ptr);  // the ring is idle by now
        if (kMode == kModeSwiglu && direct) {
            // Lanes 0..63 hold gate columns, lanes 64..127 the matching up columns. The projection is
            // rounded to the 16-bit type first, as the unfused chain stores it, so both give the same
            // bytes. The activation is shared out by tokens: the gate thread of a column takes tokens
            // 0..7, the up thread tokens 8..15, and each hands the other the eight values it needs.
            constexpr int kPitch = 9;                        // floats per column: no bank conflicts
            float* const handed = partial;                   // [2][64][9]: up for tokens 0..7, gate for 8..15
            uint8_t* const out_tile = reinterpret_cast<uint8_t*>(partial + 2 * kHalfTile * kPitch);  // [16][64]
            const int col_in_tile = nl & (kHalfTile - 1);
            const int half = nl >> 6;                        // 0: this lane holds gate values, 1: up values
            float y[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) y[j] = 0.0f;
            if (ok) {
                uint32_t v[16];
                tmem_ld_32x32b_x16(lane_taddr, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) y[j] = round_trip_16(__uint_as_float(v[j]) * scale, p.d_dtype);
            }
            {
                // a gate lane gives away tokens 8..15, an up lane tokens 0..7
                float* const dst = handed + ((1 - half) * kHalfTile + col_in_tile) * kPitch;
#pragma unroll
                for (int j = 0; j < 8; ++j) dst[j] = half == 0 ? y[8 + j] : y[j];
            }
            asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueThreads) : "memory");
            {
                const float inv_act = 1.0f / __ldg(p.act_scale);
                const float* const src = handed + (half * kHalfTile + col_in_tile) * kPitch;
                const int token0 = half * 8;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (token0 + j < p.m) {
                        const float gate = half == 0 ? y[j] : src[j];
                        const float up = half == 0 ? src[j] : y[8 + j];
                        float t = (gate / (1.0f + expf(-gate))) * up * inv_act;
                        if (p.act_fnuz) t *= 2.0f;
                        uint8_t byte = static_cast<uint8_t>(pack_e4m3x2(t, 0.0f) & 0xffu);
                        if (p.act_fnuz && byte == 0x80u) byte = 0;
                        out_tile[(token0 + j) * kHalfTile + col_in_tile] = byte;
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueThreads) : "memory");
            if (nl < kHalfTile && ok) {
                const int token = nl >> 2, piece = nl & 3;
                const int col = static_cast<int>(blockIdx.x) * kHalfTile + piece * 16;
                if (token < p.m && col < p.act_cols) {   // act_cols % 16 == 0: a piece is inside or outside
                    *reinterpret_cast<uint4*>(p.act_out + static_cast<size_t>(token) * p.act_cols + col) =
                        *reinterpret_cast<const uint4*>(out_tile + token * kHalfTile + piece * 16);
                }
            }
        } else if (ok) {
            for (int c = 0; c < p.m_pad / 16; ++c) {
                uint32_t v[16];
                tmem_ld_32x32b_x16(lane_taddr + static_cast<uint32_t>(c * 16), v);
                tmem_ld_wait();
                if (direct) {
                    if (kRowPar) {
                        // host guarantees m <= 16 here: one chunk, 16 values per thread
                        float val[16];
                        uint32_t slot[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            val[j] = __uint_as_float(v[j]);
                            slot[j] = j < p.m ? tile_slot0 + static_cast<uint32_t>(j * kTileN + nl) : 0xffffffffu;
                        }
                        if (!rowpar_exchange<16>(p.rp, epoch, slot, val, &ctrl->abort)) ok = false;
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(val[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = c * 16 + j;
                        if (ok && m < p.m && lane_valid) {
                            const size_t idx = static_cast<size_t>(m) * p.n + n;
                            const float d_in = c == 0 ? din[j] : (p.accumulate ? load_out(p.d, idx, p.d_dtype) : 0.0f);
                            store_out(p.d, idx, p.d_dtype, fmaf(__uint_as_float(v[j]), scale, d_in));
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = c * 16 + j;
                        if (m < p.m) partial[m * kTileN + nl] = __uint_as_float(v[j]);
                    }
                }
            }
        }
        if (!direct) {
            // generic-proxy writes above -> visible to the bulk-copy engine, then one thread sends
            fence_proxy_async_smem();
            cluster_wait_acquire();
            asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueThreads) : "memory");
            if (threadIdx.x == 0 && ok) {
                for (int q = 0; q < p.split; ++q) {
                    dsmem_bulk_copy(dsmem_map(recv_addr + 4u * rank * chunk, static_cast<uint32_t>(q)),
                                    ring_addr + 4u * static_cast<uint32_t>(q) * chunk, 4u * chunk,
                                    dsmem_map(recv_bar, static_cast<uint32_t>(q)));
                }
            }
            bool landed = ok && mbar_wait_bounded(recv_bar, 0u, &ctrl->abort, kRoleEpilogue);
            landed = __all_sync(0xffffffffu, landed);
            if (kMode == kModeSwiglu) {
                // This CTA owns `rows` whole token rows of the tile, starting at token t0; thread
                // tid holds lane tid of each. Same activation as in the unsplit case: the gate lane
                // of a column takes the first half of the tokens, the up lane the second half.
                const float* const recv = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(ctrl) + kCtrlBytes);
                const int per_owner = static_cast<int>(chunk) / kTileN;          // <= 8 for m <= 16, split >= 2
                const int t0 = rank * per_owner;
                const int rows = landed ? (p.m - t0 < per_owner ? p.m - t0 : per_owner) : 0;   // may be <= 0
                const int first_half = (per_owner + 1) / 2;
                constexpr int kPitch = 5;                                        // floats per column and half
                float* const handed = partial + static_cast<size_t>(p.split) * chunk;   // past the staged tile
                uint8_t* const out_tile = reinterpret_cast<uint8_t*>(handed + 2 * kHalfTile * kPitch);  // [8][64]
                const int col_in_tile = nl & (kHalfTile - 1);
                const int half = nl >> 6;
                float y[kOwned];
#pragma unroll
                for (int it = 0; it < kOwned; ++it) {
                    float sum = 0.0f;
                    if (it < rows) {
                        for (int q = 0; q < p.split; ++q) sum += recv[q * chunk + it * kTileN + nl];
                    }
                    y[it] = round_trip_16(sum * scale, p.d_dtype);
                }
#pragma unroll
                for (int it = 0; it < kOwned; ++it) {
                    const bool give = half == 0 ? it >= first_half : it < first_half;
                    if (give && it < per_owner) {
                        const int slot_in_half = half == 0 ? it - first_half : it;
                        handed[((1 - half) * kHalfTile + col_in_tile) * kPitch + slot_in_half] = y[it];
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueThreads) : "memory");
                const float inv_act = 1.0f / __ldg(p.act_scale);
#pragma unroll
                for (int it = 0; it < kOwned; ++it) {
                    const bool mine = half == 0 ? it < first_half : it >= first_half;
                    if (mine && it < rows) {
                        const int slot_in_half = half == 0 ? it : it - first_half;
                        const float other = handed[(half * kHalfTile + col_in_tile) * kPitch + slot_in_half];
                        const float gate = half == 0 ? y[it] : other;
                        const float up = half == 0 ? other : y[it];
                        float t = (gate / (1.0f + expf(-gate))) * up * inv_act;
                        if (p.act_fnuz) t *= 2.0f;
                        uint8_t byte = static_cast<uint8_t>(pack_e4m3x2(t, 0.0f) & 0xffu);
                        if (p.act_fnuz && byte == 0x80u) byte = 0;
                        out_tile[it * kHalfTile + col_in_tile] = byte;
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueThreads) : "memory");
                if (nl < 4 * rows) {
                    const int row = nl >> 2, piece = nl & 3;
                    const int col = static_cast<int>(blockIdx.x) * kHalfTile + piece * 16;
                    if (col < p.act_cols) {
                        *reinterpret_cast<uint4*>(p.act_out + static_cast<size_t>(t0 + row) * p.act_cols + col) =
                            *reinterpret_cast<const uint4*>(out_tile + row * kHalfTile + piece * 16);
                    }
                }
            } else if (landed) {
                const float* const recv = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(ctrl) + kCtrlBytes);
                float own[kOwned];
                uint32_t slot[kOwned];
#pragma unroll
                for (int it = 0; it < kOwned; ++it) {
                    const uint32_t off = threadIdx.x + it * kEpilogueThreads;
                    const int e = static_cast<int>(rank * chunk + off);
                    float sum = 0.0f;
                    if (off < chunk && e < total) {
                        for (int q = 0; q < p.split; ++q) sum += recv[q * chunk + off];
                    }
                    own[it] = sum;
                    slot[it] = (off < chunk && e < total) ? tile_slot0 + static_cast<uint32_t>(e) : 0xffffffffu;
                }
                if (kRowPar) {
                    landed = rowpar_exchange<kOwned>(p.rp, epoch, slot, own, &ctrl->abort);
                }
#pragma unroll
                for (int it = 0; it < kOwned; ++it) {
                    const uint32_t off = threadIdx.x + it * kEpilogueThreads;
                    const int e = static_cast<int>(rank * chunk + off);
                    if (landed && off < chunk && e < total) {
                        const int col = n0 + (e % kTileN);
                        if ((e % kTileN) < p.tile_rows && col < p.n) {
                            store_out(p.d, static_cast<size_t>(e / kTileN) * p.n + col, p.d_dtype,
                                      fmaf(own[it], scale, d_own[it]));
                        }
                    }
                }
                // token counts above 16 own more than kOwned elements per thread for small splits
                for (uint32_t off = threadIdx.x + kOwned * kEpilogueThreads; off < chunk; off += kEpilogueThreads) {
                    const int e = static_cast<int>(rank * chunk + off);
                    if (e >= total) break;
                    float sum = 0.0f;
                    for (int q = 0; q < p.split; ++q) sum += recv[q * chunk + off];
                    const int col = n0 + (e % kTileN);
                    if ((e % kTileN) < p.tile_rows && col < p.n) {
                        const size_t idx = static_cast<size_t>(e / kTileN) * p.n + col;
                        const float d0 = p.accumulate ? load_out(p.d, idx, p.d_dtype) : 0.0f;
                        store_out(p.d, idx, p.d_dtype, fmaf(sum, scale, d0));
                    }
                }
            }
            // the staged partial tile must outlive the copies that read it
            if (threadIdx.x == 0) bulk_copies_source_done();
        }
        if (kMode == kModeSwiglu) {
            // the next GEMM adds into this buffer: the whole grid clears it
            const size_t cta = static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x;
            const size_t ctas = static_cast<size_t>(gridDim.x) * gridDim.y;
            const size_t vecs = static_cast<size_t>(p.zero_bytes / 16);
            for (size_t i = cta * kEpilogueThreads + threadIdx.x; i < vecs; i += ctas * kEpilogueThreads) {
                reinterpret_cast<uint4*>(p.zero_ptr)[i] = make_uint4(0, 0, 0, 0);
            }
        }
    }

    if (threadIdx.x == 0) stamp(p, 6);
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) tmem_dealloc(tmem_acc, tmem_cols);
    if (kRowPar && threadIdx.x == 0) {
        // The last CTA of the grid closes the call: every CTA has read the call index by now.
        __threadfence();
        const unsigned int ctas = gridDim.x * gridDim.y;
        if (atomicAdd(p.rp.done_ctas, 1u) == ctas - 1u) {
            *p.rp.done_ctas = 0u;
            *reinterpret_cast<volatile unsigned int*>(p.rp.call_index) =
                *reinterpret_cast<volatile unsigned int*>(p.rp.call_index) + 1u;
            __threadfence();
        }
    }
    if (threadIdx.x == 0) stamp(p, 7);
}

}  // namespace hfrk
