// FP8 skinny GEMM for B200 (sm_100a):  D[m,n] <- D_in[m,n] + scale * sum_k A[m,k] * W[n,k].
//
// The operation is bound by the one pass over the weight matrix W (N*K bytes from HBM); the token
// count M is tiny. The kernel is therefore a weight streamer with a tensor-core sink:
//
//   * swap-AB: a CTA owns 128 consecutive rows of W. Those rows are the M=128 side of a
//     tcgen05.mma (kind::f8f6f4, e4m3 x e4m3 -> f32); the padded token count (16..64) is the MMA
//     N side. The accumulator D^T[128 x m_pad] lives in TMEM, one W row per TMEM lane.
//   * one elected thread streams 128x128-byte W boxes (and the matching m_pad x 128-byte A boxes)
//     with TMA, 128-byte swizzled, into a ring of shared-memory stages guarded by full/empty
//     mbarriers; one elected thread issues four K=32 MMAs per stage and commits the stage back to
//     the producer; four warps drain TMEM and write D.
//   * split-K across a thread-block cluster when N/128 tiles cannot fill the SMs: each CTA of the
//     cluster reduces a slice of the 128 x M partial tile out of its peers' shared memory (DSMEM)
//     in a fixed rank order, so the result is deterministic (the reference uses fp16 atomics:
//     csrc/op_src/skinny_gemm/consumers/mfma_16x16x32_consumer.cu:113-168).
//   * every wait on an mbarrier is bounded; a wait that runs out records a status word, lets the
//     other roles give up too, and the CTA still frees its TMEM and leaves normally.
//   * programmatic dependent launch: the weight stream of a call may start before the previous
//     kernel on the stream has finished, because W is static; A and D are only touched after
//     griddepcontrol.wait.
//
// Role of this file in the reference's terms: it replaces skinny_gemm_kernel.cu:6-79 (kernel),
// producers/*.cu (global->LDS streaming), consumers/*.cu (MFMA + atomic epilogue) and
// skinny_gemm_caller.cu:21-71 (validation, launch shape) of csrc/op_src/skinny_gemm/.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#include "../../include/hfrk_b200.h"
#include "host_common.h"
#include "ptx_sm100.cuh"
#include "elementwise_common.cuh"
#include "skinny_gemm_common.cuh"
#include "skinny_gemm_streamk.cuh"

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
//                 (split == 1 and m <= 16 only: the host guarantees both)
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

// =============================================================================== host side

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres = cudaDriverEntryPointSymbolNotFound;
        cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
        if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess) ptr = nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

struct MapKey {
    const void* base;
    uint64_t inner, outer, stride;
    uint32_t box_outer;
    bool operator==(const MapKey& o) const {
        return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride && box_outer == o.box_outer;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9E3779B97F4A7C15ull;
        h ^= (k.inner + 0x632BE59BD9B4E019ull) + (h << 6) + (h >> 2);
        h ^= (k.outer * 0xD6E8FEB86659FD93ull) + (h << 6) + (h >> 2);
        h ^= (k.stride * 0xA24BAED4963EE407ull) + (h << 6) + (h >> 2);
        h ^= k.box_outer;
        return static_cast<size_t>(h);
    }
};

// Encoding a tensor map costs a driver call; decode loops call the GEMM with the same weight
// pointers every step, so descriptors are cached by (pointer, extents, pitch, box). The cache
// holds no ownership: a stale entry for a freed-and-reused pointer is still a correct descriptor
// for that address range.
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

// 2-D uint8 tensor [outer][inner] with a pitch of `stride` bytes, boxes of 128 x box_outer bytes,
// 128-byte swizzle, zero fill outside the tensor.
int get_tensor_map(const void* base, uint64_t inner, uint64_t outer, uint64_t stride, uint32_t box_outer,
                   CUtensorMap* out) {
    MapKey key{base, inner, outer, stride, box_outer};
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        auto it = g_map_cache.find(key);
        if (it != g_map_cache.end()) {
            *out = it->second;
            return HFRK_SUCCESS;
        }
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        set_last_error("cuTensorMapEncodeTiled is not available from the driver");
        return HFRK_CUDA_ERROR;
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {stride};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), box_outer};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult res = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) {
        char msg[256];
        snprintf(msg, sizeof(msg),
                 "cuTensorMapEncodeTiled failed (%d): base=%p inner=%llu outer=%llu pitch=%llu box=128x%u",
                 static_cast<int>(res), base, static_cast<unsigned long long>(inner),
                 static_cast<unsigned long long>(outer), static_cast<unsigned long long>(stride), box_outer);
        set_last_error(msg);
        return HFRK_CUDA_ERROR;
    }
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (g_map_cache.size() > 8192) g_map_cache.clear();
    g_map_cache.emplace(key, *out);
    return HFRK_SUCCESS;
}

struct Plan {
    int split, stages, ctas, smem_bytes, m_pad, num_kblocks, tile_rows, tiles;
};

int round_up(int v, int to) { return (v + to - 1) / to * to; }

// Per-process tuning table: (padded tokens, n, k) -> (split, stages), filled by hfrk_tuning_set
// from the output of the grid search. Chips differ in how their SMs are spread over the GPCs, so
// the best cluster shape of a given projection can differ from one B200 to the next; the table
// lets a deployment pin what its own sweep found. Consulted before the built-in rule.
struct TuneKey {
    int m_pad, n, k;
    bool operator==(const TuneKey& o) const { return m_pad == o.m_pad && n == o.n && k == o.k; }
};
struct TuneKeyHash {
    size_t operator()(const TuneKey& t) const {
        return static_cast<size_t>(t.m_pad) * 1000003u ^ static_cast<size_t>(t.n) * 7919u ^ static_cast<size_t>(t.k) * 104729u;
    }
};
struct TuneValue {
    int split, stages, tile_rows;
};
std::mutex g_tune_mutex;
std::unordered_map<TuneKey, TuneValue, TuneKeyHash> g_tune_table;

bool tuning_lookup(int m_pad, int n, int k, TuneValue* out) {
    std::lock_guard<std::mutex> lock(g_tune_mutex);
    auto it = g_tune_table.find(TuneKey{m_pad, n, k});
    if (it == g_tune_table.end()) return false;
    *out = it->second;
    return true;
}

// Launch shape of the cluster kernel for one launch of m <= kMaxMPad tokens, from sweeps on B200
// (148 SMs) over the Llama-3 8B/70B projection shapes and their 2/4/8-way N and K shards:
//   * one SM cannot pull much more than 40 GB/s of weights, so every SM must stream, and two small
//     CTAs per SM hide each other's fill, drain and reduction better than one big one: with a K
//     split the ring has four 18 KiB stages (two CTAs per SM at 16 tokens);
//   * the whole grid must be resident at once, WITH MARGIN. A cluster that has to wait for a free
//     slot starts late and then streams alone at a fraction of the bandwidth, and clusters only
//     fit into one GPC, so a grid that fills the last slot on paper (288 of 296) already spills.
//     The split is the largest one with tiles * split <= 280 and at least two K blocks per CTA,
//     capped at 8 (12 below 25 tiles, 16 below 11: very narrow shards need it to reach the SMs);
//   * without a split (tiles alone cover the SMs) a ring of six stages, two CTAs per SM.
//   * tiles of fewer than 128 rows can even out a grid without a K split that is between one and
//     two CTAs per SM: 224 tiles of 128 rows put two CTAs on 76 SMs and one on the other 72, and
//     the grid ends when the doubly loaded SMs are done; 279 tiles of 103 rows load nearly every
//     SM twice. The tensor core still computes 128 lanes per tile (it idles at a few per cent
//     anyway); the lanes past the tile's rows are ignored. Measured gain on 28672 x 4096: 2.4 %.
//     Nowhere else: with clusters a taller grid crosses the residency cliff (35 clusters of 8
//     instead of 32: +45 % time), and grids of several waves got slower (57344 x 8192: +2 %).
int make_plan(int m, int n, int k, int split_req, int stages_req, Plan* plan, int tile_rows_req = 0) {
    if (m <= 0 || n <= 0 || k <= 0 || m > kMaxMPad) return HFRK_INVALID_CONFIG;
    if (tile_rows_req < kAutoTileRowsOff || tile_rows_req > kTileN || (tile_rows_req > 0 && tile_rows_req < 8))
        return HFRK_INVALID_CONFIG;
    if (split_req < 0 || split_req > kMaxSplit || stages_req < 0 || stages_req == 1 || stages_req > kMaxStages)
        return HFRK_INVALID_CONFIG;
    const int m_pad = round_up(m, 16);
    const int tiles = (n + kTileN - 1) / kTileN;
    const int nkb = (k + kBlockK - 1) / kBlockK;
    const int stage_bytes = kWStageBytes + m_pad * kBlockK;
    constexpr int kResidentTarget = 280;

    TuneValue tuned;
    if (split_req == 0 && stages_req == 0 && tile_rows_req == 0 && tuning_lookup(m_pad, n, k, &tuned)) {
        split_req = tuned.split;
        stages_req = tuned.stages;
        tile_rows_req = tuned.tile_rows;
    }
    int split = split_req;
    if (split == 0) {
        split = kResidentTarget / tiles;
        const int cap = tiles <= 10 ? kMaxSplit : (tiles <= 24 ? 12 : 8);
        if (split > cap) split = cap;
        if (split < 2 && tiles < kNumSms) split = 2;  // 141..147 tiles: two CTAs per SM still beat one
        if (split > nkb / 2) split = nkb / 2;
        if (split < 1) split = 1;
    }
    if (split > nkb) split = nkb;

    const int chunk = (((m * kTileN + split - 1) / split) + 3) & ~3;
    const int recv_bytes = split > 1 ? split * chunk * 4 : 0;
    const int fixed_bytes = 1024 + kCtrlBytes + recv_bytes;
    const int max_stages_fit = (kSmemLimit - fixed_bytes) / stage_bytes;
    int stages = stages_req != 0 ? stages_req : (split > 1 ? 4 : 6);
    if (stages_req == 0) {
        // keep two CTAs on an SM when the activation tile or the receive buffer of a larger token
        // count grows: with one CTA per SM a grid of 150-296 CTAs needs a second wave
        while (stages > 2 && 2 * (fixed_bytes + stages * stage_bytes + 1024) > 228 * 1024) --stages;
    }
    if (stages > max_stages_fit) stages = max_stages_fit;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return HFRK_INVALID_CONFIG;

    int tile_rows = tile_rows_req == kAutoTileRowsOff ? kTileN : tile_rows_req;
    if (tile_rows == 0) {
        tile_rows = kTileN;
        const int smem = fixed_bytes + stages * stage_bytes;
        if (m_pad == 16 && split == 1 && tiles > kNumSms && tiles <= kResidentTarget &&
            2 * (smem + 1024) <= 228 * 1024) {
            const int rows = (n + kResidentTarget - 1) / kResidentTarget;
            if (rows >= 64 && rows < tile_rows) tile_rows = rows;
        }
    }
    const int tiles_used = (n + tile_rows - 1) / tile_rows;

    plan->split = split;
    plan->stages = stages;
    plan->tile_rows = tile_rows;
    plan->tiles = tiles_used;
    plan->ctas = tiles_used * split;
    plan->smem_bytes = fixed_bytes + stages * stage_bytes;
    plan->m_pad = m_pad;
    plan->num_kblocks = nkb;
    return HFRK_SUCCESS;
}

int prepare_device_once() {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    HFRK_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && done[dev]) return HFRK_SUCCESS;
    HFRK_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_fp8_sm100_kernel<kModePlain>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_fp8_sm100_kernel<kModePlain>,
                                       cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_fp8_sm100_kernel<kModeRowPar>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_fp8_sm100_kernel<kModeRowPar>,
                                       cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_fp8_sm100_kernel<kModeSwiglu>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_fp8_sm100_kernel<kModeSwiglu>,
                                       cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_fp8_streamk_kernel<1>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    HFRK_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_fp8_streamk_kernel<2>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    if (dev >= 0 && dev < 64) done[dev] = true;
    return HFRK_SUCCESS;
}

int validate(const void* A, const void* W, void* D, const float* scale_dev, int m, int n, int k,
             int64_t w_row_stride, int a_kind, int w_kind, int d_dtype) {
    if (A == nullptr || W == nullptr || D == nullptr || scale_dev == nullptr) return HFRK_INVALID_CONFIG;
    if (m <= 0 || n <= 0 || k <= 0) return HFRK_INVALID_CONFIG;
    if ((a_kind != HFRK_E4M3FN && a_kind != HFRK_E4M3FNUZ) || (w_kind != HFRK_E4M3FN && w_kind != HFRK_E4M3FNUZ))
        return HFRK_BAD_DTYPE;
    if (d_dtype != HFRK_F16 && d_dtype != HFRK_BF16 && d_dtype != HFRK_F32) return HFRK_BAD_DTYPE;
    if (k % 16 != 0) return HFRK_K_NOT_DIVISIBLE;
    if (w_row_stride < k || w_row_stride % 16 != 0) return HFRK_BAD_ALIGNMENT;
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(W) & 15u) ||
        (reinterpret_cast<uintptr_t>(D) & (d_dtype == HFRK_F32 ? 3u : 1u)) ||
        (reinterpret_cast<uintptr_t>(scale_dev) & 3u))
        return HFRK_BAD_ALIGNMENT;
    return HFRK_SUCCESS;
}

// ---------------------------------------------------------------- stream-K scratch
// The stream-K kernel needs fp32 scratch for partial tiles and one counter per tile. The library
// owns it: kScratchLanes independent sets per device, allocated together on the first call on
// that device (which therefore must not happen inside a stream capture). A stream is bound to a
// lane the first time it is seen; calls on one stream are ordered, so they can share a lane, and
// up to kScratchLanes streams can run GEMMs concurrently without touching each other's scratch.
constexpr int kScratchLanes = 4;
constexpr int kSkMaxGrid = 2 * kNumSms;
constexpr int kSkMaxTiles = 65536;
constexpr size_t kLanePartialFloats = static_cast<size_t>(2) * kSkMaxGrid * kMaxMPad * kTileN;

struct DeviceScratch {
    bool ready = false;
    float* partials[kScratchLanes] = {};
    unsigned int* counters[kScratchLanes] = {};
    std::unordered_map<cudaStream_t, int> lane_of;
    int next_lane = 0;
};
std::mutex g_scratch_mutex;
DeviceScratch g_scratch[64];

int scratch_for(cudaStream_t stream, float** partials, unsigned int** counters) {
    int dev = 0;
    HFRK_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return HFRK_INVALID_CONFIG;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    DeviceScratch& sc = g_scratch[dev];
    if (!sc.ready) {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        HFRK_CUDA_TRY(cudaStreamIsCapturing(stream, &capturing));
        if (capturing != cudaStreamCaptureStatusNone) {
            set_last_error("first call on this device happened inside a stream capture: call the GEMM once "
                           "outside the capture so that its scratch memory can be allocated");
            return HFRK_CUDA_ERROR;
        }
        const size_t lane_bytes = kLanePartialFloats * sizeof(float);
        const size_t counter_bytes = static_cast<size_t>(kSkMaxTiles) * sizeof(unsigned int);
        uint8_t* block = nullptr;
        HFRK_CUDA_TRY(cudaMalloc(&block, kScratchLanes * (lane_bytes + counter_bytes)));
        HFRK_CUDA_TRY(cudaMemset(block, 0, kScratchLanes * (lane_bytes + counter_bytes)));
        for (int l = 0; l < kScratchLanes; ++l) {
            sc.partials[l] = reinterpret_cast<float*>(block + l * lane_bytes);
            sc.counters[l] = reinterpret_cast<unsigned int*>(block + kScratchLanes * lane_bytes + l * counter_bytes);
        }
        sc.ready = true;
    }
    auto it = sc.lane_of.find(stream);
    int lane;
    if (it == sc.lane_of.end()) {
        lane = sc.next_lane++ % kScratchLanes;
        if (sc.lane_of.size() > 1024) sc.lane_of.clear();
        sc.lane_of.emplace(stream, lane);
    } else {
        lane = it->second;
    }
    *partials = sc.partials[lane];
    *counters = sc.counters[lane];
    return HFRK_SUCCESS;
}

struct SkPlan {
    int grid, stages, units_per_stage, smem_bytes, m_pad, nkb, tiles;
};

// Stream-K launch shape: the grid covers the SMs `ctas_per_sm` times (never more CTAs than work
// items), and each CTA's ring takes its share of the SM's shared memory.
int make_sk_plan(int m, int n, int k, int ctas_per_sm, int stages_req, SkPlan* plan) {
    if (m <= 0 || n <= 0 || k <= 0 || m > kMaxMPad) return HFRK_INVALID_CONFIG;
    if (ctas_per_sm < 0 || ctas_per_sm > 2 || stages_req < 0 || stages_req == 1 || stages_req > kSkMaxStages)
        return HFRK_INVALID_CONFIG;
    const int m_pad = round_up(m, 16);
    const int tiles = (n + kTileN - 1) / kTileN;
    const int nkb = (k + kBlockK - 1) / kBlockK;
    if (tiles > kSkMaxTiles) return HFRK_TOO_LARGE;
    const long long units = static_cast<long long>(tiles) * nkb;
    if (units > 0x3fffffff) return HFRK_TOO_LARGE;
    if (ctas_per_sm == 0) ctas_per_sm = 2;
    // Two CTAs per SM have two MMA-issuing threads, so single-K-block stages (more of them in
    // flight) win; a lone CTA per SM needs the cheaper two-block stages to keep up.
    const int ups = ctas_per_sm == 1 ? 2 : 1;
    const int stage_bytes = ups * (kWStageBytes + m_pad * kBlockK);
    const int budget = (228 * 1024 - ctas_per_sm * 1024) / ctas_per_sm;
    int stages = stages_req != 0 ? stages_req : (budget - 1024 - kCtrlBytes) / stage_bytes;
    if (stages > kSkMaxStages) stages = kSkMaxStages;
    while (stages > 2 && 1024 + stages * stage_bytes + kCtrlBytes > kSmemLimit) --stages;
    if (stages < 2 || 1024 + stages * stage_bytes + kCtrlBytes > kSmemLimit) return HFRK_INVALID_CONFIG;
    long long grid = static_cast<long long>(kNumSms) * ctas_per_sm;
    if (grid > units) grid = units;
    plan->grid = static_cast<int>(grid);
    plan->stages = stages;
    plan->units_per_stage = ups;
    plan->smem_bytes = 1024 + stages * stage_bytes + kCtrlBytes;
    plan->m_pad = m_pad;
    plan->nkb = nkb;
    plan->tiles = tiles;
    return HFRK_SUCCESS;
}

int launch_streamk(const void* A, const void* W, void* D, const float* scale_dev, int m, int n, int k,
                   int64_t w_row_stride, int a_kind, int w_kind, int d_dtype, int accumulate, int ctas_per_sm,
                   int stages_req, int use_pdl, cudaStream_t stream, unsigned long long* stamps) {
    CUtensorMap tmap_w;
    int rc = get_tensor_map(W, static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                            static_cast<uint64_t>(w_row_stride), kTileN, &tmap_w);
    if (rc != HFRK_SUCCESS) return rc;
    float* partials = nullptr;
    unsigned int* counters = nullptr;
    rc = scratch_for(stream, &partials, &counters);
    if (rc != HFRK_SUCCESS) return rc;

    for (int m0 = 0; m0 < m; m0 += kMaxMPad) {
        const int mc = m - m0 < kMaxMPad ? m - m0 : kMaxMPad;
        SkPlan plan;
        rc = make_sk_plan(mc, n, k, ctas_per_sm, stages_req, &plan);
        if (rc != HFRK_SUCCESS) return rc;
        const uint8_t* a_chunk = static_cast<const uint8_t*>(A) + static_cast<size_t>(m0) * k;
        CUtensorMap tmap_a;
        rc = get_tensor_map(a_chunk, static_cast<uint64_t>(k), static_cast<uint64_t>(mc), static_cast<uint64_t>(k),
                            static_cast<uint32_t>(plan.m_pad), &tmap_a);
        if (rc != HFRK_SUCCESS) return rc;

        SkParams p;
        p.d = static_cast<uint8_t*>(D) + static_cast<size_t>(m0) * n * (d_dtype == HFRK_F32 ? 4 : 2);
        p.scale = scale_dev;
        p.kind_factor = (a_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f) * (w_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f);
        p.m = mc;
        p.n = n;
        p.m_pad = plan.m_pad;
        p.nkb = plan.nkb;
        p.total_units = plan.tiles * plan.nkb;
        p.stages = plan.stages;
        p.d_dtype = d_dtype;
        p.accumulate = accumulate ? 1 : 0;
        p.partials = partials;
        p.counters = counters;
        p.stamps = stamps;

        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(plan.grid), 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = static_cast<size_t>(plan.smem_bytes);
        cfg.stream = stream;
        cudaLaunchAttribute attrs[1];
        unsigned num_attrs = 0;
        if (use_pdl) {
            attrs[num_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attrs[num_attrs].val.programmaticStreamSerializationAllowed = 1;
            ++num_attrs;
        }
        cfg.attrs = attrs;
        cfg.numAttrs = num_attrs;
        if (plan.units_per_stage == 1) {
            HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_gemm_fp8_streamk_kernel<1>, tmap_w, tmap_a, p));
        } else {
            HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_gemm_fp8_streamk_kernel<2>, tmap_w, tmap_a, p));
        }
    }
    return HFRK_SUCCESS;
}

int launch_gemm(const void* A, const void* W, void* D, const float* scale_dev, int m, int n, int k,
                int64_t w_row_stride, int a_kind, int w_kind, int d_dtype, int accumulate, int variant,
                int split_req, int ctas_per_sm, int stages_req, int use_pdl, cudaStream_t stream,
                unsigned long long* stamps = nullptr, const RowparDev* rowpar = nullptr,
                int rowpar_mode = HFRK_ROWPAR_AUTO, int tile_rows_req = 0) {
    int rc = validate(A, W, D, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype);
    if (rc != HFRK_SUCCESS) return rc;
    rc = prepare_device_once();
    if (rc != HFRK_SUCCESS) return rc;
    if (variant < HFRK_VARIANT_AUTO || variant > HFRK_VARIANT_STREAMK) return HFRK_INVALID_CONFIG;
    if (variant == HFRK_VARIANT_AUTO) variant = HFRK_VARIANT_CLUSTER;
    if (rowpar != nullptr && variant != HFRK_VARIANT_CLUSTER) return HFRK_INVALID_CONFIG;
    if (variant == HFRK_VARIANT_STREAMK) {
        return launch_streamk(A, W, D, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype, accumulate,
                              ctas_per_sm, stages_req, use_pdl, stream, stamps);
    }

    const size_t out_elem = d_dtype == HFRK_F32 ? 4 : 2;
    // the fused all-reduce keeps a thread's share of the tile in registers: 16 tokens per launch
    const int m_step = rowpar != nullptr ? 16 : kMaxMPad;
    for (int m0 = 0; m0 < m; m0 += m_step) {
        const int mc = m - m0 < m_step ? m - m0 : m_step;
        Plan plan;
        // the exchange buffer of the row-parallel kernel is laid out in 128-row tiles
        rc = make_plan(mc, n, k, split_req, stages_req, &plan, rowpar != nullptr ? kAutoTileRowsOff : tile_rows_req);
        if (rc != HFRK_SUCCESS) return rc;
        CUtensorMap tmap_w;
        rc = get_tensor_map(W, static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                            static_cast<uint64_t>(w_row_stride), static_cast<uint32_t>(plan.tile_rows), &tmap_w);
        if (rc != HFRK_SUCCESS) return rc;
        const uint8_t* a_chunk = static_cast<const uint8_t*>(A) + static_cast<size_t>(m0) * k;
        CUtensorMap tmap_a;
        rc = get_tensor_map(a_chunk, static_cast<uint64_t>(k), static_cast<uint64_t>(mc), static_cast<uint64_t>(k),
                            static_cast<uint32_t>(plan.m_pad), &tmap_a);
        if (rc != HFRK_SUCCESS) return rc;

        GemmParams p;
        p.d = static_cast<uint8_t*>(D) + static_cast<size_t>(m0) * n * out_elem;
        p.scale = scale_dev;
        p.kind_factor = (a_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f) * (w_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f);
        p.m = mc;
        p.n = n;
        p.k = k;
        p.m_pad = plan.m_pad;
        p.tile_rows = plan.tile_rows;
        p.num_kblocks = plan.num_kblocks;
        p.split = plan.split;
        p.stages = plan.stages;
        p.d_dtype = d_dtype;
        p.accumulate = accumulate ? 1 : 0;
        p.stamps = stamps;
        memset(&p.rp, 0, sizeof(p.rp));
        if (rowpar != nullptr) {
            p.rp = *rowpar;
            if (rowpar_mode == HFRK_ROWPAR_AUTO) {
                // One-shot sends (world - 1) copies of this rank's fp32 partials; past about a
                // megabyte the second NVLink crossing of the two-shot costs less than that traffic.
                const unsigned long long one_shot_bytes =
                    4ull * static_cast<unsigned long long>(mc) * n * static_cast<unsigned>(p.rp.world - 1);
                p.rp.two_shot = one_shot_bytes >= kTwoShotFromBytes ? 1 : 0;
            } else {
                p.rp.two_shot = rowpar_mode == HFRK_ROWPAR_TWO_SHOT ? 1 : 0;
            }
            const unsigned tiles = static_cast<unsigned>((n + kTileN - 1) / kTileN);
            if (static_cast<unsigned long long>(tiles) * mc * kTileN > p.rp.elems_per_src) return HFRK_TOO_LARGE;
        }

        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(plan.tiles), static_cast<unsigned>(plan.split), 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = static_cast<size_t>(plan.smem_bytes);
        cfg.stream = stream;
        cudaLaunchAttribute attrs[2];
        unsigned num_attrs = 0;
        if (plan.split > 1) {
            attrs[num_attrs].id = cudaLaunchAttributeClusterDimension;
            attrs[num_attrs].val.clusterDim.x = 1;
            attrs[num_attrs].val.clusterDim.y = static_cast<unsigned>(plan.split);
            attrs[num_attrs].val.clusterDim.z = 1;
            ++num_attrs;
        }
        if (use_pdl) {
            attrs[num_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attrs[num_attrs].val.programmaticStreamSerializationAllowed = 1;
            ++num_attrs;
        }
        cfg.attrs = attrs;
        cfg.numAttrs = num_attrs;
        if (rowpar != nullptr) {
            HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_gemm_fp8_sm100_kernel<kModeRowPar>, tmap_w, tmap_a, p));
        } else {
            HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_gemm_fp8_sm100_kernel<kModePlain>, tmap_w, tmap_a, p));
        }
    }
    return HFRK_SUCCESS;
}

// Gate/up projection with the SwiGLU, the fp8 quantisation of the down projection's input and the
// zeroing of the down projection's accumulate buffer in the epilogue: one launch where the chain
// has GEMM + swiglu. W is [2 * inter, k]: `inter` gate rows, then `inter` up rows. Tile t of the
// grid takes gate rows [64t, 64t + 64) and up rows [inter + 64t, inter + 64t + 64), so that both
// halves of every output column meet in one CTA. With a K split the cluster's reduction hands every
// CTA whole token rows of the tile (not arbitrary element ranges), so the halves still meet.
int launch_gemm_swiglu(const void* A, const void* W, void* act_out, const float* scale_dev,
                       const float* act_scale_dev, void* next_buffer, int m, int inter, int k, int64_t w_row_stride,
                       int a_kind, int w_kind, int mid_dtype, int out_kind, int64_t buffer_cols, int split_req,
                       int use_pdl, cudaStream_t stream) {
    if (A == nullptr || W == nullptr || act_out == nullptr || scale_dev == nullptr || act_scale_dev == nullptr)
        return HFRK_INVALID_CONFIG;
    if (m <= 0 || inter <= 0 || k <= 0 || buffer_cols < 0) return HFRK_INVALID_CONFIG;
    if (m > 16) return HFRK_TOO_LARGE;
    if (inter % 16 != 0) return HFRK_INVALID_CONFIG;   // 16-byte pieces of the fp8 output rows
    if ((a_kind != HFRK_E4M3FN && a_kind != HFRK_E4M3FNUZ) || (w_kind != HFRK_E4M3FN && w_kind != HFRK_E4M3FNUZ) ||
        (mid_dtype != HFRK_F16 && mid_dtype != HFRK_BF16) || (out_kind != HFRK_E4M3FN && out_kind != HFRK_E4M3FNUZ))
        return HFRK_BAD_DTYPE;
    if (k % 16 != 0) return HFRK_K_NOT_DIVISIBLE;
    const size_t zero_bytes = static_cast<size_t>(m) * static_cast<size_t>(buffer_cols) * 2;
    if (zero_bytes != 0 && next_buffer == nullptr) return HFRK_INVALID_CONFIG;
    if (w_row_stride < k || w_row_stride % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15u) ||
        (reinterpret_cast<uintptr_t>(W) & 15u) || (reinterpret_cast<uintptr_t>(act_out) & 15u) ||
        (reinterpret_cast<uintptr_t>(next_buffer) & 15u) || zero_bytes % 16 != 0)
        return HFRK_BAD_ALIGNMENT;
    int rc = prepare_device_once();
    if (rc != HFRK_SUCCESS) return rc;

    CUtensorMap tmap_w, tmap_a;
    rc = get_tensor_map(W, static_cast<uint64_t>(k), static_cast<uint64_t>(2) * inter,
                        static_cast<uint64_t>(w_row_stride), kHalfTile, &tmap_w);
    if (rc != HFRK_SUCCESS) return rc;
    Plan plan;
    rc = make_plan(m, 2 * inter, k, split_req, /*stages_req=*/0, &plan, kAutoTileRowsOff);
    if (rc != HFRK_SUCCESS) return rc;
    if (plan.split > 1) {
        // the receive buffer holds whole token rows per owner: ceil(m / split) rows of 128 floats
        const int plain_chunk = (((m * kTileN + plan.split - 1) / plan.split) + 3) & ~3;
        const int row_chunk = kTileN * ((m + plan.split - 1) / plan.split);
        plan.smem_bytes += plan.split * (row_chunk - plain_chunk) * 4;
        const int stage_bytes = kWStageBytes + plan.m_pad * kBlockK;
        while (plan.stages > 2 && 2 * (plan.smem_bytes + 1024) > 228 * 1024) {
            --plan.stages;
            plan.smem_bytes -= stage_bytes;
        }
        if (plan.smem_bytes > kSmemLimit) return HFRK_INVALID_CONFIG;
    }
    rc = get_tensor_map(A, static_cast<uint64_t>(k), static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                        static_cast<uint32_t>(plan.m_pad), &tmap_a);
    if (rc != HFRK_SUCCESS) return rc;

    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.scale = scale_dev;
    p.kind_factor = (a_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f) * (w_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f);
    p.m = m;
    p.n = 2 * inter;
    p.k = k;
    p.m_pad = plan.m_pad;
    p.tile_rows = kTileN;
    p.num_kblocks = plan.num_kblocks;
    p.split = plan.split;
    p.stages = plan.stages;
    p.d_dtype = mid_dtype;
    p.accumulate = 0;
    p.act_out = static_cast<uint8_t*>(act_out);
    p.act_scale = act_scale_dev;
    p.act_cols = inter;
    p.act_fnuz = out_kind == HFRK_E4M3FNUZ ? 1 : 0;
    p.zero_ptr = static_cast<uint8_t*>(next_buffer);
    p.zero_bytes = zero_bytes;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((inter + kHalfTile - 1) / kHalfTile), static_cast<unsigned>(plan.split), 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(plan.smem_bytes);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned num_attrs = 0;
    if (plan.split > 1) {
        attrs[num_attrs].id = cudaLaunchAttributeClusterDimension;
        attrs[num_attrs].val.clusterDim.x = 1;
        attrs[num_attrs].val.clusterDim.y = static_cast<unsigned>(plan.split);
        attrs[num_attrs].val.clusterDim.z = 1;
        ++num_attrs;
    }
    if (use_pdl) {
        attrs[num_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[num_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++num_attrs;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = num_attrs;
    HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_gemm_fp8_sm100_kernel<kModeSwiglu>, tmap_w, tmap_a, p));
    return HFRK_SUCCESS;
}

}  // namespace
}  // namespace hfrk

// =============================================================================== no-allocation entry
namespace hfrk {
namespace {

// Some callers must not allocate device memory at the moment they call a GEMM: a serving engine
// that has handed the whole of HBM to its own pools at start-up (a later cudaMalloc would fail or
// fragment them), code that runs between two allocator check-points, a plug-in that is forbidden
// to touch the allocator of its host. For them the stream-K kernel is offered with its scratch in
// a fixed array that is part of the library image: nothing is allocated, ever. The price is that
// every GPU that loads the library carries the array until the process ends, that the sizes are
// capped, and that all calls share the one array.
//   partials : 2 slots per CTA x 296 CTAs x 16 tokens x 128 rows x 4 B  = 4,849,664 B
//   counters : one per 128-row tile, 4096 tiles (N <= 524,288)           =    16,384 B
constexpr int kStaticMaxTokens = 16;
constexpr int kStaticMaxTiles = 4096;
constexpr size_t kStaticPartialBytes = static_cast<size_t>(2) * kSkMaxGrid * kStaticMaxTokens * kTileN * sizeof(float);
constexpr size_t kStaticCounterBytes = static_cast<size_t>(kStaticMaxTiles) * sizeof(unsigned int);
}  // namespace
}  // namespace hfrk

static __device__ __align__(256) unsigned char g_static_scratch[hfrk::kStaticPartialBytes + hfrk::kStaticCounterBytes];

namespace hfrk {
namespace {

// In host code the array's name is only a handle for the runtime, not a device address; the
// address the kernel needs is asked for once per device, with that device current.
int static_scratch_address(unsigned char** out) {
    static std::mutex mu;
    static unsigned char* address[64] = {};
    int dev = 0;
    HFRK_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return HFRK_INVALID_CONFIG;
    std::lock_guard<std::mutex> lock(mu);
    if (address[dev] == nullptr) {
        void* ptr = nullptr;
        HFRK_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (ptr == nullptr) {
            set_last_error("cudaGetSymbolAddress returned no address for the static scratch array");
            return HFRK_CUDA_ERROR;
        }
        address[dev] = static_cast<unsigned char*>(ptr);
    }
    *out = address[dev];
    return HFRK_SUCCESS;
}

// Tensor map without the host-side cache (the cache grows a heap-allocated table).
int encode_tensor_map_uncached(const void* base, uint64_t inner, uint64_t outer, uint64_t stride, uint32_t box_outer,
                               CUtensorMap* out) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        set_last_error("cuTensorMapEncodeTiled is not available from the driver");
        return HFRK_CUDA_ERROR;
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {stride};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), box_outer};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult res = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed for the no-allocation entry point");
        return HFRK_CUDA_ERROR;
    }
    return HFRK_SUCCESS;
}

}  // namespace
}  // namespace hfrk

extern "C" int hfrk_skinny_gemm_fp8_noalloc(const void* A, const void* W, void* D, const float* scale_dev, int m,
                                            int n, int k, int64_t w_row_stride, int a_kind, int w_kind, int d_dtype,
                                            int accumulate, void* stream) {
    using namespace hfrk;
    int rc = validate(A, W, D, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype);
    if (rc != HFRK_SUCCESS) return rc;
    const int tiles = (n + kTileN - 1) / kTileN;
    if (m > kStaticMaxTokens || tiles > kStaticMaxTiles) {
        set_last_error("hfrk_skinny_gemm_fp8_noalloc: at most 16 tokens and N <= 524288 (fixed scratch array)");
        return HFRK_TOO_LARGE;
    }
    rc = prepare_device_once();
    if (rc != HFRK_SUCCESS) return rc;
    unsigned char* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc != HFRK_SUCCESS) return rc;
    SkPlan plan;
    rc = make_sk_plan(m, n, k, /*ctas_per_sm=*/2, /*stages_req=*/0, &plan);
    if (rc != HFRK_SUCCESS) return rc;
    if (plan.grid > kSkMaxGrid) return HFRK_TOO_LARGE;

    CUtensorMap tmap_w, tmap_a;
    rc = encode_tensor_map_uncached(W, static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                                    static_cast<uint64_t>(w_row_stride), kTileN, &tmap_w);
    if (rc != HFRK_SUCCESS) return rc;
    rc = encode_tensor_map_uncached(A, static_cast<uint64_t>(k), static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                                    static_cast<uint32_t>(plan.m_pad), &tmap_a);
    if (rc != HFRK_SUCCESS) return rc;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned int* counters = reinterpret_cast<unsigned int*>(scratch + kStaticPartialBytes);
    // The array keeps whatever the last call left. Partials are fully rewritten before they are
    // read; the tile counters must start at zero, so the ones this call uses are cleared here.
    HFRK_CUDA_TRY(cudaMemsetAsync(counters, 0, static_cast<size_t>(tiles) * sizeof(unsigned int), s));

    SkParams p;
    p.d = D;
    p.scale = scale_dev;
    p.kind_factor = (a_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f) * (w_kind == HFRK_E4M3FNUZ ? 0.5f : 1.0f);
    p.m = m;
    p.n = n;
    p.m_pad = plan.m_pad;
    p.nkb = plan.nkb;
    p.total_units = plan.tiles * plan.nkb;
    p.stages = plan.stages;
    p.d_dtype = d_dtype;
    p.accumulate = accumulate ? 1 : 0;
    p.partials = reinterpret_cast<float*>(scratch);
    p.counters = counters;
    p.stamps = nullptr;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(plan.grid), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(plan.smem_bytes);
    cfg.stream = s;
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
    if (plan.units_per_stage == 1) {
        HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_gemm_fp8_streamk_kernel<1>, tmap_w, tmap_a, p));
    } else {
        HFRK_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_gemm_fp8_streamk_kernel<2>, tmap_w, tmap_a, p));
    }
    return HFRK_SUCCESS;
}


// =============================================================================== row-parallel group
struct hfrk_rowpar {
    hfrk::RowparDev dev;
    uint8_t* local_block = nullptr;
    size_t block_bytes = 0;
    void* opened[hfrk::kMaxWorld] = {};   // peer mappings opened from IPC handles
    int device = 0;
    bool connected = false;
    int mode = HFRK_ROWPAR_AUTO;
};

extern "C" int hfrk_rowpar_create(int rank, int world, int max_m, int max_n, hfrk_rowpar** out) {
    if (out == nullptr || world < 1 || world > hfrk::kMaxWorld || rank < 0 || rank >= world || max_m < 1 ||
        max_n < 1)
        return HFRK_BAD_WORLD;
    const int tiles = (max_n + hfrk::kTileN - 1) / hfrk::kTileN;
    const int m_cap = max_m < 16 ? max_m : 16;  // larger M runs as launches of 16 tokens
    hfrk_rowpar* g = new hfrk_rowpar();
    g->dev.rank = rank;
    g->dev.world = world;
    g->dev.wait_cycles = hfrk::kWaitLimitCycles;
    g->dev.elems_per_src = static_cast<unsigned>(tiles) * m_cap * hfrk::kTileN;
    const size_t cells =
        (static_cast<size_t>(2) * (world + 1) * g->dev.elems_per_src * sizeof(uint2) + 255) / 256 * 256;
    g->block_bytes = cells + 256;
    cudaError_t err = cudaGetDevice(&g->device);
    if (err == cudaSuccess) err = cudaMalloc(&g->local_block, g->block_bytes);
    if (err == cudaSuccess) err = cudaMemset(g->local_block, 0, g->block_bytes);
    if (err != cudaSuccess) {
        hfrk::set_last_error(cudaGetErrorString(err));
        (void)cudaGetLastError();
        delete g;
        return HFRK_CUDA_ERROR;
    }
    g->dev.cells[rank] = reinterpret_cast<uint2*>(g->local_block);
    g->dev.call_index = reinterpret_cast<unsigned int*>(g->local_block + cells);
    g->dev.done_ctas = g->dev.call_index + 1;
    g->connected = world == 1;
    *out = g;
    return HFRK_SUCCESS;
}

extern "C" int hfrk_rowpar_ipc_handle(hfrk_rowpar* g, void* handle64_out) {
    if (g == nullptr || handle64_out == nullptr) return HFRK_BAD_WORLD;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t handle;
    HFRK_CUDA_TRY(cudaIpcGetMemHandle(&handle, g->local_block));
    memcpy(handle64_out, &handle, sizeof(handle));
    return HFRK_SUCCESS;
}

extern "C" int hfrk_rowpar_connect(hfrk_rowpar* g, const void* all_handles) {
    if (g == nullptr || all_handles == nullptr) return HFRK_BAD_WORLD;
    for (int peer = 0; peer < g->dev.world; ++peer) {
        if (peer == g->dev.rank) continue;
        cudaIpcMemHandle_t handle;
        memcpy(&handle, static_cast<const uint8_t*>(all_handles) + 64 * peer, sizeof(handle));
        void* mapped = nullptr;
        HFRK_CUDA_TRY(cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess));
        g->opened[peer] = mapped;
        g->dev.cells[peer] = static_cast<uint2*>(mapped);
    }
    g->connected = true;
    return HFRK_SUCCESS;
}

extern "C" int hfrk_rowpar_connect_pointers(hfrk_rowpar* g, void* const* peer_blocks) {
    if (g == nullptr || peer_blocks == nullptr) return HFRK_BAD_WORLD;
    for (int peer = 0; peer < g->dev.world; ++peer) {
        if (peer == g->dev.rank) continue;
        if (peer_blocks[peer] == nullptr) return HFRK_BAD_WORLD;
        g->dev.cells[peer] = static_cast<uint2*>(peer_blocks[peer]);
    }
    g->connected = true;
    return HFRK_SUCCESS;
}

extern "C" void* hfrk_rowpar_local_block(hfrk_rowpar* g) { return g == nullptr ? nullptr : g->local_block; }

extern "C" int hfrk_rowpar_destroy(hfrk_rowpar* g) {
    if (g == nullptr) return HFRK_SUCCESS;
    for (int peer = 0; peer < hfrk::kMaxWorld; ++peer) {
        if (g->opened[peer] != nullptr) (void)cudaIpcCloseMemHandle(g->opened[peer]);
    }
    if (g->local_block != nullptr) (void)cudaFree(g->local_block);
    delete g;
    return HFRK_SUCCESS;
}

extern "C" int hfrk_skinny_gemm_fp8_rowpar(hfrk_rowpar* g, const void* A, const void* W, void* D,
                                           const float* scale_dev, int m, int n, int k_shard, int64_t w_row_stride,
                                           int a_kind, int w_kind, int d_dtype, int accumulate, void* stream) {
    if (g == nullptr || !g->connected) return HFRK_BAD_WORLD;
    return hfrk::launch_gemm(A, W, D, scale_dev, m, n, k_shard, w_row_stride, a_kind, w_kind, d_dtype, accumulate,
                             HFRK_VARIANT_CLUSTER, 0, 0, 0, hfrk::default_use_pdl(), static_cast<cudaStream_t>(stream),
                             nullptr, &g->dev, g->mode);
}

extern "C" int hfrk_rowpar_set_wait_ms(hfrk_rowpar* g, int milliseconds) {
    if (g == nullptr) return HFRK_BAD_WORLD;
    if (milliseconds < 1 || milliseconds > 60000) return HFRK_INVALID_CONFIG;
    g->dev.wait_cycles = static_cast<long long>(milliseconds) * 2000000ll;   // SM clock ticks at ~2 GHz
    return HFRK_SUCCESS;
}

extern "C" int hfrk_rowpar_set_mode(hfrk_rowpar* g, int mode) {
    if (g == nullptr) return HFRK_BAD_WORLD;
    if (mode != HFRK_ROWPAR_AUTO && mode != HFRK_ROWPAR_ONE_SHOT && mode != HFRK_ROWPAR_TWO_SHOT)
        return HFRK_INVALID_CONFIG;
    g->mode = mode;
    return HFRK_SUCCESS;
}

// =============================================================================== C ABI

extern "C" int hfrk_skinny_gemm_fp8(const void* A, const void* W, void* D, const float* scale_dev, int m, int n,
                                    int k, int64_t w_row_stride, int a_kind, int w_kind, int d_dtype,
                                    int accumulate, int split_k_hint, void* stream) {
    if (split_k_hint < 0) return HFRK_INVALID_CONFIG;
    if (split_k_hint > hfrk::kMaxSplit) split_k_hint = hfrk::kMaxSplit;
    return hfrk::launch_gemm(A, W, D, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype, accumulate,
                             HFRK_VARIANT_AUTO, split_k_hint, 0, 0, hfrk::default_use_pdl(),
                             static_cast<cudaStream_t>(stream));
}

extern "C" int hfrk_skinny_gemm_fp8_swiglu(const void* A, const void* W_gate_up, void* act_out,
                                           const float* scale_dev, const float* act_scale_dev, void* next_buffer,
                                           int m, int inter, int k, int64_t w_row_stride, int a_kind, int w_kind,
                                           int mid_dtype, int out_kind, int64_t buffer_cols, void* stream) {
    return hfrk::launch_gemm_swiglu(A, W_gate_up, act_out, scale_dev, act_scale_dev, next_buffer, m, inter, k,
                                    w_row_stride, a_kind, w_kind, mid_dtype, out_kind, buffer_cols, /*split_req=*/0,
                                    hfrk::default_use_pdl(), static_cast<cudaStream_t>(stream));
}

extern "C" int hfrk_skinny_gemm_fp8_ex(const void* A, const void* W, void* D, const float* scale_dev, int m, int n,
                                       int k, int64_t w_row_stride, int a_kind, int w_kind, int d_dtype,
                                       int accumulate, int variant, int split_k, int ctas_per_sm, int num_stages,
                                       int use_pdl, void* stream) {
    return hfrk::launch_gemm(A, W, D, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype, accumulate, variant,
                             split_k, ctas_per_sm, num_stages, use_pdl, static_cast<cudaStream_t>(stream));
}

extern "C" int hfrk_skinny_gemm_fp8_profile(const void* A, const void* W, void* D, const float* scale_dev, int m,
                                            int n, int k, int64_t w_row_stride, int a_kind, int w_kind, int d_dtype,
                                            int accumulate, int variant, int split_k, int ctas_per_sm,
                                            int num_stages, int use_pdl, unsigned long long* stamps_dev,
                                            void* stream) {
    if (m > hfrk::kMaxMPad) return HFRK_TOO_LARGE;
    return hfrk::launch_gemm(A, W, D, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype, accumulate, variant,
                             split_k, ctas_per_sm, num_stages, use_pdl, static_cast<cudaStream_t>(stream), stamps_dev);
}

extern "C" int64_t hfrk_host_call_workspace_bytes(int m, int n, int k) {
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    const int64_t a_bytes = (static_cast<int64_t>(m) * k + 255) / 256 * 256;
    const int64_t d_bytes = (static_cast<int64_t>(m) * n * 4 + 255) / 256 * 256;
    return a_bytes + d_bytes;
}

namespace hfrk {
namespace {
int host_call(const void* A_host, const void* W_dev, void* D_host, const float* scale_dev, int m, int n, int k,
              int64_t w_row_stride, int a_kind, int w_kind, int d_dtype, int accumulate, void* work_dev, void* stream,
              bool synchronise);
}  // namespace
}  // namespace hfrk

extern "C" int hfrk_skinny_gemm_fp8_host(const void* A_host, const void* W_dev, void* D_host,
                                         const float* scale_dev, int m, int n, int k, int64_t w_row_stride,
                                         int a_kind, int w_kind, int d_dtype, int accumulate, void* work_dev,
                                         void* stream) {
    return hfrk::host_call(A_host, W_dev, D_host, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype,
                           accumulate, work_dev, stream, true);
}

extern "C" int hfrk_skinny_gemm_fp8_host_async(const void* A_host, const void* W_dev, void* D_host,
                                               const float* scale_dev, int m, int n, int k, int64_t w_row_stride,
                                               int a_kind, int w_kind, int d_dtype, int accumulate, void* work_dev,
                                               void* stream) {
    return hfrk::host_call(A_host, W_dev, D_host, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype,
                           accumulate, work_dev, stream, false);
}

namespace hfrk {
namespace {
int host_call(const void* A_host, const void* W_dev, void* D_host, const float* scale_dev, int m, int n, int k,
              int64_t w_row_stride, int a_kind, int w_kind, int d_dtype, int accumulate, void* work_dev, void* stream,
              bool synchronise) {
    if (A_host == nullptr || D_host == nullptr || work_dev == nullptr || m <= 0 || n <= 0 || k <= 0)
        return HFRK_INVALID_CONFIG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t a_bytes = static_cast<size_t>(m) * k;
    const size_t d_bytes = static_cast<size_t>(m) * n * (d_dtype == HFRK_F32 ? 4 : 2);
    uint8_t* a_dev = static_cast<uint8_t*>(work_dev);
    uint8_t* d_dev = a_dev + (a_bytes + 255) / 256 * 256;
    HFRK_CUDA_TRY(cudaMemcpyAsync(a_dev, A_host, a_bytes, cudaMemcpyHostToDevice, s));
    if (accumulate) HFRK_CUDA_TRY(cudaMemcpyAsync(d_dev, D_host, d_bytes, cudaMemcpyHostToDevice, s));
    int rc = hfrk::launch_gemm(a_dev, W_dev, d_dev, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype,
                               accumulate, HFRK_VARIANT_AUTO, 0, 0, 0, hfrk::default_use_pdl(), s);
    if (rc != HFRK_SUCCESS) return rc;
    HFRK_CUDA_TRY(cudaMemcpyAsync(D_host, d_dev, d_bytes, cudaMemcpyDeviceToHost, s));
    if (synchronise) HFRK_CUDA_TRY(cudaStreamSynchronize(s));
    return HFRK_SUCCESS;
}
}  // namespace
}  // namespace hfrk

extern "C" int hfrk_skinny_gemm_plan(int m, int n, int k, int variant, int split_k, int ctas_per_sm, int* out8) {
    if (out8 == nullptr || variant < HFRK_VARIANT_AUTO || variant > HFRK_VARIANT_STREAMK) return HFRK_INVALID_CONFIG;
    const int mc = m > hfrk::kMaxMPad ? hfrk::kMaxMPad : m;
    if (variant == HFRK_VARIANT_AUTO) variant = HFRK_VARIANT_CLUSTER;
    if (variant == HFRK_VARIANT_CLUSTER) {
        hfrk::Plan plan;
        int rc = hfrk::make_plan(mc, n, k, split_k, 0, &plan);
        if (rc != HFRK_SUCCESS) return rc;
        out8[0] = variant; out8[1] = plan.split; out8[2] = plan.stages; out8[3] = plan.ctas;
        out8[4] = plan.smem_bytes; out8[5] = plan.m_pad; out8[6] = plan.num_kblocks;
        out8[7] = plan.tiles;
        return HFRK_SUCCESS;
    }
    hfrk::SkPlan plan;
    int rc = hfrk::make_sk_plan(mc, n, k, ctas_per_sm, 0, &plan);
    if (rc != HFRK_SUCCESS) return rc;
    out8[0] = variant; out8[1] = 0; out8[2] = plan.stages; out8[3] = plan.grid;
    out8[4] = plan.smem_bytes; out8[5] = plan.m_pad; out8[6] = plan.nkb; out8[7] = plan.tiles;
    return HFRK_SUCCESS;
}

extern "C" int hfrk_tuning_set_ex(int m, int n, int k, int split_k, int num_stages, int tile_rows) {
    if (m <= 0 || n <= 0 || k <= 0 || split_k < 0 || split_k > hfrk::kMaxSplit || num_stages < 0 || num_stages == 1 ||
        num_stages > hfrk::kMaxStages || tile_rows < 0 || tile_rows > hfrk::kTileN || (tile_rows > 0 && tile_rows < 8))
        return HFRK_INVALID_CONFIG;
    const int m_pad = hfrk::round_up(m > hfrk::kMaxMPad ? hfrk::kMaxMPad : m, 16);
    std::lock_guard<std::mutex> lock(hfrk::g_tune_mutex);
    if (split_k == 0 && num_stages == 0 && tile_rows == 0) {
        hfrk::g_tune_table.erase(hfrk::TuneKey{m_pad, n, k});
    } else {
        hfrk::g_tune_table[hfrk::TuneKey{m_pad, n, k}] = hfrk::TuneValue{split_k, num_stages, tile_rows};
    }
    return HFRK_SUCCESS;
}

extern "C" int hfrk_tuning_set(int m, int n, int k, int split_k, int num_stages) {
    return hfrk_tuning_set_ex(m, n, k, split_k, num_stages, 0);
}

extern "C" int hfrk_tuning_clear(void) {
    std::lock_guard<std::mutex> lock(hfrk::g_tune_mutex);
    hfrk::g_tune_table.clear();
    return HFRK_SUCCESS;
}

extern "C" int hfrk_max_active_clusters(int split, int smem_bytes, int* clusters_out) {
    if (clusters_out == nullptr || split < 1 || split > hfrk::kMaxSplit || smem_bytes < 0 || smem_bytes > hfrk::kSmemLimit)
        return HFRK_INVALID_CONFIG;
    int rc = hfrk::prepare_device_once();
    if (rc != HFRK_SUCCESS) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, static_cast<unsigned>(split), 1);
    cfg.blockDim = dim3(hfrk::kThreads, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1;
    attr.val.clusterDim.y = static_cast<unsigned>(split);
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    HFRK_CUDA_TRY(cudaOccupancyMaxActiveClusters(&clusters, hfrk::skinny_gemm_fp8_sm100_kernel<hfrk::kModePlain>, &cfg));
    *clusters_out = clusters;
    return HFRK_SUCCESS;
}

extern "C" int hfrk_device_status(int clear, unsigned int* word_out) {
    unsigned int word = 0;
    HFRK_CUDA_TRY(cudaMemcpyFromSymbol(&word, hfrk::g_device_status, sizeof(word)));
    if (clear && word != 0) {
        const unsigned int zero = 0;
        HFRK_CUDA_TRY(cudaMemcpyToSymbol(hfrk::g_device_status, &zero, sizeof(zero)));
        // A kernel that gave up may have left tile counters of the stream-K scratch non-zero.
        int dev = 0;
        HFRK_CUDA_TRY(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(hfrk::g_scratch_mutex);
        if (dev >= 0 && dev < 64 && hfrk::g_scratch[dev].ready) {
            for (int l = 0; l < hfrk::kScratchLanes; ++l) {
                HFRK_CUDA_TRY(cudaMemset(hfrk::g_scratch[dev].counters[l], 0,
                                         static_cast<size_t>(hfrk::kSkMaxTiles) * sizeof(unsigned int)));
            }
        }
    }
    if (word_out != nullptr) *word_out = word;
    return word == 0 ? HFRK_SUCCESS : HFRK_DEVICE_TIMEOUT;
}
