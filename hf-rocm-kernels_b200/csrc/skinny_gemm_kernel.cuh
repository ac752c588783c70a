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
// A cell is written with ONE 8-byte scalar store, so its reader sees value and epoch together: a cell
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
    int rows_log2;       // split > 1: CTA q of a cluster finishes token rows [q << rows_log2, (q + 1) << rows_log2)
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
// A cell is ONE 64-bit scalar access: value in the low word, epoch in the high word. A scalar access
// of eight aligned bytes is single-copy atomic, so a reader never sees the new epoch beside an old
// value (the two halves of a vector access carry no such promise).
__device__ __forceinline__ void st_relaxed_sys_v2(uint2* ptr, uint32_t x, uint32_t y) {
    const unsigned long long cell = (static_cast<unsigned long long>(y) << 32) | x;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(ptr), "l"(cell) : "memory");
}

__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const uint2* ptr) {
    unsigned long long cell;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(cell) : "l"(ptr) : "memory");
    return make_uint2(static_cast<uint32_t>(cell), static_cast<uint32_t>(cell >> 32));
}

// All-reduce of the values this thread owns, fused into the GEMM epilogue. `val` holds CNT partial
// sums of which the first `valid` are in use; element i sits at index slot0 + i * 128 of the exchange
// buffer (consecutive token rows of one output column: no per-element index is kept in registers). All ranks run
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
template <int CNT, int WORLD>
__device__ __forceinline__ bool rowpar_exchange_impl(const RowparDev& rp, unsigned int epoch, uint32_t slot0, int valid,
                                                float (&val)[CNT], volatile uint32_t* abort_flag) {
    // WORLD > 0: the group size is known at compile time, so the loops over the ranks unroll to exactly
    // that many cells; WORLD == 0 is the general form (any size up to kMaxWorld).
    constexpr int kSrcs = WORLD > 0 ? WORLD : kMaxWorld;
    const int world = WORLD > 0 ? WORLD : rp.world;
    const unsigned int parity = epoch & 1u;
    const size_t sources = static_cast<size_t>(world) + 1;
    const int owner = rp.two_shot ? static_cast<int>((blockIdx.x + blockIdx.y) % static_cast<unsigned>(world)) : -1;
    const bool gather = !rp.two_shot || owner == rp.rank;   // this thread adds up the ranks' partials
    const size_t my_src = parity * sources + static_cast<size_t>(rp.rank);
    for (int peer = 0; peer < world; ++peer) {
        if (peer == rp.rank || (rp.two_shot && peer != owner)) continue;
        uint2* dst = rp.cells[peer] + my_src * rp.elems_per_src;
#pragma unroll
        for (int i = 0; i < CNT; ++i) {
            if (i < valid) st_relaxed_sys_v2(dst + slot0 + i * kTileN, __float_as_uint(val[i]), epoch);
        }
    }
    // Cells are fetched a batch at a time (4 elements x up to 3 peers, or 2 x 7, in flight per thread) and the
    // batch is re-read until every cell shows the epoch; batches of unused elements are skipped,
    // which is the common case: a thread usually owns two or three elements of the tile.
    constexpr int kBatch = kSrcs > 4 ? 2 : 4;   // cells in flight per thread: kBatch x (ranks - 1)
    bool ok = true;
    const long long start = clock64();
    const uint2* const mine = rp.cells[rp.rank] + parity * sources * rp.elems_per_src;
#pragma unroll
    for (int i0 = 0; i0 < CNT; i0 += kBatch) {
        if (i0 >= valid || !ok) continue;
        if (gather) {
            uint32_t got[kBatch][kSrcs];
            for (;;) {
                bool ready = true;
#pragma unroll
                for (int b = 0; b < kBatch; ++b) {
#pragma unroll
                    for (int src = 0; src < kSrcs; ++src) {
                        got[b][src] = 0u;
                        if (src < world && src != rp.rank && i0 + b < valid) {
                            const uint2 cell =
                                ld_relaxed_sys_v2(mine + static_cast<size_t>(src) * rp.elems_per_src + slot0 + (i0 + b) * kTileN);
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
                for (int src = 0; src < kSrcs; ++src) {
                    if (src < world) sum += (src == rp.rank) ? val[i0 + b] : __uint_as_float(got[b][src]);
                }
                val[i0 + b] = sum;
            }
            if (rp.two_shot) {
                // the owner hands the finished sums to everyone else
                const size_t fin = (parity * sources + static_cast<size_t>(world)) * rp.elems_per_src;
                for (int peer = 0; peer < world; ++peer) {
                    if (peer == rp.rank) continue;
#pragma unroll
                    for (int b = 0; b < kBatch; ++b) {
                        if (i0 + b < valid)
                            st_relaxed_sys_v2(rp.cells[peer] + fin + slot0 + (i0 + b) * kTileN, __float_as_uint(val[i0 + b]), epoch);
                    }
                }
            }
        } else {
            // not the owner: wait for the finished sums
            const uint2* const fin = mine + static_cast<size_t>(world) * rp.elems_per_src;
            uint32_t got[kBatch];
            for (;;) {
                bool ready = true;
#pragma unroll
                for (int b = 0; b < kBatch; ++b) {
                    got[b] = 0u;
                    if (i0 + b < valid) {
                        const uint2 cell = ld_relaxed_sys_v2(fin + slot0 + (i0 + b) * kTileN);
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
                if (i0 + b < valid) val[i0 + b] = __uint_as_float(got[b]);
            }
        }
    }
    return ok;
}

// The exchange for the group sizes that matter (2, 4 and 8 GPUs) is compiled for its size: the
// epilogue threads run alone on their schedulers, and the general form's loops over eight possible
// ranks, most of them predicated off, cost microseconds of issue time per call. kWorld = 0 is the
// general form.
template <int CNT, int kWorld>
__device__ __forceinline__ bool rowpar_exchange(const RowparDev& rp, unsigned int epoch, uint32_t slot0, int valid,
                                                float (&val)[CNT], volatile uint32_t* abort_flag) {
    return rowpar_exchange_impl<CNT, kWorld>(rp, epoch, slot0, valid, val, abort_flag);
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
constexpr int kEpiPitch = kTileN + 4;  // floats per token row of the transposed tile staged in shared memory
constexpr int kOwned = 8;              // token rows per owner kept in registers in the split-K reduction

__device__ __forceinline__ float round_trip_16(float x, int dtype) {
    return dtype == HFRK_BF16 ? __bfloat162float(__float2bfloat16_rn(x)) : __half2float(__float2half_rn(x));
}

// ---------------------------------------------------------------- output accessors, one per D type
// The epilogue is compiled once per output type: every warp of it runs alone on its scheduler, so
// its time is its instruction count, and a type switch per element doubled that count.
template <int DT>
__device__ __forceinline__ float load1(const void* d, size_t idx) {
    if constexpr (DT == HFRK_F32) return static_cast<const float*>(d)[idx];
    if constexpr (DT == HFRK_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(d)[idx]);
    return __half2float(static_cast<const __half*>(d)[idx]);
}

template <int DT>
__device__ __forceinline__ void store1(void* d, size_t idx, float v) {
    if constexpr (DT == HFRK_F32) {
        static_cast<float*>(d)[idx] = v;
    } else if constexpr (DT == HFRK_BF16) {
        static_cast<__nv_bfloat16*>(d)[idx] = __float2bfloat16_rn(v);
    } else {
        static_cast<__half*>(d)[idx] = __float2half_rn(v);
    }
}

template <int DT>
__device__ __forceinline__ constexpr int out_bytes() { return DT == HFRK_F32 ? 4 : 2; }

// Sixteen consecutive outputs as raw 16-byte words (two for the 16-bit types, four for float).
template <int DT>
struct Raw16 {
    uint4 q[DT == HFRK_F32 ? 4 : 2];
};

template <int DT>
__device__ __forceinline__ Raw16<DT> load_raw16(const void* d, size_t idx) {
    Raw16<DT> r;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(d) + idx * out_bytes<DT>());
#pragma unroll
    for (int i = 0; i < (DT == HFRK_F32 ? 4 : 2); ++i) r.q[i] = src[i];
    return r;
}

template <int DT>
__device__ __forceinline__ void decode16(const Raw16<DT>& r, float (&x)[16]) {
    if constexpr (DT == HFRK_F32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[4 * i] = __uint_as_float(r.q[i].x);
            x[4 * i + 1] = __uint_as_float(r.q[i].y);
            x[4 * i + 2] = __uint_as_float(r.q[i].z);
            x[4 * i + 3] = __uint_as_float(r.q[i].w);
        }
    } else {
        const uint32_t w[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float2 f;
            if constexpr (DT == HFRK_BF16) {
                f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            } else {
                f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            }
            x[2 * i] = f.x;
            x[2 * i + 1] = f.y;
        }
    }
}

template <int DT>
__device__ __forceinline__ void store16(void* d, size_t idx, const float (&y)[16]) {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(d) + idx * out_bytes<DT>());
    if constexpr (DT == HFRK_F32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dst[i] = make_uint4(__float_as_uint(y[4 * i]), __float_as_uint(y[4 * i + 1]), __float_as_uint(y[4 * i + 2]),
                                __float_as_uint(y[4 * i + 3]));
        }
    } else {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if constexpr (DT == HFRK_BF16) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
                const __half2 h = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
}

// What the epilogue functions share.
struct EpiCtx {
    Ctrl* ctrl;
    uint8_t* ring_ptr;      // start of the (by then idle) stage ring
    uint32_t recv_addr;     // shared-memory address of the receive buffer (recv_float_index)
    uint32_t recv_bar;
    uint32_t accum_bar;
    uint32_t lane_taddr;    // TMEM address of this thread's lane, column 0
    int rank;               // CTA rank in the cluster (0 without a K split)
    int n0;                 // first W row of the tile
    float scale;
};

// Receive buffer of an owner of token rows: float [sender][group][128 threads][rows per group] with
// rows per group = min(rpo, 4) = what one asynchronous store carries. The 128 threads' pieces of a
// group lie side by side, so the stores of a warp cover one contiguous run of the owner's shared
// memory; with the pieces of one thread side by side instead (a stride of 32 or 64 bytes between
// lanes once rpo reaches 8) every 16 token rows cost 1.3 us instead of 0.26 us.
__device__ __forceinline__ uint32_t recv_float_index(int sender, int tid, int row_in_owner, int rows_log2) {
    const int g_log2 = rows_log2 < 2 ? rows_log2 : 2;
    const int groups_log2 = rows_log2 - g_log2;
    return static_cast<uint32_t>(((((sender << groups_log2) + (row_in_owner >> g_log2)) * kTileN + tid) << g_log2) +
                                 (row_in_owner & ((1 << g_log2) - 1)));
}

// Sends 16 token rows (c0 .. c0 + 15) of this thread's W row to the CTAs that finish them. Token
// row r goes to CTA r >> rows_log2, row r & (rpo - 1) of this sender's block there. Rows leave
// 1, 2 or 4 at a time (min(rpo, 4)); a group never straddles two owners because its size divides
// rpo. An owner expects whole blocks, so the rows of its range past m are sent as they are.
__device__ __forceinline__ void send_partial_rows(const GemmParams& p, const EpiCtx& cx, int c0, const uint32_t (&v)[16]) {
    const int rpo = 1 << p.rows_log2;
    const uint32_t send_base = cx.recv_addr + (static_cast<uint32_t>(cx.rank) * kTileN + threadIdx.x) * (4u << p.rows_log2);
    if (rpo >= 4) {
#pragma unroll
        for (int g = 0; g < 16; g += 4) {
            const int r0 = c0 + g;
            const uint32_t q = static_cast<uint32_t>(r0 >> p.rows_log2);
            if (static_cast<int>(q << p.rows_log2) < p.m) {
                const uint32_t at = cx.recv_addr + 4u * recv_float_index(cx.rank, threadIdx.x, r0 & (rpo - 1), p.rows_log2);
                st_async_v4_b32(dsmem_map(at, q), v[g], v[g + 1], v[g + 2], v[g + 3], dsmem_map(cx.recv_bar, q));
            }
        }
    } else if (rpo == 2) {
#pragma unroll
        for (int g = 0; g < 16; g += 2) {
            const int r = c0 + g;
            if (r < p.m) {
                const uint32_t q = static_cast<uint32_t>(r >> 1);
                st_async_v2_b32(dsmem_map(send_base, q), v[g], v[g + 1], dsmem_map(cx.recv_bar, q));
            }
        }
    } else {
#pragma unroll
        for (int g = 0; g < 16; ++g) {
            const int r = c0 + g;
            if (r < p.m) {
                st_async_b32(dsmem_map(send_base, static_cast<uint32_t>(r)), v[g], dsmem_map(cx.recv_bar, static_cast<uint32_t>(r)));
            }
        }
    }
}

// Waits (bounded) for the accumulator; with a K split also for the start-up cluster barrier, after
// which the peers' receive barriers are known to exist and to be armed. False if the CTA gave up.
__device__ __forceinline__ bool wait_accumulator(const GemmParams& p, const EpiCtx& cx) {
    bool ok = mbar_wait_bounded(cx.accum_bar, 0u, &cx.ctrl->abort, kRoleEpilogue);
    ok = __all_sync(0xffffffffu, ok) && cx.ctrl->abort == 0u;
    ok = __all_sync(0xffffffffu, ok);
    if (threadIdx.x == 0) stamp(p, 5);
    tcgen05_fence_after_sync();
    if (p.split > 1) cluster_wait_acquire();
    return ok;
}

// Epilogue of the plain and the row-parallel kernel for output type DT, run by the 128 epilogue
// threads. Thread t holds TMEM lane t = W row n0 + t of the tile, 16 token rows per TMEM load.
//
// Without a K split the tile is turned in shared memory (the idle ring) so that the stores run
// along D's rows: work item (token row, 16 consecutive outputs) -> one thread, 32-byte loads of
// D_in and 32-byte stores; with 16 tokens that is exactly one item per thread, whose D_in is
// requested before the accumulator is waited for. Ragged or unaligned items fall back to
// element-wise accesses.
//
// With a K split every CTA sends its partial rows to their owners (send_partial_rows), an owner
// waits for all `split` blocks and thread t adds up and stores column t of the owner's rows.
template <int kMode, int DT, int kWorld>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, const EpiCtx& cx) {
    constexpr bool kRowPar = kMode == kModeRowPar;
    const int tid = threadIdx.x;
    const int n = cx.n0 + tid;
    const bool direct = p.split == 1;
    const int lim_cols = min(p.tile_rows, p.n - cx.n0);          // outputs of this tile that exist
    const bool lane_valid = tid < lim_cols;
    const int rpo = 1 << p.rows_log2;
    unsigned int epoch = 0;
    if (kRowPar) {
        epoch = *reinterpret_cast<volatile unsigned int*>(p.rp.call_index) + 1u;
        if (tid == 0) {
            // Once every CTA of the grid has read the call index it may move on: the last CTA to
            // say so closes the call. The count is taken here, not at the end of the kernel, so
            // that the round trip is hidden behind the wait for the accumulator; its operand is
            // derived from the loaded index, so the load is performed before the count is.
            unsigned int one;
            asm volatile("{\n\t.reg .u32 t;\n\tand.b32 t, %1, 0;\n\tadd.u32 %0, t, 1;\n\t}" : "=r"(one) : "r"(epoch));
            const unsigned int ctas = gridDim.x * gridDim.y;
            if (atomicAdd(p.rp.done_ctas, one) == ctas - 1u) {
                *p.rp.done_ctas = 0u;
                *reinterpret_cast<volatile unsigned int*>(p.rp.call_index) = epoch;
            }
        }
    }
    const uint32_t tile_slot0 = blockIdx.x * static_cast<uint32_t>(p.m * kTileN);

    // D_in of this thread's first work item, requested long before it is needed.
    const int item_row = tid >> 3, item_col = (tid & 7) * 16;
    const size_t item_idx = static_cast<size_t>(item_row) * p.n + cx.n0 + item_col;
    const bool item_vec = direct && item_row < p.m && item_col + 16 <= lim_cols &&
                          ((reinterpret_cast<uintptr_t>(p.d) + item_idx * out_bytes<DT>()) & 15u) == 0;
    Raw16<DT> din_raw;
#pragma unroll
    for (int i = 0; i < (DT == HFRK_F32 ? 4 : 2); ++i) din_raw.q[i] = make_uint4(0, 0, 0, 0);
    if (item_vec && p.accumulate) din_raw = load_raw16<DT>(p.d, item_idx);
    const int own_row0 = cx.rank << p.rows_log2;                  // first token row this CTA finishes (split > 1)
    float d_own[kOwned];
#pragma unroll
    for (int it = 0; it < kOwned; ++it) {
        const int row = own_row0 + it;
        d_own[it] = (!direct && p.accumulate && it < rpo && row < p.m && lane_valid)
                        ? load1<DT>(p.d, static_cast<size_t>(row) * p.n + n)
                        : 0.0f;
    }

    bool ok = wait_accumulator(p, cx);
    float* const tile = reinterpret_cast<float*>(cx.ring_ptr);   // [m_pad][kEpiPitch], direct path only
    if (ok) {
        for (int c = 0; c < p.m_pad; c += 16) {
            uint32_t v[16];
            tmem_ld_32x32b_x16(cx.lane_taddr + static_cast<uint32_t>(c), v);
            tmem_ld_wait();
            if (!direct) {
                send_partial_rows(p, cx, c, v);
                continue;
            }
            if (kRowPar) {
                // host guarantees m <= 16 here: one load, 16 values per thread
                float val[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) val[j] = __uint_as_float(v[j]);
                if (!rowpar_exchange<16, kWorld>(p.rp, epoch, tile_slot0 + static_cast<uint32_t>(tid), min(p.m, 16), val,
                                                 &cx.ctrl->abort))
                    ok = false;
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(val[j]);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) tile[(c + j) * kEpiPitch + tid] = __uint_as_float(v[j]);
        }
    }
    if (direct) {
        // every thread reaches the barrier, also after a wait that ran out (then nothing is stored)
        asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueThreads) : "memory");
        if (!ok || cx.ctrl->abort != 0u) return;
        const int items = p.m * 8;
        for (int item = tid; item < items; item += kEpilogueThreads) {
            const int row = item >> 3;
            if (item_col >= lim_cols) break;                     // same column group in every pass
            const float4* src = reinterpret_cast<const float4*>(tile + row * kEpiPitch + item_col);
            float x[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 f = src[i];
                x[4 * i] = f.x; x[4 * i + 1] = f.y; x[4 * i + 2] = f.z; x[4 * i + 3] = f.w;
            }
            const size_t idx = static_cast<size_t>(row) * p.n + cx.n0 + item_col;
            const bool vec = item_col + 16 <= lim_cols &&
                             ((reinterpret_cast<uintptr_t>(p.d) + idx * out_bytes<DT>()) & 15u) == 0;
            if (vec) {
                float y[16];
                if (p.accumulate) {
                    if (item == tid) {
                        decode16<DT>(din_raw, y);
                    } else {
                        decode16<DT>(load_raw16<DT>(p.d, idx), y);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) y[j] = fmaf(x[j], cx.scale, y[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) y[j] = x[j] * cx.scale;
                }
                store16<DT>(p.d, idx, y);
            } else {
#pragma unroll 1
                for (int j = 0; j < 16; ++j) {
                    if (item_col + j < lim_cols) {
                        const float d0 = p.accumulate ? load1<DT>(p.d, idx + j) : 0.0f;
                        store1<DT>(p.d, idx + j, fmaf(tile[row * kEpiPitch + item_col + j], cx.scale, d0));
                    }
                }
            }
        }
        return;
    }

    const bool owner = own_row0 < p.m;
    bool landed = ok && (!owner || mbar_wait_bounded(cx.recv_bar, 0u, &cx.ctrl->abort, kRoleEpilogue));
    landed = __all_sync(0xffffffffu, landed);
    if (!landed || !owner) return;
    const float* const recv = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(cx.ctrl) + kCtrlBytes);
    const float* const mine = recv + recv_float_index(0, tid, 0, p.rows_log2);   // [sender] at a stride of 128 * rpo
    const int sender_stride = kTileN << p.rows_log2;
    float own[kOwned];
#pragma unroll
    for (int it = 0; it < kOwned; ++it) own[it] = 0.0f;
    // rank order; each sender's rows for this thread are rpo consecutive floats
    if (rpo == 1) {
#pragma unroll 4
        for (int q = 0; q < p.split; ++q) own[0] += mine[q * sender_stride];
    } else if (rpo == 2) {
#pragma unroll 4
        for (int q = 0; q < p.split; ++q) {
            const float2 f = *reinterpret_cast<const float2*>(mine + q * sender_stride);
            own[0] += f.x; own[1] += f.y;
        }
    } else {
#pragma unroll 2
        for (int q = 0; q < p.split; ++q) {
            const float4 f = *reinterpret_cast<const float4*>(mine + q * sender_stride);
            own[0] += f.x; own[1] += f.y; own[2] += f.z; own[3] += f.w;
            if (rpo >= 8) {
                const float4 g = *reinterpret_cast<const float4*>(mine + q * sender_stride + 4 * kTileN);   // second group
                own[4] += g.x; own[5] += g.y; own[6] += g.z; own[7] += g.w;
            }
        }
    }
    if (kRowPar) {
        const int valid = max(0, min(min(rpo, kOwned), p.m - own_row0));
        if (!rowpar_exchange<kOwned, kWorld>(p.rp, epoch, tile_slot0 + static_cast<uint32_t>(own_row0 * kTileN + tid), valid,
                                             own, &cx.ctrl->abort))
            return;
    }
    if (!lane_valid) return;
    {
        const int rows = min(min(rpo, kOwned), p.m - own_row0);
        size_t idx = static_cast<size_t>(own_row0) * p.n + n;
#pragma unroll
        for (int it = 0; it < kOwned; ++it) {
            if (it < rows) store1<DT>(p.d, idx, fmaf(own[it], cx.scale, d_own[it]));
            idx += p.n;
        }
    }
    // more than 16 tokens with a small split: an owner finishes more than kOwned rows, four at a time
    for (int g = kOwned / 4; g < (rpo >> 2); ++g) {
        const int row0 = own_row0 + 4 * g;
        if (row0 >= p.m) break;
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int q = 0; q < p.split; ++q) {
            const float4 f = *reinterpret_cast<const float4*>(mine + q * sender_stride + g * 4 * kTileN);
            sum.x += f.x; sum.y += f.y; sum.z += f.z; sum.w += f.w;
        }
        const float part[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (row0 + j < p.m) {
                const size_t idx = static_cast<size_t>(row0 + j) * p.n + n;
                const float d0 = p.accumulate ? load1<DT>(p.d, idx) : 0.0f;
                store1<DT>(p.d, idx, fmaf(part[j], cx.scale, d0));
            }
        }
    }
}

// Epilogue of the gate/up kernel: fp8(silu(gate) * up / act_scale) instead of the projection, then
// the grid zeroes the down projection's accumulate buffer.
__device__ __forceinline__ void epilogue_swiglu(const GemmParams& p, const EpiCtx& cx) {
    const int tid = threadIdx.x;
    const bool direct = p.split == 1;
    const bool ok = wait_accumulator(p, cx);
    float* const partial = reinterpret_cast<float*>(cx.ring_ptr);  // the ring is idle by now
    if (direct) {
        // Lanes 0..63 hold gate columns, lanes 64..127 the matching up columns. The projection is
        // rounded to the 16-bit type first, as the unfused chain stores it, so both give the same
        // bytes. The activation is shared out by tokens: the gate thread of a column takes tokens
        // 0..7, the up thread tokens 8..15, and each hands the other the eight values it needs.
        constexpr int kPitch = 9;                        // floats per column: no bank conflicts
        float* const handed = partial;                   // [2][64][9]: up for tokens 0..7, gate for 8..15
        uint8_t* const out_tile = reinterpret_cast<uint8_t*>(partial + 2 * kHalfTile * kPitch);  // [16][64]
        const int col_in_tile = tid & (kHalfTile - 1);
        const int half = tid >> 6;                        // 0: this lane holds gate values, 1: up values
        float y[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) y[j] = 0.0f;
        if (ok) {
            uint32_t v[16];
            tmem_ld_32x32b_x16(cx.lane_taddr, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) y[j] = round_trip_16(__uint_as_float(v[j]) * cx.scale, p.d_dtype);
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
        if (tid < kHalfTile && ok) {
            const int token = tid >> 2, piece = tid & 3;
            const int col = static_cast<int>(blockIdx.x) * kHalfTile + piece * 16;
            if (token < p.m && col < p.act_cols) {   // act_cols % 16 == 0: a piece is inside or outside
                *reinterpret_cast<uint4*>(p.act_out + static_cast<size_t>(token) * p.act_cols + col) =
                    *reinterpret_cast<const uint4*>(out_tile + token * kHalfTile + piece * 16);
            }
        }
    } else {
        if (ok) {
            uint32_t v[16];
            tmem_ld_32x32b_x16(cx.lane_taddr, v);
            tmem_ld_wait();
            send_partial_rows(p, cx, 0, v);
        }
        const bool owner = (cx.rank << p.rows_log2) < p.m;
        bool landed = ok && (!owner || mbar_wait_bounded(cx.recv_bar, 0u, &cx.ctrl->abort, kRoleEpilogue));
        landed = __all_sync(0xffffffffu, landed);
        // This CTA owns `rows` whole token rows of the tile, starting at token t0; thread
        // tid holds lane tid of each. Same activation as in the unsplit case: the gate lane
        // of a column takes the first half of the tokens, the up lane the second half.
        const float* const recv = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(cx.ctrl) + kCtrlBytes);
        const int per_owner = 1 << p.rows_log2;                                      // <= 8 for m <= 16, split >= 2
        const int t0 = cx.rank << p.rows_log2;
        const int rows = landed ? (p.m - t0 < per_owner ? p.m - t0 : per_owner) : 0;   // may be <= 0
        const int first_half = (per_owner + 1) / 2;
        constexpr int kPitch = 5;                                        // floats per column and half
        float* const handed = partial;                                   // the idle ring
        uint8_t* const out_tile = reinterpret_cast<uint8_t*>(handed + 2 * kHalfTile * kPitch);  // [8][64]
        const int col_in_tile = tid & (kHalfTile - 1);
        const int half = tid >> 6;
        float y[kOwned];
#pragma unroll
        for (int it = 0; it < kOwned; ++it) {
            float sum = 0.0f;
            if (it < rows) {
                for (int q = 0; q < p.split; ++q) sum += recv[recv_float_index(q, tid, it, p.rows_log2)];
        }
            y[it] = round_trip_16(sum * cx.scale, p.d_dtype);
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
        if (tid < 4 * rows) {
            const int row = tid >> 2, piece = tid & 3;
            const int col = static_cast<int>(blockIdx.x) * kHalfTile + piece * 16;
            if (col < p.act_cols) {
                *reinterpret_cast<uint4*>(p.act_out + static_cast<size_t>(t0 + row) * p.act_cols + col) =
                    *reinterpret_cast<const uint4*>(out_tile + row * kHalfTile + piece * 16);
        }
        }
        }
    // the next GEMM adds into this buffer: the whole grid clears it
    const size_t cta = static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x;
    const size_t ctas = static_cast<size_t>(gridDim.x) * gridDim.y;
    const size_t vecs = static_cast<size_t>(p.zero_bytes / 16);
    for (size_t i = cta * kEpilogueThreads + threadIdx.x; i < vecs; i += ctas * kEpilogueThreads) {
        reinterpret_cast<uint4*>(p.zero_ptr)[i] = make_uint4(0, 0, 0, 0);
    }
}

#ifndef HFRK_MIN_CTAS
#define HFRK_MIN_CTAS 2
#endif
// kDT / kWorld: the plain and the gate/up kernel decide the output type at run time (kDT = -1); the
// row-parallel kernel is instantiated per output type and group size (2, 4, 8, or 0 = any), because
// one kernel holding every exchange variant needed 168 registers with spills and cost 2-3 us per
// call more than the plain kernel even in a group of one. It is compiled for three CTAs per SM
// (96 registers; a few tens of bytes spill in the exchange) so that it runs the launch shapes the
// planner picks for the plain kernel. A plain cap of 112 registers (3 x 192 x 112 <= 65536) does not
// do: the SM then holds two CTAs and the fused call at two GPUs goes from 22.9 to 29.5 us.
template <int kMode, int kDT = -1, int kWorld = 0>
__global__ void __launch_bounds__(kThreads, kMode == kModeRowPar ? 3 : HFRK_MIN_CTAS)
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
            // An owner of token rows expects one block of [128][rows] floats from every CTA of the
            // cluster: the rows of its range that exist in the padded tile (the last owner's range
            // may reach past it).
            if (p.split > 1 && (rank << p.rows_log2) < p.m) {
                const int first = rank << p.rows_log2;
                const int rpo = 1 << p.rows_log2;
                const int rows_sent = (first + rpo <= p.m_pad ? first + rpo : p.m_pad) - first;
                mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>(p.split) * kTileN * rows_sent * 4u);
            }
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
    // it is only waited for much later, right before partials are pushed to the peers. Only the
    // producer warp, which initialised them, arrives with release semantics: the release costs the
    // arriving thread ~1.8 us (measured from CTA entry to the end of set-up with and without a
    // cluster), and the MMA thread would spend it in front of its first K block.
    if (p.split > 1) {
        if (warp == kProducerWarp) {
            cluster_arrive_release();
        } else {
            cluster_arrive_relaxed();
        }
    }
    const uint32_t tmem_acc = ctrl->tmem_base;
    if (threadIdx.x == 0) stamp(p, 1);

    // The two single-thread loops below run alone on their schedulers, so their speed is their
    // instruction count: stage index, parity and addresses are carried along instead of being
    // derived from the block index (a division by the runtime stage count costs tens of cycles).
    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int issued = prologue;
            uint32_t s = 0, parity = 0, stage_addr = ring_addr;   // block `stages` re-uses stage 0, first round
            int k_coord = (kb_start + prologue) * kBlockK;
            for (int i = prologue; i < kb_count; ++i) {
                if (!mbar_wait_bounded(empty_bar + 8u * s, parity, &ctrl->abort, kRoleProducer)) break;
                mbar_arrive_expect_tx(full_bar + 8u * s, stage_tx);
                load_w(stage_addr, full_bar + 8u * s, k_coord, pol_w);
                tma_load_2d(stage_addr + kWStageBytes, &tmap_a, full_bar + 8u * s, k_coord, 0, pol_a);
                issued = i + 1;
                k_coord += kBlockK;
                stage_addr += stage_bytes;
                if (++s == static_cast<uint32_t>(p.stages)) {
                    s = 0;
                    stage_addr = ring_addr;
                    parity ^= 1u;
                }
            }
            if (ctrl->abort) {
                // Give the copies already in flight a bounded chance to land before the CTA exits.
                for (int st = 0; st < p.stages && st < issued; ++st) {
                    const int last = ((issued - 1 - st) / p.stages) * p.stages + st;
                    const uint32_t par = static_cast<uint32_t>(last / p.stages) & 1u;
                    const long long start = clock64();
                    while (!mbar_try_wait(full_bar + 8u * st, par)) {
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
            const uint64_t desc_fixed = umma_desc_kmajor_sw128(0u);   // everything but the address field
            uint32_t s = 0, parity = 0, stage_addr = ring_addr;
            for (int i = 0; i < kb_count; ++i) {
                if (!mbar_wait_bounded(full_bar + 8u * s, parity, &ctrl->abort, kRoleMma)) break;
                if (i == 0) stamp(p, 3);
                tcgen05_fence_after_sync();
                const uint64_t w_desc = desc_fixed + (stage_addr >> 4);
                const uint64_t a_desc = desc_fixed + ((stage_addr + kWStageBytes) >> 4);
#pragma unroll
                for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                    // +32 bytes along K inside the swizzle atom = +2 in the (address >> 4) field.
                    umma_f8f6f4(tmem_acc, w_desc + 2u * kk, a_desc + 2u * kk, idesc, (i | kk) != 0 ? 1u : 0u);
                }
                // the stage goes back to the producer only if a later block needs it
                if (i + p.stages < kb_count) umma_commit(empty_bar + 8u * s);
                stage_addr += stage_bytes;
                if (++s == static_cast<uint32_t>(p.stages)) {
                    s = 0;
                    stage_addr = ring_addr;
                    parity ^= 1u;
                }
            }
            umma_commit(accum_bar);
            stamp(p, 4);
        }
        __syncwarp();
    }

    // ---------------------------------------------------------------------- epilogue (warps 0..3)
    // split == 1: the tile goes straight from TMEM to D (through shared memory, to store along rows).
    // split  > 1: CTA q of the cluster finishes token rows [q * rpo, (q + 1) * rpo) of the tile. Every
    // CTA sends those rows of its partial tile straight from registers into q's receive buffer with
    // asynchronous stores that count their bytes on q's `recv` barrier; an owner waits (bounded)
    // until all `split` blocks have landed, adds them in rank order out of its own shared memory
    // and writes D. No staging, no copy engine and no cluster-wide barrier sit on this path; the
    // barrier issued at start-up only proves that the peers' receive barriers exist and are armed.
    const bool epilogue_warp = warp < kEpilogueThreads / 32;
    if (p.split > 1 && !epilogue_warp) cluster_wait_acquire();
    if (epilogue_warp) {
        pdl_wait_prior_grids();
        EpiCtx cx;
        cx.ctrl = ctrl;
        cx.ring_ptr = ring_ptr;
        cx.recv_addr = smem_u32(ctrl) + kCtrlBytes;
        cx.recv_bar = recv_bar;
        cx.accum_bar = accum_bar;
        cx.lane_taddr = tmem_acc + (static_cast<uint32_t>(warp * 32) << 16);
        cx.rank = rank;
        cx.n0 = n0;
        cx.scale = __ldg(p.scale) * p.kind_factor;
        if constexpr (kMode == kModeSwiglu) {
            epilogue_swiglu(p, cx);
        } else if constexpr (kDT >= 0) {
            epilogue_store<kMode, kDT, kWorld>(p, cx);
        } else {
            if (p.d_dtype == HFRK_BF16) {
                epilogue_store<kMode, HFRK_BF16, kWorld>(p, cx);
            } else if (p.d_dtype == HFRK_F16) {
                epilogue_store<kMode, HFRK_F16, kWorld>(p, cx);
            } else {
                epilogue_store<kMode, HFRK_F32, kWorld>(p, cx);
            }
        }
    }

    if (threadIdx.x == 0) stamp(p, 6);
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) tmem_dealloc(tmem_acc, tmem_cols);
    if (threadIdx.x == 0) stamp(p, 7);
}

}  // namespace hfrk
