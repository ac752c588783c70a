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
// The kernel itself is in skinny_gemm_kernel.cuh; this file holds the tensor maps, the launch
// planning, the launchers and the C ABI. In the reference's terms the two files replace
// skinny_gemm_kernel.cu:6-79 (kernel), producers/*.cu (global->LDS streaming), consumers/*.cu (MFMA
// + atomic epilogue) and skinny_gemm_caller.cu:21-71 (validation, launch shape) of
// csrc/op_src/skinny_gemm/.
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
#include "device_model.cuh"
#include "skinny_gemm_kernel.cuh"
#include "skinny_gemm_streamk.cuh"

namespace hfrk {

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
    int rows_log2;        // split > 1: token rows finished per CTA of a cluster = 1 << rows_log2
};

// Token rows each CTA of a cluster finishes in the split-K reduction: the smallest power of two
// that is at least ceil(m / split) (a power of two so that a thread's 1, 2 or 4 consecutive rows
// always belong to one owner and can leave in one vector store).
int rows_per_owner_log2(int m, int split) {
    const int need = (m + split - 1) / split;
    int lg = 0;
    while ((1 << lg) < need) ++lg;
    return lg;
}

// Receive buffer of the split-K reduction: split x 128 x rows-per-owner floats (layout: recv_float_index).
int recv_buffer_bytes(int m, int split) {
    return split > 1 ? split * kTileN * 4 * (1 << rows_per_owner_log2(m, split)) : 0;
}

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

// Shared memory one CTA of the cluster kernel takes: alignment slack, the ring, the control block
// and the receive buffer of the split-K reduction.
int plan_smem_bytes(int m, int m_pad, int split, int stages) {
    return 1024 + stages * (kWStageBytes + m_pad * kBlockK) + kCtrlBytes + recv_buffer_bytes(m, split);
}

// CTAs of the kernel that fit on one SM: shared memory decides (the registers allow three).
int ctas_per_sm(int smem_bytes) {
    const int by_smem = kSmemPerSm / (smem_bytes + kSmemCtaReserve);
    return by_smem < kModelMaxPerSm ? by_smem : kModelMaxPerSm;
}

// Launch shapes measured best on B200 for the Llama-3 8B/70B decode projections and their K shards
// (16 tokens and fewer), in the reference's tradition of a per-shape table (hf_rocm_kernels/
// operators/skinny_gemm/wrapped.py:42-102). An entry is only used if the device holds all its
// clusters at once (the measured capacity decides); otherwise the rule below takes over.
struct BuiltinShape {
    int n, k, split, stages;
};
constexpr BuiltinShape kBuiltinShapes[] = {
    {6144, 4096, 7, 3},    // 8B qkv
    {4096, 4096, 7, 5},    // 8B o_proj (as good as 8 x 3 between calls of its own shape, 0.4 us better between qkv and gate_up)
    {4096, 14336, 8, 5},   // 8B down
    {10240, 8192, 5, 3},   // 70B qkv
    {8192, 8192, 6, 3},    // 70B o_proj
    {57344, 8192, 1, 3},   // 70B gate_up
    {8192, 28672, 6, 3},   // 70B down
    {8192, 14336, 6, 3},   // 70B down, K over 2 GPUs
    {8192, 7168, 6, 3},    // 70B down, K over 4 GPUs
    {8192, 3584, 6, 3},    // 70B down, K over 8 GPUs
    {5120, 8192, 6, 4},    // 70B qkv, N over 2 GPUs
    {14336, 8192, 2, 5},   // 70B gate_up, N over 4 GPUs
};

// Launch shape of the cluster kernel for one launch of m <= kMaxMPad tokens. What the measurements
// on B200 say (traces of consecutive calls in a graph, sweeps over the Llama-3 shapes and shards):
//   * a call in a chain of dependent launches costs latency, not bandwidth, until the matrix
//     reaches ~100 MB: dependency release, activation load, MMA issue, reduction, exit. More CTAs
//     shorten every CTA's K range and put more loads in flight, so the K split is the largest one
//     whose clusters are ALL resident at once. Residency is the cliff: a cluster that waits for a
//     free slot starts when others leave and streams alone (5120 x 8192: 10.0 us with 40 clusters
//     of 6, 14.6 us with 40 clusters of 7 on a chip that holds 39 of them). The capacity comes
//     from the device model (measured per chip), never from a constant;
//   * three CTAs per SM (a ring of three 18 KiB stages) beat two (four stages) on most shapes:
//     the third slot lets part of the NEXT call's grid move in and start its weight stream while
//     this call drains;
//   * at least two K blocks per CTA; no split once the tiles alone cover the SMs (then six
//     stages, two CTAs per SM, or three stages when that saves a wave: 448 tiles on 444 slots);
//   * tiles of fewer than 128 rows even out a grid without a K split that is between one and two
//     CTAs per SM: 224 tiles of 128 rows put two CTAs on 76 SMs and one on the other 72; 256
//     tiles of 112 rows spread more evenly. The tensor core still computes 128 lanes per tile; the
//     lanes past the tile's rows are ignored. The height stays a multiple of 16, the width of the
//     epilogue's row-wise stores.
int make_plan(const DeviceModel& dm, int m, int n, int k, int split_req, int stages_req, Plan* plan,
              int tile_rows_req = 0, int max_per_sm = kModelMaxPerSm) {
    if (m <= 0 || n <= 0 || k <= 0 || m > kMaxMPad) return HFRK_INVALID_CONFIG;
    if (tile_rows_req < kAutoTileRowsOff || tile_rows_req > kTileN || (tile_rows_req > 0 && tile_rows_req < 8))
        return HFRK_INVALID_CONFIG;
    if (split_req < 0 || split_req > kMaxSplit || stages_req < 0 || stages_req == 1 || stages_req > kMaxStages)
        return HFRK_INVALID_CONFIG;
    const int m_pad = round_up(m, 16);
    const int tiles = (n + kTileN - 1) / kTileN;
    const int nkb = (k + kBlockK - 1) / kBlockK;
    const int stage_bytes = kWStageBytes + m_pad * kBlockK;
    const int two_per_sm = 2 * dm.sms;

    // all clusters of (split, stages) resident at once on this device?
    auto resident = [&](int split, int stages) {
        const int smem = plan_smem_bytes(m, m_pad, split, stages);
        if (smem > kSmemLimit) return false;
        const int per_sm = ctas_per_sm(smem) < max_per_sm ? ctas_per_sm(smem) : max_per_sm;
        // one cluster to spare: at the exact capacity a straggler of the previous grid keeps the last one out
        return per_sm >= 1 && tiles < dm.capacity[split][per_sm];
    };

    TuneValue tuned;
    if (split_req == 0 && stages_req == 0 && tile_rows_req == 0) {
        if (tuning_lookup(m_pad, n, k, &tuned)) {
            split_req = tuned.split;
            stages_req = tuned.stages;
            tile_rows_req = tuned.tile_rows;
        } else if (m_pad == 16) {
            for (const BuiltinShape& b : kBuiltinShapes) {
                if (b.n == n && b.k == k && (b.split == 1 || resident(b.split, b.stages))) {
                    split_req = b.split;
                    stages_req = b.stages;
                    break;
                }
            }
        }
    }
    int split = split_req;
    int stages = stages_req;
    if (split == 0) {
        split = 1;
        if (tiles < dm.sms) {
            // largest resident split; a ring of three stages lets three CTAs share an SM, four stages
            // two. Up to 16 tokens more CTAs win; with equal CTAs the longer ring does.
            // Above 16 tokens the activation tile and the receive buffer grow and the choices thin
            // out: a ring of two stages may be all that lets three CTAs share an SM. There the bytes
            // in flight decide (CTAs x stages), marked down by a quarter when an owner finishes more
            // than eight token rows (the reduction then runs past its register path); equal scores
            // go to more CTAs. 8192 x 8192, 48 tokens: 15.4 us with 64 clusters of 6 on two stages,
            // 18.2 us with clusters of 4 on three; 6144 x 4096, 32 tokens: 7.7 us with clusters of 5
            // on four stages, 8.9 us with clusters of 7 on two.
            int best_ctas = 0;
            long best_score = 0;
            const int ring_choices[3] = {2, 3, 4};
            for (int choice = m_pad > 16 ? 0 : 1; choice < 3; ++choice) {
                const int ring = stages_req != 0 ? stages_req : ring_choices[choice];
                for (int s = kMaxSplit; s >= 2; --s) {
                    if (nkb / s < 2) continue;
                    if (!resident(s, ring)) continue;
                    const int ctas = tiles * s;
                    bool better;
                    if (m_pad > 16) {
                        const long score = static_cast<long>(ctas) * ring * (rows_per_owner_log2(m, s) > 3 ? 3 : 4);
                        better = score > best_score || (score == best_score && ctas > best_ctas);
                        if (better) best_score = score;
                    } else {
                        better = ctas >= best_ctas;
                    }
                    if (better) {
                        best_ctas = ctas;
                        split = s;
                        if (stages_req == 0) stages = ring;
                    }
                    break;   // smaller splits of this ring have fewer CTAs
                }
            }
        }
    }
    if (split > nkb) split = nkb;
    if (split < 1) split = 1;

    const int fixed_bytes = 1024 + kCtrlBytes + recv_buffer_bytes(m, split);
    const int max_stages_fit = (kSmemLimit - fixed_bytes) / stage_bytes;
    if (stages == 0) {
        if (split > 1) {
            stages = 4;
        } else {
            // three stages (three CTAs per SM) when two per SM would need one more wave than three
            const int waves2 = (tiles + two_per_sm - 1) / two_per_sm;
            const int waves3 = (tiles + 3 * dm.sms - 1) / (3 * dm.sms);
            stages = (m_pad == 16 && waves3 < waves2) ? 3 : 6;
        }
        // keep two CTAs on an SM when the activation tile or the receive buffer of a larger token
        // count grows: with one CTA per SM a grid of 150-296 CTAs needs a second wave
        while (stages > 2 && 2 * (fixed_bytes + stages * stage_bytes + kSmemCtaReserve) > kSmemPerSm) --stages;
    }
    // a ring longer than the CTA's K range only takes shared memory from the next call's CTAs
    const int blocks_per_cta = (nkb + split - 1) / split;
    if (stages_req == 0 && stages > blocks_per_cta) stages = blocks_per_cta < 2 ? 2 : blocks_per_cta;
    if (stages > max_stages_fit) stages = max_stages_fit;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return HFRK_INVALID_CONFIG;

    int tile_rows = tile_rows_req == kAutoTileRowsOff ? kTileN : tile_rows_req;
    if (tile_rows == 0) {
        tile_rows = kTileN;
        const int smem = fixed_bytes + stages * stage_bytes;
        const int slots = two_per_sm - two_per_sm / 18;   // two CTAs per SM, a few slots spare
        if (m_pad == 16 && split == 1 && tiles > dm.sms && tiles <= slots && ctas_per_sm(smem) >= 2) {
            // a multiple of 16 rows: the epilogue stores 16 outputs at a time, and a tile that ends on half
            // a piece finishes it element by element (28672 x 4096: 21.6 us with 104 rows, 20.5 us with 112)
            const int rows = round_up((n + slots - 1) / slots, 16);
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
    plan->rows_log2 = split > 1 ? rows_per_owner_log2(m, split) : 0;
    return HFRK_SUCCESS;
}

// The row-parallel kernel for an output type and a group size (sizes other than 2, 4, 8 share the
// general form).
using GemmKernel = void (*)(const CUtensorMap, const CUtensorMap, const GemmParams);
template <int kDT>
GemmKernel rowpar_kernel_for_world(int world) {
    switch (world) {
        case 2: return skinny_gemm_fp8_sm100_kernel<kModeRowPar, kDT, 2>;
        case 4: return skinny_gemm_fp8_sm100_kernel<kModeRowPar, kDT, 4>;
        case 8: return skinny_gemm_fp8_sm100_kernel<kModeRowPar, kDT, 8>;
        default: return skinny_gemm_fp8_sm100_kernel<kModeRowPar, kDT, 0>;
    }
}
const void* rowpar_kernel(int d_dtype, int world) {
    GemmKernel fn = d_dtype == HFRK_BF16 ? rowpar_kernel_for_world<HFRK_BF16>(world)
                    : d_dtype == HFRK_F16 ? rowpar_kernel_for_world<HFRK_F16>(world)
                                          : rowpar_kernel_for_world<HFRK_F32>(world);
    return reinterpret_cast<const void*>(fn);
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
    for (int dt = 0; dt < 3; ++dt) {
        for (int world : {0, 2, 4, 8}) {
            const void* fn = rowpar_kernel(dt, world);
            HFRK_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
            HFRK_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        }
    }
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
        rc = make_plan(device_model(stream), mc, n, k, split_req, stages_req, &plan,
                       rowpar != nullptr ? kAutoTileRowsOff : tile_rows_req,
                       kModelMaxPerSm);   // the row-parallel instantiations are compiled for three CTAs per SM too
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
        p.rows_log2 = plan.rows_log2;
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
            void* args[3] = {&tmap_w, &tmap_a, &p};
            HFRK_CUDA_TRY(cudaLaunchKernelExC(&cfg, rowpar_kernel(d_dtype, p.rp.world), args));
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
    rc = make_plan(device_model(stream), m, 2 * inter, k, split_req, /*stages_req=*/0, &plan, kAutoTileRowsOff);
    if (rc != HFRK_SUCCESS) return rc;
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
    p.rows_log2 = plan.rows_log2;
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
    unsigned long long* stamps = nullptr;   // diagnostic: per-CTA time stamps of the next calls
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
                             g->stamps, &g->dev, g->mode);
}

extern "C" int hfrk_rowpar_set_wait_ms(hfrk_rowpar* g, int milliseconds) {
    if (g == nullptr) return HFRK_BAD_WORLD;
    if (milliseconds < 1 || milliseconds > 60000) return HFRK_INVALID_CONFIG;
    g->dev.wait_cycles = static_cast<long long>(milliseconds) * 2000000ll;   // SM clock ticks at ~2 GHz
    return HFRK_SUCCESS;
}

extern "C" int hfrk_rowpar_set_stamps(hfrk_rowpar* g, unsigned long long* stamps_dev) {
    if (g == nullptr) return HFRK_BAD_WORLD;
    g->stamps = stamps_dev;
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
    // Page-locked host memory is addressable from the device: the epilogue then reads the bias from
    // D_host and writes the result to it over PCIe itself (at most a few hundred kilobytes), which
    // saves two copy submissions per call. Pageable memory takes the staged route.
    void* d_direct = nullptr;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, D_host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer != nullptr) {
        d_direct = attr.devicePointer;
    } else {
        (void)cudaGetLastError();
    }
    if (d_direct != nullptr) {
        int rc = hfrk::launch_gemm(a_dev, W_dev, d_direct, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype,
                                   accumulate, HFRK_VARIANT_AUTO, 0, 0, 0, hfrk::default_use_pdl(), s);
        if (rc != HFRK_SUCCESS) return rc;
    } else {
        if (accumulate) HFRK_CUDA_TRY(cudaMemcpyAsync(d_dev, D_host, d_bytes, cudaMemcpyHostToDevice, s));
        int rc = hfrk::launch_gemm(a_dev, W_dev, d_dev, scale_dev, m, n, k, w_row_stride, a_kind, w_kind, d_dtype,
                                   accumulate, HFRK_VARIANT_AUTO, 0, 0, 0, hfrk::default_use_pdl(), s);
        if (rc != HFRK_SUCCESS) return rc;
        HFRK_CUDA_TRY(cudaMemcpyAsync(D_host, d_dev, d_bytes, cudaMemcpyDeviceToHost, s));
    }
    if (synchronise) HFRK_CUDA_TRY(cudaStreamSynchronize(s));
    return HFRK_SUCCESS;
}
}  // namespace
}  // namespace hfrk

// =============================================================================== host batch
namespace hfrk {
namespace {

constexpr size_t kBatchMergeBytes = 512 * 1024;   // largest merged activation copy; smallest result group
constexpr int kBatchEvents = 64;

// Per device: the library's copy stream and a ring of events (an event may be recorded again while
// an older wait on it is pending: a wait refers to the record that preceded it).
struct BatchResources {
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t events[kBatchEvents] = {};
    int next_event = 0;
    bool ready = false;
};
std::mutex g_batch_mutex;
BatchResources g_batch[64];

int batch_resources(BatchResources** out) {
    int dev = 0;
    HFRK_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return HFRK_INVALID_CONFIG;
    BatchResources& r = g_batch[dev];
    if (!r.ready) {
        HFRK_CUDA_TRY(cudaStreamCreateWithFlags(&r.copy_stream, cudaStreamNonBlocking));
        for (int i = 0; i < kBatchEvents; ++i) {
            HFRK_CUDA_TRY(cudaEventCreateWithFlags(&r.events[i], cudaEventDisableTiming));
        }
        r.ready = true;
    }
    *out = &r;
    return HFRK_SUCCESS;
}

size_t out_elem_bytes(int d_dtype) { return d_dtype == HFRK_F32 ? 4 : 2; }
size_t align16(size_t v) { return (v + 15) & ~static_cast<size_t>(15); }

bool batch_call_valid(const hfrk_host_call& c) {
    return c.A_host != nullptr && c.W_dev != nullptr && c.D_host != nullptr && c.scale_dev != nullptr && c.m > 0 &&
           c.n > 0 && c.k > 0 && (c.d_dtype == HFRK_F16 || c.d_dtype == HFRK_BF16 || c.d_dtype == HFRK_F32);
}

}  // namespace
}  // namespace hfrk

extern "C" int64_t hfrk_host_batch_workspace_bytes(const hfrk_host_call* calls, int count) {
    if (calls == nullptr || count <= 0) return 0;
    size_t total = 0;
    for (int i = 0; i < count; ++i) {
        if (!hfrk::batch_call_valid(calls[i])) return 0;
        // activations are packed as on the host (k % 16 == 0 keeps every block 16-byte aligned); outputs padded to 16
        total += hfrk::align16(static_cast<size_t>(calls[i].m) * calls[i].k);
        total += hfrk::align16(static_cast<size_t>(calls[i].m) * calls[i].n * hfrk::out_elem_bytes(calls[i].d_dtype));
    }
    return static_cast<int64_t>(total + 256);
}

extern "C" int hfrk_skinny_gemm_fp8_host_batch(const hfrk_host_call* calls, int count, void* work_dev,
                                               int64_t work_bytes, void* stream) {
    using namespace hfrk;
    if (calls == nullptr || count <= 0 || work_dev == nullptr) return HFRK_INVALID_CONFIG;
    if (work_bytes < hfrk_host_batch_workspace_bytes(calls, count) || hfrk_host_batch_workspace_bytes(calls, count) == 0)
        return HFRK_INVALID_CONFIG;
    for (int i = 0; i < count; ++i) {
        if (calls[i].k % 16 != 0) return HFRK_K_NOT_DIVISIBLE;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> lock(g_batch_mutex);
    BatchResources* res = nullptr;
    int rc = batch_resources(&res);
    if (rc != HFRK_SUCCESS) return rc;
    auto next_event = [&]() {
        cudaEvent_t e = res->events[res->next_event];
        res->next_event = (res->next_event + 1) % kBatchEvents;
        return e;
    };

    // device layout: all activation blocks, then all output blocks
    uint8_t* const base = static_cast<uint8_t*>(work_dev);
    size_t a_total = 0;
    for (int i = 0; i < count; ++i) a_total += align16(static_cast<size_t>(calls[i].m) * calls[i].k);
    uint8_t* const d_base = base + ((a_total + 255) & ~static_cast<size_t>(255));

    // activations: host-contiguous runs merged into copies of at most kBatchMergeBytes, on the copy
    // stream; needs_event[i] = the event the compute stream waits for before call i (or none)
    cudaEvent_t needs_event[1024] = {};
    if (count > 1024) return HFRK_TOO_LARGE;
    {
        // the scratch may still be in use by what was queued on `stream` before (the previous batch)
        cudaEvent_t before = next_event();
        HFRK_CUDA_TRY(cudaEventRecord(before, s));
        HFRK_CUDA_TRY(cudaStreamWaitEvent(res->copy_stream, before, 0));
    }
    {
        size_t dev_off = 0;
        int i = 0;
        while (i < count) {
            const uint8_t* host0 = static_cast<const uint8_t*>(calls[i].A_host);
            size_t run = 0;
            int j = i;
            // the first block is kept small so that the first GEMM does not wait for the whole step's input
            const size_t limit = i == 0 ? kBatchMergeBytes / 4 : kBatchMergeBytes;
            while (j < count && run < limit) {
                const size_t bytes = static_cast<size_t>(calls[j].m) * calls[j].k;   // a multiple of 16
                if (static_cast<const uint8_t*>(calls[j].A_host) != host0 + run) break;
                run += bytes;
                ++j;
            }
            cudaError_t merged = cudaMemcpyAsync(base + dev_off, host0, run, cudaMemcpyHostToDevice, res->copy_stream);
            if (merged != cudaSuccess && j > i + 1) {
                // blocks that follow each other in the address space but come from different page-locked
                // allocations cannot travel as one copy (refused at submission): one copy per block then
                (void)cudaGetLastError();
                size_t done = 0;
                for (int t = i; t < j; ++t) {
                    const size_t bytes = static_cast<size_t>(calls[t].m) * calls[t].k;
                    HFRK_CUDA_TRY(cudaMemcpyAsync(base + dev_off + done, calls[t].A_host, bytes, cudaMemcpyHostToDevice,
                                                  res->copy_stream));
                    done += bytes;
                }
            } else {
                HFRK_CUDA_TRY(merged);
            }
            // D_in of the chunk's accumulating calls travels with it, so that nothing but kernels sits
            // on the compute stream (a copy between two kernels would end their overlap)
            for (int t = i; t < j; ++t) {
                if (!calls[t].accumulate) continue;
                size_t off = 0;
                for (int u = 0; u < t; ++u)
                    off += align16(static_cast<size_t>(calls[u].m) * calls[u].n * out_elem_bytes(calls[u].d_dtype));
                HFRK_CUDA_TRY(cudaMemcpyAsync(d_base + off, calls[t].D_in_host != nullptr ? calls[t].D_in_host : calls[t].D_host,
                                              static_cast<size_t>(calls[t].m) * calls[t].n * out_elem_bytes(calls[t].d_dtype),
                                              cudaMemcpyHostToDevice, res->copy_stream));
            }
            cudaEvent_t e = next_event();
            HFRK_CUDA_TRY(cudaEventRecord(e, res->copy_stream));
            needs_event[i] = e;
            dev_off += run;
            i = j;
        }
    }

    // results leave in about three groups: each group's copy overlaps the next group's GEMMs, and
    // every group costs one dependency between the two streams
    size_t out_total = 0;
    for (int i = 0; i < count; ++i) out_total += static_cast<size_t>(calls[i].m) * calls[i].n * out_elem_bytes(calls[i].d_dtype);
    const size_t group_target = out_total / 3 > kBatchMergeBytes ? out_total / 3 : kBatchMergeBytes;
    size_t a_off = 0, d_off = 0;
    size_t group_bytes = 0;
    int group_first = 0;
    size_t group_first_off = 0;
    auto flush_group = [&](int last) -> int {
        // results of calls group_first..last: wait for the last GEMM, then copy out on the copy stream,
        // merging calls whose host blocks follow each other as their device blocks do
        cudaEvent_t e = next_event();
        HFRK_CUDA_TRY(cudaEventRecord(e, s));
        HFRK_CUDA_TRY(cudaStreamWaitEvent(res->copy_stream, e, 0));
        size_t off = group_first_off;
        int i = group_first;
        while (i <= last) {
            uint8_t* host0 = static_cast<uint8_t*>(calls[i].D_host);
            size_t run = 0, dev_run = 0;
            int j = i;
            while (j <= last) {
                const size_t bytes = static_cast<size_t>(calls[j].m) * calls[j].n * out_elem_bytes(calls[j].d_dtype);
                if (static_cast<uint8_t*>(calls[j].D_host) != host0 + run || run != dev_run) break;
                run += bytes;
                dev_run += align16(bytes);
                ++j;
            }
            cudaError_t merged = cudaMemcpyAsync(host0, d_base + off, run, cudaMemcpyDeviceToHost, res->copy_stream);
            if (merged != cudaSuccess && j > i + 1) {
                (void)cudaGetLastError();   // neighbours from different page-locked allocations, as above
                size_t done = 0;
                for (int t = i; t < j; ++t) {
                    const size_t bytes = static_cast<size_t>(calls[t].m) * calls[t].n * out_elem_bytes(calls[t].d_dtype);
                    HFRK_CUDA_TRY(cudaMemcpyAsync(calls[t].D_host, d_base + off + done, bytes, cudaMemcpyDeviceToHost,
                                                  res->copy_stream));
                    done += bytes;
                }
            } else {
                HFRK_CUDA_TRY(merged);
            }
            // device blocks are padded to 16 bytes: a run only continues while no padding intervened
            for (int t = i; t < j; ++t)
                off += align16(static_cast<size_t>(calls[t].m) * calls[t].n * out_elem_bytes(calls[t].d_dtype));
            i = j;
        }
        return HFRK_SUCCESS;
    };

    for (int i = 0; i < count; ++i) {
        const hfrk_host_call& c = calls[i];
        const size_t a_bytes = static_cast<size_t>(c.m) * c.k;
        const size_t d_bytes = static_cast<size_t>(c.m) * c.n * out_elem_bytes(c.d_dtype);
        if (needs_event[i] != nullptr) HFRK_CUDA_TRY(cudaStreamWaitEvent(s, needs_event[i], 0));
        rc = launch_gemm(base + a_off, c.W_dev, d_base + d_off, c.scale_dev, c.m, c.n, c.k, c.w_row_stride, c.a_kind,
                         c.w_kind, c.d_dtype, c.accumulate, HFRK_VARIANT_AUTO, 0, 0, 0, default_use_pdl(), s);
        if (rc != HFRK_SUCCESS) return rc;
        if (group_bytes == 0) {
            group_first = i;
            group_first_off = d_off;
        }
        group_bytes += d_bytes;
        a_off += a_bytes;
        d_off += align16(d_bytes);
        // also right before the last call: its result is all that is left to copy when the GEMMs end
        if (group_bytes >= group_target || i >= count - 2) {
            rc = flush_group(i);
            if (rc != HFRK_SUCCESS) return rc;
            group_bytes = 0;
        }
    }
    cudaEvent_t done = next_event();
    HFRK_CUDA_TRY(cudaEventRecord(done, res->copy_stream));
    HFRK_CUDA_TRY(cudaStreamWaitEvent(s, done, 0));
    return HFRK_SUCCESS;
}

extern "C" int hfrk_skinny_gemm_plan(int m, int n, int k, int variant, int split_k, int ctas_per_sm, int* out8) {
    if (out8 == nullptr || variant < HFRK_VARIANT_AUTO || variant > HFRK_VARIANT_STREAMK) return HFRK_INVALID_CONFIG;
    const int mc = m > hfrk::kMaxMPad ? hfrk::kMaxMPad : m;
    if (variant == HFRK_VARIANT_AUTO) variant = HFRK_VARIANT_CLUSTER;
    if (variant == HFRK_VARIANT_CLUSTER) {
        hfrk::Plan plan;
        int rc = hfrk::make_plan(hfrk::device_model(nullptr), mc, n, k, split_k, 0, &plan);
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

extern "C" int hfrk_device_model_get(int* sms_out, int* capacity_out, int* measured_out) {
    const hfrk::DeviceModel dm = hfrk::device_model(nullptr);
    if (sms_out != nullptr) *sms_out = dm.sms;
    if (measured_out != nullptr) *measured_out = dm.measured ? 1 : 0;
    if (capacity_out != nullptr) {
        for (int split = 0; split <= hfrk::kModelMaxSplit; ++split) {
            for (int per_sm = 0; per_sm <= hfrk::kModelMaxPerSm; ++per_sm) {
                capacity_out[split * (hfrk::kModelMaxPerSm + 1) + per_sm] = dm.capacity[split][per_sm];
            }
        }
    }
    return HFRK_SUCCESS;
}

extern "C" int hfrk_device_model_override(int sms, const int* capacity) {
    std::lock_guard<std::mutex> lock(hfrk::model_detail::mutex());
    if (capacity == nullptr) {
        hfrk::model_detail::override_on() = false;
        return HFRK_SUCCESS;
    }
    if (sms < 1) return HFRK_INVALID_CONFIG;
    hfrk::DeviceModel& dm = hfrk::model_detail::override_model();
    dm.sms = sms;
    dm.measured = false;
    for (int split = 0; split <= hfrk::kModelMaxSplit; ++split) {
        for (int per_sm = 0; per_sm <= hfrk::kModelMaxPerSm; ++per_sm) {
            dm.capacity[split][per_sm] = capacity[split * (hfrk::kModelMaxPerSm + 1) + per_sm];
        }
    }
    hfrk::model_detail::override_on() = true;
    return HFRK_SUCCESS;
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
