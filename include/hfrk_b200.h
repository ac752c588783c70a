/*
 * hfrk_b200.h - C ABI of the B200 (sm_100a) FP8 skinny GEMM library, libhfrk_b200.so.
 *
 * The GEMM:        D[m,n] <- (accumulate ? D_in[m,n] : 0) + scale * sum_k A[m,k] * W[n,k]
 *   A  [M,K]  fp8 e4m3, row-major, contiguous
 *   W  [N,K]  fp8 e4m3, row-major with a row stride of w_row_stride elements
 *   D  [M,N]  fp16 or bf16, row-major, contiguous, updated in place
 *   scale     one fp32 value read ON THE DEVICE (the product scale_a * scale_w)
 *
 * Every pointer is a plain device pointer unless the name says "host". Nothing here takes or
 * returns a torch type; the torch op `_HFRK_C::skinny_gemm_tb` is a thin shim over these calls.
 *
 * The entry points stand where the reference (huggingface/hf-rocm-kernels) has
 *   csrc/op_src/skinny_gemm/skinny_gemm_binding.cu:16-42   (tensor -> pointers, shapes, stream)
 *   csrc/op_src/skinny_gemm/skinny_gemm_caller.cu:21-71    (validation, grid/block, dispatch)
 *   csrc/op_src/skinny_gemm/skinny_gemm_kernel.cu:6-79     (the device kernel)
 * and keep its convention of returning a status int instead of throwing
 * (csrc/op_src/skinny_gemm/skinny_gemm_caller.cu:9-17). The two element-wise kernels that sit
 * between the GEMMs of a decoder layer (hfrk_residual_rms, hfrk_swiglu_fp8) are declared further
 * down with the reference files they replace.
 */
#ifndef HFRK_B200_H_
#define HFRK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------
 * 0..6 are the reference's SkinnyGemmReturnCode values (skinny_gemm_caller.cu:9-17); the B200
 * kernel never needs 1, 2, 4, 5 (no warp-tile, lane or queue knobs) but keeps the numbering so
 * that callers that log the code read the same meaning. Codes >= 7 are new. */
enum hfrk_status {
    HFRK_SUCCESS = 0,
    HFRK_M_ABOVE_WARPTILE_M = 1,        /* never returned */
    HFRK_N_NOT_EVEN = 2,                /* never returned: odd N is handled */
    HFRK_K_NOT_DIVISIBLE = 3,           /* K must be a multiple of 16 (TMA row pitch) */
    HFRK_TOO_MANY_WARPS = 4,            /* never returned */
    HFRK_QSIZE_TOO_SMALL = 5,           /* never returned */
    HFRK_INVALID_CONFIG = 6,            /* m, n, k <= 0, or a tuning value out of range */
    HFRK_BAD_ALIGNMENT = 7,             /* base pointer or W row stride not 16-byte aligned */
    HFRK_BAD_DTYPE = 8,                 /* unknown fp8 kind or output dtype */
    HFRK_CUDA_ERROR = 9,                /* a CUDA runtime/driver call failed (see hfrk_last_error) */
    HFRK_DEVICE_TIMEOUT = 10,           /* a bounded device-side wait ran out (pipeline or peer) */
    HFRK_BAD_WORLD = 11,                /* row-parallel: rank/world/peer table inconsistent */
    HFRK_TOO_LARGE = 12                 /* a size exceeds a documented fixed capacity */
};

/* fp8 encodings. E4M3FNUZ operands are reinterpreted bit-for-bit as E4M3FN and the result is
 * multiplied by 0.5 per FNUZ operand on the device: for every bit pattern the reference's
 * quantiser can emit (hf_rocm_kernels/utils/fp8.py:17-29) value_fnuz == value_fn / 2 exactly. */
enum hfrk_fp8_kind { HFRK_E4M3FN = 0, HFRK_E4M3FNUZ = 1 };
/* F32 output exists for unfused multi-GPU baselines (partial sums that a library all-reduce adds). */
enum hfrk_out_dtype { HFRK_F16 = 0, HFRK_BF16 = 1, HFRK_F32 = 2 };

/* The two kernels behind the GEMM.
 *   CLUSTER : one CTA per (128-row tile, K split); the K splits of a tile form a thread-block
 *             cluster and reduce through distributed shared memory. No scratch memory.
 *             This is what AUTO picks.
 *   STREAMK : the (tile, K block) work items are cut into equal ranges over a grid sized to the
 *             SM count; partial tiles meet in library-owned fp32 scratch and the last CTA to
 *             arrive reduces them in a fixed order. Balanced for any shape, but its reduction
 *             goes through L2 and costs more than the in-cluster one at these sizes. */
enum hfrk_variant { HFRK_VARIANT_AUTO = 0, HFRK_VARIANT_CLUSTER = 1, HFRK_VARIANT_STREAMK = 2 };

/* Single-GPU skinny GEMM on `stream` (a cudaStream_t passed as void*), asynchronous, no host
 * synchronisation. The kernel this entry point launches (the cluster kernel) needs no scratch and
 * the call allocates no device memory; the first call on a device sets the kernels' attributes,
 * so make one call per device before capturing into a CUDA graph. Only the stream-K variant
 * (hfrk_skinny_gemm_fp8_ex with HFRK_VARIANT_STREAMK) owns scratch: about 80 MB per device,
 * allocated on its first use (before any capture) and kept until the process ends, in four lanes
 * so that calls on up to four streams of a device may overlap.
 * Replaces skinny_gemm_tb / skinny_gemm() of the reference
 * (csrc/op_src/skinny_gemm/skinny_gemm_binding.cu:16-42, skinny_gemm_caller.cu:21-71).
 *   a_kind, w_kind : enum hfrk_fp8_kind       d_dtype : enum hfrk_out_dtype
 *   accumulate     : 1 = D += result (the reference's contract, wrapped.py:115), 0 = overwrite
 *   split_k_hint   : 0 = choose automatically; >= 1 = requested K split (clamped to what the
 *                    launch supports). The reference's split_k argument maps here.
 * The launch uses programmatic dependent launch unless the environment has HFRK_PDL=0: the
 * weight stream may begin while the previous kernel on `stream` is still running (A, D and the
 * scale are only read after it has finished). That previous kernel must therefore not write W. */
int hfrk_skinny_gemm_fp8(const void* A, const void* W, void* D, const float* scale_dev,
                         int m, int n, int k, int64_t w_row_stride,
                         int a_kind, int w_kind, int d_dtype, int accumulate,
                         int split_k_hint, void* stream);

/* Same operation with the launch shape pinned by the caller (benchmark sweeps, tuning):
 *   variant     : enum hfrk_variant
 *   split_k     : CLUSTER only; 0 = automatic, else 1..16
 *   ctas_per_sm : STREAMK only; 0 = automatic, else 1 or 2 (grid = 148 * ctas_per_sm)
 *   num_stages  : 0 = automatic, else 2..12 (CLUSTER, 16 KiB stages) or 2..8 (STREAMK, 32 KiB)
 *   use_pdl     : 1 = launch with programmatic stream serialisation so the weight stream of this
 *                 call may start while the previous kernel on the stream drains. Only safe when
 *                 nothing earlier on the stream writes W.
 * Takes the place of the reference's nine tuning ints
 * (csrc/op_src/skinny_gemm/skinny_gemm_caller.cu:28-32). */
int hfrk_skinny_gemm_fp8_ex(const void* A, const void* W, void* D, const float* scale_dev,
                            int m, int n, int k, int64_t w_row_stride,
                            int a_kind, int w_kind, int d_dtype, int accumulate,
                            int variant, int split_k, int ctas_per_sm, int num_stages, int use_pdl,
                            void* stream);

/* Host-buffer form of the same call, for callers whose activations live in host memory:
 * copies A host->device, runs the GEMM against the device-resident weights W_dev with D in host
 * memory, and synchronises `stream`. When D_host is page-locked the kernel reads (accumulate=1)
 * and writes it directly over PCIe; pageable memory is staged through `work_dev` with copies.
 * `work_dev` is caller-owned device scratch of at least hfrk_host_call_workspace_bytes(m, n, k)
 * bytes. Weights stay on the device: they are model state, as in the reference where they are
 * torch CUDA tensors (hf_rocm_kernels/operators/skinny_gemm/wrapped.py:28-35). */
int hfrk_skinny_gemm_fp8_host(const void* A_host, const void* W_dev, void* D_host,
                              const float* scale_dev, int m, int n, int k, int64_t w_row_stride,
                              int a_kind, int w_kind, int d_dtype, int accumulate,
                              void* work_dev, void* stream);
int64_t hfrk_host_call_workspace_bytes(int m, int n, int k);
/* The same work queued on `stream` WITHOUT the final synchronisation: D_host holds the result once
 * the caller has synchronised the stream. A_host, D_host (page-locked, or the copies are not
 * asynchronous) and work_dev must stay untouched until then; calls that share a work_dev must
 * share the stream. Lets a decode step queue all of its projections and wait once. */
int hfrk_skinny_gemm_fp8_host_async(const void* A_host, const void* W_dev, void* D_host,
                                    const float* scale_dev, int m, int n, int k, int64_t w_row_stride,
                                    int a_kind, int w_kind, int d_dtype, int accumulate,
                                    void* work_dev, void* stream);

/* One decode step's worth of host-buffer calls in ONE library call. A caller that drives the GEMMs
 * one by one from an interpreter pays more for submitting a call than the GPU needs to run it; here
 * the whole list is queued by one native loop:
 *   * activations go host->device on a copy stream owned by the library, neighbouring host blocks
 *     merged into copies of up to 512 KiB (one cudaMemcpyAsync per merged block, D_in of the
 *     block's accumulating calls behind it), each followed by an event that `stream` waits for
 *     only before the first GEMM that needs it;
 *   * nothing but the GEMMs runs on `stream`, in list order, so consecutive calls overlap as they
 *     do for device-resident callers;
 *   * results go device->host on the copy stream in about three groups, each behind an event
 *     recorded after the group's last GEMM, so that a group's copy overlaps the next group's GEMMs;
 *   * `stream` finally waits for the last copy: the caller synchronises `stream` once and finds
 *     every D_host filled.
 * work_dev: device scratch of at least hfrk_host_batch_workspace_bytes(calls, count) bytes; host
 * buffers should be page-locked (pageable ones make the copies synchronous, still correct) and
 * must stay untouched until `stream` has been synchronised. Returns the first failing call's
 * status. No counterpart in the reference, whose callers hold activations in CUDA tensors
 * (hf_rocm_kernels/operators/skinny_gemm/wrapped.py:104-128). */
typedef struct hfrk_host_call {
    const void* A_host;      /* [m, k] fp8 */
    const void* W_dev;       /* [n, k] fp8 on the device, row pitch w_row_stride */
    void* D_host;            /* [m, n] in/out */
    const float* scale_dev;
    int m, n, k;
    int64_t w_row_stride;
    int a_kind, w_kind, d_dtype, accumulate;
    const void* D_in_host;   /* accumulate != 0: where D_in is read from; NULL = from D_host itself. A
                              * separate, read-only bias-filled buffer spares the caller the refill of
                              * D_host before every step. */
} hfrk_host_call;
int64_t hfrk_host_batch_workspace_bytes(const hfrk_host_call* calls, int count);
int hfrk_skinny_gemm_fp8_host_batch(const hfrk_host_call* calls, int count, void* work_dev,
                                    int64_t work_bytes, void* stream);

/* ---- row-parallel (K split over GPUs) GEMM with the all-reduce fused into its epilogue ---------
 * Rank r of `world` holds columns [r*K/world, (r+1)*K/world) of A and W. Every rank calls
 * hfrk_skinny_gemm_fp8_rowpar with its shard; every rank ends with the full
 *     D = D_in + scale * sum_r (A_r . W_r^T)
 * (D_in must be the same on all ranks). Inside the kernel each thread writes the partial sums it
 * owns into every peer's exchange buffer as 8-byte {value, call number} cells (plain stores over
 * NVLink; a cell is valid once it carries the current call number, so no flag or fence is
 * needed), polls its own buffer for the peers' cells (bounded, ~2 s: HFRK_DEVICE_TIMEOUT through
 * hfrk_device_status) and adds the contributions in rank order, so all ranks produce
 * bit-identical results (hfrk_rowpar_set_mode describes the second exchange scheme). One process
 * per GPU: create -> exchange the 64-byte IPC handles by any host-side all-gather -> connect.
 * The reference has no multi-GPU path at all (no collective call site exists in its tree); this
 * stands where the benchmark specification asks for "GEMM + allreduce" in combined_ops.
 * All ranks must issue the same sequence of calls on a group. A group serves one stream at a time.
 *   max_m, max_n : largest call the group will see (sizes the exchange buffer:
 *                  2 * (world + 1) * min(max_m,16) * roundup(max_n,128) * 8 bytes). */
typedef struct hfrk_rowpar hfrk_rowpar;
int hfrk_rowpar_create(int rank, int world, int max_m, int max_n, hfrk_rowpar** out);
int hfrk_rowpar_ipc_handle(hfrk_rowpar* group, void* handle64_out);
int hfrk_rowpar_connect(hfrk_rowpar* group, const void* all_handles /* world x 64 bytes, by rank */);
/* Same-process alternative to the IPC route (all ranks' devices driven by one process with peer
 * access enabled): the exchange blocks of all ranks, from hfrk_rowpar_local_block. */
int hfrk_rowpar_connect_pointers(hfrk_rowpar* group, void* const* peer_blocks);
void* hfrk_rowpar_local_block(hfrk_rowpar* group);
int hfrk_rowpar_destroy(hfrk_rowpar* group);
/* How the partial tiles cross NVLink. ONE_SHOT: every rank sends its fp32 partials to every peer
 * and each adds them up itself (one crossing of latency, (world-1) copies of the partials out of
 * every GPU). TWO_SHOT: each CTA position has an owner rank that receives the partials, adds them
 * in rank order and sends the sums back (two crossings, about 2/world of the traffic). AUTO (the
 * default) takes ONE_SHOT while the one-shot traffic per GPU, 4*m*n*(world-1) bytes, is below
 * 1 MiB. Every rank of the group must use the same mode for the same call. */
enum hfrk_rowpar_mode { HFRK_ROWPAR_AUTO = 0, HFRK_ROWPAR_ONE_SHOT = 1, HFRK_ROWPAR_TWO_SHOT = 2 };
int hfrk_rowpar_set_mode(hfrk_rowpar* group, int mode);
/* Diagnostic: later calls of this group record per-CTA time stamps into stamps_dev[cta][8] as
 * hfrk_skinny_gemm_fp8_profile does (NULL = off). No counterpart in the reference. */
int hfrk_rowpar_set_stamps(hfrk_rowpar* group, unsigned long long* stamps_dev);
/* How long the kernel waits for a peer's partial sums before it gives up, in milliseconds of SM
 * clock at ~2 GHz (1..60000; the default is about two seconds). A call whose peer does not
 * deliver in time leaves D untouched for the elements concerned, sets the device status word
 * (HFRK_DEVICE_TIMEOUT, role 4) and returns normally: the context stays usable, the group does
 * not (its ranks no longer agree on the call number) and should be destroyed. */
int hfrk_rowpar_set_wait_ms(hfrk_rowpar* group, int milliseconds);
int hfrk_skinny_gemm_fp8_rowpar(hfrk_rowpar* group, const void* A_shard, const void* W_shard, void* D,
                                const float* scale_dev, int m, int n, int k_shard, int64_t w_row_stride,
                                int a_kind, int w_kind, int d_dtype, int accumulate, void* stream);

/* The GEMM for callers that must not allocate device memory when they call it: an inference
 * server whose own pools already own all of HBM (a late cudaMalloc fails or fragments them), code
 * that runs between allocator check-points, a plug-in barred from its host's allocator. It runs
 * the stream-K kernel with its scratch (fp32 partial tiles + tile counters) in a fixed array
 * inside the library image -- 4,866,048 bytes that every GPU loading the library holds until the
 * process exits -- and calls no cudaMalloc, cudaFree or any allocating routine, on any call.
 * Limits: m <= 16 and n <= 524,288, otherwise HFRK_TOO_LARGE (hfrk_last_error says why); the
 * caller still passes A, W, D and the scale. The first call on a device looks up the array's
 * device address (cudaGetSymbolAddress, with that device current) and, with CUDA's lazy module
 * loading, is also the moment the driver loads the library's module onto that device, the array
 * included: make that first call at start-up, before any stream capture and BEFORE the caller's own
 * pools take the rest of HBM (or run with CUDA_MODULE_LOADING=EAGER), or it can fail for lack of
 * the very memory the entry point promises not to ask for later. All calls share the one array, which keeps what the last call left:
 * the tile counters a call uses are cleared on `stream` before its kernel, partials are always
 * written before they are read; two calls that overlap on the GPU (different streams) race on it.
 * Plain launch (no programmatic dependent launch). It has no counterpart in the reference. */
int hfrk_skinny_gemm_fp8_noalloc(const void* A, const void* W, void* D, const float* scale_dev,
                                 int m, int n, int k, int64_t w_row_stride,
                                 int a_kind, int w_kind, int d_dtype, int accumulate, void* stream);

/* Plain SIMT (no TMA, no tensor core) kernel for the same operation. It exists to bisect faults
 * in the tensor-core path and as an on-device cross-check at sizes where a CPU check is slow.
 * It is never selected by hfrk_skinny_gemm_fp8. No counterpart in the reference. */
int hfrk_skinny_gemm_fp8_simt(const void* A, const void* W, void* D, const float* scale_dev,
                              int m, int n, int k, int64_t w_row_stride,
                              int a_kind, int w_kind, int d_dtype, int accumulate, void* stream);

/* hfrk_skinny_gemm_fp8_ex (m <= 64) that also records, per CTA, eight %globaltimer samples (ns)
 * into stamps_dev[cta][8]: 0 kernel entry, 1 set-up done, 2 first loads issued, 3 first stage
 * landed, 4 last MMA issued, 5 accumulator complete, 6 output written, 7 TMEM released.
 * stamps_dev holds grid CTAs * 8 uint64 (the plan query gives the CTA count). A profiling aid
 * with no counterpart in the reference. */
int hfrk_skinny_gemm_fp8_profile(const void* A, const void* W, void* D, const float* scale_dev,
                                 int m, int n, int k, int64_t w_row_stride,
                                 int a_kind, int w_kind, int d_dtype, int accumulate,
                                 int variant, int split_k, int ctas_per_sm, int num_stages, int use_pdl,
                                 unsigned long long* stamps_dev, void* stream);

/* Launch shape for (m, n, k) and the given pins (for logs and tests; no GPU work).
 * out[0]=variant chosen, out[1]=split_k (0 for STREAMK), out[2]=num_stages, out[3]=grid CTAs,
 * out[4]=dynamic shared memory bytes, out[5]=padded token count (MMA N), out[6]=K blocks of 128,
 * out[7]=tiles along N (of out[3]/out[1] CTAs; a tile is at most 128 rows). Returns a status code. */
int hfrk_skinny_gemm_plan(int m, int n, int k, int variant, int split_k, int ctas_per_sm, int* out8);

/* ---- the element-wise kernels either side of the GEMM in a decoder layer -------------------
 * Both quantise the input of the next projection to fp8 and zero the buffer that projection
 * accumulates into (the GEMM computes D += ...), so a layer is GEMM, one of these, GEMM, ...
 * with nothing in between. Both are launched as programmatic dependents (unless HFRK_PDL=0):
 * the weight prefetch of the GEMM after them overlaps them.
 *
 * Output encodings. HFRK_OUT_E4M3FNUZ writes the bytes the reference writes: value / scale in
 * e4m3fnuz, where callers pass the DOUBLED scale of hf_rocm_kernels/utils/fp8.py:31-33. The
 * bytes saturate at +-224 (0x7e), as utils/fp8.py:19-20 clamps, not at the +-240 (0x7f) of the
 * HIP conversion: 0x7f is NaN to a consumer that multiplies the bytes natively as e4m3fn, as the
 * GEMM here does. Negative zero is written as 0x00 (utils/fp8.py:26-30). A NaN input comes out as
 * 0x7f/0xff, the NaN of e4m3fn, which that consumer propagates (a reader that decodes the bytes as
 * true e4m3fnuz would see +-240 there). HFRK_OUT_E4M3FN writes value / scale in e4m3fn, saturating
 * at +-448. */
enum hfrk_norm_out { HFRK_OUT_SAME = 0, HFRK_OUT_E4M3FN = 1, HFRK_OUT_E4M3FNUZ = 2 };

/* out[r, c] = fp8( silu(gate_up[r, c]) * gate_up[r, hidden + c] / scale ),  c < hidden;
 * next_buffer[rows, buffer_cols] (16-bit elements) <- 0.
 *   gate_up [rows, 2*hidden] fp16 or bf16 (in_dtype: enum hfrk_out_dtype), contiguous
 *   out     [rows, hidden]   one byte per element, out_kind HFRK_E4M3FN or HFRK_E4M3FNUZ
 *   scale_dev                one fp32 on the device
 * hidden % 8 == 0 with gate_up 16-byte and out 8-byte aligned takes 16-byte loads; anything else
 * (or force_scalar != 0) takes the element-by-element kernel. rows == 0 is a no-op.
 * Replaces swiglu() of the reference (csrc/op_src/swiglu/swiglu_dispatch.cu:8-42; op schema
 * csrc/torch_bindings.cpp:31-35). */
int hfrk_swiglu_fp8(const void* gate_up, const float* scale_dev, void* out, void* next_buffer,
                    int rows, int hidden, int64_t buffer_cols, int in_dtype, int out_kind,
                    int force_scalar, void* stream);

/* residual <- input + residual (in place, rounded to the 16-bit type);
 * output <- residual * rsqrt(mean(residual^2) + epsilon) * weight, written in the 16-bit type
 * (out_kind HFRK_OUT_SAME, scale_dev may be NULL) or divided by *scale_dev and written as fp8
 * (HFRK_OUT_E4M3FN / HFRK_OUT_E4M3FNUZ); with fp8 output also next_buffer[rows, buffer_cols]
 * (16-bit elements) <- 0. With 16-bit output next_buffer is left alone, as in the reference
 * (residual_rms_dispatch.cu:33-43).
 *   input, residual [rows, cols], weight [cols]: fp16 or bf16 (dtype: enum hfrk_out_dtype)
 *   num_threads : CTA size, a multiple of 32 in [32, 1024]; anything else lets the library choose
 * One CTA per row. cols % 8 == 0 with 16-byte aligned tensors takes 16-byte loads; anything else
 * (or force_scalar != 0) the element-by-element kernel. rows == 0 is a no-op.
 * Replaces residual_rms() of the reference (csrc/op_src/residual_rms/residual_rms_dispatch.cu:8-63;
 * op schema csrc/torch_bindings.cpp:25-29). */
int hfrk_residual_rms(const void* input, void* residual, const void* weight, const float* scale_dev,
                      float epsilon, void* output, void* next_buffer, int rows, int cols,
                      int64_t buffer_cols, int dtype, int out_kind, int num_threads, int force_scalar,
                      void* stream);

/* The gate/up projection of an MLP block with swiglu folded into its epilogue: one launch in
 * place of hfrk_skinny_gemm_fp8 + hfrk_swiglu_fp8, with the same bytes as result.
 *   act_out[m, inter] <- fp8( silu(g) * u / *act_scale_dev ),  next_buffer[m, buffer_cols] <- 0
 *   where [g | u] = round16( *scale_dev * A[m, k] . W_gate_up[2*inter, k]^T )
 * W_gate_up holds the `inter` gate rows followed by the `inter` up rows (the layout the unfused
 * chain uses); a CTA's tile is 64 gate rows plus the matching 64 up rows. mid_dtype (HFRK_F16 or
 * HFRK_BF16) is the type the unfused chain would have stored the projection in: the epilogue
 * rounds to it before the activation so that fused and unfused results are identical bytes.
 * Limits: m <= 16 (HFRK_TOO_LARGE), inter % 16 == 0, no bias. K is split over a cluster as in the
 * plain GEMM when the matrix has too few tiles for the SMs; the reduction then hands every CTA
 * whole token rows, so the result does not depend on the split.
 * act_out and next_buffer 16-byte aligned. No counterpart in the reference, whose
 * combined_ops/llama_mlp.py:29-47 runs the two kernels one after the other. */
int hfrk_skinny_gemm_fp8_swiglu(const void* A, const void* W_gate_up, void* act_out,
                                const float* scale_dev, const float* act_scale_dev, void* next_buffer,
                                int m, int inter, int k, int64_t w_row_stride, int a_kind, int w_kind,
                                int mid_dtype, int out_kind, int64_t buffer_cols, void* stream);

/* Pins the launch shape of (m, n, k) for every later automatic call in this process: split_k and
 * num_stages as in hfrk_skinny_gemm_fp8_ex (0 = leave that one to the built-in rule; both 0 = drop
 * the entry). Token counts share an entry per multiple of 16. Fed from the JSON the grid search
 * writes (hf_rocm_kernels/benchmarks/skinny_gemm/grid_search.py); stands where the reference has
 * its hard-coded per-shape table (hf_rocm_kernels/operators/skinny_gemm/wrapped.py:42-102). */
int hfrk_tuning_set(int m, int n, int k, int split_k, int num_stages);
/* The same with the tile height: tile_rows = W rows per CTA, 8..128 (0 = the built-in rule, which
 * picks the smallest height that keeps the number of waves of the 128-row grid, so that the last
 * wave loads every SM alike). All three 0 = drop the entry. */
int hfrk_tuning_set_ex(int m, int n, int k, int split_k, int num_stages, int tile_rows);
int hfrk_tuning_clear(void);

/* What the launch planner knows about the current device: the SM count and, for cluster sizes
 * 1..16 and 1..3 CTAs per SM, how many clusters the chip holds at once, written to
 * capacity_out[17 * 4] as [cluster size][CTAs per SM]. The capacities are MEASURED on the first
 * call on a device (a probe kernel whose CTAs wait a bounded 50 us for each other; about 50 ms
 * once per device and process): clusters live inside one GPC and chips differ in how their SMs
 * are spread over the GPCs. That first call must not come inside a stream capture; if it does, an
 * estimate is used until a later call can measure (*measured_out = 0). Any pointer may be NULL.
 * Stands where the reference hard-codes its CU count (csrc/op_src/skinny_gemm/core.cu:24). */
int hfrk_device_model_get(int* sms_out, int* capacity_out, int* measured_out);
/* Replaces the device model by the given one for every later plan in this process (capacity as in
 * hfrk_device_model_get; NULL = back to the real device). For tests of the planner, which can
 * then run without a GPU, and for planning on behalf of another chip. */
int hfrk_device_model_override(int sms, const int* capacity);


/* How many clusters of `split` CTAs of the GEMM kernel with `smem_bytes` of dynamic shared memory
 * the current device can hold at once (cudaOccupancyMaxActiveClusters): the figure the launch
 * heuristic needs, exposed for tuning scripts. Clusters must fit inside one GPC, so the answer
 * depends on how the SMs of this particular chip are spread over its GPCs. */
int hfrk_max_active_clusters(int split, int smem_bytes, int* clusters_out);

/* Device-side status word of the current device: 0, or the HFRK_DEVICE_TIMEOUT details packed
 * as (code << 24 | role << 16 | block index & 0xffff). Reads it with a synchronous copy, and
 * clears it when `clear` is non-zero. Kernels only ever write it when a bounded wait runs out. */
int hfrk_device_status(int clear, unsigned int* word_out);

/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* hfrk_last_error(void);

/* Library version: major*10000 + minor*100 + patch. */
int hfrk_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HFRK_B200_H_ */
