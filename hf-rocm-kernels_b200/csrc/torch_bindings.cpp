// Registers torch.ops._HFRK_C.skinny_gemm_tb, .swiglu, .residual_rms and .increment with the schemas of
// the reference (csrc/torch_bindings.cpp:20-41 of huggingface/hf-rocm-kernels) and forwards to the C ABI
// of libhfrk_b200.so. This file is the only place where torch types meet the kernel library; it
// does what csrc/op_src/skinny_gemm/skinny_gemm_binding.cu:16-42 does in the reference: pull
// pointers, shapes and the W pitch out of the tensors, pick the current stream of A's device and
// return the launcher's status code.
#include <Python.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/all.h>
#include <torch/library.h>

#include "../../include/hfrk_b200.h"

namespace {

int fp8_kind_of(const torch::Tensor& t) {
    if (t.scalar_type() == at::ScalarType::Float8_e4m3fn) return HFRK_E4M3FN;
    if (t.scalar_type() == at::ScalarType::Float8_e4m3fnuz) return HFRK_E4M3FNUZ;
    return -1;
}

int out_kind_of(const torch::Tensor& t) {
    if (t.scalar_type() == at::ScalarType::Half) return HFRK_F16;
    if (t.scalar_type() == at::ScalarType::BFloat16) return HFRK_BF16;
    return -1;
}

}  // namespace

// A [m,k] row-major fp8; B [k,n] with stride(0) == 1, i.e. the row-major weight W [n,k] seen
// transposed, W's row pitch being B.stride(1); D [m,n] fp16/bf16 updated in place
// (D += scale * A.B); scale_tensor one fp32 on the device. split_k > 0 requests that K split,
// 0 lets the library choose; the other eight integers belonged to the reference's MI300X kernel
// and are ignored.
int64_t skinny_gemm_tb(torch::Tensor& A, torch::Tensor& B, torch::Tensor& D, torch::Tensor& scale_tensor,
                       int64_t split_k, int64_t A_producers, int64_t B_producers, int64_t consumers,
                       int64_t a_lanes, int64_t b_lanes, int64_t qsize, int64_t op_m, int64_t ops) {
    (void)A_producers; (void)B_producers; (void)consumers; (void)a_lanes;
    (void)b_lanes; (void)qsize; (void)op_m; (void)ops;
    if (A.dim() != 2 || B.dim() != 2 || B.stride(0) != 1 || !A.is_contiguous() || !D.is_contiguous() ||
        A.size(1) != B.size(0) || D.numel() != A.size(0) * B.size(1) || scale_tensor.numel() != 1 ||
        scale_tensor.scalar_type() != at::ScalarType::Float) {
        return HFRK_INVALID_CONFIG;
    }
    const int a_kind = fp8_kind_of(A), w_kind = fp8_kind_of(B), d_kind = out_kind_of(D);
    if (a_kind < 0 || w_kind < 0 || d_kind < 0) return HFRK_BAD_DTYPE;
    if (split_k < 0) return HFRK_INVALID_CONFIG;

    const at::cuda::OptionalCUDAGuard device_guard(device_of(A));
    const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int64_t m = A.size(0), k = A.size(1), n = B.size(1);
    if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return HFRK_INVALID_CONFIG;
    return hfrk_skinny_gemm_fp8(A.data_ptr(), B.data_ptr(), D.data_ptr(),
                                static_cast<const float*>(scale_tensor.data_ptr()), static_cast<int>(m),
                                static_cast<int>(n), static_cast<int>(k), B.stride(1), a_kind, w_kind, d_kind,
                                /*accumulate=*/1, static_cast<int>(split_k > 16 ? 16 : split_k), stream);
}

// The same GEMM for graph tracers: an op that returns an int cannot be captured into a traced graph,
// so this form returns nothing and raises on a non-zero status. No counterpart in the reference.
void skinny_gemm_inplace(torch::Tensor& A, torch::Tensor& B, torch::Tensor& D, torch::Tensor& scale_tensor,
                         int64_t split_k) {
    const int64_t status = skinny_gemm_tb(A, B, D, scale_tensor, split_k, 1, 1, 1, 1, 1, 12, 16, 4);
    TORCH_CHECK(status == HFRK_SUCCESS, "skinny_gemm: status ", status, " (see hfrk_b200.h)");
}

// Gate/up projection with swiglu in its epilogue (hfrk_skinny_gemm_fp8_swiglu): A [m, k] fp8, B the
// [k, 2*inter] view (stride(0) == 1) of the row-major gate/up weight, act_out [m, inter] fp8,
// next_buffer [m, any] 16-bit zeroed. mid_bf16 names the 16-bit type the unfused chain would have
// stored the projection in. No counterpart in the reference.
void skinny_gemm_swiglu(torch::Tensor& A, torch::Tensor& B, torch::Tensor& act_out, torch::Tensor& scale_tensor,
                        torch::Tensor& act_scale_tensor, torch::Tensor& next_buffer, bool mid_bf16) {
    TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && B.stride(0) == 1 && A.is_contiguous() && act_out.is_contiguous() &&
                    A.size(1) == B.size(0) && B.size(1) % 2 == 0 && act_out.numel() == A.size(0) * (B.size(1) / 2),
                "skinny_gemm_swiglu: expected A [m, k], B [k, 2*inter] column-major, act_out [m, inter]");
    TORCH_CHECK(scale_tensor.numel() == 1 && act_scale_tensor.numel() == 1 &&
                    scale_tensor.scalar_type() == at::ScalarType::Float &&
                    act_scale_tensor.scalar_type() == at::ScalarType::Float,
                "skinny_gemm_swiglu: the two scales must hold one fp32 each");
    const int a_kind = fp8_kind_of(A), w_kind = fp8_kind_of(B), out_kind = fp8_kind_of(act_out);
    TORCH_CHECK(a_kind >= 0 && w_kind >= 0 && out_kind >= 0, "skinny_gemm_swiglu: A, B and act_out must be e4m3");
    const int64_t m = A.size(0), k = A.size(1), inter = B.size(1) / 2;
    TORCH_CHECK(next_buffer.is_contiguous() && next_buffer.element_size() == 2 &&
                    (next_buffer.numel() == 0 || next_buffer.size(0) == m),
                "skinny_gemm_swiglu: next_buffer must be a contiguous 16-bit [m, .] matrix");
    TORCH_CHECK(m <= INT32_MAX && inter <= INT32_MAX && k <= INT32_MAX, "skinny_gemm_swiglu: extent above 2^31");
    const at::cuda::OptionalCUDAGuard device_guard(device_of(A));
    const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int status = hfrk_skinny_gemm_fp8_swiglu(
        A.data_ptr(), B.data_ptr(), act_out.data_ptr(), static_cast<const float*>(scale_tensor.data_ptr()),
        static_cast<const float*>(act_scale_tensor.data_ptr()), next_buffer.data_ptr(), static_cast<int>(m),
        static_cast<int>(inter), static_cast<int>(k), B.stride(1), a_kind, w_kind, mid_bf16 ? HFRK_BF16 : HFRK_F16,
        out_kind, m == 0 ? 0 : next_buffer.numel() / m, stream);
    TORCH_CHECK(status == HFRK_SUCCESS, "skinny_gemm_swiglu: status ", status, " (", hfrk_last_error(), ")");
}

// gate_up [rows, 2*hidden] fp16/bf16 -> output [rows, hidden] fp8 (e4m3fnuz as in the reference, or
// e4m3fn), next_buffer [rows, any] 16-bit zeroed. Stands where the reference has
// csrc/op_src/swiglu/swiglu_dispatch.cu:8-42. num_threads belonged to the reference's launch and is
// ignored; force_scalar selects the element-by-element kernel as it does there.
void swiglu(torch::Tensor& gate_up, torch::Tensor& scale_tensor, torch::Tensor& output, torch::Tensor& next_buffer,
            int64_t num_threads, bool force_scalar) {
    (void)num_threads;
    TORCH_CHECK(gate_up.dim() == 2 && gate_up.size(1) % 2 == 0 && gate_up.is_contiguous(),
                "swiglu: gate_up must be a contiguous [rows, 2*hidden] matrix");
    const int64_t rows = gate_up.size(0), hidden = gate_up.size(1) / 2;
    TORCH_CHECK(output.is_contiguous() && output.numel() == rows * hidden, "swiglu: output must be [rows, hidden]");
    TORCH_CHECK(next_buffer.is_contiguous() && next_buffer.element_size() == 2 &&
                    (next_buffer.numel() == 0 || next_buffer.size(0) == rows),
                "swiglu: next_buffer must be a contiguous 16-bit [rows, .] matrix");
    TORCH_CHECK(scale_tensor.numel() == 1 && scale_tensor.scalar_type() == at::ScalarType::Float,
                "swiglu: scale_tensor must hold one fp32");
    const int in_kind = out_kind_of(gate_up), out_kind = fp8_kind_of(output);
    TORCH_CHECK(in_kind >= 0, "swiglu: gate_up must be fp16 or bf16");
    TORCH_CHECK(out_kind >= 0, "swiglu: output must be float8_e4m3fnuz or float8_e4m3fn");
    TORCH_CHECK(rows <= INT32_MAX && hidden <= INT32_MAX, "swiglu: extent above 2^31");
    const at::cuda::OptionalCUDAGuard device_guard(device_of(gate_up));
    const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int64_t buffer_cols = rows == 0 ? 0 : next_buffer.numel() / rows;
    const int status = hfrk_swiglu_fp8(gate_up.data_ptr(), static_cast<const float*>(scale_tensor.data_ptr()),
                                       output.data_ptr(), next_buffer.data_ptr(), static_cast<int>(rows),
                                       static_cast<int>(hidden), buffer_cols, in_kind, out_kind,
                                       force_scalar ? 1 : 0, stream);
    TORCH_CHECK(status == HFRK_SUCCESS, "swiglu: status ", status, " (", hfrk_last_error(), ")");
}

// input, residual [rows, cols] and weight [cols] fp16/bf16; residual updated in place; output fp8
// (scale_tensor defined) or the 16-bit type (scale_tensor undefined, i.e. None in Python);
// next_buffer zeroed. Stands where the reference has
// csrc/op_src/residual_rms/residual_rms_dispatch.cu:8-63.
void residual_rms(torch::Tensor& input, torch::Tensor& residual, torch::Tensor& weight, torch::Tensor& scale_tensor,
                  double epsilon, torch::Tensor& output, torch::Tensor& next_buffer, int64_t num_threads,
                  bool force_scalar) {
    TORCH_CHECK(input.dim() == 2 && input.is_contiguous() && residual.is_contiguous() && weight.is_contiguous() &&
                    residual.sizes() == input.sizes() && weight.numel() == input.size(1),
                "residual_rms: input and residual must be contiguous [rows, cols], weight [cols]");
    const int dtype = out_kind_of(input);
    TORCH_CHECK(dtype >= 0 && residual.scalar_type() == input.scalar_type() &&
                    weight.scalar_type() == input.scalar_type(),
                "residual_rms: input, residual and weight must share fp16 or bf16");
    const int64_t rows = input.size(0), cols = input.size(1);
    TORCH_CHECK(output.is_contiguous() && output.numel() == rows * cols, "residual_rms: output must be [rows, cols]");
    TORCH_CHECK(next_buffer.is_contiguous() && next_buffer.element_size() == 2 &&
                    (next_buffer.numel() == 0 || next_buffer.size(0) == rows),
                "residual_rms: next_buffer must be a contiguous 16-bit [rows, .] matrix");
    int out_kind;
    const float* scale_ptr = nullptr;
    if (output.scalar_type() == input.scalar_type()) {
        out_kind = HFRK_OUT_SAME;
    } else {
        const int fp8 = fp8_kind_of(output);
        TORCH_CHECK(fp8 >= 0, "residual_rms: output must be the input's dtype, float8_e4m3fnuz or float8_e4m3fn");
        TORCH_CHECK(scale_tensor.defined() && scale_tensor.numel() == 1 &&
                        scale_tensor.scalar_type() == at::ScalarType::Float,
                    "residual_rms: an fp8 output needs a one-element fp32 scale_tensor");
        out_kind = fp8 == HFRK_E4M3FNUZ ? HFRK_OUT_E4M3FNUZ : HFRK_OUT_E4M3FN;
        scale_ptr = static_cast<const float*>(scale_tensor.data_ptr());
    }
    TORCH_CHECK(rows <= INT32_MAX && cols <= INT32_MAX, "residual_rms: extent above 2^31");
    const at::cuda::OptionalCUDAGuard device_guard(device_of(input));
    const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int64_t buffer_cols = rows == 0 ? 0 : next_buffer.numel() / rows;
    const int status = hfrk_residual_rms(input.data_ptr(), residual.data_ptr(), weight.data_ptr(), scale_ptr,
                                         static_cast<float>(epsilon), output.data_ptr(), next_buffer.data_ptr(),
                                         static_cast<int>(rows), static_cast<int>(cols), buffer_cols, dtype, out_kind,
                                         static_cast<int>(num_threads), force_scalar ? 1 : 0, stream);
    TORCH_CHECK(status == HFRK_SUCCESS, "residual_rms: status ", status, " (", hfrk_last_error(), ")");
}

// The reference's registration smoke test (csrc/op_src/increment/increment_op.cu:3): x += 1 through ATen.
void increment(torch::Tensor& x) { x.add_(1); }

TORCH_LIBRARY(_HFRK_C, ops) {
    ops.def("increment(Tensor! x) -> ()");
    ops.impl("increment", torch::kCUDA, &increment);
    ops.def(
        "residual_rms(Tensor input, Tensor! residual, Tensor weight, Tensor scale_tensor, float epsilon, Tensor! "
        "output, Tensor! next_buffer, int num_threads, bool force_scalar) -> ()");
    ops.impl("residual_rms", torch::kCUDA, &residual_rms);
    ops.def(
        "swiglu(Tensor gate_up, Tensor scale_tensor, Tensor! output, Tensor! next_buffer, int num_threads, "
        "bool force_scalar) -> ()");
    ops.impl("swiglu", torch::kCUDA, &swiglu);
    ops.def(
        "skinny_gemm_tb(Tensor A, Tensor B, Tensor! D, Tensor scale_tensor, int split_k, int A_producers, "
        "int B_producers, int consumers, int a_lanes, int b_lanes, int qsize, int op_m, int ops) -> int");
    ops.impl("skinny_gemm_tb", torch::kCUDA, &skinny_gemm_tb);
    ops.def("skinny_gemm_inplace(Tensor A, Tensor B, Tensor! D, Tensor scale_tensor, int split_k) -> ()");
    ops.impl("skinny_gemm_inplace", torch::kCUDA, &skinny_gemm_inplace);
    ops.def(
        "skinny_gemm_swiglu(Tensor A, Tensor B, Tensor! act_out, Tensor scale_tensor, Tensor act_scale_tensor, "
        "Tensor! next_buffer, bool mid_bf16) -> ()");
    ops.impl("skinny_gemm_swiglu", torch::kCUDA, &skinny_gemm_swiglu);
}

// Shape-only implementations for the Meta key, so that graph tracers (torch.compile, fake tensors)
// can step over the ops: every op works in place on tensors the caller allocated, so there is
// nothing to compute. The reference registers none; a serving engine that compiles its model needs them.
int64_t skinny_gemm_tb_meta(torch::Tensor&, torch::Tensor&, torch::Tensor&, torch::Tensor&, int64_t, int64_t, int64_t,
                            int64_t, int64_t, int64_t, int64_t, int64_t, int64_t) {
    return HFRK_SUCCESS;
}
void skinny_gemm_inplace_meta(torch::Tensor&, torch::Tensor&, torch::Tensor&, torch::Tensor&, int64_t) {}
void skinny_gemm_swiglu_meta(torch::Tensor&, torch::Tensor&, torch::Tensor&, torch::Tensor&, torch::Tensor&,
                             torch::Tensor&, bool) {}
void swiglu_meta(torch::Tensor&, torch::Tensor&, torch::Tensor&, torch::Tensor&, int64_t, bool) {}
void residual_rms_meta(torch::Tensor&, torch::Tensor&, torch::Tensor&, torch::Tensor&, double, torch::Tensor&,
                       torch::Tensor&, int64_t, bool) {}
void increment_meta(torch::Tensor&) {}

TORCH_LIBRARY_IMPL(_HFRK_C, Meta, ops) {
    ops.impl("skinny_gemm_tb", &skinny_gemm_tb_meta);
    ops.impl("skinny_gemm_inplace", &skinny_gemm_inplace_meta);
    ops.impl("skinny_gemm_swiglu", &skinny_gemm_swiglu_meta);
    ops.impl("swiglu", &swiglu_meta);
    ops.impl("residual_rms", &residual_rms_meta);
    ops.impl("increment", &increment_meta);
}

// `import hf_rocm_kernels._HFRK_C` only has to load this shared object so that the static
// registration above runs; the module itself is empty.
PyMODINIT_FUNC PyInit__HFRK_C(void) {
    static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, "_HFRK_C", nullptr, 0, nullptr, nullptr, nullptr, nullptr, nullptr};
    return PyModule_Create(&module);
}
