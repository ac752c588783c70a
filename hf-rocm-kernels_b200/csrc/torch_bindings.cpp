// Registers torch.ops._HFRK_C.skinny_gemm_tb with the schema of the reference
// (csrc/torch_bindings.cpp:38-41 of huggingface/hf-rocm-kernels) and forwards to the C ABI of
// libhfrk_b200.so. This file is the only place where torch types meet the kernel library; it
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

TORCH_LIBRARY(_HFRK_C, ops) {
    ops.def(
        "skinny_gemm_tb(Tensor A, Tensor B, Tensor! D, Tensor scale_tensor, int split_k, int A_producers, "
        "int B_producers, int consumers, int a_lanes, int b_lanes, int qsize, int op_m, int ops) -> int");
    ops.impl("skinny_gemm_tb", torch::kCUDA, &skinny_gemm_tb);
}

// `import hf_rocm_kernels._HFRK_C` only has to load this shared object so that the static
// registration above runs; the module itself is empty.
PyMODINIT_FUNC PyInit__HFRK_C(void) {
    static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, "_HFRK_C", nullptr, 0, nullptr};
    return PyModule_Create(&module);
}
