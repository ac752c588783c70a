"""The operators inside a traced graph: ``torch.compile(fullgraph=True)`` over the package's Python
API must capture all of them (no graph break) and give the bytes of eager execution. This is what
a serving engine that compiles its model needs; the reference registers no shape-only
implementations and its GEMM op returns an int, which a traced graph cannot hold, so the wrapper
switches to a form of the same op that returns nothing while tracing."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_the_python_api_compiles_without_graph_breaks(native_build):
    from hf_rocm_kernels import residual_rms, skinny_gemm, swiglu
    from hf_rocm_kernels.utils.fp8 import fp8_quantize_e4m3fn

    dev = torch.device("cuda:0")
    torch.manual_seed(5)
    w_q, w_s = fp8_quantize_e4m3fn(torch.randn(2048, 1024, device=dev) * 0.02)
    a_q, a_s = fp8_quantize_e4m3fn(torch.randn(4, 1024, device=dev))
    scale = a_s * w_s
    gamma = torch.ones(1024, dtype=torch.bfloat16, device=dev)

    def layer(a_q, scale):
        out = torch.zeros((4, 2048), dtype=torch.bfloat16, device=dev)
        skinny_gemm(a_q, w_q.t(), scale, out)
        act = swiglu(out, scale * 1000, out_dtype=torch.float8_e4m3fn)
        x = out[:, :1024].contiguous()
        normed, res = residual_rms(x, x.clone(), gamma, 1e-5, scale * 1000, out_dtype=torch.float8_e4m3fn)
        return out, act, normed, res

    def as_bytes(t):
        return t.view(torch.uint8) if t.dtype.itemsize == 1 else t

    eager = layer(a_q, scale)
    compiled = torch.compile(layer, backend="aot_eager", fullgraph=True)
    for _ in range(2):
        got = compiled(a_q, scale)
        torch.cuda.synchronize()
        assert all(torch.equal(as_bytes(g), as_bytes(e)) for g, e in zip(got, eager))


def test_the_mlp_block_compiles_without_graph_breaks(native_build):
    from hf_rocm_kernels.combined_ops import llama_mlp_combined_ops
    from hf_rocm_kernels.utils.fp8 import fp8_quantize_e4m3fn

    dev = torch.device("cuda:0")
    torch.manual_seed(6)
    tokens, hidden, inter = 8, 1024, 2048
    attn = torch.randn(tokens, hidden, device=dev).bfloat16()
    residual = torch.randn(tokens, hidden, device=dev).bfloat16()
    gamma = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
    w_gu, s_gu = fp8_quantize_e4m3fn(torch.randn(2 * inter, hidden, device=dev) * 0.02)
    w_dn, s_dn = fp8_quantize_e4m3fn(torch.randn(hidden, inter, device=dev) * 0.02)
    s_in = torch.tensor([4.0 / 448], device=dev)
    s_act = torch.tensor([16.0 / 448], device=dev)

    def block(attn, residual):
        return llama_mlp_combined_ops(attn, residual, gamma, 1e-5, w_gu.t(), s_in, s_in * s_gu, w_dn.t(), s_act,
                                      s_act * s_dn)

    want_out, want_res = block(attn, residual.clone())
    compiled = torch.compile(block, backend="aot_eager", fullgraph=True)
    got_out, got_res = compiled(attn, residual.clone())
    torch.cuda.synchronize()
    assert torch.equal(got_out, want_out) and torch.equal(got_res, want_res)
