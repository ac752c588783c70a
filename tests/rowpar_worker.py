"""One rank of the row-parallel parity test (launched by torchrun from test_gpu_rowpar.py).

Every rank draws the WHOLE problem from the same seed on CPU, keeps its K shard, runs the fused
GEMM + all-reduce, and checks its full result against the oracle's whole-K product. Also checks
that all ranks hold bit-identical results, that repeated calls (epoch/parity reuse of the exchange
buffer, including inside a CUDA graph) stay correct, and the unfused NCCL baseline."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (os.path.join(ROOT, "hf-rocm-kernels_b200"), os.path.join(ROOT, "oracle")):
    sys.path.insert(0, path)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import oracle  # noqa: E402
from hf_rocm_kernels import _capi  # noqa: E402
from hf_rocm_kernels.benchmarks.skinny_gemm import workloads as wl  # noqa: E402
from hf_rocm_kernels.combined_ops import RowParallelSkinnyGemm, skinny_gemm_then_allreduce  # noqa: E402


def tensor_parallel_mlp(group, dev, rank, world) -> None:
    """llama_mlp_combined_ops with the gate/up weight split by columns and the down weight by rows
    over the ranks, against the same block on one GPU with the whole weights. The partial sums are
    added in another order than one GPU's K loop, so the results agree to the GEMM's tolerance, not
    bit for bit; the ranks among themselves must agree bit for bit."""
    from hf_rocm_kernels.combined_ops import llama_mlp_combined_ops
    from hf_rocm_kernels.utils.fp8 import fp8_quantize_e4m3fn

    tokens, hidden, inter = 16, 2048, 1024 * world
    gen = torch.Generator().manual_seed(99)
    attn = torch.randn(tokens, hidden, generator=gen).bfloat16().to(dev)
    residual = torch.randn(tokens, hidden, generator=gen).bfloat16().to(dev)
    rms_w = (1 + 0.1 * torch.randn(hidden, generator=gen)).bfloat16().to(dev)
    q_gu, s_gu = fp8_quantize_e4m3fn((torch.randn(2 * inter, hidden, generator=gen) * 0.02).to(dev))
    q_dn, s_dn = fp8_quantize_e4m3fn((torch.randn(hidden, inter, generator=gen) * 0.02).to(dev))
    s_in = torch.tensor([4.0 / 448], device=dev)
    s_act = torch.tensor([16.0 / 448], device=dev)

    whole, whole_res = llama_mlp_combined_ops(attn, residual.clone(), rms_w, 1e-5, q_gu.t(), s_in, s_in * s_gu,
                                              q_dn.t(), s_act, s_act * s_dn)
    shard = inter // world
    lo, hi = rank * shard, (rank + 1) * shard
    gu_shard = torch.cat([q_gu.view(torch.uint8)[lo:hi], q_gu.view(torch.uint8)[inter + lo:inter + hi]])
    gu_shard = gu_shard.view(torch.float8_e4m3fn)                       # [2 * shard, hidden]: gate_r then up_r
    dn_shard = q_dn[:, lo:hi]                                           # [hidden, shard], row pitch of the whole
    outs = []
    for _ in range(2):
        out, res = llama_mlp_combined_ops(attn, residual.clone(), rms_w, 1e-5, gu_shard.t(), s_in, s_in * s_gu,
                                          dn_shard.t(), s_act, s_act * s_dn, down_row_parallel=group)
        torch.cuda.synchronize()
        outs.append(out)
        assert torch.equal(res, whole_res)
    assert _capi.device_status(clear=True)[0] == 0
    assert torch.equal(outs[0], outs[1])
    gathered = [torch.empty_like(outs[0]) for _ in range(world)]
    dist.all_gather(gathered, outs[0])
    assert all(torch.equal(g, outs[0]) for g in gathered), "ranks disagree on the MLP block"
    diff = (outs[0].float() - whole.float()).abs()
    # one bf16 step at the value, plus one at the block's typical magnitude for outputs that cancel to
    # almost nothing (their float32 partial sums are added in a different order)
    bound = whole.float().abs() * 2.0 ** -7 + whole.float().abs().mean() * 2.0 ** -7
    assert bool((diff <= bound).all()), float((diff - bound).max())


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    c_oracle = oracle.load_c_oracle()
    c_oracle.set_threads(max(1, len(os.sched_getaffinity(0)) // world))

    # the benchmark's row-parallel configuration exactly (M in {1,2,8,16}, N=8192, K=28672), then shapes
    # that reach the other code paths: a bias, ragged N, one token on a wide matrix, more than 16 tokens
    shapes = wl.cases(3) + [wl.Case(3, 101, "down_m16_bias", 16, 8192, 28672, bias=True),
                            wl.Case(3, 102, "small_m3", 3, 1000, 2048 * world),
                            wl.Case(3, 103, "wide_m1", 1, 20480, 1024 * world),
                            wl.Case(3, 104, "m40", 40, 1024, 512 * world, bias=True)]
    group = RowParallelSkinnyGemm(max_m=64, max_n=20480)
    for case in shapes:
        inp = wl.make_inputs(case, device="cpu")
        lo, hi = wl.k_split_cols(case.k, world, rank)
        a_sh = inp["a"][:, lo:hi].contiguous().to(dev)
        w_full = inp["w"].to(dev)
        w_sh = w_full[:, lo:hi]                      # column slice: keeps the full row pitch
        s = inp["scale"].to(dev)
        d0 = inp["d_in"].to(dev) if inp["d_in"] is not None else torch.zeros((case.m, case.n), dtype=torch.bfloat16, device=dev)
        scale = float(inp["scale"][0])
        a_q, w_q = inp["a"].view(torch.uint8).numpy(), inp["w"].view(torch.uint8).numpy()
        d32 = None if inp["d_in"] is None else inp["d_in"].float().numpy()
        ref = c_oracle.skinny_gemm(a_q, w_q, scale, d32)
        floor = oracle.accumulation_floor(a_q, w_q, scale)

        outs = []
        # both exchange schemes (and the automatic choice), back to back on the same buffer; with
        # three calls each, both parities of the buffer are reused under either scheme
        for mode in ("one_shot", "one_shot", "two_shot", "two_shot", "two_shot", "one_shot", "auto"):
            group.set_mode(mode)
            out = d0.clone()
            group(a_sh, w_sh, s, out)
            torch.cuda.synchronize()
            outs.append(out)
        group.set_mode("auto")
        code, word = _capi.device_status(clear=True)
        assert code == 0, f"rank {rank}: device status {word:#x}"
        for out in outs:
            res = oracle.compare(out.float().cpu().numpy(), ref, case.k, scale, oracle.BF16, floor)
            assert res["hard_violations"] == 0 and res["nan_out"] == 0, (rank, case.name, res)
            assert res["violations"] <= oracle.strict_exception_cap(case.k, res["count"]), (rank, case.name, res)
            assert torch.equal(out, outs[0])
        # every rank holds the same bits
        gathered = [torch.empty_like(outs[0]) for _ in range(world)]
        dist.all_gather(gathered, outs[0])
        assert all(torch.equal(g, outs[0]) for g in gathered), f"ranks disagree on {case.name}"

        # unfused baseline: fp32 partials + NCCL all-reduce
        base = d0.clone()
        partial = torch.empty((case.m, case.n), dtype=torch.float32, device=dev)
        skinny_gemm_then_allreduce(a_sh, w_sh, s, base, partial)
        torch.cuda.synchronize()
        res = oracle.compare(base.float().cpu().numpy(), ref, case.k, scale, oracle.BF16, floor)
        assert res["hard_violations"] == 0, (rank, case.name, "baseline", res)

    # CUDA graph: the call index lives on the device, so replays keep the ranks in step
    case = shapes[0]
    inp = wl.make_inputs(case, device="cpu")
    lo, hi = wl.k_split_cols(case.k, world, rank)
    a_sh, w_sh, s = inp["a"][:, lo:hi].contiguous().to(dev), inp["w"].to(dev)[:, lo:hi], inp["scale"].to(dev)
    out = torch.zeros((case.m, case.n), dtype=torch.bfloat16, device=dev)
    expect = torch.zeros_like(out)
    group(a_sh, w_sh, s, expect)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            group(a_sh, w_sh, s, out, accumulate=False, stream=stream)
            group(a_sh, w_sh, s, out, accumulate=False, stream=stream)
        for _ in range(5):
            graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, expect)
    assert _capi.device_status(clear=True)[0] == 0

    tensor_parallel_mlp(group, dev, rank, world)
    dist.barrier()
    group.close()
    print("ROWPAR_OK", rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
