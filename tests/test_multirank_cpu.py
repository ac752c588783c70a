"""The two sharding modes as multi-process programs on CPU (gloo, world size 2 and 4): each rank
draws the whole problem from the seed, keeps its shard, computes its part with the oracle and the
ranks exchange results the way the GPU path does -- nothing for the N split (the output columns
are disjoint), a sum of fp32 partials taken in rank order for the K split. Checks the sharding
helpers, that scales taken from the full tensors make shard results compose, and that the
rank-ordered sum every rank computes is identical and within the parity bound of the whole GEMM.
A third mode runs the tensor-parallel MLP block (column-sharded gate/up + swiglu, row-sharded down)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, mode: str, failures) -> None:
    for path in (os.path.join(ROOT, "hf-rocm-kernels_b200"), os.path.join(ROOT, "oracle")):
        if path not in sys.path:
            sys.path.insert(0, path)
    import oracle
    from hf_rocm_kernels.benchmarks.skinny_gemm import workloads as wl

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if mode == "mlp":
            _mlp_block_shards(rank, world, oracle)
            return
        case = wl.Case(2 if mode == "n" else 3, 77, "mini", 5, 64 * world * 2, 512 * world, bias=(mode == "k"))
        inp = wl.make_inputs(case)                           # same seed on every rank -> same tensors
        a_q, w_q = inp["a"].view(torch.uint8).numpy(), inp["w"].view(torch.uint8).numpy()
        scale = float(inp["scale"][0])
        d_in = None if inp["d_in"] is None else inp["d_in"].float().numpy()
        whole = oracle.reference_skinny_gemm(a_q, w_q, scale, d_in)
        if mode == "n":
            lo, hi = wl.n_split_rows(case.n, world, rank)
            mine = torch.from_numpy(oracle.reference_skinny_gemm(a_q, w_q[lo:hi], scale))
            pieces = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(pieces, mine)                    # only to check: the data path needs no collective
            assert np.array_equal(torch.cat(pieces, dim=1).numpy(), whole)
            assert (hi - lo) * world == case.n and lo == rank * (hi - lo)
        else:
            lo, hi = wl.k_split_cols(case.k, world, rank)
            assert lo % 16 == 0 and (hi - lo) * world == case.k
            # fp32 partial of this shard with scale 1 (what the kernel keeps before the exchange)
            partial = torch.from_numpy(oracle.reference_skinny_gemm(a_q[:, lo:hi], w_q[:, lo:hi], 1.0))
            gathered = [torch.empty_like(partial) for _ in range(world)]
            dist.all_gather(gathered, partial)
            total = np.zeros_like(gathered[0].numpy())
            for src in range(world):                          # rank order, identical on every rank
                total = total + gathered[src].numpy()
            out = (total.astype(np.float64) * np.float64(np.float32(scale)) + d_in.astype(np.float64)).astype(np.float32)
            res = oracle.compare(out, whole, case.k, scale, oracle.BF16, oracle.accumulation_floor(a_q, w_q, scale))
            assert res["hard_violations"] == 0 and res["violations"] == 0, res
            mine = torch.from_numpy(out)
            everyone = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(everyone, mine)
            assert all(torch.equal(e, mine) for e in everyone)
    except Exception as exc:  # report instead of hanging the peers
        failures.put((rank, repr(exc)))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def _mlp_block_shards(rank: int, world: int, oracle) -> None:
    """The tensor-parallel MLP block of ``llama_mlp_combined_ops(down_row_parallel=...)`` with the
    oracles: rank r holds the gate rows and the up rows [r*I/g, (r+1)*I/g) of the gate/up weight,
    stacked gate first, and the matching K columns of the down weight. Its swiglu output must be
    the column slice of the whole block's, and the rank-ordered sum of the down partials the whole
    block's result."""
    import elementwise_oracle as ew

    tokens, hidden, inter = 5, 256, 64 * world
    rng = np.random.default_rng(1234)                        # same seed on every rank -> same tensors
    a_q = oracle.quantize_e4m3fn(rng.standard_normal((tokens, hidden)).astype(np.float32), 4.0 / 448)
    w_gu = oracle.quantize_e4m3fn(rng.standard_normal((2 * inter, hidden)).astype(np.float32), 4.0 / 448)
    w_dn = oracle.quantize_e4m3fn(rng.standard_normal((hidden, inter)).astype(np.float32), 4.0 / 448)
    s_gu, s_act, s_dn = (4.0 / 448) ** 2 * 0.05, 16.0 / 448, (16.0 / 448) * (4.0 / 448)

    def gate_up_then_swiglu(w_rows):
        proj = oracle.reference_skinny_gemm(a_q, w_rows, s_gu)                # fp32 [tokens, 2 * cols]
        return ew.reference_swiglu(proj.astype(np.float16), s_act, oracle.F16, oracle.E4M3FN)

    act_whole = gate_up_then_swiglu(w_gu)
    whole = oracle.reference_skinny_gemm(act_whole, w_dn, s_dn)

    shard = inter // world
    lo, hi = rank * shard, (rank + 1) * shard
    w_gu_shard = np.concatenate([w_gu[lo:hi], w_gu[inter + lo:inter + hi]])     # gate_r then up_r
    act_shard = gate_up_then_swiglu(w_gu_shard)
    assert np.array_equal(act_shard, act_whole[:, lo:hi]), "a column shard of gate/up gives that slice of swiglu"

    partial = torch.from_numpy(oracle.reference_skinny_gemm(act_shard, w_dn[:, lo:hi], 1.0))
    gathered = [torch.empty_like(partial) for _ in range(world)]
    dist.all_gather(gathered, partial)
    total = np.zeros_like(partial.numpy())
    for src in range(world):                                  # rank order, identical on every rank
        total = total + gathered[src].numpy()
    out = (total.astype(np.float64) * np.float64(np.float32(s_dn))).astype(np.float32)
    res = oracle.compare(out, whole, inter, s_dn, oracle.BF16, oracle.accumulation_floor(act_whole, w_dn, s_dn))
    assert res["hard_violations"] == 0 and res["violations"] == 0, res
    mine = torch.from_numpy(out)
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    assert all(torch.equal(e, mine) for e in everyone)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("mode", ["n", "k", "mlp"])
def test_sharded_oracle_composes(world, mode, native_build):
    ctx = mp.get_context("spawn")
    failures = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, failures)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert failures.empty(), failures.get()
