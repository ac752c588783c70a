"""Benchmark of the FP8 skinny GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-detail]

One *step* is one pass over the Llama-3-8B decode projections (configuration 1 of the benchmark
specification: M in {1,2,4,8,16} x {qkv 6144x4096 (+bias), o_proj 4096x4096, gate_up 28672x4096,
down 4096x14336}, 20 calls), every call on its own weight matrix, so a step streams 1.09 GB of
distinct weights -- about nine times the L2 -- and nothing is re-read from cache between calls or
between steps. The 20 calls are captured once in a CUDA graph through the public torch op (the
reference times its op the same way: operators/skinny_gemm/benchmarking_fn.py:62-92) and the graph
is replayed once per step.

Printed: ONE JSON line. ``value`` is the achieved HBM bandwidth over the timed steps (algorithmic
bytes of every call / device time, inputs resident in HBM), whole job over all ranks. ``e2e`` is
the same metric through the C ABI's host-buffer call: activations (and the bias) come from pinned
host memory and the result is read back to the host inside the timed region, every call; weights
stay resident (they are model state). With N > 1 (launched by torchrun, one rank per GPU) every
rank runs the same per-GPU workload on its own shard of a column-parallel layer, no collective on
the data path: weak scaling.

``--impl reference`` times the CPU port of the reference's semantics (oracle/cpu_baseline.py) on
the host cores instead; rank 0 only.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "hf-rocm-kernels_b200"))

METRIC = "fp8_skinny_gemm_hbm_bandwidth"
UNIT = "TB/s"
WORKLOAD = "llama3_8b_decode_projections_fp8_e4m3_bf16out_M1-16 (configuration 1)"
L2_BYTES = 126 * 1024 * 1024   # B200; replaced by the device's own figure once a GPU is in hand (run_ours)


def measured_hbm_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy kernel)"
    except Exception:
        return 6650.0, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU through NVML (read-only queries)
    every few milliseconds while the timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        self.index = index
        self.sm = []
        self.mask = 0
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.recording = threading.Event()
        self.thread = None
        self.error = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            # CUDA_VISIBLE_DEVICES may renumber devices: resolve the NVML handle through the PCI bus id
            import torch

            bus = torch.cuda.get_device_properties(self.index).pci_bus_id if hasattr(
                torch.cuda.get_device_properties(self.index), "pci_bus_id") else None
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            if bus is not None:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    if int(pynvml.nvmlDeviceGetPciInfo(h).bus) == int(bus):
                        self.handle = h
                        break
            self.nvml = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # NVML missing: report it rather than fail the benchmark
            self.error = repr(exc)[:120]
            return
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()

    def begin(self):
        """Samples taken from here on count: the thread is started earlier so that the first,
        slow NVML queries fall outside the timed region."""
        self.recording.set()

    def _poll(self):
        while not self.stop_flag.is_set():
            try:
                mhz = float(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
                reasons = int(self.nvml.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                if self.recording.is_set():
                    self.sm.append(mhz)
                    self.mask |= reasons
            except Exception as exc:
                self.error = repr(exc)[:120]
                return
            time.sleep(0.002)

    def stop(self):
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=1)
        reasons = sorted(name for name, bit in self.REASONS.items() if self.mask & bit)
        out = {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
               "reasons": reasons, "samples": len(self.sm)}
        if self.error:
            out["error"] = self.error
        return out


def build_workload(dev, wl, torch):
    """Per case: inputs on the device (drawn by a device generator: values N(0,1), per-tensor
    e4m3fn quantisation) plus, for the e2e leg, page-locked host copies of the per-step inputs: all
    activations of a step in one block and all outputs in another, as a serving loop would hold them."""
    cases = wl.cases(1)
    a_block = torch.empty(sum(c.m * c.k for c in cases), dtype=torch.uint8).pin_memory()
    d_block = torch.empty(sum(c.m * c.n for c in cases), dtype=torch.bfloat16).pin_memory()
    items, a_off, d_off = [], 0, 0
    for case in cases:
        inp = wl.make_inputs(case, device=str(dev))
        d0 = inp["d_in"] if inp["d_in"] is not None else torch.zeros((case.m, case.n), dtype=torch.bfloat16, device=dev)
        a_host = a_block[a_off:a_off + case.m * case.k].view(torch.float8_e4m3fn).view(case.m, case.k)
        d_host = d_block[d_off:d_off + case.m * case.n].view(case.m, case.n)
        a_host.copy_(inp["a"].cpu())
        d_host.copy_(d0.cpu())
        a_off += case.m * case.k
        d_off += case.m * case.n
        items.append({
            "case": case, "a": inp["a"], "w": inp["w"], "scale": inp["scale"], "d0": d0, "d": d0.clone(),
            "a_host": a_host, "d_host": d_host, "d0_host": d0.cpu().pin_memory(),
        })
    return items


def self_check(items, capi, wl, torch, dev):
    """Run before any number is printed, so that a timed kernel that does not do the work cannot
    produce a figure. (1) One seeded case (configuration 1, qkv with bias, 16 tokens, drawn on the
    CPU as the parity tests draw it) against the CPU oracle under the parity tests' criterion:
    nothing beyond tolerance + accumulation floor, and (K = 4096 here) nothing beyond the stated
    bound itself. (2) Every 16-token shape of the step against the SIMT diagnostic kernel (an
    independent code path: no TMA, no tensor core): both round to bf16, so they may sit one bf16
    step apart plus the two kernels' fp32 summation-order difference."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle  # the checker

    case = wl.cases(1)[16]
    inp = wl.make_inputs(case, device="cpu")
    out = inp["d_in"].to(dev).clone()
    capi.check(capi.skinny_gemm(inp["a"].to(dev), inp["w"].to(dev), out, inp["scale"].to(dev)))
    torch.cuda.synchronize()
    a_q, w_q = inp["a"].view(torch.uint8).numpy(), inp["w"].view(torch.uint8).numpy()
    scale = float(inp["scale"][0])
    ref = oracle.load_c_oracle().skinny_gemm(a_q, w_q, scale, inp["d_in"].float().numpy())
    res = oracle.compare(out.float().cpu().numpy(), ref, case.k, scale, oracle.BF16,
                         oracle.accumulation_floor(a_q, w_q, scale))
    if res["hard_violations"] or res["nan_out"] or res["violations"] > oracle.strict_exception_cap(case.k, res["count"]):
        raise RuntimeError(f"self-check against the oracle failed on {case.name}: {res}")
    summary = {"oracle_case": case.name, "count": res["count"], "beyond_stated_bound": res["violations"],
               "beyond_bound_plus_floor": res["hard_violations"], "max_err_over_tol": round(res["max_err_over_tol"], 3)}

    for it in items:
        if it["case"].m != 16:
            continue
        got = it["d0"].clone()
        want = it["d0"].clone()
        capi.check(capi.skinny_gemm(it["a"], it["w"], got, it["scale"]))
        capi.check(capi.skinny_gemm_simt(it["a"], it["w"], want, it["scale"]))
        torch.cuda.synchronize()
        k = it["case"].k
        bound = want.float().abs() * 2.0 ** -7 + 2e-3 * (k ** 0.5) * float(it["scale"][0]) + 1e-30
        over = int(((got.float() - want.float()).abs() > bound).sum().item())
        if over > oracle.MAX_STRICT_EXCEPTIONS:
            raise RuntimeError(f"self-check against the SIMT kernel failed for {it['case'].name}: {over} elements differ")
    return summary


def time_case_rotating(it, skinny_gemm, torch, warmups=8, iters=24):
    """us per call of one case the way the reference measures it: one graph of G back-to-back calls
    on G different weight matrices (G matrices total at least twice the L2), replayed."""
    case = it["case"]
    g_count = max(8, -(-2 * L2_BYTES // case.weight_bytes))
    pool = [it["w"]] + [it["w"].clone() for _ in range(g_count - 1)]
    for k, extra in enumerate(pool[1:]):  # make the copies different matrices
        extra.view(torch.uint8).copy_(torch.roll(it["w"].view(torch.uint8), shifts=k + 1, dims=0))
    out = it["d0"].clone()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        skinny_gemm(it["a"], pool[0].t(), it["scale"], out)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for w in pool:
                skinny_gemm(it["a"], w.t(), it["scale"], out)
        times = []
        for i in range(warmups + iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            e1.synchronize()
            if i >= warmups:
                times.append(e0.elapsed_time(e1) * 1000.0 / g_count)
    del pool
    return statistics.median(times)


def time_scaled_mm_rotating(it, torch, warmups=8, iters=24):
    """us per call of torch._scaled_mm (cuBLASLt's fp8 GEMM) on the same case with the same method
    (graph of G calls on G different weight matrices), as the reference compares its kernel with
    _scaled_mm (hf_rocm_kernels/benchmarks/skinny_gemm/all_knobs.py:34-56). The bias, where the case
    has one, goes in as _scaled_mm's own bias argument. None if cuBLASLt refuses the shape."""
    case = it["case"]
    g_count = max(8, -(-2 * L2_BYTES // case.weight_bytes))
    pool = [it["w"]] + [it["w"].clone() for _ in range(g_count - 1)]
    one = torch.ones((), dtype=torch.float32, device=it["a"].device)
    bias = it["d0"][0].contiguous() if case.bias else None
    try:
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            def call(w):
                return torch._scaled_mm(it["a"], w.t(), scale_a=it["scale"].reshape(()), scale_b=one, bias=bias,
                                        out_dtype=torch.bfloat16)
            call(pool[0])
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for w in pool:
                    call(w)
            times = []
            for i in range(warmups + iters):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                graph.replay()
                e1.record(stream)
                e1.synchronize()
                if i >= warmups:
                    times.append(e0.elapsed_time(e1) * 1000.0 / g_count)
        return statistics.median(times)
    except Exception:
        torch.cuda.synchronize()
        return None
    finally:
        del pool


def run_ours(args):
    import torch
    import torch.distributed as dist

    import hf_rocm_kernels
    from hf_rocm_kernels import _capi as capi
    from hf_rocm_kernels.benchmarks.skinny_gemm import workloads as wl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    global L2_BYTES
    L2_BYTES = int(torch.cuda.get_device_properties(dev).L2_cache_size)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    items = build_workload(dev, wl, torch)
    check_summary = self_check(items, capi, wl, torch, dev)
    step_bytes = sum(it["case"].algorithmic_bytes() for it in items)
    step_weight_bytes = sum(it["case"].weight_bytes for it in items)

    # ---- the device-resident leg: one CUDA graph of the 20 calls, through the torch op
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for it in items:
            hf_rocm_kernels.skinny_gemm(it["a"], it["w"].t(), it["scale"], it["d"])
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for it in items:
                hf_rocm_kernels.skinny_gemm(it["a"], it["w"].t(), it["scale"], it["d"])
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        stream.synchronize()
        barrier()
        sampler.begin()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        e1.synchronize()
        device_ms = e0.elapsed_time(e1)
        # K steps of ~0.23 ms are over before the sampler (one NVML query per ~2 ms) has seen much: the
        # same graph keeps running, untimed, until the clock record covers at least 60 ms of this load
        extra_replays = 0
        if rank == 0:
            window_start = time.perf_counter()
            while time.perf_counter() - window_start < 0.06:
                for _ in range(10):
                    graph.replay()
                stream.synchronize()
                extra_replays += 10
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        if clocks is not None:
            clocks["window"] = f"the timed region plus {extra_replays} further replays of the same graph (same load, untimed)"

    # ---- the end-to-end leg: host buffers through the C ABI, copies inside the timed region. A step
    # hands its 20 calls to the library in ONE call (hfrk_skinny_gemm_fp8_host_batch): activations and
    # the bias-filled outputs go host->device, the GEMMs run, the results come back device->host on
    # the library's copy stream while later GEMMs run, and the step waits once for all results, as a
    # decode step would.
    batch = capi.HostBatch([(it["a_host"], it["w"], it["d_host"], it["scale"], it["case"].bias,
                             it["d0_host"] if it["case"].bias else None) for it in items], dev)
    lanes = [(torch.cuda.Stream(), torch.empty(max(capi.lib.hfrk_host_call_workspace_bytes(c.m, c.n, c.k)
                                                   for c in wl.cases(1)), dtype=torch.uint8, device=dev))]
    e2e_stream = torch.cuda.Stream()
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        # the bias-filled D_in of the qkv calls is read from its own page-locked buffer (D_in_host), the
        # results land in d_host: nothing for the caller to refill between steps
        capi.check(batch.queue(e2e_stream))
        e2e_stream.synchronize()

    for _ in range(2):
        e2e_step()
    # the batch must return what the single synchronous host call returns, and what the device-resident call returns
    for probe in (items[0], items[-1], items[16]):
        expect_host = probe["d0_host"].clone()
        capi.check(capi.skinny_gemm_host(probe["a_host"], probe["w"], expect_host, probe["scale"], lanes[0][1],
                                         accumulate=probe["case"].bias))
        on_device = probe["d0"].clone()
        capi.check(capi.skinny_gemm(probe["a"], probe["w"], on_device, probe["scale"]))
        torch.cuda.synchronize()
        if not (torch.equal(expect_host, probe["d_host"]) and torch.equal(on_device.cpu(), probe["d_host"])):
            raise RuntimeError(f"end-to-end leg: batch, single host call and device call disagree on {probe['case'].name}")
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1000.0
    barrier()
    h2d = sum(c.m * c.k + (2 * c.m * c.n if c.bias else 0) for c in wl.cases(1))
    d2h = sum(2 * c.m * c.n for c in wl.cases(1))

    # ---- multi-GPU extras: configuration 2 (N split, no collective) and 3 (K split, fused all-reduce)
    multi = multi_gpu_extras(torch, dist, capi, wl, dev, rank, world) if world > 1 else None

    # ---- per-case times (rank 0 of a single-GPU run only; bounded)
    detail = None
    if world == 1 and not args.no_detail:
        detail = []
        for it in items:
            us = time_case_rotating(it, hf_rocm_kernels.skinny_gemm, torch)
            lt = time_scaled_mm_rotating(it, torch)
            c = it["case"]
            detail.append({"case": c.name, "us_per_call": round(us, 2),
                           "hbm_tbps": round(c.algorithmic_bytes() / us / 1e6, 3),
                           "weight_tbps": round(c.weight_bytes / us / 1e6, 3),
                           "frac_of_peak": round(c.algorithmic_bytes() / us / 1e3 / measured_hbm_peak_gbs()[0], 3),
                           "scaled_mm_us": None if lt is None else round(lt, 2)})

    # ---- configuration 2 with all of N on this GPU (its g = 1 column): the Llama-3-70B projections
    detail_70b = None
    if world == 1 and not args.no_detail:
        detail_70b = []
        for c in wl.cases(2):
            inp = wl.make_inputs(c, device=str(dev))
            it = {"case": c, "a": inp["a"], "w": inp["w"], "scale": inp["scale"],
                  "d0": torch.zeros((c.m, c.n), dtype=torch.bfloat16, device=dev)}
            us = time_case_rotating(it, hf_rocm_kernels.skinny_gemm, torch, warmups=4, iters=12)
            lt = time_scaled_mm_rotating(it, torch, warmups=4, iters=12)
            detail_70b.append({"case": c.name, "us_per_call": round(us, 2),
                               "weight_tbps": round(c.weight_bytes / us / 1e6, 3),
                               "frac_of_peak": round(c.algorithmic_bytes() / us / 1e3 / measured_hbm_peak_gbs()[0], 3),
                               "scaled_mm_us": None if lt is None else round(lt, 2)})
            del it, inp
            torch.cuda.empty_cache()

    layer_block = mlp_block_detail(torch, dev) if world == 1 and not args.no_detail else None

    status_code, status_word = capi.device_status(clear=True)
    if status_code != 0:
        raise RuntimeError(f"device status word {status_word:#x}: a bounded wait ran out during the benchmark")

    # ---- max over ranks
    times = torch.tensor([device_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    device_ms, e2e_ms = times.tolist()

    if rank == 0:
        peak_gbs, peak_source = measured_hbm_peak_gbs()
        ms_per_step = device_ms / args.steps
        value = world * step_bytes / (ms_per_step * 1e-3) / 1e12
        per_gpu_gbs = step_bytes / (ms_per_step * 1e-3) / 1e9
        e2e_value = world * step_bytes / (e2e_ms / e2e_steps * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (f32 accumulate, bf16 out)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "calls_per_step": len(items),
                       "weight_bytes_per_step": step_weight_bytes, "algorithmic_bytes_per_step": step_bytes,
                       "l2": "each call has its own weight matrix; a step streams 1.09 GB (>> 126 MB L2)",
                       "timing": "CUDA events on the launching stream around K graph replays, max over ranks",
                       "us_per_call_mean": round(ms_per_step * 1e3 / len(items), 3),
                       "weight_stream_tbps": round(world * step_weight_bytes / (ms_per_step * 1e-3) / 1e12, 4)},
            "roofline": {"bound": "hbm", "achieved": round(per_gpu_gbs, 1), "peak": peak_gbs, "unit": "GB/s",
                         "frac": round(per_gpu_gbs / peak_gbs, 4),
                         "frac_of_nominal_8000_gbs": round(per_gpu_gbs / 8000.0, 4),
                         # ncu dram__bytes_read+write per launch = 1.00-1.03 x the algorithmic bytes on the two
                         # captured single calls (17 MB and 118 MB); scaled to this step's average launch
                         "traffic": int(1.02 * step_bytes / len(items)), "traffic_unit": "bytes/launch",
                         "algorithmic_bytes_per_launch": int(step_bytes / len(items)), "peak_source": peak_source,
                         "kernel": "skinny_gemm_fp8_sm100_kernel", "launches": args.steps * len(items)},
            "e2e": {"value": round(e2e_value, 4), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "note": "host activations/bias in, host results out, every call, through hfrk_skinny_gemm_fp8_host_batch (one library call per step); weights resident; copies by cudaMemcpyAsync from/to page-locked memory inside the timed region; the step waits once for all results"},
            "gpu_launches": args.steps * len(items),
            "self_check": check_summary,
            "clocks": clocks,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline(torch, wl)
        if detail is not None and detail_70b is not None:
            timed = [d for d in detail + detail_70b if d["scaled_mm_us"] is not None]
            line["vs_cublaslt"] = {"wins": sum(1 for d in timed if d["us_per_call"] < d["scaled_mm_us"]),
                                   "of": len(timed), "not_run_by_cublaslt": len(detail) + len(detail_70b) - len(timed),
                                   "what": "cases where this library's us_per_call is below torch._scaled_mm's, "
                                           "same graph-of-rotating-weights timing"}
        if detail is not None:
            line["detail"] = detail
        if detail_70b is not None:
            line["detail_llama3_70b"] = detail_70b
        if layer_block is not None:
            line["layer_block"] = layer_block
        if multi is not None:
            line["multi_gpu"] = multi
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def mlp_block_detail(torch, dev, tokens=16):
    """The Llama-3-8B MLP block through hf_rocm_kernels.combined_ops.llama_mlp_combined_ops, as three
    launches (residual_rms -> gate/up GEMM with swiglu in its epilogue -> down GEMM) and as the
    reference's four (swiglu as its own kernel), and the two element-wise kernels on their own, each
    from a CUDA graph of back-to-back calls. Four weight sets rotate so
    that weights come from HBM (4 x 176 MB >> L2). Not part of the headline figure."""
    from hf_rocm_kernels.combined_ops import llama_mlp_combined_ops
    from hf_rocm_kernels.utils.benchmarking import time_graph_us
    from hf_rocm_kernels.utils.fp8 import fp8_quantize_e4m3fn

    hidden, inter, sets = 4096, 14336, 4
    gen = torch.Generator(device=dev).manual_seed(7)
    attn = torch.randn(tokens, hidden, device=dev, generator=gen).bfloat16()
    residual = torch.randn(tokens, hidden, device=dev, generator=gen).bfloat16()
    rms_weight = torch.ones(hidden, device=dev).bfloat16()
    gate_up = [fp8_quantize_e4m3fn(torch.randn(2 * inter, hidden, device=dev, generator=gen) * 0.02)
               for _ in range(sets)]
    down = [fp8_quantize_e4m3fn(torch.randn(hidden, inter, device=dev, generator=gen) * 0.02) for _ in range(sets)]
    s_in = torch.tensor([4.0 / 448], device=dev)
    s_act = torch.tensor([16.0 / 448], device=dev)
    scales = [(s_in * gate_up[j][1], s_act * down[j][1]) for j in range(sets)]

    def block(i, fuse=None):
        j = i % sets
        llama_mlp_combined_ops(attn, residual, rms_weight, 1e-5, gate_up[j][0].t(), s_in, scales[j][0],
                               down[j][0].t(), s_act, scales[j][1], fuse_swiglu=fuse)

    chain_us = time_graph_us(block, graph_size=8, warmups=5, iterations=20)
    four_us = time_graph_us(lambda i: block(i, False), graph_size=8, warmups=5, iterations=20)
    normed = torch.empty(tokens, hidden, dtype=torch.float8_e4m3fn, device=dev)
    gu = torch.zeros(tokens, 2 * inter, dtype=torch.bfloat16, device=dev)
    act = torch.empty(tokens, inter, dtype=torch.float8_e4m3fn, device=dev)
    out = torch.zeros(tokens, hidden, dtype=torch.bfloat16, device=dev)
    rms_us = time_graph_us(lambda i: torch.ops._HFRK_C.residual_rms(attn, residual, rms_weight, s_in, 1e-5, normed,
                                                                    gu, 0, False), 16, 5, 20)
    swiglu_us = time_graph_us(lambda i: torch.ops._HFRK_C.swiglu(gu, s_act, act, out, 0, False), 16, 5, 20)
    weight_bytes = 3 * inter * hidden
    return {"block": "llama3-8b mlp, residual_rms -> gate_up (+swiglu in the epilogue) -> down", "tokens": tokens,
            "us_per_block": round(chain_us, 2), "weight_tbps": round(weight_bytes / chain_us / 1e6, 3),
            "launches_per_block": 3, "us_per_block_four_launches": round(four_us, 2),
            "residual_rms_alone_us": round(rms_us, 2), "swiglu_alone_us": round(swiglu_us, 2)}


def _graph_time_us(torch, dist, dev, fns, reps=20, warm=5):
    """Median microseconds per call of a graph of len(fns) calls, max over ranks."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        fns[0]()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for fn in fns:
                fn()
        times = []
        for i in range(warm + reps):
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            e1.synchronize()
            if i >= warm:
                times.append(e0.elapsed_time(e1) * 1000.0 / len(fns))
    t = torch.tensor([statistics.median(times)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _all_ranks_agree(torch, dist, flag: bool, dev) -> bool:
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def multi_gpu_parity(torch, dist, capi, wl, dev, rank, world):
    """Correctness of the two sharding modes on this run's GPUs, before anything is timed.

    Every rank draws the WHOLE seeded problem on its GPU (same seed, same generator: identical
    tensors on every rank), keeps its shard and runs the library. Checked, outside any timed region:
      * configuration 3 (the exact grid: M in {1,2,8,16}, N=8192, K=28672 split over the ranks): the
        fused GEMM + all-reduce under the one-shot, the two-shot and the automatic exchange gives the
        same bits under all three and on all ranks, and rank 0 compares them with the CPU oracle's
        whole-K product under the parity tolerance;
      * configuration 2: N-split shards, gathered, against the oracle's whole product;
      * the tensor-parallel MLP block (gate/up split by columns, down split by rows with the fused
        all-reduce) against the same block on one GPU.
    The oracle is used here as the checker only. Raises if anything disagrees."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle  # checker, rank 0 only does the arithmetic

    from hf_rocm_kernels.combined_ops import RowParallelSkinnyGemm

    c_oracle = oracle.load_c_oracle() if rank == 0 else None
    report = {"cases": 0, "strict_bound_exceptions": 0}

    def oracle_check(out_full, inp, case, label):
        """rank 0: out_full [M,N] against the exact product; returns ok."""
        ok = True
        if rank == 0:
            a_q = inp["a"].view(torch.uint8).cpu().numpy()
            w_q = inp["w"].view(torch.uint8).cpu().numpy()
            scale = float(inp["scale"][0])
            d32 = None if inp["d_in"] is None else inp["d_in"].float().cpu().numpy()
            ref = c_oracle.skinny_gemm(a_q, w_q, scale, d32)
            floor = oracle.accumulation_floor(a_q, w_q, scale)
            res = oracle.compare(out_full.float().cpu().numpy(), ref, case.k, scale, oracle.BF16, floor)
            ok = (res["hard_violations"] == 0 and res["nan_out"] == 0 and
                  res["violations"] <= oracle.strict_exception_cap(case.k, res["count"]))
            report["strict_bound_exceptions"] += res["violations"]
            if not ok:
                print(f"multi-GPU parity: {label} failed: {res}", file=sys.stderr, flush=True)
        report["cases"] += 1
        return _all_ranks_agree(torch, dist, ok, dev)

    # ---- configuration 3: K split, all-reduce fused into the epilogue
    group = RowParallelSkinnyGemm(max_m=16, max_n=8192)
    identical = True
    for case in wl.cases(3):
        inp = wl.make_inputs(case, device=str(dev))
        lo, hi = wl.k_split_cols(case.k, world, rank)
        a_sh = inp["a"][:, lo:hi].contiguous()
        w_sh = inp["w"][:, lo:hi]                       # column slice: keeps the full row pitch
        outs = []
        for mode in ("one_shot", "two_shot", "auto", "one_shot"):
            group.set_mode(mode)
            out = torch.zeros((case.m, case.n), dtype=torch.bfloat16, device=dev)
            group(a_sh, w_sh, inp["scale"], out)
            outs.append(out)
        torch.cuda.synchronize()
        group.set_mode("auto")
        code, word = capi.device_status(clear=True)
        same = code == 0 and all(torch.equal(o, outs[0]) for o in outs)
        gathered = [torch.empty_like(outs[0]) for _ in range(world)]
        dist.all_gather(gathered, outs[0])
        same = same and all(torch.equal(g, outs[0]) for g in gathered)
        identical = _all_ranks_agree(torch, dist, same, dev) and identical
        if not oracle_check(outs[0], inp, case, f"config 3 {case.name} world {world}"):
            raise RuntimeError(f"fused GEMM + all-reduce disagrees with the oracle on {case.name}")
        del inp, a_sh, w_sh
    if not identical:
        raise RuntimeError("fused GEMM + all-reduce: ranks or exchange schemes disagree bit-wise (or a wait ran out)")
    report["config3"] = "ok"
    report["ranks_bit_identical"] = True

    # ---- configuration 2: N split, no collective; slices gathered only for the check
    for index in (4, 1, 11):   # 70b qkv m=4, o_proj m=1, down m=16
        case = wl.cases(2)[index]
        inp = wl.make_inputs(case, device=str(dev))
        lo, hi = wl.n_split_rows(case.n, world, rank)
        piece = torch.zeros((case.m, hi - lo), dtype=torch.bfloat16, device=dev)
        capi.check(capi.skinny_gemm(inp["a"], inp["w"][lo:hi], piece, inp["scale"]))
        torch.cuda.synchronize()
        pieces = [torch.empty_like(piece) for _ in range(world)]
        dist.all_gather(pieces, piece)
        if not oracle_check(torch.cat(pieces, dim=1), inp, case, f"config 2 {case.name} world {world}"):
            raise RuntimeError(f"N-split shards disagree with the oracle on {case.name}")
        del inp
    report["config2"] = "ok"

    # ---- the tensor-parallel MLP block against the block on one GPU
    report["tp_mlp"] = "ok" if _tp_mlp_matches(torch, dist, capi, group, dev, rank, world) else "FAILED"
    torch.cuda.synchronize()
    dist.barrier()
    group.close()
    if report["tp_mlp"] != "ok":
        raise RuntimeError("tensor-parallel MLP block disagrees with the single-GPU block")
    torch.cuda.empty_cache()
    return report


def _tp_mlp_matches(torch, dist, capi, group, dev, rank, world) -> bool:
    from hf_rocm_kernels.combined_ops import llama_mlp_combined_ops
    from hf_rocm_kernels.utils.fp8 import fp8_quantize_e4m3fn

    tokens, hidden, inter = 16, 4096, 1024 * world
    gen = torch.Generator(device=dev).manual_seed(99)
    attn = torch.randn(tokens, hidden, generator=gen, device=dev).bfloat16()
    residual = torch.randn(tokens, hidden, generator=gen, device=dev).bfloat16()
    rms_w = (1 + 0.1 * torch.randn(hidden, generator=gen, device=dev)).bfloat16()
    q_gu, s_gu = fp8_quantize_e4m3fn(torch.randn(2 * inter, hidden, generator=gen, device=dev) * 0.02)
    q_dn, s_dn = fp8_quantize_e4m3fn(torch.randn(hidden, inter, generator=gen, device=dev) * 0.02)
    s_in = torch.tensor([4.0 / 448], device=dev)
    s_act = torch.tensor([16.0 / 448], device=dev)
    whole, whole_res = llama_mlp_combined_ops(attn, residual.clone(), rms_w, 1e-5, q_gu.t(), s_in, s_in * s_gu,
                                              q_dn.t(), s_act, s_act * s_dn)
    shard = inter // world
    lo, hi = rank * shard, (rank + 1) * shard
    gu_shard = torch.cat([q_gu.view(torch.uint8)[lo:hi], q_gu.view(torch.uint8)[inter + lo:inter + hi]])
    gu_shard = gu_shard.view(torch.float8_e4m3fn)
    dn_shard = q_dn[:, lo:hi]
    out, res = llama_mlp_combined_ops(attn, residual.clone(), rms_w, 1e-5, gu_shard.t(), s_in, s_in * s_gu,
                                      dn_shard.t(), s_act, s_act * s_dn, down_row_parallel=group)
    torch.cuda.synchronize()
    ok = capi.device_status(clear=True)[0] == 0 and torch.equal(res, whole_res)
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    ok = ok and all(torch.equal(g, out) for g in gathered)
    # The partial sums meet in another order than one GPU's K loop: one bf16 step at the value plus
    # one at the block's typical magnitude for outputs that cancel to almost nothing.
    diff = (out.float() - whole.float()).abs()
    bound = whole.float().abs() * 2.0 ** -7 + whole.float().abs().mean() * 2.0 ** -7
    ok = ok and bool((diff <= bound).all())
    return _all_ranks_agree(torch, dist, ok, dev)


def multi_gpu_extras(torch, dist, capi, wl, dev, rank, world):
    """Strong-scaling figures of the two sharding modes, all ranks in step, after their parity check."""
    from hf_rocm_kernels.combined_ops import RowParallelSkinnyGemm, skinny_gemm_then_allreduce

    out = {"world": world, "parity": multi_gpu_parity(torch, dist, capi, wl, dev, rank, world),
           "config2_n_split": [], "config3_k_split_fused_allreduce": []}
    scale = torch.full((1,), 1e-4, device=dev)

    def rand_fp8(rows, cols):
        return torch.randint(0, 120, (rows, cols), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)

    # configuration 2: each rank holds N/world rows of the 70B projections; no collective
    # Beside each shard time stands the time of the WHOLE matrix on one GPU, measured in the same
    # run on the same GPUs (max over ranks), so that efficiency = t_whole / (world * t_shard) can be
    # read from this one line.
    efficiencies = []
    for name, (n, k) in wl.LLAMA3_70B.items():
        rows = n // world
        copies = max(8, -(-2 * L2_BYTES // (rows * k)))
        ws = [rand_fp8(rows, k) for _ in range(copies)]
        whole_copies = max(8, -(-2 * L2_BYTES // (n * k)))
        whole = [rand_fp8(n, k) for _ in range(whole_copies)]
        for m in (1, 4, 16):
            a = rand_fp8(m, k)
            d = torch.zeros((m, rows), dtype=torch.bfloat16, device=dev)
            d_whole = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
            us = _graph_time_us(torch, dist, dev, [lambda w=w: capi.check(capi.skinny_gemm(a, w, d, scale)) for w in ws])
            us_whole = _graph_time_us(torch, dist, dev,
                                      [lambda w=w: capi.check(capi.skinny_gemm(a, w, d_whole, scale)) for w in whole],
                                      reps=10, warm=3)
            eff = us_whole / (world * us)
            efficiencies.append(eff)
            out["config2_n_split"].append({"case": f"70b_{name}_m{m}", "rows_per_gpu": rows, "us_per_call": round(us, 2),
                                           "us_whole_matrix_one_gpu": round(us_whole, 2), "efficiency": round(eff, 3),
                                           "aggregate_weight_tbps": round(n * k / us / 1e6, 3)})
        del ws, whole
        torch.cuda.empty_cache()
    out["config2_efficiency_min"] = round(min(efficiencies), 3)
    out["config2_efficiency_mean"] = round(sum(efficiencies) / len(efficiencies), 3)
    # configuration 3: K split of the 70B down projection, all-reduce fused into the epilogue
    n, k = 8192, 28672
    k_shard = k // world
    group = RowParallelSkinnyGemm(max_m=16, max_n=n)
    copies = max(8, -(-2 * L2_BYTES // (n * k_shard)))
    ws = [rand_fp8(n, k_shard) for _ in range(copies)]
    for m in (1, 2, 8, 16):
        a = rand_fp8(m, k_shard)
        d = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
        partial = torch.empty((m, n), dtype=torch.float32, device=dev)
        fused = _graph_time_us(torch, dist, dev, [lambda w=w: group(a, w, scale, d) for w in ws])
        unfused = _graph_time_us(torch, dist, dev,
                                 [lambda w=w: skinny_gemm_then_allreduce(a, w, scale, d, partial) for w in ws])
        local = _graph_time_us(torch, dist, dev, [lambda w=w: capi.check(capi.skinny_gemm(a, w, d, scale)) for w in ws])
        out["config3_k_split_fused_allreduce"].append({
            "m": m, "k_per_gpu": k_shard, "us_fused": round(fused, 2), "us_gemm_plus_nccl_allreduce": round(unfused, 2),
            "us_local_gemm_only": round(local, 2), "nvlink_bytes_out_per_gpu": (world - 1) * 4 * m * n})
    torch.cuda.synchronize()
    dist.barrier()
    # a timed exchange that ran out of time would leave D untouched and look fast: the status word tells
    code, word = capi.device_status(clear=True)
    if not _all_ranks_agree(torch, dist, code == 0, dev):
        raise RuntimeError(f"a bounded wait ran out during the multi-GPU timing (status word {word:#x} on rank {rank})")
    out["status_after_timing"] = "ok"
    group.close()
    return out


def load_workloads_standalone():
    """workloads.py loaded by file path: it imports torch only, so the CPU arm never loads the
    package (whose __init__ loads the CUDA libraries)."""
    import importlib.util

    path = os.path.join(ROOT, "hf-rocm-kernels_b200", "hf_rocm_kernels", "benchmarks", "skinny_gemm", "workloads.py")
    spec = importlib.util.spec_from_file_location("hfrk_workloads_standalone", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = module
    spec.loader.exec_module(module)
    return module


CPU_SAMPLE = "one whole step: the 20 calls of the workload once (1.09 GB of weights) on the host cores"


def cpu_sample(torch, wl):
    """The CPU arm's step: all 20 calls of the workload, the same step the GPU arm times."""
    picked = wl.cases(1)
    return picked, [wl.make_inputs(c, device="cpu") for c in picked]


def cpu_baseline(torch, wl):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_baseline as port  # the oracle's timed leg; the only use of oracle/ in this file

    picked, inputs = cpu_sample(torch, wl)
    seconds = port.time_cases(inputs, repeats=2)
    seconds_wide = port.time_cases_predequantised(inputs, repeats=2)
    nbytes = sum(c.algorithmic_bytes() for c in picked)
    return {"value": round(nbytes / seconds / 1e12, 6), "unit": UNIT, "cores": port.host_threads(), "kind": "port",
            "sample": CPU_SAMPLE + ", dequantise + fp32 matmul, torch CPU, best of 2",
            "value_weights_predequantised": round(nbytes / seconds_wide / 1e12, 6)}


def run_reference(args):
    """The reference's semantics on the host cores (it has no CUDA path and no CPU code of its own
    for this op; oracle/cpu_baseline.py ports reference.py:18-25 + wrapped.py:115)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import torch

    wl = load_workloads_standalone()
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_baseline as port

    picked, inputs = cpu_sample(torch, wl)
    nbytes = sum(c.algorithmic_bytes() for c in picked)
    torch.set_num_threads(port.host_threads())
    for _ in range(max(args.warmup, 1)):
        port.time_cases(inputs, repeats=0)
    start = time.perf_counter()
    for _ in range(args.steps):
        for inp in inputs:
            port.skinny_gemm_cpu(inp["a"], inp["w"], inp["scale"], inp["d_in"])
    seconds = time.perf_counter() - start
    ms_per_step = seconds / args.steps * 1e3
    value = nbytes / (ms_per_step * 1e-3) / 1e12
    sample = "each step = " + CPU_SAMPLE
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 6), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": round(ms_per_step, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (f32 accumulate, bf16 out)",
        "data": "synthetic", "config": {"workload": WORKLOAD, "calls_per_step": len(picked), "sample": sample},
        "cpu_baseline": {"value": round(value, 6), "unit": UNIT, "cores": port.host_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 6), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--no-detail", action="store_true", help="skip the per-case table")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
