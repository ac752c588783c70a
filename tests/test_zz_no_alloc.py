"""The no-allocation entry point against the ordinary one, through the C ABI.

``hfrk_skinny_gemm_fp8_noalloc`` exists for callers that may not allocate device memory when they
call the GEMM (a server whose pools own all of HBM, a plug-in barred from the allocator): its
scratch is a fixed array inside the library. This file is collected last on purpose, so that a run
that stops at the first failure has already been through every other test; it passes on its own in
a fresh process as well as after the rest of the suite.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi(native_build):
    from hf_rocm_kernels import _capi

    return _capi


def _inputs(case, dev):
    from hf_rocm_kernels.benchmarks.skinny_gemm import workloads as wl

    inp = wl.make_inputs(case, device="cpu")
    d0 = inp["d_in"] if inp["d_in"] is not None else torch.zeros((case.m, case.n), dtype=torch.bfloat16)
    return inp["a"].to(dev), inp["w"].to(dev), inp["scale"].to(dev), d0.to(dev), inp


@pytest.mark.parametrize("shape", [(16, 4096, 4096, True), (5, 1000, 1040, False), (1, 6144, 4096, True),
                                   (13, 4104, 5120, False)])
def test_noalloc_entry_matches_the_ordinary_one_twice_in_a_row(capi, oracle_mod, c_oracle, shape):
    from hf_rocm_kernels.benchmarks.skinny_gemm import workloads as wl

    m, n, k, bias = shape
    dev = torch.device("cuda:0")
    case = wl.Case(7, m * 7 + n, "noalloc", m, n, k, bias=bias)
    a, w, s, d0, inp = _inputs(case, dev)

    expected = d0.clone()
    capi.check(capi.skinny_gemm(a, w, expected, s))                    # the existing entry point
    torch.cuda.synchronize()

    # same tolerance as the parity tests: the stated bound (+ accumulation floor) against the oracle,
    # and against the existing entry point the two kernels may differ by that bound at most twice
    a_q, w_q = inp["a"].view(torch.uint8).numpy(), inp["w"].view(torch.uint8).numpy()
    scale = float(inp["scale"][0])
    d32 = None if inp["d_in"] is None else inp["d_in"].float().numpy()
    ref = c_oracle.skinny_gemm(a_q, w_q, scale, d32)
    floor = oracle_mod.accumulation_floor(a_q, w_q, scale)
    tol = oracle_mod.tolerance(ref, k, scale, oracle_mod.BF16) + floor

    results = []
    outs = [d0.clone() for _ in range(3)]                               # made before the memory is read
    torch.cuda.synchronize()
    for call in range(3):                                               # calls in a row share the array
        out = outs[call]
        free_before = torch.cuda.mem_get_info(dev)[0]
        capi.check(capi.skinny_gemm_noalloc(a, w, out, s))
        torch.cuda.synchronize()
        if call > 0:
            # past the first call on the device (which loads the module and looks up the array) a call
            # allocates nothing: the device's free memory does not move across it
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        assert capi.device_status(clear=True)[0] == 0
        res = oracle_mod.compare(out.float().cpu().numpy(), ref, k, scale, oracle_mod.BF16, floor)
        assert res["hard_violations"] == 0 and res["nan_out"] == 0, res
        diff = (out.float() - expected.float()).abs().cpu().numpy()
        assert (diff <= 2 * tol).all()
        results.append(out)
    assert torch.equal(results[0], results[1])


def test_noalloc_entry_rejects_sizes_beyond_its_fixed_array(capi):
    dev = torch.device("cuda:0")
    a = torch.zeros((17, 256), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    w = torch.zeros((128, 256), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    d = torch.zeros((17, 128), dtype=torch.bfloat16, device=dev)
    s = torch.ones(1, device=dev)
    assert capi.skinny_gemm_noalloc(a, w, d, s) == 12                   # HFRK_TOO_LARGE: more than 16 tokens
    assert b"16 tokens" in capi.lib.hfrk_last_error()
    # more than 4096 tiles of 128 rows (N > 524,288): the tile counters of the fixed array run out
    n_big = 4097 * 128
    a1 = torch.zeros((1, 16), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    w_big = torch.zeros((n_big, 16), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    d_big = torch.zeros((1, n_big), dtype=torch.bfloat16, device=dev)
    assert capi.skinny_gemm_noalloc(a1, w_big, d_big, s) == 12
    n_ok = 4096 * 128
    assert capi.skinny_gemm_noalloc(a1, w_big[:n_ok], d_big[:, :n_ok].contiguous(), s) == 0
    torch.cuda.synchronize()
