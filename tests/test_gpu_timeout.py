"""A wait inside a kernel that runs out must end the call with a status word, not hang the GPU.

The only wait that another party can starve is the row-parallel exchange: a rank polls its
exchange buffer for its peers' partial sums. Here rank 0 of a two-rank group runs alone; the
"peer" is a second buffer in the same process that nothing ever writes, so the poll runs out
after the (shortened) limit. No fault, no trap, no endless loop: the kernel returns by itself, the
host reads the status, and the same context runs the next GEMM correctly.
"""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["one_shot", "two_shot"])
def test_a_peer_that_never_delivers_ends_the_call_with_a_status(native_build, mode):
    from hf_rocm_kernels import _capi as capi

    lib = capi.lib
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    assert capi.device_status(clear=True)[0] == 0
    m, n, k = 4, 1024, 512
    lone, lender = ctypes.c_void_p(), ctypes.c_void_p()
    capi.check(lib.hfrk_rowpar_create(0, 2, 16, n, ctypes.byref(lone)))
    capi.check(lib.hfrk_rowpar_create(1, 2, 16, n, ctypes.byref(lender)))     # only lends its buffer
    try:
        blocks = (ctypes.c_void_p * 2)(None, lib.hfrk_rowpar_local_block(lender))
        capi.check(lib.hfrk_rowpar_connect_pointers(lone, blocks))
        capi.check(lib.hfrk_rowpar_set_wait_ms(lone, 100))
        capi.check(lib.hfrk_rowpar_set_mode(lone, {"one_shot": capi.ROWPAR_ONE_SHOT,
                                                   "two_shot": capi.ROWPAR_TWO_SHOT}[mode]))
        assert lib.hfrk_rowpar_set_wait_ms(lone, 0) == 6

        a = torch.randint(0, 120, (m, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        w = torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        scale = torch.tensor([1e-3], device=dev)
        d = torch.full((m, n), 3.0, dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        started = time.perf_counter()
        status = lib.hfrk_skinny_gemm_fp8_rowpar(lone, a.data_ptr(), w.data_ptr(), d.data_ptr(), scale.data_ptr(),
                                                 m, n, k, k, capi.E4M3FN, capi.E4M3FN, capi.BF16, 1,
                                                 torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        assert status == 0                      # the launch itself succeeded
        assert elapsed < 5.0, f"the bounded wait took {elapsed:.1f} s"
        code, word = capi.device_status(clear=True)
        assert code == 10, "the kernel must report HFRK_DEVICE_TIMEOUT"
        assert word >> 24 == 10 and (word >> 16) & 0xFF == 4, f"status word {word:#x}: expected role 4 (peer)"
        assert bool((d == 3.0).all()), "elements whose sums never arrived must not be written"
        assert capi.device_status(clear=True)[0] == 0
    finally:
        lib.hfrk_rowpar_destroy(lone)
        lib.hfrk_rowpar_destroy(lender)

    # the context is still good: a plain GEMM gives the right answer
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
    check = torch.zeros_like(out)
    capi.check(capi.skinny_gemm(a, w, out, scale))
    capi.check(capi.skinny_gemm_simt(a, w, check, scale))
    torch.cuda.synchronize()
    assert capi.device_status(clear=True)[0] == 0
    # both kernels round to bf16: one step apart at most (a step is 2**-7 of the value)
    assert bool(((out.float() - check.float()).abs() <= check.float().abs() * 2.0 ** -7 + 1e-3).all())
