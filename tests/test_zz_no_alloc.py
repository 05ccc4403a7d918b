"""The allocation-free split-K entry point against the regular launch entry.

``kcg_gemm_bf16_splitk_noalloc`` exists for callers that may not allocate device memory when they reach
the GEMM (a fixed memory pool, a serving loop with a frozen budget, a process whose free HBM is owned by
another allocator): its split-K workspace is a fixed array inside the library's device image instead of
memory the library allocates on first use. Both entries run the same kernel code at the same config, and the
split-K reduction sums partials in split order, so the outputs must agree exactly; the test also holds them
to the bf16 tolerance of the other GPU tests (2e-2 on max relative error). Two calls in a row check that the
shared array, which keeps the previous call's contents, is cleared where it must be.

Collected last on purpose: a failure here cannot hide the result of any other test in a run that stops
at the first failure. It passes alone in a fresh process as well as after the rest of the suite.
"""
import ctypes

import pytest
import torch

from codegendemo_b200 import _lib
from codegendemo_b200.kcg.matmul_op import build_kernel, default_config
from codegendemo_b200.kcg.Utils import DeviceInfo, EnumKernelDType as E
from oracle import oracle

pytestmark = pytest.mark.gpu


def _noalloc(a, b, c, M, N, K, synchronize=1):
    lib = _lib.get_lib()
    stream = DeviceInfo.get_cuda_stream(0)
    return lib.kcg_gemm_bf16_splitk_noalloc(0, ctypes.c_uint64(stream), ctypes.c_uint64(a.data_ptr()),
                                            ctypes.c_uint64(b.data_ptr()), ctypes.c_uint64(c.data_ptr()), M, N, K,
                                            synchronize)


def _warm_up_noalloc_entry():
    """The first call on a device loads the library's device image (the built-in workspace included): that
    one-time cost is made here, so that the calls measured below are steady-state calls."""
    x = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda:0")
    y = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda:0")
    z = torch.empty(128, 256, dtype=torch.bfloat16, device="cuda:0")
    assert _noalloc(x, y, z, 128, 256, 256) == 0, _lib.get_lib().kcg_last_error()


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    torch.cuda.set_device(0)
    lib = _lib.get_lib()
    _warm_up_noalloc_entry()
    shapes = [(256, 512, 2048), (128, 4096, 1024)]  # second call: other shape, more tiles, same shared array
    for call, (M, N, K) in enumerate(shapes):
        A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=10 + call)
        a, b = A.cuda(), B.cuda()
        # existing entry: the JIT-compiled kernel of the same config, workspace allocated by the library
        kpm = default_config(M, N, K, E.bfloat16, BLOCK_SIZE_M=128, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, NUM_STAGES=4,
                             LOCAL_SPLIT_U=4, BLOCK_MAPPING=8)
        _, kern = build_kernel(kpm, 0)
        c_ref = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        kern.run(a, b, c_ref)
        kern.checkStatus()
        # new entry: no allocation between here and the result
        c_new = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        torch.cuda.synchronize()
        # free bytes as the driver counts them: unlike torch's own counters this also sees an allocation made
        # inside the library
        free_before, _ = torch.cuda.mem_get_info(0)
        rc = _noalloc(a, b, c_new, M, N, K)
        assert rc == 0, lib.kcg_last_error()
        free_after, _ = torch.cuda.mem_get_info(0)
        assert free_after == free_before, f"device memory changed by {free_before - free_after} bytes across the call"
        err = oracle.rel_errors(c_new, c_ref.float())
        assert err["max_rel"] <= oracle.TOL_16BIT and not err["nan"], (call, err)
        assert torch.equal(c_new, c_ref), f"call {call}: outputs differ from the regular entry"
        # and both agree with the CPU oracle
        assert oracle.rel_errors(c_new, oracle.host_matmul(A, B))["max_rel"] <= oracle.TOL_16BIT


def test_noalloc_entry_leaves_the_callers_current_device_alone():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs a second GPU to be the caller's current device")
    torch.cuda.set_device(1)
    try:
        x = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda:0")
        y = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda:0")
        z = torch.empty(128, 256, dtype=torch.bfloat16, device="cuda:0")
        assert _noalloc(x, y, z, 128, 256, 256) == 0
        assert torch.cuda.current_device() == 1
    finally:
        torch.cuda.set_device(0)


def test_noalloc_entry_rejects_what_does_not_fit():
    lib = _lib.get_lib()
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda:0")
    p = x.data_ptr()
    big = lib.kcg_gemm_bf16_splitk_noalloc(0, 0, p, p, p, 4096, 4096, 4096, 0)  # 4*M*N floats > built-in workspace
    assert big == _lib.E_TOO_LARGE and b"too large for the built-in workspace" in lib.kcg_last_error()
    odd = lib.kcg_gemm_bf16_splitk_noalloc(0, 0, p, p, p, 100, 256, 256, 0)
    assert odd == _lib.E_BAD_CONFIG
    short_k = lib.kcg_gemm_bf16_splitk_noalloc(0, 0, p, p, p, 128, 256, 128, 0)
    assert short_k == _lib.E_BAD_CONFIG
