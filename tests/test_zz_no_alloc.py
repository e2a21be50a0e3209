"""The allocation-free Linear entry point against the regular plan / launch path.  GPU only.

Some hosts of this library may not allocate device memory at all once they are running: a
runtime that plans every byte of the device itself, or a serving loop that cannot afford the
device-wide synchronisation cudaMalloc implies.  rt_linear_q8_0_static_scratch serves them by
keeping its scratch (the dequantised weight) in an array built into the library.  This test
calls it through the C ABI twice in a row, with different weights the second time so that the
array's leftover contents would show, and compares each result with the regular entry point's.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import numpy as np
import pytest

import oracle
import ratchet_b200 as rb
from ratchet_b200 import DType, Device, GpuBuffer, Tensor, _lib
from util import make_lhs, round_to

pytestmark = pytest.mark.gpu


def _regular(gpu, w_t, x, bias, epilogue):
    y = w_t.gemm(Tensor.from_data(x, gpu, DType.F16), Tensor.from_data(bias, gpu, DType.F16) if bias is not None else None,
                 False, True, True, epilogue=epilogue).resolve()
    return y.to(Device.CPU).to_numpy()


def _static(gpu, w_t, x, bias, epilogue):
    lib = _lib.load()
    rows, k = x.shape
    n = w_t.shape[0]
    xd = Tensor.from_data(x, gpu, DType.F16)
    bd = Tensor.from_data(bias, gpu, DType.F16) if bias is not None else None
    out = GpuBuffer(gpu, rows * n * 2)
    _lib.check(lib.rt_linear_q8_0_static_scratch(gpu._h, w_t.ptr, xd.ptr, bd.ptr if bd is not None else None, out.ptr,
                                                 rows, n, k, epilogue, None))
    gpu.sync()
    return Tensor([rows, n], DType.F16, gpu, out).to(Device.CPU).to_numpy()


def test_static_scratch_linear_matches_the_regular_path_twice(gpu):
    # the second weight is smaller than the first: part of the first one's dequantised copy stays behind in the array
    cases = [((1536, 384), 1500, True, rb.EPILOGUE_GELU_TANH, 301), ((256, 768), 777, False, rb.EPILOGUE_NONE, 302)]
    for (n, k), rows, has_bias, epilogue, seed in cases:
        w_cpu, wv = make_lhs(DType.Q8_0H, (n, k), np.random.default_rng(seed), 0.02)
        w_t = w_cpu.to(gpu)
        x = round_to(DType.F16, np.random.default_rng(seed + 1).standard_normal((rows, k))).astype(np.float16)
        bias = (round_to(DType.F16, np.random.default_rng(seed + 2).standard_normal(n) * 0.02).astype(np.float16)
                if has_bias else None)
        want = _regular(gpu, w_t, x, bias, epilogue)
        got = _static(gpu, w_t, x, bias, epilogue)
        assert got.shape == want.shape
        assert oracle.rel_l2(got.astype(np.float32), want.astype(np.float32)) <= 1e-3
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))  # same kernels, same bits
        # and against the oracle, so that agreeing with each other is not the only evidence
        truth = oracle.matmul_truth(wv, x.astype(np.float32), None if bias is None else bias.astype(np.float32),
                                    1, 1, 1, n, rows, k, False, True, True, epilogue)
        assert oracle.rel_l2(got.astype(np.float32).reshape(-1), oracle.f64_to_f16(truth).astype(np.float32)) <= 1e-3


def test_static_scratch_calls_leave_free_device_memory_unchanged(gpu):
    """The property the entry point exists for: with operands and output in place, calls through it take no device
    memory (cudaMemGetInfo reads the same before and after)."""
    import torch
    lib = _lib.load()
    n, k, rows = 512, 1024, 300
    w_cpu, _ = make_lhs(DType.Q8_0H, (n, k), np.random.default_rng(311), 0.02)
    w_t = w_cpu.to(gpu)
    xd = Tensor.from_data(np.random.default_rng(312).standard_normal((rows, k)).astype(np.float16), gpu, DType.F16)
    out = GpuBuffer(gpu, rows * n * 2)
    call = lambda: _lib.check(lib.rt_linear_q8_0_static_scratch(gpu._h, w_t.ptr, xd.ptr, None, out.ptr, rows, n, k, 0, None))
    call()       # the first call on a device looks the array's address up
    gpu.sync()
    free_before, _ = torch.cuda.mem_get_info(gpu.ordinal)
    for _ in range(20):
        call()
    gpu.sync()
    free_after, _ = torch.cuda.mem_get_info(gpu.ordinal)
    assert free_after == free_before, (free_before, free_after)


def test_static_scratch_refuses_weights_beyond_its_array(gpu):
    lib = _lib.load()
    n, k = 4096, 2048  # 16 MiB of f16 weights > the 8 MiB array
    dummy = GpuBuffer(gpu, 1 << 20)
    st = lib.rt_linear_q8_0_static_scratch(gpu._h, dummy.ptr, dummy.ptr + 4096, None, dummy.ptr + 8192, 16, n, k, 0, None)
    assert st == _lib.RT_ERR_UNSUPPORTED
    assert b"built-in array holds" in lib.rt_last_error()
    # an inner extent beyond 32 bits is a shape error, not a wrapped size
    st = lib.rt_linear_q8_0_static_scratch(gpu._h, dummy.ptr, dummy.ptr + 4096, None, dummy.ptr + 8192, 16, 1, 1 << 33, 0, None)
    assert st == _lib.RT_ERR_SHAPE
    # operands that are not 16-byte aligned are refused before anything is launched
    st = lib.rt_linear_q8_0_static_scratch(gpu._h, dummy.ptr + 2, dummy.ptr + 4096, None, dummy.ptr + 8192, 16, 64, 64, 0, None)
    assert st == _lib.RT_ERR_ARG
    st = lib.rt_linear_q8_0_static_scratch(gpu._h, dummy.ptr, dummy.ptr + 4096 + 4, None, dummy.ptr + 8192, 16, 64, 64, 0, None)
    assert st == _lib.RT_ERR_ARG and b"16-byte aligned" in lib.rt_last_error()
