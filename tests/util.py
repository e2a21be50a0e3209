"""Shared helpers of the parity tests: seeded problems, the oracle's answer, the library's answer."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

import oracle
import ratchet_b200 as rb
from ratchet_b200 import DType, Device, Quantization, Quantizer, Tensor

TRANS_KINDS = {  # crates/ratchet-core/src/ops/matmul.rs:720-753 of the reference
    "None": (False, False, False), "LHS": (True, False, False), "LHSAndOut": (True, False, True),
    "RHS": (False, True, False), "RHSAndOut": (False, True, True), "Out": (False, False, True),
}

# rel-L2 bars of the path (f16 / bf16 activations, f32 activations)
TOL = {DType.F16: 1e-3, DType.BF16: 1e-3, DType.F32: 1e-5}


@dataclass
class Problem:
    lhs_dt: DType
    act_dt: DType
    lhs_shape: tuple
    rhs_shape: tuple
    trans: tuple = (False, False, False)
    bias: bool = False
    epilogue: int = 0
    seed: int = 0
    w_std: float = 1.0
    bias_dt: Optional[DType] = None


def round_to(dt: DType, x: np.ndarray) -> np.ndarray:
    """f32 values rounded to `dt`, returned as f32."""
    x = np.asarray(x, dtype=np.float32)
    if dt == DType.F16:
        return x.astype(np.float16).astype(np.float32)
    if dt == DType.BF16:
        return rb.bf16_bits_to_f32(rb.f32_to_bf16_bits(x)).reshape(x.shape)
    return x


def make_lhs(dt: DType, shape, rng, std):
    """Returns (CPU Tensor in the library's layout, f32 array of the exact operand values)."""
    w = (rng.standard_normal(shape) * std).astype(np.float32)
    numel = w.size
    if dt in (DType.Q8_0F, DType.Q8_0H):
        buf = oracle.q8_quantize_f(w)
        if dt == DType.Q8_0H:
            buf = oracle.q8_f_to_h(buf, numel)
            vals = oracle.q8_dequantize_h(buf, numel).astype(np.float32)
        else:
            vals = oracle.q8_dequantize_f(buf, numel)
        return Tensor.from_quantized(buf, dt, shape), vals.reshape(shape)
    if dt == DType.Q4_K:
        buf = oracle.q4k_quantize(w)
        return Tensor.from_quantized(buf, dt, shape), oracle.q4k_dequantize(buf, numel).reshape(shape)
    vals = round_to(dt, w)
    return Tensor.from_data(vals, dt=dt), vals


def dims(p: Problem):
    tl, tr, to = p.trans
    a, b = list(p.lhs_shape), list(p.rhs_shape)
    if len(a) < 2:
        a.insert(int(tl), 1)      # implicit m (matmul.rs:296-298)
    if len(b) < 2:
        b.insert(int(not tr), 1)  # implicit n (matmul.rs:299-301)
    m, ka = a[-2], a[-1]
    kb, n = b[-2], b[-1]
    if tl:
        m, ka = ka, m
    if tr:
        kb, n = n, kb
    assert ka == kb
    return m, n, ka


def run_problem(p: Problem, gpu):
    """Runs one Matmul node through the library; returns (result f32, truth f64 rounded to dtype as f32,
    truth f64 unrounded, faithful f32 or None, kernel name)."""
    rng = np.random.default_rng(p.seed)
    tl, tr, to = p.trans
    lhs_t, lhs_vals = make_lhs(p.lhs_dt, p.lhs_shape, np.random.default_rng(p.seed + 1000), p.w_std)
    x = round_to(p.act_dt, rng.standard_normal(p.rhs_shape).astype(np.float32))
    rhs_t = Tensor.from_data(x, dt=p.act_dt)
    M, N, K = dims(p)
    bias_t = bias_vals = None
    if p.bias:
        bdt = p.bias_dt or p.act_dt
        blen = M if to else N
        bias_vals = round_to(bdt, (np.random.default_rng(p.seed + 2000).standard_normal(blen) * max(p.w_std, 0.02)).astype(np.float32))
        bias_t = Tensor.from_data(bias_vals, dt=bdt)

    out = lhs_t.to(gpu).gemm(rhs_t.to(gpu), bias_t.to(gpu) if bias_t is not None else None, tl, tr, to,
                             epilogue=p.epilogue)
    kernel = rb._lib.load().rt_plan_kernel(gpu.plan_for(out.op.desc)).decode()
    got = out.resolve().to(Device.CPU).to_f32().reshape(-1)

    a_stack = int(np.prod(p.lhs_shape[:-2])) if len(p.lhs_shape) > 2 else 1
    b_stack = int(np.prod(p.rhs_shape[:-2])) if len(p.rhs_shape) > 2 else 1
    stacks = max(a_stack, b_stack)
    truth = oracle.matmul_truth(lhs_vals, x, bias_vals, stacks, a_stack, b_stack, M, N, K, tl, tr, to, p.epilogue)
    if p.act_dt == DType.F16:
        truth_r = oracle.f64_to_f16(truth).astype(np.float32)
    elif p.act_dt == DType.BF16:
        truth_r = oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(truth))
    else:
        truth_r = truth.astype(np.float32)
    faithful = None
    if p.act_dt in (DType.F16, DType.F32) and p.lhs_dt != DType.Q4_K:
        faithful = oracle.matmul_faithful(lhs_vals, x, bias_vals, stacks, a_stack, b_stack, M, N, K, tl, tr, to,
                                          p.epilogue, "f16" if p.act_dt == DType.F16 else "f32")
    return got, truth_r, truth, faithful, kernel


def check_problem(p: Problem, gpu, tol: Optional[float] = None):
    got, truth_r, truth, faithful, kernel = run_problem(p, gpu)
    tol = tol if tol is not None else TOL[p.act_dt]
    assert got.shape == truth_r.shape, (got.shape, truth_r.shape)
    assert np.all(np.isfinite(got)), f"non-finite output from {kernel}"
    err = oracle.rel_l2(got, truth_r)
    assert err <= tol, f"{kernel}: rel-L2 {err:.3e} > {tol:.0e} for {p}"
    return err, kernel
