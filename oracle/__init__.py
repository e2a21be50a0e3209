"""CPU oracle for ratchet-core's Matmul path: TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline / reference legs import
this package, as the checker and the timed CPU baseline.  The product package never
imports it.

`ratchet_oracle.c` restates the reference's arithmetic in C (citations in that file);
`shape_rules.py` restates the reference's shape / dtype rules in Python.  The functions
below are thin numpy wrappers over the C library.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libratchet_oracle.so")
_lib = None

QK8_0 = 32
QK_K = 256
Q4K_BLOCK_BYTES = 144


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside it (gcc, OpenMP when available)."""
    src = os.path.join(_HERE, "ratchet_oracle.c")
    if (force or not os.path.exists(_LIB_PATH)
            or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)):
        subprocess.run(["make", "-C", _HERE, "-B", "libratchet_oracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_q8_nbytes.restype = ctypes.c_int64
        _lib.orc_q8_nbytes.argtypes = [ctypes.c_int64, ctypes.c_int]
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    return ctypes.c_int64(int(v))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_cores() -> int:
    """Threads = the cores this process may run on, whatever OMP_NUM_THREADS says (torchrun exports 1)."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(ctypes.c_int(n))
    return num_threads()


# ----------------------------------------------------------------------------- conversions

def f64_to_f16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float64)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f64_to_f16(_p(x), _p(out), _i64(x.size))
    return out.view(np.float16)


def f64_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float64)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f64_to_bf16(_p(x), _p(out), _i64(x.size))
    return out


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    return f64_to_bf16_bits(np.asarray(x, dtype=np.float32).astype(np.float64))


# ----------------------------------------------------------------------------- Q8_0

def q8_segments(numel: int, scale_bytes: int):
    out = (ctypes.c_int64 * 4)()
    lib().orc_q8_segments(_i64(numel), ctypes.c_int(scale_bytes), out)
    return [(int(out[0]), int(out[1])), (int(out[2]), int(out[3]))]


def q8_nbytes(numel: int, scale_bytes: int) -> int:
    return int(lib().orc_q8_nbytes(_i64(numel), ctypes.c_int(scale_bytes)))


def q8_quantize_f(x: np.ndarray) -> np.ndarray:
    """sint8_quantize: f32 -> Q8_0F buffer (codes | pad | f32 scales | pad) as uint8."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.size % QK8_0 == 0
    out = np.empty(q8_nbytes(x.size, 4), dtype=np.uint8)
    lib().orc_q8_quantize_f(_p(x), _i64(x.size), _p(out))
    return out


def q8_f_to_h(buf_f: np.ndarray, numel: int) -> np.ndarray:
    out = np.empty(q8_nbytes(numel, 2), dtype=np.uint8)
    lib().orc_q8_f_to_h(_p(np.ascontiguousarray(buf_f)), _i64(numel), _p(out))
    return out


def q8_quantize_h(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return q8_f_to_h(q8_quantize_f(x), x.size)


def q8_dequantize_f(buf: np.ndarray, numel: int) -> np.ndarray:
    out = np.empty(numel, dtype=np.float32)
    lib().orc_q8_dequantize_f(_p(np.ascontiguousarray(buf)), _i64(numel), _p(out))
    return out


def q8_dequantize_h(buf: np.ndarray, numel: int) -> np.ndarray:
    out = np.empty(numel, dtype=np.uint16)
    lib().orc_q8_dequantize_h(_p(np.ascontiguousarray(buf)), _i64(numel), _p(out))
    return out.view(np.float16)


def q8_transcode_gguf(blocks: np.ndarray, scale_bytes: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    assert blocks.size % 34 == 0
    nb = blocks.size // 34
    out = np.empty(q8_nbytes(nb * QK8_0, scale_bytes), dtype=np.uint8)
    lib().orc_q8_transcode_gguf(_p(blocks), _i64(nb), ctypes.c_int(scale_bytes), _p(out))
    return out


# ----------------------------------------------------------------------------- Q4_K

def q4k_nbytes(numel: int) -> int:
    assert numel % QK_K == 0
    return numel // QK_K * Q4K_BLOCK_BYTES


def q4k_quantize(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(q4k_nbytes(x.size), dtype=np.uint8)
    lib().orc_q4k_quantize(_p(x), _i64(x.size), _p(out))
    return out


def q4k_dequantize(buf: np.ndarray, numel: int) -> np.ndarray:
    out = np.empty(numel, dtype=np.float32)
    lib().orc_q4k_dequantize(_p(np.ascontiguousarray(buf)), _i64(numel), _p(out))
    return out


# ----------------------------------------------------------------------------- GELU / matmul

def gelu_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    lib().orc_gelu_f32(_p(x), _p(y), _i64(x.size))
    return y


def silu_f32(v: np.ndarray) -> np.ndarray:
    """silu(v) = v * sigmoid(v) in f32, with the reference's two-branch sigmoid
    (crates/ratchet-core/src/ops/unary.rs:121-131,165-175): exp(v) / (1 + exp(v)) for v >= 0 (NaN once
    exp(v) overflows), 1 / (1 + exp(-v)) below."""
    v = np.asarray(v, dtype=np.float32)
    one = np.float32(1)
    with np.errstate(over="ignore", invalid="ignore"):
        pos = np.exp(v) / (one + np.exp(v))
        neg = one / (one + np.exp(-v))
        return (v * np.where(v >= 0, pos, neg)).astype(np.float32)


def silu_mul(full: np.ndarray, act_dt: str = "f16") -> np.ndarray:
    """The Phi-3 gate/up fold, crates/ratchet-models/src/phi3/mlp.rs:31-39: `full` [..., 2*ff] is the gate_up
    Linear's output (values of dtype `act_dt` held in f32), gate = [..., :ff], up = [..., ff:], result
    up * cast(silu(full(gate))) with every tensor of the chain in `act_dt`.  bf16 (no reference counterpart)
    rounds the product only."""
    full = np.asarray(full, dtype=np.float32)
    ff = full.shape[-1] // 2
    gate, up = full[..., :ff], full[..., ff:]
    sv = silu_f32(gate)
    with np.errstate(over="ignore", invalid="ignore"):
        if act_dt == "f16":
            return (up.astype(np.float16) * sv.astype(np.float16)).astype(np.float32)
        if act_dt == "bf16":
            return bf16_bits_to_f32(f64_to_bf16_bits((up * sv).astype(np.float64))).reshape(up.shape)
        return (up * sv).astype(np.float32)


def silu_mul_truth(full64: np.ndarray) -> np.ndarray:
    """The same fold in f64 without intermediate roundings."""
    full64 = np.asarray(full64, dtype=np.float64)
    ff = full64.shape[-1] // 2
    gate, up = full64[..., :ff], full64[..., ff:]
    with np.errstate(over="ignore"):
        return up * gate / (1.0 + np.exp(-gate))


def _mm_args(A, B, bias, stacks, a_stack, b_stack, M, N, K, ta, tb, to, epilogue):
    return [_i64(stacks), _i64(a_stack), _i64(b_stack), _i64(M), _i64(N), _i64(K),
            ctypes.c_int(int(ta)), ctypes.c_int(int(tb)), ctypes.c_int(int(to)),
            ctypes.c_int(int(epilogue))]


def matmul_truth(A, B, bias, stacks, a_stack, b_stack, M, N, K, trans_a, trans_b, trans_out,
                 epilogue=0) -> np.ndarray:
    """fp64-accumulated result as a flat f64 array in the output's memory order."""
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    assert A.size == a_stack * M * K and B.size == b_stack * K * N
    bp = None
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        bp = _p(bias)
    out = np.empty(stacks * M * N, dtype=np.float64)
    lib().orc_matmul_truth(_p(A), _p(B), bp, _p(out),
                           *_mm_args(A, B, bias, stacks, a_stack, b_stack, M, N, K,
                                     trans_a, trans_b, trans_out, epilogue))
    return out


def matmul_faithful(A, B, bias, stacks, a_stack, b_stack, M, N, K, trans_a, trans_b, trans_out,
                    epilogue=0, act_dt="f32") -> np.ndarray:
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    assert A.size == a_stack * M * K and B.size == b_stack * K * N
    bp = None
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        bp = _p(bias)
    out = np.empty(stacks * M * N, dtype=np.float32)
    lib().orc_matmul_faithful(_p(A), _p(B), bp, _p(out),
                              *_mm_args(A, B, bias, stacks, a_stack, b_stack, M, N, K,
                                        trans_a, trans_b, trans_out, epilogue),
                              ctypes.c_int(1 if act_dt == "f16" else 0))
    return out


def gemv_faithful(W, x, bias, N, K, act_dt="f32") -> np.ndarray:
    W = np.ascontiguousarray(W, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    bp = None
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        bp = _p(bias)
    out = np.empty(N, dtype=np.float32)
    lib().orc_gemv_faithful(_p(W), _p(x), bp, _p(out), _i64(N), _i64(K),
                            ctypes.c_int(1 if act_dt == "f16" else 0))
    return out


def q8h_gemv_packed(wbuf: np.ndarray, N: int, K: int, x16: np.ndarray, bias16=None) -> np.ndarray:
    """Timed CPU baseline: shader-faithful Q8_0H GEMV straight from the packed buffer."""
    x16 = np.ascontiguousarray(x16, dtype=np.float16)
    y = np.empty(N, dtype=np.float16)
    bp = None
    if bias16 is not None:
        bias16 = np.ascontiguousarray(bias16, dtype=np.float16)
        bp = _p(bias16)
    lib().orc_q8h_gemv_packed(_p(wbuf), _i64(N), _i64(K), _p(x16), bp, _p(y))
    return y


def rel_l2(y, ref) -> float:
    y = np.asarray(y, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    den = float(np.linalg.norm(ref))
    num = float(np.linalg.norm(y - ref))
    return num / den if den > 0 else num
