"""Generates qmatmul.npz: quantised and f16 matmuls whose expected values never pass through this
repository's code (run once in the build container, output committed).

    GGUF blocks (random, written here byte by byte)
      -> gguf.quants.dequantize (the gguf Python package's decoder; Q8_0 values rounded to f16 as the
         reference's f16 path holds them)
      -> torch.matmul in float64 (+ bias, + tanh GELU), rounded once to f16
The reference's own tests take torch.matmul as ground truth the same way
(crates/ratchet-core/src/ops/matmul.rs:663-718); its loader hands the kernels GGUF Q8_0 blocks
transcoded to split segments (crates/ratchet-loader/src/gguf/dtype.rs:44-110).  Q4_K has no
arithmetic in the reference; the published GGUF format, as gguf-py decodes it, is the pin.
Dense f16 cases use torch's own half matmul on the CPU.

Usage:  python tests/golden/make_qmatmul_golden.py
"""
import os

import numpy as np
import torch
import torch.nn.functional as F
from gguf import GGMLQuantizationType, quants

HERE = os.path.dirname(os.path.abspath(__file__))


def q8_blocks(rng, n_blocks):
    d = rng.uniform(2e-4, 6e-4, size=n_blocks).astype(np.float16)   # weights of about N(0, 0.02)
    qs = np.clip(np.round(rng.standard_normal((n_blocks, 32)) * 45), -127, 127).astype(np.int8)
    blocks = np.zeros((n_blocks, 34), dtype=np.uint8)
    blocks[:, :2] = d.view(np.uint8).reshape(n_blocks, 2)
    blocks[:, 2:] = qs.view(np.uint8)
    return blocks


def q4k_blocks(rng, n_blocks):
    blocks = rng.integers(0, 256, size=(n_blocks, 144), dtype=np.uint8)
    d = rng.uniform(1e-4, 4e-4, size=n_blocks).astype(np.float16)
    dmin = rng.uniform(1e-4, 4e-4, size=n_blocks).astype(np.float16)
    blocks[:, 0:2] = d.view(np.uint8).reshape(n_blocks, 2)
    blocks[:, 2:4] = dmin.view(np.uint8).reshape(n_blocks, 2)
    return blocks


def expected(w, x, bias, gelu):
    """out[b, m, n] = sum_k x[b, m, k] w[n, k] (+ bias[n]) in float64, rounded once to f16."""
    y = torch.matmul(torch.from_numpy(x.astype(np.float64)), torch.from_numpy(w.astype(np.float64)).T)
    if bias is not None:
        y = y + torch.from_numpy(bias.astype(np.float64))
    if gelu:
        y = F.gelu(y, approximate="tanh")
    return y.numpy().astype(np.float16)


def main():
    torch.set_num_threads(1)
    rng = np.random.default_rng(20240611)
    out = {}
    cases = []
    # (name, format, N, K, x rows, bias, gelu)
    spec = [("q8_gemv", "q8", 256, 512, 1, False, False), ("q8_gemv_phi2_k", "q8", 96, 2560, 1, True, False),
            ("q8_skinny", "q8", 128, 256, 5, True, True), ("q8_gemm", "q8", 192, 384, 40, True, True),
            ("q4k_gemv", "q4k", 64, 1024, 1, False, False), ("q4k_skinny", "q4k", 48, 512, 5, True, False),
            ("q4k_gemm", "q4k", 128, 512, 48, True, True)]
    for name, fmt, N, K, M, has_bias, gelu in spec:
        if fmt == "q8":
            blocks = q8_blocks(rng, N * K // 32)
            w = quants.dequantize(blocks, GGMLQuantizationType.Q8_0).astype(np.float32).reshape(N, K)
            # with f16 scales the reference's kernels hold the dequantised weight as f16: f16(q) * d rounded to f16
            # (crates/ratchet-core/src/ops/gemm.rs:395-409), i.e. the exact product q * d rounded once
            w = w.astype(np.float16).astype(np.float32)
        else:
            blocks = q4k_blocks(rng, N * K // 256)
            w = quants.dequantize(blocks, GGMLQuantizationType.Q4_K).astype(np.float32).reshape(N, K)
        x = rng.standard_normal((1, M, K)).astype(np.float16)
        bias = (rng.standard_normal(N) * 0.02).astype(np.float16) if has_bias else None
        out[name + "_blocks"] = blocks
        out[name + "_x"] = x
        if bias is not None:
            out[name + "_bias"] = bias
        out[name + "_y"] = expected(w, x.astype(np.float32), None if bias is None else bias.astype(np.float32), gelu)
        out[name + "_meta"] = np.array([N, K, M, int(has_bias), int(gelu)], dtype=np.int32)
        cases.append(name)
    # dense f16: torch's half matmul (f32 accumulation, one rounding)
    for name, (B, M, K, N) in {"f16_a": (1, 33, 96, 40), "f16_b": (2, 64, 80, 72)}.items():
        a = (rng.standard_normal((B, M, K)) * 0.5).astype(np.float16)
        b = (rng.standard_normal((B, K, N)) * 0.5).astype(np.float16)
        out[name + "_a"], out[name + "_b"] = a, b
        out[name + "_c"] = torch.matmul(torch.from_numpy(a), torch.from_numpy(b)).numpy()
    out["quant_cases"] = np.array(cases)
    np.savez_compressed(os.path.join(HERE, "qmatmul.npz"), **out)
    print("wrote qmatmul.npz:", cases, os.path.getsize(os.path.join(HERE, "qmatmul.npz")), "bytes")


if __name__ == "__main__":
    main()
