"""Generates the fixtures in this folder (run once in the build container, outputs committed).

The reference (FL33TW00D/ratchet) holds no golden vectors for Matmul: its tests compare
against PyTorch at run time (crates/ratchet-core/src/ops/matmul.rs:663-718,
crates/ratchet-core/src/ops/unary.rs:372-400).  These fixtures freeze that same ground
truth, plus the gguf Python package's decoders for the two block formats, so that the
oracle is pinned without torch or gguf at test time:

  q8_gguf.npz     random GGUF Q8_0 blocks  -> gguf.quants.dequantize (f32)
  q4k_gguf.npz    random GGUF Q4_K blocks  -> gguf.quants.dequantize (f32)
  sgemm.npz       f32 matmul, the reference tests' property space (6 transpose kinds,
                  bias on/off, B in 1..3) and its fixed regression shapes at reduced size
                  -> torch.matmul (+ torch.add) in f32
  gelu.npz        torch.nn.functional.gelu(approximate="tanh") in f32

Usage:  python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch
import torch.nn.functional as F
from gguf import GGMLQuantizationType, quants

HERE = os.path.dirname(os.path.abspath(__file__))
TRANS_KINDS = {  # matmul.rs:720-753
    "None": (False, False, False), "LHS": (True, False, False), "LHSAndOut": (True, False, True),
    "RHS": (False, True, False), "RHSAndOut": (False, True, True), "Out": (False, False, True),
}


def q8_blocks(rng, n_blocks):
    d = (rng.uniform(1e-4, 5e-2, size=n_blocks)).astype(np.float16)
    qs = rng.integers(-127, 128, size=(n_blocks, 32), dtype=np.int8)
    blocks = np.zeros((n_blocks, 34), dtype=np.uint8)
    blocks[:, :2] = d.view(np.uint8).reshape(n_blocks, 2)
    blocks[:, 2:] = qs.view(np.uint8)
    return blocks


def q4k_blocks(rng, n_blocks):
    blocks = rng.integers(0, 256, size=(n_blocks, 144), dtype=np.uint8)
    d = rng.uniform(1e-4, 2e-3, size=n_blocks).astype(np.float16)
    dmin = rng.uniform(1e-4, 2e-3, size=n_blocks).astype(np.float16)
    blocks[:, 0:2] = d.view(np.uint8).reshape(n_blocks, 2)
    blocks[:, 2:4] = dmin.view(np.uint8).reshape(n_blocks, 2)
    return blocks


def torch_matmul(a, b, bias, tl, tr, to):
    ta, tb = torch.from_numpy(a), torch.from_numpy(b)
    if tl:
        ta = ta.transpose(-1, -2)
    if tr:
        tb = tb.transpose(-1, -2)
    c = torch.matmul(ta, tb)
    if bias is not None:
        c = torch.add(c, torch.from_numpy(bias))
    if to:
        c = c.transpose(-1, -2)
    return np.ascontiguousarray(c.numpy())


def main():
    torch.set_num_threads(1)
    rng = np.random.default_rng(20240607)

    b8 = q8_blocks(rng, 96)
    np.savez_compressed(os.path.join(HERE, "q8_gguf.npz"), blocks=b8,
                        dequant=quants.dequantize(b8, GGMLQuantizationType.Q8_0).astype(np.float32))

    b4 = q4k_blocks(rng, 24)
    np.savez_compressed(os.path.join(HERE, "q4k_gguf.npz"), blocks=b4,
                        dequant=quants.dequantize(b4, GGMLQuantizationType.Q4_K).astype(np.float32))

    cases = {}
    idx = 0
    for name, (tl, tr, to) in TRANS_KINDS.items():
        for (B, M, K, N) in [(1, 5, 7, 3), (2, 33, 40, 17), (3, 24, 32, 40), (1, 1, 70, 45), (2, 37, 1, 29)]:
            for has_bias in (False, True):
                if to and has_bias:  # matmul.rs:786-789: the reference tests drop bias with trans_out
                    continue
                a = rng.standard_normal((B, K, M) if tl else (B, M, K)).astype(np.float32)
                b = rng.standard_normal((B, N, K) if tr else (B, K, N)).astype(np.float32)
                bias = rng.standard_normal(N).astype(np.float32) if has_bias else None
                c = torch_matmul(a, b, bias, tl, tr, to)
                key = f"c{idx:03d}"
                cases[key + "_a"], cases[key + "_b"], cases[key + "_c"] = a, b, c
                if bias is not None:
                    cases[key + "_bias"] = bias
                cases[key + "_meta"] = np.array([int(tl), int(tr), int(to), int(has_bias)], dtype=np.int32)
                idx += 1
    # fixed regression shapes of the reference's tests at reduced size
    # debug_gemm (matmul.rs:854-890): [2,222,252]^T x [1,222,238] + bias, broadcast batch
    a = rng.standard_normal((2, 58, 62)).astype(np.float32)
    b = rng.standard_normal((1, 58, 46)).astype(np.float32)
    bias = rng.standard_normal(46).astype(np.float32)
    key = f"c{idx:03d}"
    cases[key + "_a"], cases[key + "_b"], cases[key + "_bias"] = a, b, bias
    cases[key + "_c"] = torch_matmul(a, b, bias, True, False, False)
    cases[key + "_meta"] = np.array([1, 0, 0, 1], dtype=np.int32)
    idx += 1
    # debug_gemv (matmul.rs:892-926): [1,51865,384] x [1,1,384]^T, trans_out; rows not a multiple of 4
    a = rng.standard_normal((1, 1037, 96)).astype(np.float32)
    b = rng.standard_normal((1, 1, 96)).astype(np.float32)
    key = f"c{idx:03d}"
    cases[key + "_a"], cases[key + "_b"] = a, b
    cases[key + "_c"] = torch_matmul(a, b, None, False, True, True)
    cases[key + "_meta"] = np.array([0, 1, 1, 0], dtype=np.int32)
    idx += 1
    # test_qgemm (matmul.rs:831-852): [6,1500,64] x [6,64,1500], all stacks equal
    a = rng.standard_normal((6, 50, 64)).astype(np.float32)
    b = rng.standard_normal((6, 64, 50)).astype(np.float32)
    key = f"c{idx:03d}"
    cases[key + "_a"], cases[key + "_b"] = a, b
    cases[key + "_c"] = torch_matmul(a, b, None, False, False, False)
    cases[key + "_meta"] = np.array([0, 0, 0, 0], dtype=np.int32)
    idx += 1
    cases["n_cases"] = np.array([idx], dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, "sgemm.npz"), **cases)

    x = np.concatenate([np.linspace(-12, 12, 481), rng.standard_normal(512) * 3]).astype(np.float32)
    y = F.gelu(torch.from_numpy(x), approximate="tanh").numpy()
    np.savez_compressed(os.path.join(HERE, "gelu.npz"), x=x, y=y)
    print("wrote fixtures:", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
