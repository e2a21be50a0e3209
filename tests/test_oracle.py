"""The oracle against the committed fixtures (torch.matmul, F.gelu, gguf-py decoders).  CPU only."""
import os

import numpy as np
import pytest

import oracle
from oracle import shape_rules

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_q8_decode_matches_gguf_bit_exact():
    g = np.load(os.path.join(GOLDEN, "q8_gguf.npz"))
    n = g["dequant"].size
    buf_f = oracle.q8_transcode_gguf(g["blocks"], 4)
    got = oracle.q8_dequantize_f(buf_f, n)
    assert np.array_equal(got.view(np.uint32), g["dequant"].reshape(-1).view(np.uint32))
    # f16 scales: f16(q)*d rounded to f16 == the f32 product rounded once
    buf_h = oracle.q8_transcode_gguf(g["blocks"], 2)
    got_h = oracle.q8_dequantize_h(buf_h, n)
    assert np.array_equal(got_h.view(np.uint16), g["dequant"].reshape(-1).astype(np.float16).view(np.uint16))


def test_q8_layout_follows_segments():
    # blocks.rs:61-74: codes padded to 256 B, then scales padded to 256 B
    assert oracle.q8_segments(10240 * 2560, 2) == [(0, 26214400), (26214400, 1638400)]
    assert oracle.q8_segments(10240 * 2560, 4) == [(0, 26214400), (26214400, 3276800)]
    assert oracle.q8_segments(1536 * 384, 2) == [(0, 589824), (589824, 36864)]
    assert oracle.q8_segments(96, 2) == [(0, 256), (256, 256)]
    g = np.load(os.path.join(GOLDEN, "q8_gguf.npz"))
    blocks = g["blocks"][:3]  # 96 values: both segments need padding
    buf = oracle.q8_transcode_gguf(blocks, 2)
    assert buf.size == 512
    assert np.array_equal(buf[:96], blocks[:, 2:].reshape(-1))
    assert not buf[96:256].any() and not buf[262:].any()
    assert np.array_equal(buf[256:262], blocks[:, :2].reshape(-1))


def test_q8_quantizer_properties():
    rng = np.random.default_rng(5)
    w = (rng.standard_normal(32 * 257) * 0.02).astype(np.float32)
    buf = oracle.q8_quantize_f(w)
    codes = buf[: w.size].view(np.int8)
    d = buf[oracle.q8_segments(w.size, 4)[1][0]:][: w.size // 32 * 4].view(np.float32)
    # quant.rs:57-61: d = amax / 127 in f32
    amax = np.abs(w.reshape(-1, 32)).max(axis=1)
    assert np.array_equal(d, (amax / np.float32(127.0)).astype(np.float32))
    assert codes.min() >= -127 and codes.max() <= 127
    assert np.all(np.abs(codes.reshape(-1, 32)).max(axis=1) == 127)
    # round half away from zero of x / d
    q = w.reshape(-1, 32) / d[:, None]
    want = np.where(q >= 0, np.floor(q + np.float32(0.5)), np.ceil(q - np.float32(0.5))).astype(np.int8)
    assert np.array_equal(codes.reshape(-1, 32), want)
    deq = oracle.q8_dequantize_f(buf, w.size)
    assert np.all(np.abs(deq - w) <= np.repeat(d, 32) * 0.5000001)
    # an all-zero block: d = 0, x/d = NaN -> code 0 (Rust `as i32`)
    z = np.zeros(64, dtype=np.float32)
    bz = oracle.q8_quantize_f(z)
    assert not bz.any()


def test_q8_close_to_gguf_quantizer():
    """gguf-py rounds half to even and multiplies by 1/d, so codes may differ by one in rare ties."""
    from gguf import GGMLQuantizationType, quants
    rng = np.random.default_rng(6)
    w = (rng.standard_normal((64, 256)) * 0.02).astype(np.float32)
    ours = oracle.q8_quantize_f(w)[: w.size].view(np.int8).astype(np.int32)
    theirs = quants.quantize(w, GGMLQuantizationType.Q8_0).reshape(-1, 34)[:, 2:].reshape(-1).view(np.int8).astype(np.int32)
    diff = np.abs(ours - theirs)
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3


def test_q4k_decode_matches_gguf_bit_exact():
    g = np.load(os.path.join(GOLDEN, "q4k_gguf.npz"))
    got = oracle.q4k_dequantize(g["blocks"].reshape(-1), g["dequant"].size)
    assert np.array_equal(got.view(np.uint32), g["dequant"].reshape(-1).view(np.uint32))


def test_q4k_encoder_round_trip():
    rng = np.random.default_rng(7)
    w = (rng.standard_normal(256 * 48) * 0.02).astype(np.float32)
    deq = oracle.q4k_dequantize(oracle.q4k_quantize(w), w.size)
    assert oracle.rel_l2(deq, w) < 0.09  # 4-bit affine per 32 values
    # decode(encode(decode(blocks))) is a fixed point of the codec's value set
    again = oracle.q4k_dequantize(oracle.q4k_quantize(deq), w.size)
    assert oracle.rel_l2(again, deq) < 0.03


def test_gelu_matches_torch_fixture():
    g = np.load(os.path.join(GOLDEN, "gelu.npz"))
    assert np.abs(oracle.gelu_f32(g["x"]) - g["y"]).max() < 1e-6


@pytest.mark.parametrize("key", [f"c{i:03d}" for i in range(int(np.load(os.path.join(GOLDEN, "sgemm.npz"))["n_cases"][0]))])
def test_matmul_oracles_match_torch_fixture(key):
    z = np.load(os.path.join(GOLDEN, "sgemm.npz"))
    a, b, c = z[key + "_a"], z[key + "_b"], z[key + "_c"]
    tl, tr, to, hb = (int(v) for v in z[key + "_meta"])
    bias = z[key + "_bias"] if hb else None
    M, K = (a.shape[-1], a.shape[-2]) if tl else (a.shape[-2], a.shape[-1])
    N = b.shape[-2] if tr else b.shape[-1]
    stacks = max(a.shape[0], b.shape[0])
    # the shape rule first (matmul.rs:284-361)
    assert shape_rules.compute_c_shape(a.shape, b.shape, tl, tr, to) == list(c.shape)
    truth = oracle.matmul_truth(a, b, bias, stacks, a.shape[0], b.shape[0], M, N, K, tl, tr, to)
    faithful = oracle.matmul_faithful(a, b, bias, stacks, a.shape[0], b.shape[0], M, N, K, tl, tr, to, 0, "f32")
    # the reference's own bar against torch: all_close(1e-4, 1e-4) (matmul.rs:827)
    assert np.allclose(truth.astype(np.float32), c.reshape(-1), rtol=1e-4, atol=1e-4)
    assert np.allclose(faithful, c.reshape(-1), rtol=1e-4, atol=1e-4)


def test_f16_faithful_oracle_distance_from_truth():
    """The reference's f16 path (f16 products, f32 sums) sits a few 1e-4 from the truth: inside 1e-3."""
    rng = np.random.default_rng(8)
    M, N, K = 48, 40, 2560
    w = (rng.standard_normal((M, K)) * 0.02).astype(np.float32)
    buf = oracle.q8_quantize_h(w)
    wv = oracle.q8_dequantize_h(buf, w.size).astype(np.float32)
    x = rng.standard_normal((N, K)).astype(np.float16).astype(np.float32)
    truth = oracle.matmul_truth(wv, x, None, 1, 1, 1, M, N, K, False, True, True)
    truth_r = oracle.f64_to_f16(truth).astype(np.float32)
    faith = oracle.matmul_faithful(wv, x, None, 1, 1, 1, M, N, K, False, True, True, 0, "f16")
    err = oracle.rel_l2(faith, truth_r)
    assert 1e-5 < err < 1e-3
    # the GEMV order (32 lane partials, gemv.rs:492-553) agrees with the GEMM order to f32 rounding
    gv = oracle.gemv_faithful(wv, x[0], None, M, K, "f16")
    gm = oracle.matmul_faithful(wv, x[0:1], None, 1, 1, 1, M, 1, K, False, True, True, 0, "f16")
    assert oracle.rel_l2(gv, gm) < 1e-3


def test_packed_cpu_baseline_equals_faithful_oracle():
    rng = np.random.default_rng(9)
    N, K = 64, 512
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    buf = oracle.q8_quantize_h(w)
    wv = oracle.q8_dequantize_h(buf, w.size).astype(np.float32)
    x = rng.standard_normal(K).astype(np.float16)
    b = (rng.standard_normal(N) * 0.02).astype(np.float16)
    y = oracle.q8h_gemv_packed(buf, N, K, x, b)
    ref = oracle.matmul_faithful(wv, x.astype(np.float32)[None, :], b.astype(np.float32), 1, 1, 1, N, 1, K,
                                 False, True, True, 0, "f16")
    assert np.array_equal(y.astype(np.float32), ref)


def test_bf16_rounding_single():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e38, 3.4e38, 1e-40, 0.1], dtype=np.float64)
    bits = oracle.f64_to_bf16_bits(x)
    import torch
    want = torch.tensor(x, dtype=torch.float64).to(torch.float32).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, want)


def _qmatmul_cases():
    z = np.load(os.path.join(GOLDEN, "qmatmul.npz"))
    for name in z["quant_cases"]:
        name = str(name)
        N, K, M, has_bias, gelu = (int(v) for v in z[name + "_meta"])
        yield name, z[name + "_blocks"], z[name + "_x"], (z[name + "_bias"] if has_bias else None), z[name + "_y"], N, K, M, gelu


def test_truth_oracle_over_decoded_blocks_matches_gguf_py_plus_torch():
    """GGUF blocks -> this oracle's decode -> this oracle's fp64 matmul (+ bias, + GELU), against the same blocks
    through gguf-py's decoder and torch.matmul in float64: the expected values never touched this repository's code."""
    for name, blocks, x, bias, want, N, K, M, gelu in _qmatmul_cases():
        if name.startswith("q8"):
            w = oracle.q8_dequantize_h(oracle.q8_transcode_gguf(blocks, 2), N * K).astype(np.float32)
        else:
            w = oracle.q4k_dequantize(blocks.reshape(-1), N * K)
        truth = oracle.matmul_truth(w.reshape(N, K), x.astype(np.float32), None if bias is None else bias.astype(np.float32),
                                    1, 1, 1, N, M, K, False, True, True, gelu)
        got = oracle.f64_to_f16(truth).reshape(want.shape)
        # one rounding on both sides: equal up to rare last-digit flips (the two GELUs evaluate tanh differently)
        ulp = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
        assert ulp.max() <= 1 and (ulp != 0).mean() < 0.01, (name, int(ulp.max()), float((ulp != 0).mean()))


def test_truth_oracle_f16_dense_matches_torch_half_matmul():
    z = np.load(os.path.join(GOLDEN, "qmatmul.npz"))
    for name in ("f16_a", "f16_b"):
        a, b, c = z[name + "_a"], z[name + "_b"], z[name + "_c"]
        B, M, K = a.shape
        N = b.shape[2]
        truth = oracle.matmul_truth(a.astype(np.float32), b.astype(np.float32), None, B, B, B, M, N, K, False, False, False)
        got = oracle.f64_to_f16(truth).reshape(c.shape)
        assert oracle.rel_l2(got.astype(np.float32), c.astype(np.float32)) <= 2e-4  # torch sums in f32
