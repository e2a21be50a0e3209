"""Host-side rules of the library (no GPU): C ABI surface, shapes, dtypes, layouts, quantisers."""
import ctypes
import os
import re
from ctypes import byref

import numpy as np
import pytest

import oracle
import ratchet_b200 as rb
from oracle import shape_rules
from ratchet_b200 import DType, InvariantError, Matmul, Quantization, Quantizer, ShapeError, Tensor, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "ratchet_b200.h")).read()
    names = set(re.findall(r"\b(rt_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 30
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing
    assert "sm_100a" in _lib.load().rt_version().decode()


def test_public_structs_have_the_layout_the_ctypes_mirror_assumes():
    """sizeof / offsetof as the library was compiled against the ctypes Structures of _lib.py (the same check a
    Rust -sys crate would make of its #[repr(C)] structs)."""
    lib = _lib.load()
    buf = (ctypes.c_uint64 * 64)()
    n = lib.rt_abi_layout(buf, 64)
    S, L = ctypes.sizeof, _lib
    off = lambda t, f: getattr(t, f).offset
    want = [
        S(L.rt_shape), off(L.rt_shape, "dims"), S(L.rt_segment),
        S(L.rt_matmul_desc), off(L.rt_matmul_desc, "lhs_shape"), off(L.rt_matmul_desc, "rhs_shape"), off(L.rt_matmul_desc, "bias_shape"),
        off(L.rt_matmul_desc, "has_bias"), off(L.rt_matmul_desc, "epilogue"),
        S(L.rt_gemm_spec), off(L.rt_gemm_spec, "out_dt"), off(L.rt_gemm_spec, "lhs_stack"), off(L.rt_gemm_spec, "dim_inner"), off(L.rt_gemm_spec, "is_gemv"),
        S(L.rt_launch_opts), off(L.rt_launch_opts, "outs"), off(L.rt_launch_opts, "out_ld"), off(L.rt_launch_opts, "out_col"),
        S(L.rt_dispatch), off(L.rt_dispatch, "opts"),
        S(L.rt_gguf_value), off(L.rt_gguf_value, "str"),
        S(L.rt_gguf_tensor_info), off(L.rt_gguf_tensor_info, "shape"), off(L.rt_gguf_tensor_info, "nbytes"),
        S(L.rt_usage_record), off(L.rt_usage_record, "producer"), S(L.rt_node_tensors),
        S(L.rt_mlp_desc), off(L.rt_mlp_desc, "fc2"), off(L.rt_mlp_desc, "w1"), off(L.rt_mlp_desc, "out"),
    ]
    assert n == len(want)
    assert [int(buf[i]) for i in range(n)] == want
    # rt_dispatch embeds its options by value
    assert off(L.rt_dispatch, "opts") + S(L.rt_launch_opts) == S(L.rt_dispatch)


def test_no_device_is_a_loud_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(rb.RatchetError) as e:
        rb.Device.request_device(rb.DeviceRequest.GPU)
    assert "no CPU path" in str(e.value)
    # and a CPU tensor cannot be resolved
    a = Tensor.from_data(np.ones((4, 4), dtype=np.float32))
    with pytest.raises(rb.RatchetError):
        a.matmul(a).resolve()


def _desc(lhs_dt, rhs_dt, a, b, tl, tr, to, bias=None, bias_dt=None, epilogue=0):
    d = _lib.rt_matmul_desc()
    d.lhs_dt, d.rhs_dt = int(lhs_dt), int(rhs_dt)
    d.lhs_shape, d.rhs_shape = _lib.rt_shape.of(a), _lib.rt_shape.of(b)
    d.trans_lhs, d.trans_rhs, d.trans_out = int(tl), int(tr), int(to)
    d.has_bias = int(bias is not None)
    if bias is not None:
        d.bias_shape = _lib.rt_shape.of(bias)
        d.bias_dt = int(bias_dt if bias_dt is not None else rhs_dt)
    d.epilogue = epilogue
    return d


def _spec(d):
    s = _lib.rt_gemm_spec()
    st = _lib.load().rt_matmul_spec(byref(d), byref(s))
    return st, s


def test_compute_c_shape_property_space_matches_restated_rules():
    rng = np.random.default_rng(11)
    n_ok = n_err = 0
    for _ in range(3000):
        ra, rbk = rng.integers(1, 5), rng.integers(1, 5)
        a = [int(v) for v in rng.integers(1, 5, size=ra)]
        b = [int(v) for v in rng.integers(1, 5, size=rbk)]
        tl, tr, to = (bool(v) for v in rng.integers(0, 2, size=3))
        if rng.random() < 0.7:  # make the inner dims agree most of the time
            ka = (a[-2] if tl else a[-1]) if ra >= 2 else a[0]
            if rbk >= 2:
                b[-1 if tr else -2] = ka
            else:
                b[0] = ka
        try:
            want = shape_rules.compute_c_shape(a, b, tl, tr, to)
        except shape_rules.ShapeError:
            want = None
        if want is None:
            with pytest.raises(ShapeError):
                Matmul.compute_c_shape(a, b, tl, tr, to)
            n_err += 1
        else:
            assert Matmul.compute_c_shape(a, b, tl, tr, to) == want, (a, b, tl, tr, to)
            n_ok += 1
    assert n_ok > 500 and n_err > 200


def test_compute_c_shape_agrees_with_torch_matmul_shapes():
    import torch
    rng = np.random.default_rng(12)
    for _ in range(300):
        batch_a = [int(v) for v in rng.integers(1, 4, size=rng.integers(0, 3))]
        batch_b = [int(v) for v in rng.integers(1, 4, size=rng.integers(0, 3))]
        m, k, n = (int(v) for v in rng.integers(1, 6, size=3))
        a, b = batch_a + [m, k], batch_b + [k, n]
        try:
            want = list(torch.matmul(torch.empty(a), torch.empty(b)).shape)
        except RuntimeError:
            with pytest.raises(ShapeError):
                Matmul.compute_c_shape(a, b, False, False, False)
            continue
        assert Matmul.compute_c_shape(a, b, False, False, False) == want


def test_config_shapes_and_routing():
    # the five benchmark configurations as W.gemm(X, b, false, true, true) (linear.rs:23)
    cases = [
        (DType.F32, DType.F32, [10240, 2560], [1, 128, 2560], [1, 128, 10240], 10240, 128, 2560, 0),
        (DType.Q8_0H, DType.F16, [10240, 2560], [1, 1, 2560], [1, 1, 10240], 10240, 1, 2560, 1),
        (DType.Q8_0H, DType.F16, [2560, 10240], [1, 1, 10240], [1, 1, 2560], 2560, 1, 10240, 1),
        (DType.Q8_0H, DType.F16, [1536, 384], [1, 1500, 384], [1, 1500, 1536], 1536, 1500, 384, 0),
        (DType.Q4_K, DType.F16, [8192, 3072], [1, 16, 3072], [1, 16, 8192], 8192, 16, 3072, 0),
        (DType.Q8_0H, DType.BF16, [10240, 2560], [4, 2048, 2560], [4, 2048, 10240], 10240, 2048, 2560, 0),
    ]
    for lhs_dt, rhs_dt, a, b, out, M, N, K, gemv in cases:
        st, s = _spec(_desc(lhs_dt, rhs_dt, a, b, False, True, True, bias=[a[0]]))
        assert st == _lib.RT_OK, _lib.load().rt_last_error()
        assert s.out_shape.tolist() == out
        assert (s.dim_lhs_outer, s.dim_rhs_outer, s.dim_inner, s.is_gemv) == (M, N, K, gemv)
        assert s.out_dt == int(rhs_dt)
        assert s.lhs_stack == 1 and s.rhs_stack == b[0] and s.stacks == b[0]


def test_stacking_rules_follow_gemmspec():
    # all stacks equal, or one side broadcast from 1 (matmul.rs:90-94)
    ok = [([6, 8, 4], [6, 4, 8]), ([2, 8, 4], [1, 4, 8]), ([8, 4], [3, 4, 8]), ([2, 3, 8, 4], [2, 3, 4, 8]),
          ([1, 1, 8, 4], [2, 3, 4, 8])]
    for a, b in ok:
        st, s = _spec(_desc(DType.F32, DType.F32, a, b, False, False, False))
        assert st == _lib.RT_OK
        want = shape_rules.gemm_spec(a, b, s.out_shape.tolist(), False, False, False)
        assert (s.lhs_stack, s.rhs_stack, s.out_stack) == (want.lhs_stack, want.rhs_stack, want.out_stack)
    # per-dimension broadcast passes compute_c_shape but trips the stack assertion in the reference
    for a, b in [([2, 1, 8, 4], [1, 3, 4, 8]), ([2, 3, 8, 4], [1, 3, 4, 8])]:
        assert Matmul.compute_c_shape(a, b, False, False, False)
        st, _ = _spec(_desc(DType.F32, DType.F32, a, b, False, False, False))
        assert st == _lib.RT_ERR_INVARIANT
        with pytest.raises(shape_rules.InvariantError):
            shape_rules.gemm_spec(a, b, Matmul.compute_c_shape(a, b, False, False, False), False, False, False)


def test_guards_match_the_reference_panics_and_errors():
    f32, f16 = DType.F32, DType.F16
    # check_dtypes (matmul.rs:454-477)
    for l, r in [(f32, f16), (f16, f32), (DType.Q8_0H, f32), (DType.Q8_0F, DType.BF16), (DType.I32, DType.I32),
                 (f16, DType.Q8_0H)]:
        st, _ = _spec(_desc(l, r, [32, 32], [32, 32], False, False, False))
        assert st == _lib.RT_ERR_DTYPE, (l, r)
        with pytest.raises(shape_rules.InvariantError):
            shape_rules.check_dtypes(l.name, r.name)
    for l, r in shape_rules.ALLOWED_PAIRS:
        st, _ = _spec(_desc(DType[l], DType[r], [32, 32], [32, 32], False, False, False))
        assert st == _lib.RT_OK
    # bias dtype must equal the rhs dtype
    st, _ = _spec(_desc(f32, f32, [8, 4], [4, 8], False, False, False, bias=[8], bias_dt=f16))
    assert st == _lib.RT_ERR_DTYPE
    # Matmul::new: bias must be a vector; quantised lhs cannot be transposed (matmul.rs:266-272)
    st, _ = _spec(_desc(f32, f32, [8, 4], [4, 8], False, False, False, bias=[2, 4]))
    assert st == _lib.RT_ERR_INVARIANT
    st, _ = _spec(_desc(DType.Q8_0F, f32, [32, 64], [32, 8], True, False, False))
    assert st == _lib.RT_ERR_INVARIANT
    # ka != kb is an error, not a panic (matmul.rs:333-335)
    st, _ = _spec(_desc(f32, f32, [8, 4], [5, 8], False, False, False))
    assert st == _lib.RT_ERR_SHAPE
    assert "ka != kb: 4 != 5" in _lib.load().rt_last_error().decode()
    # block formats run along K
    st, _ = _spec(_desc(DType.Q8_0H, f16, [64, 48], [48, 8], False, False, False))
    assert st == _lib.RT_ERR_SHAPE
    st, _ = _spec(_desc(DType.Q4_K, f16, [64, 128], [128, 8], False, False, False))
    assert st == _lib.RT_ERR_SHAPE
    # the Python mirror raises where the reference panics
    a = Tensor.from_data(np.zeros((8, 4), dtype=np.float32))
    with pytest.raises(InvariantError):
        a.gemm(Tensor.from_data(np.zeros((4, 8), dtype=np.float16)), None, False, False, False)
    with pytest.raises(ShapeError):
        a.matmul(Tensor.from_data(np.zeros((5, 8), dtype=np.float32)))


def test_bias_length_rules():
    f32 = DType.F32
    assert _spec(_desc(f32, f32, [8, 4], [4, 6], False, False, False, bias=[6]))[0] == _lib.RT_OK
    assert _spec(_desc(f32, f32, [8, 4], [4, 6], False, False, False, bias=[8]))[0] == _lib.RT_ERR_SHAPE
    assert _spec(_desc(f32, f32, [8, 4], [4, 6], False, False, True, bias=[8]))[0] == _lib.RT_OK   # gemm.rs:468-476
    assert _spec(_desc(f32, f32, [8, 4], [1, 4], False, True, False, bias=[8]))[0] == _lib.RT_OK   # gemv.rs:476-490
    assert _spec(_desc(f32, f32, [8, 4], [1, 4], False, True, False, bias=[1]))[0] == _lib.RT_OK


def test_segments_follow_blocks_rs():
    for numel in (32, 96, 256, 8192, 1536 * 384, 10240 * 2560):
        assert DType.Q8_0H.segments(numel) == oracle.q8_segments(numel, 2)
        assert DType.Q8_0F.segments(numel) == oracle.q8_segments(numel, 4)
        assert DType.Q8_0H.nbytes(numel) == oracle.q8_nbytes(numel, 2)
    # plain types: max(bytes, 16) rounded up to 4 (dtype/mod.rs:88-92)
    assert DType.F32.segments(1) == [(0, 16)]
    assert DType.F16.segments(9) == [(0, 20)]
    assert DType.F16.segments(1000) == [(0, 2000)]
    assert DType.Q4_K.segments(8192 * 3072) == [(0, 14155776)]
    with pytest.raises(ShapeError):
        DType.Q8_0H.segments(33)
    assert DType.Q8_0H.activation_dt() == DType.F16 and DType.Q8_0F.activation_dt() == DType.F32
    assert DType.F16.size_of() == 2 and DType.Q8_0H.is_quantized() and not DType.F32.is_quantized()


def test_host_quantizers_equal_the_oracle_bit_for_bit():
    rng = np.random.default_rng(13)
    w = (rng.standard_normal((96, 160)) * 0.02).astype(np.float32)
    w[3, :32] = 0.0  # an all-zero block
    w[5, 7] = 1e-30
    t = Tensor.from_data(w)
    qz = Quantizer(Quantization.SInt8)
    qf, qh = qz.sint8_quantize(t), qz.sint8_quantize(t, DType.Q8_0H)
    assert np.array_equal(qf.to_numpy(), oracle.q8_quantize_f(w))
    assert np.array_equal(qh.to_numpy(), oracle.q8_quantize_h(w))
    assert np.array_equal(qz.sint8_dequantize(qf).to_numpy().reshape(-1), oracle.q8_dequantize_f(qf.to_numpy(), w.size))
    assert np.array_equal(qz.sint8_dequantize(qh).to_numpy().reshape(-1),
                          oracle.q8_dequantize_h(qh.to_numpy(), w.size).astype(np.float32))
    w4 = (rng.standard_normal((8, 512)) * 0.02).astype(np.float32)
    q4 = Quantizer.q4k_quantize(Tensor.from_data(w4))
    assert np.array_equal(q4.to_numpy(), oracle.q4k_quantize(w4))
    assert np.array_equal(q4.to_f32().reshape(-1), oracle.q4k_dequantize(q4.to_numpy(), w4.size))


def test_host_decoders_match_gguf_fixtures():
    g = np.load(os.path.join(GOLDEN, "q8_gguf.npz"))
    n = g["dequant"].size
    t = rb.transcode_gguf_q8_0(g["blocks"], [n // 32, 32], DType.Q8_0F)
    assert np.array_equal(t.to_numpy(), oracle.q8_transcode_gguf(g["blocks"], 4))
    assert np.array_equal(t.to_f32().reshape(-1).view(np.uint32), g["dequant"].reshape(-1).view(np.uint32))
    th = rb.transcode_gguf_q8_0(g["blocks"], [n // 32, 32], DType.Q8_0H)
    assert np.array_equal(th.to_numpy(), oracle.q8_transcode_gguf(g["blocks"], 2))
    g4 = np.load(os.path.join(GOLDEN, "q4k_gguf.npz"))
    got = Quantizer.dequantize_bytes(g4["blocks"].reshape(-1), DType.Q4_K, g4["dequant"].size)
    assert np.array_equal(got.view(np.uint32), g4["dequant"].reshape(-1).view(np.uint32))


def test_host_f16_conversion_is_ieee():
    # every f16 scale value survives Q8_0H quantise -> dequantise of a block whose amax hits it
    bits = np.arange(0, 0x7C00, dtype=np.uint16)
    f = bits.view(np.float16).astype(np.float32)
    rng = np.random.default_rng(14)
    d = (rng.uniform(0, 70000, size=4096)).astype(np.float32)
    d = np.concatenate([d, f[::7], f[1:] - np.diff(f) / 2])  # ties between neighbours
    x = np.zeros((d.size, 32), dtype=np.float32)
    x[:, 0] = d * np.float32(127.0)
    ok = np.isfinite(x[:, 0])
    x = x[ok]
    q = Quantizer(Quantization.SInt8).sint8_quantize(Tensor.from_data(x), DType.Q8_0H).to_numpy()
    off = DType.Q8_0H.segments(x.size)[1][0]
    got = q[off: off + 2 * x.shape[0]].view(np.uint16)
    want = (np.abs(x).max(axis=1) / np.float32(127.0)).astype(np.float32).astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_lazy_graph_shapes_without_a_device():
    # Linear builds W.gemm(x, b, false, true, true): out [B, M, N] in the activation dtype
    w = Quantizer(Quantization.SInt8).sint8_quantize(Tensor.from_data(np.ones((64, 32), dtype=np.float32)), DType.Q8_0H)
    x = Tensor.from_data(np.ones((2, 5, 32), dtype=np.float16))
    y = rb.Linear(w, Tensor.from_data(np.ones(64, dtype=np.float32))).schedule(x)
    assert y.shape == [2, 5, 64] and y.dt == DType.F16 and not y.resolved()
    z = rb.Linear(Tensor.from_data(np.ones((16, 64), dtype=np.float16))).schedule(y)
    assert z.shape == [2, 5, 16]
    assert z.execution_order()[-1] is z


def test_silu_mul_epilogue_halves_the_linear_output_and_rejects_other_forms():
    """RT_EPILOGUE_SILU_MUL (the gate/up fold of phi3/mlp.rs:31-39): only the Linear form takes it, the weight
    has an even number of rows, and the node's output is [.., rows/2]."""
    SILU = _lib.RT_EPILOGUE_SILU_MUL
    st, s = _spec(_desc(DType.Q8_0H, DType.F16, [16384, 3072], [1, 7, 3072], False, True, True, epilogue=SILU))
    assert st == _lib.RT_OK and s.out_shape.tolist() == [1, 7, 8192]
    assert s.dim_lhs_outer == 16384 and s.dim_rhs_outer == 7 and s.dim_inner == 3072
    out = _lib.rt_shape()
    d = _desc(DType.F16, DType.F16, [64, 32], [5, 32], False, True, True, bias=[64], epilogue=SILU)
    assert _lib.load().rt_matmul_out_shape(byref(d), byref(out)) == _lib.RT_OK and out.tolist() == [5, 32]
    st, _ = _spec(_desc(DType.F16, DType.F16, [63, 32], [5, 32], False, True, True, epilogue=SILU))
    assert st == _lib.RT_ERR_SHAPE
    for trans in [(False, False, False), (False, True, False), (True, False, True)]:
        a = [32, 64] if trans[0] else [64, 32]
        b = [5, 32] if trans[1] else [32, 5]
        st, _ = _spec(_desc(DType.F16, DType.F16, a, b, *trans, epilogue=SILU))
        assert st == _lib.RT_ERR_INVARIANT, trans
    st, _ = _spec(_desc(DType.F16, DType.F16, [64, 32], [5, 32], False, True, True, epilogue=3))
    assert st == _lib.RT_ERR_ARG


def test_oracle_silu_follows_the_two_branch_sigmoid():
    """ops/unary.rs:121-131: exp(v)/(1+exp(v)) for v >= 0, which is NaN once exp(v) overflows; 1/(1+exp(-v)) below,
    which underflows to -0 * ... = -0."""
    import oracle
    v = np.array([0.0, 1.0, -1.0, 20.0, -20.0, 88.0, 89.0, -100.0, 65504.0], dtype=np.float32)
    s = oracle.silu_f32(v)
    assert s[0] == 0.0 and abs(s[1] - 0.7310586) < 1e-6 and abs(s[2] + 0.26894143) < 1e-6
    assert abs(s[3] - 20.0) < 1e-5 and abs(s[4]) < 1e-7 and abs(s[5] - 88.0) < 1e-4
    assert np.isnan(s[6]) and np.isnan(s[8]) and s[7] == 0.0
    full = np.array([[1.0, -2.0, 3.0, 0.5]], dtype=np.float32)  # gate = [1, -2], up = [3, 0.5]
    got = oracle.silu_mul(full, "f16")
    want = np.array([[3.0 * np.float16(0.7310586), 0.5 * np.float16(-2.0 * 0.11920292)]], dtype=np.float16)
    assert np.array_equal(got.astype(np.float16), want)
