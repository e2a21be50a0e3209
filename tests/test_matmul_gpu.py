"""Parity of the CUDA path against the oracle, through the host mirror and the C ABI.  GPU only."""
import os

import numpy as np
import pytest

import oracle
import ratchet_b200 as rb
from ratchet_b200 import DType, Device, Linear, Quantization, Quantizer, Tensor
from util import TOL, TRANS_KINDS, Problem, check_problem, make_lhs, round_to, run_problem

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
F32, F16, BF16, Q8H, Q8F, Q4K = DType.F32, DType.F16, DType.BF16, DType.Q8_0H, DType.Q8_0F, DType.Q4_K


# ----------------------------------------------------------------------------- dequantised weights: bit-exact

@pytest.mark.parametrize("dt", [Q8H, Q8F, Q4K])
def test_device_dequant_is_bit_exact(gpu, dt):
    rng = np.random.default_rng(21)
    shape = (96, 768)
    t, vals = make_lhs(dt, shape, rng, 0.02)
    got = t.to(gpu).dequantize_on_device()
    if dt == Q8H:
        assert got.dtype == np.float16
        assert np.array_equal(got.view(np.uint16), vals.astype(np.float16).view(np.uint16))
    else:
        assert np.array_equal(got.view(np.uint32), vals.view(np.uint32))


def test_device_dequant_matches_gguf_fixtures(gpu):
    g = np.load(os.path.join(GOLDEN, "q8_gguf.npz"))
    n = g["dequant"].size
    t = rb.transcode_gguf_q8_0(g["blocks"], [n // 32, 32], Q8F, gpu)
    assert np.array_equal(t.dequantize_on_device().reshape(-1).view(np.uint32), g["dequant"].reshape(-1).view(np.uint32))
    g4 = np.load(os.path.join(GOLDEN, "q4k_gguf.npz"))
    n4 = g4["dequant"].size
    t4 = Tensor.from_quantized(g4["blocks"].reshape(-1), Q4K, [n4 // 256, 256], gpu)
    assert np.array_equal(t4.dequantize_on_device().reshape(-1).view(np.uint32), g4["dequant"].reshape(-1).view(np.uint32))


def test_quantised_matmul_fixtures_from_gguf_py_and_torch(gpu):
    """GGUF blocks through the library's loader path (transcode for Q8_0, raw super-blocks for Q4_K) and kernels,
    against values that gguf-py's decoder and torch.matmul in float64 produced (tests/golden/make_qmatmul_golden.py):
    GEMV, skinny and GEMM shapes, with bias and GELU."""
    z = np.load(os.path.join(GOLDEN, "qmatmul.npz"))
    for name in z["quant_cases"]:
        name = str(name)
        N, K, M, has_bias, gelu = (int(v) for v in z[name + "_meta"])
        if name.startswith("q8"):
            w = rb.transcode_gguf_q8_0(z[name + "_blocks"], [N, K], Q8H, gpu)
        else:
            w = Tensor.from_quantized(z[name + "_blocks"].reshape(-1), Q4K, [N, K], gpu)
        bias = Tensor.from_data(z[name + "_bias"], gpu) if has_bias else None
        y = w.gemm(Tensor.from_data(z[name + "_x"], gpu), bias, False, True, True, epilogue=gelu).resolve().to(Device.CPU)
        want = z[name + "_y"].astype(np.float32)
        assert y.shape == list(want.shape)
        assert oracle.rel_l2(y.to_f32().reshape(-1), want.reshape(-1)) <= TOL[F16], name
    for name in ("f16_a", "f16_b"):
        y = Tensor.from_data(z[name + "_a"], gpu).matmul(Tensor.from_data(z[name + "_b"], gpu)).resolve().to(Device.CPU)
        assert oracle.rel_l2(y.to_f32().reshape(-1), z[name + "_c"].astype(np.float32).reshape(-1)) <= TOL[F16], name


# ----------------------------------------------------------------------------- dense f32: the reference's own test space

@pytest.mark.parametrize("i", range(int(np.load(os.path.join(GOLDEN, "sgemm.npz"))["n_cases"][0])))
def test_sgemm_fixture(gpu, i):
    z = np.load(os.path.join(GOLDEN, "sgemm.npz"))
    key = f"c{i:03d}"
    a, b, c = z[key + "_a"], z[key + "_b"], z[key + "_c"]
    tl, tr, to, hb = (bool(v) for v in z[key + "_meta"])
    bias = Tensor.from_data(z[key + "_bias"], gpu) if hb else None
    out = Tensor.from_data(a, gpu).gemm(Tensor.from_data(b, gpu), bias, tl, tr, to).resolve().to(Device.CPU)
    assert out.shape == list(c.shape)
    # the reference's bar: ground.all_close(&ours, 1e-4, 1e-4) (matmul.rs:827)
    assert np.allclose(out.to_numpy(), c, rtol=1e-4, atol=1e-4)


def test_sgemm_property_space(gpu):
    """SGEMMProblem (matmul.rs:743-756): B 1..3, M/K/N 1..256, bias, six transpose kinds; f32 and f16."""
    rng = np.random.default_rng(22)
    kinds = list(TRANS_KINDS.values())
    for case in range(48):
        B, M, K, N = int(rng.integers(1, 4)), *(int(v) for v in rng.integers(1, 257, size=3))
        tl, tr, to = kinds[case % 6]
        dt = F32 if case % 2 == 0 else F16
        lhs = (B, K, M) if tl else (B, M, K)
        rhs = (B, N, K) if tr else (B, K, N)
        check_problem(Problem(dt, dt, lhs, rhs, (tl, tr, to), bias=bool(rng.integers(0, 2)), seed=100 + case), gpu)


def test_sgemm_property_space_at_tensor_core_sizes(gpu):
    """The same space with extents up to 700 x 1600 x 700 (most cases reach the tensor-core GEMMs, with ragged last
    tiles, inner dimensions that need padding, and an rhs that has to be transposed first), bf16 as a third dtype, and
    one operand's batch broadcast against the other's."""
    rng = np.random.default_rng(23)
    kinds = list(TRANS_KINDS.values())
    seen = set()
    for case in range(36):
        B = int(rng.integers(1, 4))
        M, N = (int(v) for v in rng.integers(1, 701, size=2))
        K = int(rng.integers(1, 1601))
        tl, tr, to = kinds[case % 6]
        dt = [F32, F16, BF16][case % 3]
        bl, br = (B, B) if case % 4 else ((1, B) if case % 8 else (B, 1))
        lhs = (bl, K, M) if tl else (bl, M, K)
        rhs = (br, N, K) if tr else (br, K, N)
        _, kernel = check_problem(Problem(dt, dt, lhs, rhs, (tl, tr, to), bias=bool(rng.integers(0, 2)), seed=300 + case,
                                          w_std=1.0 / np.sqrt(K)), gpu)
        seen.add(kernel.split("_")[0] + "_" + kernel.split("_")[1])
    assert any(k.startswith("gemm_umma") for k in seen), seen


def test_reference_regression_shapes(gpu):
    # debug_gemm (matmul.rs:854-890): transposed lhs, broadcast batch, extents not multiples of 32
    check_problem(Problem(F32, F32, (2, 222, 252), (1, 222, 238), (True, False, False), bias=True, seed=31), gpu)
    # debug_gemv (matmul.rs:892-926): 51865 rows, trans_out
    for dt in (F32, F16):
        _, kernel = check_problem(Problem(dt, dt, (1, 51865, 384), (1, 1, 384), (False, True, True), seed=32), gpu)
        assert "gemv" in kernel
    # test_qgemm (matmul.rs:831-852): Q8_0F [6,1500,64] x [6,64,1500], all stacks equal
    check_problem(Problem(Q8F, F32, (6, 1500, 64), (6, 64, 1500), (False, False, False), seed=33), gpu)
    # quantised GEMV at the Whisper logits shape
    check_problem(Problem(Q8H, F16, (51865, 384), (1, 1, 384), (False, True, True), seed=34, w_std=0.02), gpu)


def test_every_matmul_call_site_of_the_models(gpu):
    """The forms and shape families of each `matmul` / `gemm` call in the reference's models."""
    nn = (False, False, False)
    # attention scores q·kT (k permuted beforehand, so plain matmul) in f32 after .full(), then
    # softmax(w)·v in the cache dtype: phi2/attn.rs:139-151, phi3/attn.rs:144-155,
    # moondream/text_model.rs:87-98 -- rank 4, all stacks equal; prefill (S = T) and decode (S = 1)
    for heads, hd, S, T in [(32, 80, 48, 48), (32, 80, 1, 200), (32, 96, 1, 64)]:
        check_problem(Problem(F32, F32, (1, heads, S, hd), (1, heads, hd, T), nn, seed=51), gpu)
        check_problem(Problem(F16, F16, (1, heads, S, T), (1, heads, T, hd), nn, seed=52), gpu)
    # whisper/mha.rs:109-124: scores and values both in the activation dtype, encoder length 1500
    for dt in (F32, F16):
        check_problem(Problem(dt, dt, (1, 6, 1500, 64), (1, 6, 64, 1500), nn, seed=53), gpu)
        check_problem(Problem(dt, dt, (1, 6, 1500, 1500), (1, 6, 1500, 64), nn, seed=54), gpu)
        check_problem(Problem(dt, dt, (1, 6, 1, 64), (1, 6, 64, 1500), nn, seed=55), gpu)  # decoder cross-attention
    # moondream/vision_encoder.rs:58-61: 729 patches, 16 heads of 72
    check_problem(Problem(F32, F32, (1, 16, 729, 72), (1, 16, 72, 729), nn, seed=56), gpu)
    check_problem(Problem(F16, F16, (1, 16, 729, 729), (1, 16, 729, 72), nn, seed=57), gpu)
    # crates/ratchet-core/tests/attn_tests.rs:56-65,129-153
    check_problem(Problem(F32, F32, (1, 128, 256), (256, 256), nn, seed=58), gpu)
    check_problem(Problem(F32, F32, (1, 64, 384), (1, 384, 384), nn, seed=59), gpu)
    # nn::Linear (linear.rs:23) at the shapes the configs do not name
    lin = (False, True, True)
    check_problem(Problem(Q8H, F16, (51200, 2560), (1, 1, 2560), lin, bias=True, seed=60, w_std=0.02), gpu)  # Phi-2 lm_head
    check_problem(Problem(Q8H, F16, (16384, 3072), (1, 1, 3072), lin, seed=61, w_std=0.02), gpu)             # Phi-3 gate_up
    check_problem(Problem(Q8H, F16, (3072, 8192), (1, 7, 8192), lin, seed=62, w_std=0.02), gpu)              # Phi-3 down, short prompt
    check_problem(Problem(Q8H, F16, (2048, 1152), (1, 729, 1152), lin, bias=True, seed=63, w_std=0.02), gpu)  # Moondream projection
    check_problem(Problem(F16, F16, (384, 384), (1, 1500, 384), lin, seed=64, w_std=0.05), gpu)              # Whisper k (no bias)


def test_rank_and_broadcast_forms(gpu):
    check_problem(Problem(F32, F32, (7, 5), (5,), (False, False, False), seed=41), gpu)           # implicit n
    check_problem(Problem(F32, F32, (5,), (5, 9), (False, False, False), seed=42), gpu)           # implicit m
    check_problem(Problem(F32, F32, (3, 2, 17, 5), (3, 2, 5, 9), (False, False, False), seed=43), gpu)
    check_problem(Problem(F16, F16, (17, 40), (3, 2, 40, 9), (False, False, False), bias=True, seed=44), gpu)
    check_problem(Problem(F32, F32, (4, 33, 20), (1, 20, 65), (False, False, True), seed=45), gpu)
    check_problem(Problem(BF16, BF16, (2, 64, 96), (2, 96, 48), (False, False, False), bias=True, seed=46), gpu)


def test_empty_and_degenerate(gpu):
    a = Tensor.from_data(np.zeros((0, 4), dtype=np.float32), gpu)
    b = Tensor.from_data(np.ones((4, 3), dtype=np.float32), gpu)
    out = a.matmul(b).resolve().to(Device.CPU)
    assert out.shape == [0, 3]
    # K = 0: an empty sum, only the bias survives
    a = Tensor.from_data(np.zeros((5, 0), dtype=np.float32), gpu)
    b = Tensor.from_data(np.zeros((0, 3), dtype=np.float32), gpu)
    bias = Tensor.from_data(np.array([1.0, 2.0, 3.0], dtype=np.float32), gpu)
    out = a.gemm(b, bias, False, False, False).resolve().to(Device.CPU).to_numpy()
    assert np.array_equal(out, np.tile(np.array([1.0, 2.0, 3.0], dtype=np.float32), (5, 1)))
    check_problem(Problem(F32, F32, (1, 1), (1, 1), seed=47), gpu)


def test_launch_rejects_aliasing_and_null(gpu):
    lib = rb._lib.load()
    a = Tensor.from_data(np.ones((8, 8), dtype=np.float32), gpu)
    out = a.matmul(a)
    plan = gpu.plan_for(out.op.desc)
    assert lib.rt_matmul_launch(plan, a.ptr, a.ptr, None, a.ptr, None) == rb._lib.RT_ERR_INVARIANT
    assert lib.rt_matmul_launch(plan, None, a.ptr, None, a.ptr, None) == rb._lib.RT_ERR_ARG
    # the same invariant when the node is bound into an executable
    from ctypes import byref, c_void_p
    node = (rb._lib.rt_dispatch * 1)()
    node[0].plan, node[0].lhs, node[0].rhs, node[0].out = plan, a.ptr, a.ptr, a.ptr
    exe = c_void_p()
    assert lib.rt_executable_create(gpu._h, node, 1, 0, byref(exe)) == rb._lib.RT_ERR_INVARIANT


def test_streaming_gemv_rejects_misaligned_operands(gpu):
    """The Q8_0 streaming kernel fetches rows with bulk copies and activations with 16-byte loads: an offset device
    pointer is refused with an error code, not handed to the kernel."""
    lib = rb._lib.load()
    w, _ = make_lhs(Q8H, (1000, 2560), np.random.default_rng(1), 0.02)
    w = w.to(gpu)
    x = Tensor.from_data(np.zeros((1, 2, 2560), dtype=np.float16), gpu)
    node = w.gemm(x, None, False, True, True)
    plan = gpu.plan_for(node.op.desc)
    assert lib.rt_plan_kernel(plan).decode().startswith("q8_gemv_mma")
    out = rb.GpuBuffer(gpu, 2 * 1000 * 2)
    assert lib.rt_matmul_launch(plan, w.ptr, x.ptr + 4, None, out.ptr, None) == rb._lib.RT_ERR_ARG
    assert lib.rt_matmul_launch(plan, w.ptr + 8, x.ptr, None, out.ptr, None) == rb._lib.RT_ERR_ARG
    assert b"16-byte aligned" in lib.rt_last_error()
    assert lib.rt_matmul_launch(plan, w.ptr, x.ptr, None, out.ptr, None) == rb._lib.RT_OK
    gpu.sync()


@pytest.mark.parametrize("lhs_dt,act", [(Q8H, F16), (Q8H, BF16), (Q4K, F16), (F32, F32), (F16, F16)])
def test_tensor_core_gemm_rejects_misaligned_operands(gpu, lhs_dt, act):
    """Its tensor maps and its dequantise / cast pre-passes need 16-byte aligned operands: refused with an error code
    before anything is launched."""
    lib = rb._lib.load()
    w, _ = make_lhs(lhs_dt, (512, 512), np.random.default_rng(1), 0.02)
    w = w.to(gpu)
    np_dt = np.float32 if act == F32 else np.float16
    x = Tensor.from_data(np.zeros((1, 130, 512), dtype=np.float32), gpu, act)
    node = w.gemm(x, None, False, True, True)
    plan = gpu.plan_for(node.op.desc)
    assert lib.rt_plan_kernel(plan).decode().startswith("gemm_umma"), lib.rt_plan_kernel(plan)
    out = rb.GpuBuffer(gpu, 130 * 512 * 4 + 64)
    assert lib.rt_matmul_launch(plan, w.ptr, x.ptr + 4, None, out.ptr, None) == rb._lib.RT_ERR_ARG
    assert lib.rt_matmul_launch(plan, w.ptr + 8, x.ptr, None, out.ptr, None) == rb._lib.RT_ERR_ARG
    assert b"16-byte aligned" in lib.rt_last_error()
    # an output that is only element-aligned is fine: the epilogue falls back to narrower stores
    assert lib.rt_matmul_launch(plan, w.ptr, x.ptr, None, out.ptr + x.dt.size_of(), None) == rb._lib.RT_OK
    assert lib.rt_matmul_launch(plan, w.ptr, x.ptr, None, out.ptr, None) == rb._lib.RT_OK
    gpu.sync()


def test_plans_are_cached_by_the_library_and_kept_weights_follow_their_buffers(gpu):
    """rt_matmul_plan hands equal descriptions the same plan (the KernelKey cache's role).  A quantised weight
    flagged constant is dequantised once and the copy kept by pointer; when the weight's buffer is freed and its
    block reused for another weight, the stale copy must not be used."""
    from ctypes import byref, c_void_p
    lib = rb._lib.load()
    shape, rows = (512, 256), 64
    x = round_to(F16, np.random.default_rng(7).standard_normal((1, rows, 256)))
    xd = Tensor.from_data(x, gpu, F16)
    results = []
    for seed in (11, 12):
        w_t, wv = make_lhs(Q8H, shape, np.random.default_rng(seed), 0.02)
        w_dev = w_t.to(gpu)
        node = w_dev.gemm(xd, None, False, True, True)
        h1, h2 = c_void_p(), c_void_p()
        rb._lib.check(lib.rt_matmul_plan(gpu._h, byref(node.op.desc), byref(h1)))
        rb._lib.check(lib.rt_matmul_plan(gpu._h, byref(node.op.desc), byref(h2)))
        assert h1.value == h2.value
        assert lib.rt_plan_kernel(h1).decode().endswith("_dequant_prepass")
        for _ in range(2):  # the second launch takes the kept copy
            y = w_dev.gemm(xd, None, False, True, True).resolve().to(Device.CPU)
            truth = oracle.matmul_truth(wv, x, None, 1, 1, 1, shape[0], rows, shape[1], False, True, True)
            assert oracle.rel_l2(y.to_f32().reshape(-1), oracle.f64_to_f16(truth).astype(np.float32)) <= TOL[F16], seed
        results.append(w_dev.ptr)
        del w_dev, node, y  # the buffer goes back to the pool: the next weight of this size gets the same block
    assert results[0] == results[1], "the pool did not reuse the block: the test did not exercise the stale-copy case"


# ----------------------------------------------------------------------------- Q8_0 GEMV (decode)

@pytest.mark.parametrize("shape,seed", [((10240, 2560), 102), ((2560, 10240), 112)])
def test_q8_gemv_phi2_shapes(gpu, shape, seed):
    """The Phi-2 MLP decode GEMVs: x f16 [1,1,K], W Q8_0H [N,K] from N(0,0.02), out f16 [1,1,N]."""
    N, K = shape
    for bias in (False, True):
        p = Problem(Q8H, F16, shape, (1, 1, K), (False, True, True), bias=bias, seed=seed, w_std=0.02)
        got, truth_r, truth, faithful, kernel = run_problem(p, gpu)
        assert kernel.startswith("q8_gemv_umma_h"), kernel
        err = oracle.rel_l2(got, truth_r)
        err_ref = oracle.rel_l2(faithful, truth_r)
        assert err <= 1e-3, (kernel, err)
        assert err <= err_ref + 1e-4  # int8 products of 15-bit activation digits: at least as close to the truth as the reference's f16 arithmetic
    # f32 scales with f16 activations (extension) and the reference's (Q8_0F, F32) pair
    _, kernel = check_problem(Problem(Q8F, F16, shape, (1, 1, K), (False, True, True), bias=True, seed=seed, w_std=0.02), gpu)
    assert kernel.startswith("q8_gemv_mma_f")
    check_problem(Problem(Q8F, F32, shape, (1, 1, K), (False, True, True), bias=True, seed=seed, w_std=0.02), gpu)


def _decode_chain(gpu, shapes, seed, with_bias):
    rng = np.random.default_rng(seed)
    x0 = rng.standard_normal(shapes[0][1]).astype(np.float16)
    h = Tensor.from_data(x0, gpu)
    x_dev, nodes, host = h, [], []
    for i, shape in enumerate(shapes):
        w_t, w_vals = make_lhs(Q8H, shape, np.random.default_rng(seed + 10 + i), 0.02 if shape[1] < 8192 else 0.01)
        b_vals = b_t = None
        if with_bias[i]:
            b_vals = round_to(F16, (np.random.default_rng(seed + 50 + i).standard_normal(shape[0]) * 0.02).astype(np.float32))
            b_t = Tensor.from_data(b_vals, gpu, F16)
        epi = rb.EPILOGUE_GELU_TANH if i % 2 == 0 else 0
        h = w_t.to(gpu).gemm(h, b_t, False, True, True, epilogue=epi)
        nodes.append(h)
        host.append((w_vals, b_vals, epi))
    return x_dev, nodes, host


@pytest.mark.parametrize("shapes", [
    [(2560, 2560), (2560, 2560), (2560, 2560)],                        # no K split: clusters of one
    [(10240, 2560), (2560, 10240), (8192, 2560), (2560, 8192)],        # fc1 / fc2: K split four ways on every second node
], ids=["square_x3", "phi2_mlp_x2"])
def test_q8_gemv_chain_is_one_kernel_and_matches_node_by_node(gpu, monkeypatch, shapes):
    """A decode step's GEMVs as ONE persistent kernel (rows handed from node to node as tagged words): every
    node's output agrees with node-by-node dispatch and meets the bar against the fp64 oracle."""
    x_dev, nodes, host = _decode_chain(gpu, shapes, 4100, [True, False, False, True][:len(shapes)])
    nodes[-1].resolve()
    exe = rb.Executable(gpu, nodes, use_graph=True)
    assert exe.kernel.startswith("q8_gemv_chain"), exe.kernel
    assert exe.launches == 1
    monkeypatch.setenv("RT_GEMV_CHAIN", "0")
    exe_nodes = rb.Executable(gpu, nodes, use_graph=True)
    assert exe_nodes.kernel == "graph" and exe_nodes.launches == len(shapes)
    for trial in range(3):  # new input every time: the outputs must really be recomputed
        x = np.random.default_rng(4200 + trial).standard_normal(shapes[0][1]).astype(np.float16)
        x_dev.write(x)
        exe_nodes.dispatch()
        gpu.sync()
        want = [n.to(Device.CPU).to_numpy().reshape(-1).copy() for n in nodes]
        for n in nodes:
            n.write(np.zeros(n.numel(), dtype=np.float16))
        exe.dispatch()
        exe.dispatch()  # back to back: every dispatch has its own tag
        gpu.sync()
        got = [n.to(Device.CPU).to_numpy().reshape(-1).copy() for n in nodes]
        h = x.astype(np.float32)
        for i, (w_vals, b_vals, epi) in enumerate(host):
            # same products, another order of the f32 sums: a last f16 digit here and there, fed forward
            assert oracle.rel_l2(got[i].astype(np.float32), want[i].astype(np.float32)) <= TOL[F16], f"node {i} differs from node-by-node dispatch"
            M, K = shapes[i]
            truth = oracle.matmul_truth(w_vals, h, b_vals, 1, 1, 1, M, 1, K, False, True, True, epi)
            assert oracle.rel_l2(got[i].astype(np.float32), oracle.f64_to_f16(truth).astype(np.float32)) <= TOL[F16]
            h = got[i].astype(np.float32)  # the next node's input is what this one wrote


@pytest.mark.parametrize("shapes,kind", [
    ([(4096, 10240), (2560, 4096)], "chain"),   # K = 10240 splits four ways, K = 4096 two ways: both in one kernel
    ([(2560, 2560), (512, 2560)], "graph"),     # 512 rows are too few for the tensor-memory GEMV: one launch per node
], ids=["mixed_k_splits", "not_eligible"])
def test_q8_gemv_lists_chain_or_graph(gpu, shapes, kind):
    x_dev, nodes, host = _decode_chain(gpu, shapes, 4300, [False, True])
    nodes[-1].resolve()
    exe = rb.Executable(gpu, nodes, use_graph=True)
    assert exe.kernel.startswith("q8_gemv_chain") if kind == "chain" else exe.kernel == "graph", exe.kernel
    for n in nodes:
        n.write(np.zeros(n.numel(), dtype=np.float16))
    exe.dispatch()
    gpu.sync()
    h = x_dev.to(Device.CPU).to_numpy().reshape(-1).astype(np.float32)
    for i, (w_vals, b_vals, epi) in enumerate(host):
        M, K = shapes[i]
        got = nodes[i].to(Device.CPU).to_numpy().reshape(-1)
        truth = oracle.matmul_truth(w_vals, h, b_vals, 1, 1, 1, M, 1, K, False, True, True, epi)
        assert oracle.rel_l2(got.astype(np.float32), oracle.f64_to_f16(truth).astype(np.float32)) <= TOL[F16]
        h = got.astype(np.float32)


def _reference_gemv_f16(w_codes, w_scales, x16):
    """The reference's Q8_0H GEMV arithmetic in numpy (gemv.rs:470-480): code times scale rounded to f16, times x
    in f16, widened to f32 and summed.  IEEE semantics for NaN and infinities come with numpy's float16."""
    with np.errstate(all="ignore"):
        inter = (w_codes.astype(np.float16).reshape(w_codes.shape[0], -1, 32) * w_scales[:, :, None]).astype(np.float16)
        prod = (inter.reshape(w_codes.shape[0], -1) * x16[None, :]).astype(np.float16)
        return prod.astype(np.float32).sum(axis=1, dtype=np.float32)


@pytest.mark.parametrize("as_list", [True, False], ids=["executable", "single_launch"])
def test_q8_gemv_propagates_nan_and_infinities(gpu, as_list):
    """NaN, +inf, -inf and a 60000-magnitude outlier among N(0,1) activations: every output row is NaN, +inf, -inf or
    finite exactly where the reference's f16 arithmetic makes it so, and the finite rows meet the usual bar."""
    M, K = 4096, 2560
    rng = np.random.default_rng(4700)
    w = (rng.standard_normal((M, K)) * 0.02).astype(np.float32)
    w[7, 64:96] = 0.0            # a row whose weights are zero where an infinity sits: 0 * inf = NaN
    buf = oracle.q8_quantize_h(w)
    codes = buf[:M * K].view(np.int8).reshape(M, K)
    scales = buf[(M * K + 255) // 256 * 256:][:M * K // 32 * 2].view(np.float16).reshape(M, K // 32)
    wv = oracle.q8_dequantize_h(buf, M * K).astype(np.float32).reshape(M, K)
    w_t = Tensor.from_quantized(buf, Q8H, (M, K), gpu)
    w2_t, w2v = make_lhs(Q8H, (M, M), np.random.default_rng(4701), 0.02)
    w2_t = w2_t.to(gpu)
    cases = {
        "outlier": [(100, 60000.0)],
        "nan": [(5, np.nan)],
        "pos_inf": [(70, np.inf)],
        "two_inf_one_block": [(64, np.inf), (65, -np.inf)],
        "inf_and_nan_far_apart": [(33, -np.inf), (2000, np.nan)],
    }
    for name, edits in cases.items():
        x = rng.standard_normal(K).astype(np.float16)
        for pos, val in edits:
            x[pos] = np.float16(val)
        xd = Tensor.from_data(x, gpu)
        y1 = w_t.gemm(xd, None, False, True, True)
        if as_list:
            y2 = w2_t.gemm(y1, None, False, True, True)
            y2.resolve()
            exe = rb.Executable(gpu, [y1, y2])
            assert exe.kernel.startswith("q8_gemv_chain"), exe.kernel
            y1.write(np.zeros(M, dtype=np.float16))
            exe.dispatch()
            gpu.sync()
        else:
            y1.resolve()
        got = y1.to(Device.CPU).to_numpy().reshape(-1).astype(np.float32)
        want = _reference_gemv_f16(codes, scales, x)
        for kind, f in (("nan", np.isnan), ("+inf", np.isposinf), ("-inf", np.isneginf)):
            assert np.array_equal(f(got), f(want)), (name, kind, int(f(got).sum()), int(f(want).sum()))
        fin = np.isfinite(want)
        if fin.any():
            truth = oracle.matmul_truth(wv, x.astype(np.float32), None, 1, 1, 1, M, 1, K, False, True, True)
            assert oracle.rel_l2(got[fin], oracle.f64_to_f16(truth).astype(np.float32)[fin]) <= TOL[F16], name
        if as_list:
            # the second node reads the first one's rows: whatever is not finite there spreads the same way
            got2 = y2.to(Device.CPU).to_numpy().reshape(-1).astype(np.float32)
            codes2 = w2_t.to(Device.CPU).to_numpy()[:M * M].view(np.int8).reshape(M, M)
            scales2 = w2_t.to(Device.CPU).to_numpy()[(M * M + 255) // 256 * 256:][:M * M // 32 * 2].view(np.float16).reshape(M, M // 32)
            want2 = _reference_gemv_f16(codes2, scales2, y1.to(Device.CPU).to_numpy().reshape(-1))
            for kind, f in (("nan", np.isnan), ("+inf", np.isposinf), ("-inf", np.isneginf)):
                assert np.array_equal(f(got2), f(want2)), (name, "node 2", kind)


def test_q8_gemv_chain_is_deterministic(gpu):
    """Same input, same bits, dispatch after dispatch: the CTAs hand rows on through polled words and K slices
    meet in a fixed order, so nothing may depend on which CTA is early."""
    shapes = [(10240, 2560), (2560, 10240), (10240, 2560), (2560, 10240), (10240, 2560), (2560, 10240)]
    x_dev, nodes, host = _decode_chain(gpu, shapes, 4600, [True, False, False, True, False, False])
    nodes[-1].resolve()
    exe = rb.Executable(gpu, nodes, use_graph=True)
    assert exe.kernel.startswith("q8_gemv_chain"), exe.kernel
    exe.dispatch()
    gpu.sync()
    first = [n.to(Device.CPU).to_numpy().reshape(-1).copy() for n in nodes]
    for trial in range(12):
        for _ in range(25):
            exe.dispatch()
        gpu.sync()
        for i, n in enumerate(nodes):
            got = n.to(Device.CPU).to_numpy().reshape(-1)
            assert np.array_equal(got.view(np.uint16), first[i].view(np.uint16)), f"dispatch {25 * (trial + 1)}: node {i} changed"


def test_q8_gemv_chain_tag_wraps(gpu, monkeypatch):
    """The dispatch tag is 16 bits wide: dispatches across the wrap from 65535 to 1 stay correct."""
    shapes = [(2560, 2560), (2560, 2560)]
    x_dev, nodes, host = _decode_chain(gpu, shapes, 4400, [False, False])
    nodes[-1].resolve()
    monkeypatch.setenv("RT_CHAIN_TAG_START", "65532")
    exe = rb.Executable(gpu, nodes, use_graph=True)
    assert exe.kernel.startswith("q8_gemv_chain"), exe.kernel
    for trial in range(8):
        x = np.random.default_rng(4500 + trial).standard_normal(shapes[0][1]).astype(np.float16)
        x_dev.write(x)
        exe.dispatch()
        gpu.sync()
        h = x.astype(np.float32)
        for i, (w_vals, b_vals, epi) in enumerate(host):
            M, K = shapes[i]
            got = nodes[i].to(Device.CPU).to_numpy().reshape(-1)
            truth = oracle.matmul_truth(w_vals, h, b_vals, 1, 1, 1, M, 1, K, False, True, True, epi)
            assert oracle.rel_l2(got.astype(np.float32), oracle.f64_to_f16(truth).astype(np.float32)) <= TOL[F16], (trial, i)
            h = got.astype(np.float32)


def test_q8_gemv_chain_bounded_wait_runs_out_and_the_next_dispatch_is_right(gpu, monkeypatch):
    """A wait that can never be satisfied: one dispatch publishes its rows under a tag no reader waits for, with the
    readers' budget cut to about a millisecond.  The kernel must come back by itself (nothing faults or spins on),
    the next synchronisation must name the failure, and the dispatch after that must be correct again."""
    shapes = [(2560, 2560), (2560, 2560), (2560, 2560)]
    x_dev, nodes, host = _decode_chain(gpu, shapes, 4800, [False, False, False])
    nodes[-1].resolve()
    monkeypatch.setenv("RT_CHAIN_WAIT_CYCLES", "2000000")
    monkeypatch.setenv("RT_CHAIN_TEST_WRONG_TAG", "1")
    exe = rb.Executable(gpu, nodes, use_graph=True)
    assert exe.kernel.startswith("q8_gemv_chain"), exe.kernel
    exe.dispatch()
    with pytest.raises(rb.RatchetError) as err:
        gpu.sync()
    assert err.value.status == rb._lib.RT_ERR_CUDA and "gave up a bounded wait" in str(err.value)
    gpu.sync()  # the flag was taken: the device is usable
    x = np.random.default_rng(4801).standard_normal(shapes[0][1]).astype(np.float16)
    x_dev.write(x)
    exe.dispatch()
    gpu.sync()
    h = x.astype(np.float32)
    for i, (w_vals, b_vals, epi) in enumerate(host):
        M, K = shapes[i]
        got = nodes[i].to(Device.CPU).to_numpy().reshape(-1)
        truth = oracle.matmul_truth(w_vals, h, b_vals, 1, 1, 1, M, 1, K, False, True, True, epi)
        assert oracle.rel_l2(got.astype(np.float32), oracle.f64_to_f16(truth).astype(np.float32)) <= TOL[F16], i
        h = got.astype(np.float32)


def test_q8_gemv_shapes_and_forms(gpu):
    for N, K in [(16, 32), (15, 64), (17, 96), (33, 2560), (1000, 352), (4096, 4096), (7, 8192)]:
        check_problem(Problem(Q8H, F16, (N, K), (1, K), (False, True, True), bias=True, seed=N + K, w_std=0.05), gpu)
    # non-transposed vector [K,1] and no trans_out: out [N,1]
    check_problem(Problem(Q8H, F16, (64, 256), (256, 1), (False, False, False), seed=51, w_std=0.05), gpu)
    # batched vectors against one weight (the reference's GEMV does not broadcast W; GEMMSpec does)
    check_problem(Problem(Q8H, F16, (96, 128), (3, 1, 128), (False, True, True), bias=True, seed=52, w_std=0.05), gpu)
    # batched weights
    check_problem(Problem(Q8H, F16, (3, 96, 128), (3, 1, 128), (False, True, True), seed=53, w_std=0.05), gpu)
    # fused GELU epilogue
    check_problem(Problem(Q8H, F16, (512, 1024), (1, 1024), (False, True, True), bias=True, epilogue=1, seed=54, w_std=0.05), gpu)


@pytest.mark.parametrize("nv", [2, 3, 5, 8])
def test_q8_skinny_gemm_streams_weights_once(gpu, nv):
    for to in (True, False):
        _, kernel = check_problem(Problem(Q8H, F16, (1000, 2560), (1, nv, 2560), (False, True, to), bias=True,
                                          seed=60 + nv, w_std=0.02), gpu)
        assert f"nv{nv}" in kernel


# ----------------------------------------------------------------------------- Q8_0 GEMM (prefill)

def test_q8_gemm_whisper_mlp_chain(gpu):
    """The Whisper-tiny encoder MLP: A f16 [1,1500,384] -> Q8_0 [1536,384] + b -> GELU -> Q8_0 [384,1536] + b."""
    rng = np.random.default_rng(103)
    w1_t, w1 = make_lhs(Q8H, (1536, 384), np.random.default_rng(1103), 0.02)
    w2_t, w2 = make_lhs(Q8H, (384, 1536), np.random.default_rng(1104), 0.02)
    b1 = round_to(F16, np.random.default_rng(2103).standard_normal(1536) * 0.02)
    b2 = round_to(F16, np.random.default_rng(2104).standard_normal(384) * 0.02)
    x = round_to(F16, rng.standard_normal((1, 1500, 384)))
    fc1 = Linear(w1_t.to(gpu), Tensor.from_data(b1, gpu, F16), epilogue=rb.EPILOGUE_GELU_TANH)
    fc2 = Linear(w2_t.to(gpu), Tensor.from_data(b2, gpu, F16))
    y = fc2.schedule(fc1.schedule(Tensor.from_data(x, gpu, F16))).resolve().to(Device.CPU)
    assert y.shape == [1, 1500, 384] and y.dt == F16
    # oracle: hidden rounded to f16 between the two GEMMs, as the reference's graph does
    h = oracle.matmul_truth(w1, x, b1, 1, 1, 1, 1536, 1500, 384, False, True, True, 1)
    h16 = oracle.f64_to_f16(h).astype(np.float32)
    t = oracle.matmul_truth(w2, h16, b2, 1, 1, 1, 384, 1500, 1536, False, True, True, 0)
    assert oracle.rel_l2(y.to_f32().reshape(-1), oracle.f64_to_f16(t).astype(np.float32)) <= 1e-3
    # and against the shader-faithful chain
    hf = oracle.matmul_faithful(w1, x, b1, 1, 1, 1, 1536, 1500, 384, False, True, True, 1, "f16")
    tf = oracle.matmul_faithful(w2, hf, b2, 1, 1, 1, 384, 1500, 1536, False, True, True, 0, "f16")
    assert oracle.rel_l2(y.to_f32().reshape(-1), tf) <= 2e-3


def test_q8_gemm_forms(gpu):
    for (N, K, M) in [(64, 32, 9), (100, 96, 33), (1536, 384, 200), (257, 512, 129)]:
        check_problem(Problem(Q8H, F16, (N, K), (2, M, K), (False, True, True), bias=True, seed=N + M, w_std=0.03), gpu)
        check_problem(Problem(Q8H, F16, (N, K), (K, M), (False, False, False), seed=N + M + 1, w_std=0.03), gpu)
    check_problem(Problem(Q8F, F32, (128, 256), (3, 50, 256), (False, True, True), bias=True, seed=71, w_std=0.03), gpu)
    check_problem(Problem(Q8H, BF16, (320, 256), (2, 70, 256), (False, True, True), bias=True, epilogue=1, seed=72,
                          w_std=0.03, bias_dt=F16), gpu)


@pytest.mark.parametrize("wshape,xshape,bias,epi", [
    ((1536, 384), (1, 1500, 384), True, 1),      # Whisper fc1 in the reference's default dtypes
    ((10240, 2560), (1, 128, 2560), True, 0),    # Phi-2 fc1, 128 rows
    ((520, 352), (3, 33, 352), False, 0),        # ragged, batched rows over one weight
])
def test_q8f_f32_prefill_takes_the_tf32x3_gemm(gpu, wshape, xshape, bias, epi):
    """The reference's default pair (Q8_0F weights, f32 activations; dtype/mod.rs:77-83) in the Linear form: weights
    dequantised to f32 as (i8)q * d (quant.rs:114-120), then the 3 x TF32 tensor-core GEMM; the f32 bar holds."""
    err, kernel = check_problem(Problem(Q8F, F32, wshape, xshape, (False, True, True), bias=bias, epilogue=epi, seed=wshape[0] + xshape[1],
                                        w_std=0.02), gpu)
    assert kernel.startswith("gemm_umma_tf32x3_Q8_0F_F32") and "dequant_prepass" in kernel, kernel
    assert err <= 1e-5
    # as an executable with the weight flagged constant: the f32 copy is kept, dispatch after dispatch gives the same bits
    w_t, _ = make_lhs(Q8F, wshape, np.random.default_rng(9), 0.02)
    x = Tensor.from_data(np.random.default_rng(10).standard_normal(xshape).astype(np.float32), gpu, F32)
    node = w_t.to(gpu).gemm(x, None, False, True, True)
    first = node.resolve().to(Device.CPU).to_numpy().copy()
    exe = rb.Executable(gpu, [node])
    node.write(np.zeros(node.numel(), dtype=np.float32))
    exe.dispatch()
    exe.dispatch()
    gpu.sync()
    assert np.array_equal(node.to(Device.CPU).to_numpy(), first)


def test_dense_f32_phi2_fc1(gpu):
    """Dense f32 Phi-2 fc1 prefill: A f32 [1,128,2560], W f32 [10240,2560] N(0,0.02) rhs-transposed, b f32."""
    err, kernel = check_problem(Problem(F32, F32, (10240, 2560), (1, 128, 2560), (False, True, True), bias=True, seed=101,
                                        w_std=0.02), gpu)
    assert kernel.startswith("gemm_umma_tf32x3"), kernel
    assert err <= 1e-5


# ----------------------------------------------------------------------------- Q4_K

@pytest.mark.parametrize("M", [1, 16, 512])
def test_q4k_phi3_shapes(gpu, M):
    """The Phi-3 shaped Q4_K projection: W Q4_K [8192,3072] from N(0,0.02), x f16 [M,3072], out f16 [M,8192]."""
    check_problem(Problem(Q4K, F16, (8192, 3072), (1, M, 3072), (False, True, True), seed=104, w_std=0.02), gpu)


def test_q4k_gemv_shapes_and_vectors(gpu, monkeypatch):
    """The streaming Q4_K kernel: ragged rows, K slices over a cluster, 1..16 activation vectors, both output orders."""
    monkeypatch.setenv("RT_Q4K_UMMA", "0")
    for N, K in [(16, 256), (37, 512), (1000, 1024), (3072, 8192), (5, 4096)]:
        _, kernel = check_problem(Problem(Q4K, F16, (N, K), (1, K), (False, True, True), bias=True, seed=N + K, w_std=0.02), gpu)
        assert kernel.startswith("q4k_gemv_mma"), kernel
    for nv in (2, 7, 8, 9, 16):
        for to in (True, False):
            _, kernel = check_problem(Problem(Q4K, F16, (520, 1536), (1, nv, 1536), (False, True, to), bias=True, epilogue=1,
                                              seed=90 + nv, w_std=0.02), gpu)
            assert f"nv{nv}" in kernel, kernel
    check_problem(Problem(Q4K, F16, (3, 64, 512), (3, 1, 512), (False, True, True), seed=91, w_std=0.02), gpu)  # batched weights
    check_problem(Problem(Q4K, F16, (64, 512), (4, 1, 512), (False, True, True), seed=92, w_std=0.02), gpu)     # broadcast weight


def test_q4k_skinny_gemm_walks_row_groups(gpu, monkeypatch):
    """More row groups than SMs and 2..16 vectors: a CTA keeps the activations and walks several row
    groups (two at a time, one per half of its warps).  Ragged last group, a last CTA with fewer
    groups, both output orders, bias + GELU, K split over a cluster, batched weights."""
    monkeypatch.setenv("RT_Q4K_UMMA", "0")
    for nv in (2, 5, 8, 9, 16):
        for to in (True, False):
            _, kernel = check_problem(Problem(Q4K, F16, (2405, 768), (1, nv, 768), (False, True, to), bias=True, epilogue=1,
                                              seed=190 + nv, w_std=0.02), gpu)
            assert f"nv{nv}_split1_walk2" in kernel, kernel
    _, kernel = check_problem(Problem(Q4K, F16, (4100, 8192), (1, 16, 8192), (False, True, True), seed=196, w_std=0.02), gpu)
    assert "nv16_split4_walk7" in kernel, kernel
    _, kernel = check_problem(Problem(Q4K, F16, (3, 2405, 512), (3, 4, 512), (False, True, True), bias=True, seed=197, w_std=0.02), gpu)
    assert "walk4" in kernel, kernel
    _, kernel = check_problem(Problem(Q4K, F16, (8192, 3072), (1, 8, 3072), (False, True, True), seed=198, w_std=0.02), gpu)
    assert "nv8_split1_walk4x4buf" in kernel, kernel


@pytest.mark.parametrize("wshape,nv,name", [
    ((8192, 3072), 1, "nv1_rb111_split2"),     # Phi-3 decode: 74 clusters of two CTAs, 111 rows each
    ((8192, 3072), 16, "nv16_rb111_split2"),
    ((3072, 8192), 1, "nv1_rb84_split4"),      # the down projection: K = 8192 over clusters of four
    ((3072, 8192), 5, "nv5_rb84_split4"),
    ((16384, 3072), 3, "nv3_rb111_split1"),    # more rows than 148 x 111: one CTA per cluster
    ((8191, 1024), 8, "nv8_"),                 # ragged last cluster
    ((5000, 2048), 9, "nv9_"),
    ((4100, 8192), 16, "nv16_"),
])
def test_q4k_gemv_through_tensor_memory(gpu, monkeypatch, wshape, nv, name):
    """Q4_K weights of a size that fills the machine (opt-in route, RT_Q4K_UMMA=1): raw super-blocks by TMA, nibbles to
    int8 codes in shared memory, tcgen05.mma against the activations' digits.  1..16 vectors, both output orders, bias
    and GELU."""
    monkeypatch.setenv("RT_Q4K_UMMA", "1")
    for to in ((True, False) if nv > 1 else (True,)):
        _, kernel = check_problem(Problem(Q4K, F16, wshape, (1, nv, wshape[1]), (False, True, to), bias=True, epilogue=nv % 2,
                                          seed=300 + nv + wshape[0], w_std=0.02), gpu)
        assert kernel.startswith("q4k_gemv_umma") and name in kernel, kernel
    if nv == 1:  # the vector form of the reference's GEMV call: rhs [K], no transposes
        _, kernel = check_problem(Problem(Q4K, F16, wshape, (wshape[1],), (False, False, False), seed=77, w_std=0.02), gpu)
        assert kernel.startswith("q4k_gemv_umma"), kernel


def test_q4k_gemv_through_tensor_memory_matches_the_streaming_kernel_and_propagates_nan(gpu, monkeypatch):
    """Same weights, same activations through both Q4_K kernels: within the bar of each other on finite inputs; a NaN
    and infinities in the activations come out as IEEE arithmetic on the decoded weights gives them (0 * inf and
    inf - inf are NaN, anything else with an infinity is that infinity)."""
    M, K, nv = 8192, 3072, 4
    monkeypatch.setenv("RT_Q4K_UMMA", "1")
    w_t, wv = make_lhs(Q4K, (M, K), np.random.default_rng(411), 0.02)
    x = round_to(F16, np.random.default_rng(412).standard_normal((nv, K)).astype(np.float32))
    x[0, 5], x[1, 700], x[1, 701], x[2, 3000] = np.nan, np.inf, -np.inf, np.inf  # vector 3 stays finite
    w_d, x_d = w_t.to(gpu), Tensor.from_data(x, gpu, F16)
    node = w_d.gemm(x_d, None, False, True, True)
    assert rb._lib.load().rt_plan_kernel(gpu.plan_for(node.op.desc)).decode().startswith("q4k_gemv_umma")
    y_new = node.resolve().to(Device.CPU).to_f32().reshape(nv, M)
    with np.errstate(invalid="ignore"):
        want = (wv.astype(np.float64) @ x.astype(np.float64).T).T  # [nv][M]
    assert np.array_equal(np.isnan(y_new), np.isnan(want))
    assert np.all(np.isnan(y_new[0])) and np.isnan(y_new[1]).sum() > M // 4 and np.isinf(y_new[2]).sum() > M // 2
    inf = np.isinf(want)
    assert np.array_equal(np.isinf(y_new), inf) and np.array_equal(np.sign(y_new[inf]), np.sign(want[inf]))
    fin = np.isfinite(want)
    assert oracle.rel_l2(y_new[fin], oracle.f64_to_f16(want[fin]).astype(np.float32)) <= TOL[F16]
    monkeypatch.setenv("RT_Q4K_UMMA", "0")
    node_old = w_d.gemm(x_d, None, False, True, True)
    assert rb._lib.load().rt_plan_kernel(gpu.plan_for(node_old.op.desc)).decode().startswith("q4k_gemv_mma")
    y_old = node_old.resolve().to(Device.CPU).to_f32().reshape(nv, M)
    assert oracle.rel_l2(y_new[3], y_old[3]) <= 2e-3


def test_q4k_forms(gpu):
    check_problem(Problem(Q4K, F16, (40, 256), (1, 256), (False, True, True), bias=True, seed=81, w_std=0.02), gpu)
    check_problem(Problem(Q4K, F16, (2, 33, 512), (2, 512, 7), (False, False, False), seed=82, w_std=0.02), gpu)
    check_problem(Problem(Q4K, BF16, (64, 768), (5, 768), (False, True, True), bias=True, seed=83, w_std=0.02), gpu)


# ----------------------------------------------------------------------------- bf16 prefill at reduced rows

def test_q8_bf16_prefill_row_slice(gpu):
    """A slice of the rows of the bf16 prefill Linear: A bf16 [1,256,2560], W Q8_0H [10240,2560], f16 bias, GELU."""
    check_problem(Problem(Q8H, BF16, (10240, 2560), (1, 256, 2560), (False, True, True), bias=True, epilogue=1,
                          seed=105, w_std=0.02, bias_dt=F16), gpu)


# ----------------------------------------------------------------------------- tensor-core GEMM (tcgen05)

def test_umma_dense_forms(gpu):
    """Both operands K-major (the nn::Linear form), f16 and bf16, ragged extents, both output orders."""
    for dt in (F16, BF16):
        for to in (True, False):
            _, kernel = check_problem(Problem(dt, dt, (300, 520), (2, 700, 520), (False, True, to), bias=True,
                                              seed=201, w_std=0.05), gpu)
            assert kernel.startswith("gemm_umma"), kernel
    # batched weights, K with a tail below one 64-wide step, N not a multiple of 8 (scalar stores)
    _, kernel = check_problem(Problem(F16, F16, (3, 257, 200), (3, 190, 200), (False, True, True), seed=202, w_std=0.05), gpu)
    assert kernel.startswith("gemm_umma"), kernel
    _, kernel = check_problem(Problem(F16, F16, (513, 1024), (1, 130, 1024), (False, True, True), bias=True, epilogue=1,
                                      seed=203, w_std=0.03), gpu)
    assert kernel.startswith("gemm_umma"), kernel


def test_umma_tf32x3_dense_f32_forms(gpu):
    """Dense f32 on the tensor cores (three TF32 MMAs per product) must keep the f32 bar of 1e-5: ragged
    extents, K with a tail below one 32-wide step, both output orders, batches, bias, GELU."""
    cases = [
        Problem(F32, F32, (300, 520), (2, 700, 520), (False, True, True), bias=True, seed=301, w_std=0.05),
        Problem(F32, F32, (300, 520), (2, 700, 520), (False, True, False), bias=True, seed=302, w_std=0.05),
        Problem(F32, F32, (3, 257, 204), (3, 190, 204), (False, True, True), seed=303, w_std=0.05),
        Problem(F32, F32, (513, 1024), (1, 131, 1024), (False, True, True), bias=True, epilogue=1, seed=304, w_std=0.03),
        Problem(F32, F32, (1024, 4096), (1, 256, 4096), (False, True, True), seed=305, w_std=1.0),  # long sums, large values
    ]
    for p in cases:
        err, kernel = check_problem(p, gpu)
        assert kernel.startswith("gemm_umma_tf32x3"), kernel
        assert err <= 1e-5, (kernel, err)


@pytest.mark.parametrize("w_rows,x_rows,name", [
    (128, 18944, "bn128"), (96, 18944, "bn96"), (80, 18944, "bn80"), (40, 500, "bn64"),  # one tile column: split in the GEMM
    (256, 9472, "bn128_presplit"), (192, 9472, "bn96_presplit"), (10240, 128, "bn80_presplit"), (300, 1400, "bn64_presplit"),
])
def test_umma_tf32x3_tile_widths(gpu, w_rows, x_rows, name):
    """Every tile width of the f32 tensor-core GEMM, with the activations split inside the GEMM (one tile
    column) and by the pass ahead of it (several)."""
    err, kernel = check_problem(Problem(F32, F32, (w_rows, 328), (1, x_rows, 328), (False, True, True), bias=True,
                                        seed=310 + w_rows % 97, w_std=0.05), gpu)
    assert kernel == "gemm_umma_tf32x3_F32_F32_" + name, kernel
    assert err <= 1e-5, (kernel, err)


def test_attention_products_take_the_tensor_core_gemm(gpu):
    """q.kT and softmax.v of the models: rank 4, no transposes, rhs stored [K][N].  A transposing pass makes
    the rhs K-major for the tensor-core GEMMs (16-bit operands whose K is not a multiple of 8 are zero-padded on the way)."""
    nn = (False, False, False)
    cases = [
        (Problem(F16, F16, (1, 32, 1, 1024), (1, 32, 1024, 80), nn, seed=401), "rowvec_mat_F16", "_ksplit10"),               # decode, values: k rows split
        (Problem(F32, F32, (1, 1, 1000), (3, 1000, 50), nn, bias=True, seed=417), "rowvec_mat_F32", "_ksplit15"),           # ragged chunks, broadcast lhs
        (Problem(F16, F16, (1, 32, 1, 80), (1, 32, 80, 1024), nn, seed=415), "rowvec_mat_F16", ""),                          # decode, scores: one row
        (Problem(F16, F16, (1, 32, 16, 1024), (1, 32, 1024, 80), nn, seed=412), "gemm_umma_F16_F16", "_rhs_transposed"),     # 16 rows, values
        (Problem(F16, F16, (1, 32, 512, 512), (1, 32, 512, 80), nn, seed=402), "gemm_umma_F16_F16", "_rhs_transposed"),      # prefill, values
        (Problem(BF16, BF16, (2, 4, 100, 64), (2, 4, 64, 72), nn, seed=403), "gemm_umma_BF16_BF16", "_rhs_transposed"),
        (Problem(F32, F32, (1, 32, 512, 80), (1, 32, 80, 512), nn, seed=404), "gemm_umma_tf32x3", "_rhs_transposed"),        # prefill, scores
        (Problem(F16, F16, (3, 300, 96), (1, 96, 200), nn, bias=True, seed=405), "gemm_umma_F16_F16", "_rhs_transposed"),      # broadcast rhs, bias
        (Problem(F32, F32, (1, 32, 1, 80), (1, 32, 80, 1024), nn, seed=406), "rowvec_mat_F32", ""),                          # decode scores in f32: one row
        (Problem(BF16, BF16, (3, 1, 77), (1, 77, 131), nn, bias=True, epilogue=1, seed=413), "rowvec_mat_BF16", ""),          # odd N, broadcast rhs, bias + GELU
        (Problem(F32, F32, (77,), (77, 260), nn, bias=True, seed=416), "rowvec_mat_F32", ""),                               # vector lhs
        (Problem(F32, F32, (2, 5, 8, 80), (2, 5, 80, 256), nn, seed=414), "gemm_simt", ""),                                  # f32 below 16 rows
        (Problem(F16, F16, (1, 6, 300, 64), (1, 6, 64, 300), nn, seed=407), "gemm_umma_F16_F16", "_rhs_transposed"),         # rows of 300: element stores
        (Problem(BF16, BF16, (1, 2, 130, 64), (1, 2, 64, 1501), nn, bias=True, seed=409), "gemm_umma_BF16_BF16", "_rhs_transposed"),  # odd row length
        (Problem(F16, F16, (1, 6, 64, 300), (1, 6, 300, 64), nn, seed=408), "gemm_umma_F16_F16", "_rhs_transposed_kpad304"),  # K % 8 != 0: zero-padded
        (Problem(BF16, BF16, (2, 3, 200, 1501), (2, 3, 1501, 64), nn, bias=True, seed=410), "gemm_umma_BF16_BF16", "_kpad1504"),    # odd K
        (Problem(F32, F32, (1, 6, 64, 302), (1, 6, 302, 64), nn, seed=411), "gemm_simt", ""),                                # f32: K % 4 != 0
        (Problem(F16, F16, (1, 4, 300, 12), (1, 4, 12, 601), nn, bias=True, seed=418), "gemm_umma_F16_F16", "_kpad16"),      # K below one tile step, odd N
        (Problem(F16, F16, (2, 129, 8), (2, 8, 1024), nn, seed=419), "gemm_umma_F16_F16", "_rhs_transposed"),               # K = 8
    ]
    for prob, prefix, suffix in cases:
        _, kernel = check_problem(prob, gpu)
        assert kernel.startswith(prefix) and kernel.endswith(suffix), (prob, kernel)


def test_short_prompts_take_the_tensor_core_gemm(gpu):
    """9..15 activation rows (more than the streaming GEMV kernels take, fewer than one MMA column
    block): the tensor-core GEMM with the missing rows zero-filled by the tile loads."""
    for nv in (9, 15):
        for lhs, dt in ((Q8H, F16), (F16, F16), (BF16, BF16), (F32, F32)):
            for to in (True, False):
                _, kernel = check_problem(Problem(lhs, dt, (1000, 512), (1, nv, 512), (False, True, to), bias=True,
                                                  epilogue=0 if dt == F32 else 1, seed=200 + nv, w_std=0.02), gpu)
                if lhs == Q8H and to:  # the Linear form: one pass of the streaming kernel, two groups of eight MMA columns
                    assert kernel.startswith(f"q8_gemv_mma_h_nv{nv}_"), kernel
                else:
                    assert kernel.startswith("gemm_umma"), kernel
    # the same at a decode shape, with bias and GELU, f32 scales too
    for lhs in (Q8H, Q8F):
        for nv in (9, 12, 16, 17, 24):
            _, kernel = check_problem(Problem(lhs, F16, (10240, 2560), (1, nv, 2560), (False, True, True), bias=True, epilogue=1,
                                              seed=230 + nv, w_std=0.02), gpu)
            assert (f"_nv{nv}_" if nv <= 16 else f"_nv16+{nv - 16}_") in kernel, kernel  # 17..24: a pass of 16, then the rest


def test_skinny_q8_routes_by_vectors_and_weight_size(gpu):
    """9..16 vectors: one pass of the streaming kernel; 17..24: a pass of 16 and a pass of the rest, except against
    weights of 32 Mi values or more, where two passes cost more than the tensor-core GEMM."""
    lib = rb._lib.load()
    for (wshape, nv, want) in [((16384, 3072), 16, "q8_gemv_mma_h_nv16_"), ((16384, 3072), 17, "gemm_umma_Q8_0H_F16"),
                               ((10240, 2560), 24, "q8_gemv_mma_h_nv16+8_"), ((3072, 8192), 20, "q8_gemv_mma_h_nv16+4_")]:
        _, kernel = check_problem(Problem(Q8H, F16, wshape, (1, nv, wshape[1]), (False, True, True), bias=True, seed=nv, w_std=0.02), gpu)
        assert kernel.startswith(want), kernel


def test_umma_takes_the_prefill_configs(gpu):
    lib = rb._lib.load()
    for lhs_dt, act, wshape, xshape in [(Q8H, F16, (1536, 384), (1, 1500, 384)), (Q8H, F16, (384, 1536), (1, 1500, 1536)),
                                        (Q4K, F16, (8192, 3072), (1, 512, 3072)), (Q8H, BF16, (10240, 2560), (4, 2048, 2560))]:
        w = Tensor(list(wshape), lhs_dt, gpu)
        x = Tensor(list(xshape), act, gpu)
        node = w.gemm(x, None, False, True, True)
        assert lib.rt_plan_kernel(gpu.plan_for(node.op.desc)).decode().startswith("gemm_umma"), (lhs_dt, wshape)


@pytest.mark.parametrize("lhs_dt,act,wshape,xshape,bias,epi", [
    (Q8H, F16, (5120, 512), (1, 2048, 512), True, 1),      # 8 x 20 tiles of 256 x 256
    (F16, F16, (5000, 256), (2, 1000, 256), True, 0),      # ragged rows and columns, two batches over one weight
    (BF16, BF16, (4096, 320), (1, 2560, 320), False, 1),   # K = 5 blocks of 64
    (Q8H, BF16, (10240, 512), (1, 1030, 512), True, 1),    # rows that end in a pair's first CTA
    (Q4K, F16, (8192, 512), (1, 1200, 512), False, 0),
    (F16, F16, (3, 2048, 256), (3, 1000, 256), False, 0),  # a weight per batch: three stacks of ragged row tiles
])
def test_gemm_on_cta_pairs_matches_the_oracle_and_the_single_cta_kernel(gpu, monkeypatch, lhs_dt, act, wshape, xshape, bias, epi):
    """Large GEMMs run 256 x 256 tiles on pairs of CTAs (tcgen05 cta_group::2: each CTA stages its 128 rows of the
    activations and half of the tile's weight rows): the result meets the bar against the oracle on sampled rows and
    has the bits of the one-CTA kernel (same products, same order of the K blocks)."""
    rng = np.random.default_rng(sum(wshape) + sum(xshape))
    w_t, wv = make_lhs(lhs_dt, wshape, np.random.default_rng(5 + wshape[0]), 0.05)
    x = round_to(act, rng.standard_normal(xshape).astype(np.float32))
    bdt = F16 if act == BF16 else act
    b = round_to(bdt, rng.standard_normal(wshape[0]).astype(np.float32) * 0.1) if bias else None
    w_d, x_d = w_t.to(gpu), Tensor.from_data(x, gpu, act)
    b_d = Tensor.from_data(b, gpu, bdt) if bias else None
    node = w_d.gemm(x_d, b_d, False, True, True, epilogue=epi)
    assert "pair256x256" in rb._lib.load().rt_plan_kernel(gpu.plan_for(node.op.desc)).decode()
    got = node.resolve().to(Device.CPU)
    monkeypatch.setenv("RT_GEMM_PAIR", "0")
    node1 = w_d.gemm(x_d, b_d, False, True, True, epilogue=epi)
    assert "pair" not in rb._lib.load().rt_plan_kernel(gpu.plan_for(node1.op.desc)).decode()
    assert np.array_equal(got.to_numpy().reshape(-1), node1.resolve().to(Device.CPU).to_numpy().reshape(-1))
    if len(wshape) == 3:  # batched weights: check batch 1 against its own weight
        N, K = wshape[1:]
        rows_total = xshape[1]
        got_f = got.to_f32().reshape(wshape[0], rows_total, N)[1]
        rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, rows_total - 1], np.random.default_rng(1).integers(0, rows_total, size=40)]))
        truth = oracle.matmul_truth(wv[1], x[1][rows], None, 1, 1, 1, N, len(rows), K, False, True, True, epi)
        assert oracle.rel_l2(got_f[rows], oracle.f64_to_f16(truth).astype(np.float32).reshape(len(rows), N)) <= TOL[act]
        return
    N, K = wshape
    rows_total = int(np.prod(xshape[:-1]))
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, rows_total - 1], np.random.default_rng(1).integers(0, rows_total, size=40)]))
    truth = oracle.matmul_truth(wv, x.reshape(rows_total, K)[rows], b, 1, 1, 1, N, len(rows), K, False, True, True, epi)
    truth_r = (oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(truth)) if act == BF16 else oracle.f64_to_f16(truth).astype(np.float32))
    assert oracle.rel_l2(got.to_f32().reshape(rows_total, N)[rows], truth_r.reshape(len(rows), N)) <= TOL[act]


@pytest.mark.parametrize("N,K,rows,widths,kernel_part", [
    (10240, 512, 1536, [3424, 3408, 3408], "pair256x256"),   # windows that end inside a 64-column block: the TMA stores clip
    (768, 256, 200, [272, 256, 240], "bn"),                   # the one-CTA kernel's scatter
])
def test_scattered_outputs_on_one_gpu(gpu, N, K, rows, widths, kernel_part):
    """The N-sharded prefill form with every shard on ONE GPU: each shard's GEMM writes its column window into TWO
    full-width output buffers (rt_matmul_launch_ex with n_out = 2, the peer-store epilogue with local "peers").  Both
    buffers end up holding the unsharded Linear's result, bit for bit, and nothing outside a window is touched."""
    from ctypes import byref
    lib = rb._lib.load()
    w_t, wv = make_lhs(Q8H, (N, K), np.random.default_rng(31), 0.03)
    b = round_to(F16, np.random.default_rng(32).standard_normal(N).astype(np.float32) * 0.1)
    x = round_to(BF16, np.random.default_rng(33).standard_normal((rows, K)).astype(np.float32))
    x_d = Tensor.from_data(x, gpu, BF16)
    whole = w_t.to(gpu).gemm(x_d, Tensor.from_data(b, gpu, F16), False, True, True, epilogue=rb.EPILOGUE_GELU_TANH)
    want = whole.resolve().to(Device.CPU).to_numpy().reshape(rows, N)
    outs = [Tensor([rows, N], BF16, gpu, rb.GpuBuffer(gpu, rows * N * 2)) for _ in range(2)]
    for o in outs:
        o.write(np.full(rows * N, 0x7FC0, dtype=np.uint16))  # bf16 NaN: an unwritten element would show
    c0 = 0
    for wd in widths:
        shard = rb.shard_rows(w_t, c0, c0 + wd).to(gpu)
        bias = Tensor.from_data(np.ascontiguousarray(b[c0:c0 + wd]), gpu, F16)
        node = shard.gemm(x_d, bias, False, True, True, epilogue=rb.EPILOGUE_GELU_TANH)
        plan = gpu.plan_for(node.op.desc)
        assert kernel_part in lib.rt_plan_kernel(plan).decode(), lib.rt_plan_kernel(plan).decode()
        opts = rb._lib.rt_launch_opts()
        opts.flags, opts.n_out = rb._lib.RT_LAUNCH_LHS_CONSTANT, 2
        opts.outs[0], opts.outs[1] = outs[0].ptr, outs[1].ptr
        opts.out_ld, opts.out_col = N, c0
        rb._lib.check(lib.rt_matmul_launch_ex(plan, shard.ptr, x_d.ptr, bias.ptr, None, None, byref(opts)))
        c0 += wd
    gpu.sync()
    for o in outs:
        assert np.array_equal(o.to(Device.CPU).to_numpy().reshape(rows, N), want)


@pytest.mark.parametrize("M", [2048, 8192], ids=["4x2048", "4x8192"])
def test_q8_bf16_prefill_full_size_sampled(gpu, M):
    """The sharded prefill workload at full size on one GPU: A bf16 [4,M,2560], W Q8_0H [10240,2560], f16 bias,
    fused GELU, with M = 2048 and the long form M = 8192 (32768 rows).  The oracle finishes a sample of the output
    rows in seconds; every sampled row is compared."""
    B, K, N = 4, 2560, 10240
    w_t, wv = make_lhs(Q8H, (N, K), np.random.default_rng(1105), 0.02)
    x = round_to(BF16, np.random.default_rng(105).standard_normal((B, M, K)).astype(np.float32))
    bias = round_to(F16, np.random.default_rng(2105).standard_normal(N) * 0.02)
    y = w_t.to(gpu).gemm(Tensor.from_data(x, gpu, BF16), Tensor.from_data(bias, gpu, F16), False, True, True,
                         epilogue=rb.EPILOGUE_GELU_TANH).resolve().to(Device.CPU)
    assert y.shape == [B, M, N]
    got = y.to_f32().reshape(B * M, N)
    rows = np.random.default_rng(5).choice(B * M, size=48, replace=False)
    rows = np.concatenate([rows, [0, 127, 128, B * M - 1]])
    xs = x.reshape(B * M, K)[rows]
    truth = oracle.matmul_truth(wv, xs, bias, 1, 1, 1, N, len(rows), K, False, True, True, 1)
    truth_r = oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(truth)).reshape(len(rows), N)
    assert oracle.rel_l2(got[rows], truth_r) <= 1e-3
    # a checksum over everything else: column sums of the output against the sampled rows' scale
    assert np.all(np.isfinite(got))


def test_repeated_dispatch_is_bitwise_stable(gpu):
    """The kernels with scratch passes, walking CTAs or several issuers give the same bits on every dispatch:
    their reductions run in a fixed order and their scratch is rewritten each time."""
    rng = np.random.default_rng(77)
    cases = [
        (Q4K, F16, (8192, 3072), (1, 16, 3072), (False, True, True)),      # row-walking Q4_K kernel
        (Q8H, F16, (10240, 2560), (1, 12, 2560), (False, True, True)),     # two passes of the streaming kernel
        (F32, F32, (10240, 2560), (1, 128, 2560), (False, True, True)),    # pre-split + two issuers
        (F16, F16, (1, 6, 200, 1500), (1, 6, 1500, 64), (False, False, False)),  # transposed + K-padded
    ]
    for lhs_dt, act_dt, lsh, rsh, tr in cases:
        w, _ = make_lhs(lhs_dt, lsh, rng, 0.02)
        x = Tensor.from_data(rng.standard_normal(rsh).astype(np.float32), gpu, act_dt)
        y = w.to(gpu).gemm(x, None, *tr)
        y.resolve()
        exe = rb.Executable(gpu, [y])
        first = None
        for _ in range(25):
            exe.dispatch()
            gpu.sync()
            got = y.to(Device.CPU).storage.copy()
            if first is None:
                first = got
            assert np.array_equal(got, first), (lhs_dt, lsh)


# ----------------------------------------------------------------------------- a seeded sweep over the routing boundaries

@pytest.mark.parametrize("lhs_dt,act", [(Q8H, F16), (Q8F, F32), (Q8F, F16), (Q8H, BF16), (Q4K, F16), (Q4K, BF16), (F16, F16), (BF16, BF16), (F32, F32)])
def test_seeded_sweep_of_linear_forms_across_the_routing_boundaries(gpu, lhs_dt, act):
    """Row counts on both sides of every switch between kernels (1 | 2..8 | 9..24 | 25.. | whole 128- and 256-row tiles),
    weight rows that are no multiple of any tile, with and without bias and GELU, flattened batches; every case
    against the oracle at the activation type's tolerance, and every kernel name collected so that the sweep is known
    to have crossed the boundaries."""
    rng = np.random.default_rng(int(lhs_dt) * 31 + int(act))
    kstep = 256 if lhs_dt == Q4K else 32
    rows_pool = [1, 2, 3, 8, 9, 16, 17, 24, 25, 31, 32, 33, 100, 127, 128, 129, 255, 256, 257, 300, 513]
    seen = set()
    for case in range(len(rows_pool)):
        rows = rows_pool[case]
        N = int(rng.choice([8, 24, 40, 128, 136, 200, 520, 1000, 1544]))
        K = int(rng.integers(1, 9)) * kstep if case % 3 else int(rng.choice([1, 4, 10])) * 256
        batch = int(rng.choice([1, 1, 2, 3])) if rows <= 130 else 1
        bias = bool(rng.integers(0, 2))
        epi = int(rng.integers(0, 2)) if bias else 0
        bias_dt = F16 if (act == BF16 and lhs_dt != BF16) else None
        kw = dict(bias=bias, epilogue=epi, seed=1000 + case, w_std=0.03)
        if bias_dt is not None:
            kw["bias_dt"] = bias_dt
        prob = Problem(lhs_dt, act, (N, K), (batch, rows, K), (False, True, True), **kw)
        if lhs_dt == Q4K and act == BF16:
            # Q4_K weights are rounded to f16 for the tensor cores (2^-12 relative).  Against a truth that is itself
            # rounded to bf16 that shows as whole-ulp flips (2^-8 each) on a few percent of the elements, which puts
            # the rel-L2 of rounded against rounded near 9e-4 with a sample spread that crosses 1e-3 on small outputs.
            # The statement that does not depend on where the truth happens to fall between two bf16 values: the
            # result is as close to the exact product as the correctly rounded one is, within 10 %.
            got, truth_r, truth, _, kernel = run_problem(prob, gpu)
            assert np.all(np.isfinite(got))
            exact = truth.reshape(-1)
            assert oracle.rel_l2(got, exact) <= 1.10 * oracle.rel_l2(truth_r, exact), (kernel, prob)
            assert oracle.rel_l2(got, truth_r) <= 1.5e-3, (kernel, prob)
        else:
            _, kernel = check_problem(prob, gpu)
        seen.add(kernel.split("<")[0].split("(")[0])
    assert len(seen) >= 2, seen


# ----------------------------------------------------------------------------- bf16 activations outside f16's range

@pytest.mark.parametrize("lhs_dt", [Q8H, Q4K])
@pytest.mark.parametrize("trans_out", [True, False])
def test_bf16_activations_outside_the_f16_range_against_quantised_weights(gpu, lhs_dt, trans_out):
    """The tensor-core GEMM multiplies f16 weights by activations cast from bf16 to f16; the cast takes a power of two
    out of every activation row and the epilogue puts it back, so rows of any bf16 magnitude come out at the tolerance
    of ordinary ones, and infinities and NaNs arrive where the exact product has them."""
    N, K, rows = 264, 512, 70
    w_t, wv = make_lhs(lhs_dt, (N, K), np.random.default_rng(5), 0.03)
    rng = np.random.default_rng(6)
    x = rng.standard_normal((rows, K)).astype(np.float32)
    mags = {0: 1e6, 1: 3e38 / 16, 2: 1e-20, 3: 1e-33, 4: 70000.0, 5: 1.0}
    for r, m in mags.items():
        x[r] *= np.float32(m)
    x[6, :] = 0.0                     # a row of zeros: factor 1
    x[7, 10] = np.inf                 # one infinity among ordinary values
    x[8, 11] = np.nan                 # one NaN
    x[9, :] *= np.float32(1e-30)
    x[9, 5] = np.float32(1e30)        # 2^200 between the largest and the rest of the row: the rest underflows, harmlessly
    x = round_to(BF16, x)
    xt = Tensor.from_data(x.reshape(1, rows, K), gpu, BF16)
    out = w_t.to(gpu).gemm(xt, None, False, True, trans_out)
    kernel = rb._lib.load().rt_plan_kernel(gpu.plan_for(out.op.desc)).decode()
    assert kernel.startswith("gemm_umma_"), kernel
    got = out.resolve().to(Device.CPU).to_f32().reshape((rows, N) if trans_out else (N, rows))
    if not trans_out:
        got = got.T
    with np.errstate(all="ignore"):
        truth = x.astype(np.float64) @ wv.astype(np.float64).T
        truth_r = oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(truth)).reshape(rows, N)
    for r in range(rows):
        if r == 6:
            assert np.all(got[r] == 0.0)
        elif r == 7:
            assert np.array_equal(got[r], truth_r[r], equal_nan=True), "one infinity: +-inf by the sign of its weight"
            assert np.all(np.isinf(got[r]) | np.isnan(got[r]))
        elif r == 8:
            assert np.all(np.isnan(got[r]))
        else:
            fin = np.isfinite(truth_r[r])  # 3e38/16 times a sum of 512 terms may leave bf16's range in the truth too
            assert np.array_equal(np.isfinite(got[r]), fin), r
            assert oracle.rel_l2(got[r][fin], truth_r[r][fin]) <= (2e-3 if lhs_dt == Q4K else 1e-3), (r, kernel)


# ----------------------------------------------------------------------------- infinities and NaNs on every route

@pytest.mark.parametrize("lhs_dt,act,N,K,rows", [
    (Q8H, F16, 256, 512, 4),      # streaming GEMV kernel, several vectors
    (Q8H, F16, 256, 512, 20),     # the same in passes
    (Q8H, F16, 264, 512, 70),     # tensor-core GEMM
    (Q8F, F32, 264, 512, 70),     # 3 x TF32
    (F32, F32, 264, 512, 70),
    (F16, F16, 264, 512, 70),
    (BF16, BF16, 264, 512, 70),
    (Q8H, BF16, 264, 512, 70),
    (Q4K, F16, 264, 512, 1),
    (Q4K, F16, 264, 512, 12),
    (Q4K, F16, 264, 512, 70),
    (F32, F32, 24, 32, 5),        # below every tensor-core threshold
    (Q8F, F32, 24, 32, 5),
])
def test_infinities_and_nans_stay_in_their_rows(gpu, lhs_dt, act, N, K, rows):
    """One activation row holds an infinity, one a NaN: those output rows are what the exact product has there
    (+-inf by the weight's sign, NaN against a zero weight; all NaN), and every other row is bit for bit what it is
    without the two."""
    w_t, wv = make_lhs(lhs_dt, (N, K), np.random.default_rng(15), 0.03)
    x = round_to(act, np.random.default_rng(16).standard_normal((rows, K)).astype(np.float32))
    r_inf, r_nan = (0, rows - 1) if rows > 1 else (0, None)
    xs = x.copy()
    xs[r_inf, 7] = np.inf
    if r_nan is not None and r_nan != r_inf:
        xs[r_nan, 9] = np.nan

    def run(a):
        out = w_t.to(gpu).gemm(Tensor.from_data(a.reshape(1, rows, K), gpu, act), None, False, True, True)
        name = rb._lib.load().rt_plan_kernel(gpu.plan_for(out.op.desc)).decode()
        return out.resolve().to(Device.CPU).to_f32().reshape(rows, N), name

    clean, kernel = run(x)
    got, _ = run(xs)
    assert np.all(np.isfinite(clean)), kernel
    for r in range(rows):
        if r == r_inf:
            w7 = wv[:, 7]
            want_nan = w7 == 0
            assert np.array_equal(np.isnan(got[r]), want_nan), kernel
            assert np.array_equal(got[r][~want_nan], np.where(w7 > 0, np.inf, -np.inf)[~want_nan].astype(np.float32)), kernel
        elif r == r_nan:
            assert np.all(np.isnan(got[r])), kernel
        else:
            assert np.array_equal(got[r], clean[r]), (kernel, r)


# ----------------------------------------------------------------------------- a seeded sweep over decode chains

@pytest.mark.parametrize("seed", range(6))
def test_seeded_decode_chains_against_the_oracle(gpu, seed):
    """Decode chains of two to six Q8_0H GEMVs with widths drawn from the models' (and a few that are no multiple of
    the kernel's row groups), bias on some nodes, GELU on every second: whatever form the executable takes (the
    persistent kernel where every node is eligible, else a graph of single launches), every node's output meets the
    bar against the fp64 oracle fed with the previous node's actual output, twice in a row."""
    rng = np.random.default_rng(5200 + seed)
    dims = [2560, 10240, 3072, 8192, 4096, 5120, 3200, 6400, 2048]
    n = int(rng.integers(2, 7))
    widths = [int(rng.choice(dims)) for _ in range(n + 1)]
    shapes = [(widths[i + 1], widths[i]) for i in range(n)]
    x_dev, nodes, host = _decode_chain(gpu, shapes, 5300 + seed, [bool(rng.integers(0, 2)) for _ in range(n)])
    nodes[-1].resolve()
    exe = rb.Executable(gpu, nodes, use_graph=True)
    for trial in range(2):
        x = np.random.default_rng(5400 + seed + trial).standard_normal(shapes[0][1]).astype(np.float16)
        x_dev.write(x)
        for nd in nodes:
            nd.write(np.zeros(nd.numel(), dtype=np.float16))
        exe.dispatch()
        gpu.sync()
        h = x.astype(np.float32)
        for i, (w_vals, b_vals, epi) in enumerate(host):
            M, K = shapes[i]
            got = nodes[i].to(Device.CPU).to_numpy().reshape(-1).astype(np.float32)
            truth = oracle.matmul_truth(w_vals, h, b_vals, 1, 1, 1, M, 1, K, False, True, True, epi)
            assert np.all(np.isfinite(got)), (exe.kernel, shapes, i)
            assert oracle.rel_l2(got, oracle.f64_to_f16(truth).astype(np.float32)) <= TOL[F16], (exe.kernel, shapes, i)
            h = got
