"""The MLP block as one executable, the gate/up SiLU fold, and executables whose intermediates live in one
planned arena: parity against the oracle, through the host mirror and the C ABI.  GPU only."""
import ctypes

import numpy as np
import pytest

import oracle
import ratchet_b200 as rb
from ratchet_b200 import MLP, DType, Device, Executable, Linear, Tensor, _lib
from util import TOL, make_lhs, round_to

pytestmark = pytest.mark.gpu
F32, F16, BF16, Q8H, Q8F, Q4K = DType.F32, DType.F16, DType.BF16, DType.Q8_0H, DType.Q8_0F, DType.Q4_K
ACT_NAME = {F16: "f16", BF16: "bf16", F32: "f32"}


def _ulps_apart_f16(a, b):
    """Distance in f16 steps between two f16 arrays (NaN only ever equals NaN)."""
    def key(v):
        bits = v.astype(np.float16).view(np.uint16).astype(np.int32)
        return np.where(bits & 0x8000, -(bits & 0x7FFF), bits)
    d = np.abs(key(a) - key(b))
    nan_a, nan_b = np.isnan(a), np.isnan(b)
    d[nan_a & nan_b] = 0
    d[nan_a ^ nan_b] = 1 << 20
    return d


def _kernel_of(gpu, node):
    return _lib.load().rt_plan_kernel(gpu.plan_for(node.op.desc)).decode()


# ----------------------------------------------------------------------------- RT_EPILOGUE_SILU_MUL, one node

@pytest.mark.parametrize("lhs_dt,act,wshape,xshape,bias,route", [
    (Q8H, F16, (16384, 3072), (1, 1, 3072), False, "+silu_mul"),             # Phi-3 gate_up, decode
    (Q8H, F16, (16384, 3072), (1, 16, 3072), False, "+silu_mul"),            # 16 rows: two streaming passes
    (Q8H, F16, (2048, 1024), (1, 9, 1024), True, "+silu_mul"),               # one streaming pass with two groups of MMA columns
    (Q8H, F16, (2048, 1024), (1, 17, 1024), True, "+silu_mul"),              # a pass of 16 and a pass of one
    (Q8H, F16, (2048, 1024), (1, 24, 1024), False, "+silu_mul"),
    (Q8H, F16, (2048, 1024), (1, 25, 1024), True, "paired_tiles"),           # the first row count of the tensor-core GEMM
    (Q4K, F16, (2048, 1024), (1, 16, 1024), True, "+silu_mul"),
    (Q4K, F16, (2048, 1024), (1, 17, 1024), True, "paired_tiles"),
    (Q8H, F16, (16384, 3072), (1, 512, 3072), False, "paired_tiles"),        # prefill: the tensor-core GEMM folds the pairs
    (Q8H, F16, (512, 256), (3, 40, 256), True, "paired_tiles"),              # batched rows over one weight, bias on both halves
    (F16, F16, (200, 64), (1, 300, 64), True, "paired_tiles"),               # ff = 100: not a multiple of 8, ragged tiles
    (F16, F16, (2 * 104, 128), (1, 130, 128), False, "paired_tiles"),        # ff = 104: vector stores with a ragged last tile
    (F16, F16, (2 * 328, 64), (2, 129, 64), True, "paired_tiles"),           # several tile columns, two row tiles per batch
    (BF16, BF16, (512, 128), (1, 200, 128), True, "paired_tiles"),
    (Q8H, BF16, (1024, 256), (1, 256, 256), False, "paired_tiles"),
    (Q4K, F16, (16384, 3072), (1, 512, 3072), False, "paired_tiles"),
    (Q4K, F16, (1024, 512), (1, 1, 512), False, "+silu_mul"),
    (Q8F, F32, (256, 128), (1, 5, 128), True, "+silu_mul"),                  # f32: the reference's default activation dtype
    (F32, F32, (512, 256), (1, 64, 256), True, "+silu_mul"),                 # TF32x3 GEMM, then the fold
    (F16, F16, (64, 32), (1, 2, 32), True, "+silu_mul"),                     # CUDA-core route
], ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else str(getattr(v, "name", v)))
def test_silu_mul_node_is_the_fold_of_the_plain_node(gpu, lhs_dt, act, wshape, xshape, bias, route):
    """up * cast(silu(full(gate))) (phi3/mlp.rs:31-39) as one node: the same as folding the library's own plain
    node with the oracle's restatement of the chain (a last digit may differ where device and host exp differ in
    the last bit), and within the path's bar of the f64 truth."""
    rng = np.random.default_rng(sum(wshape) + sum(xshape))
    w_t, wv = make_lhs(lhs_dt, wshape, np.random.default_rng(77 + wshape[0]), 0.05 if wshape[1] <= 512 else 0.02)
    x = round_to(act, rng.standard_normal(xshape).astype(np.float32))
    b = round_to(act, rng.standard_normal(wshape[0]).astype(np.float32) * 0.1) if bias else None
    w_d, x_d = w_t.to(gpu), Tensor.from_data(x, gpu, act)
    b_d = Tensor.from_data(b, gpu, act) if bias else None
    node = w_d.gemm(x_d, b_d, False, True, True, epilogue=rb.EPILOGUE_SILU_MUL)
    plain = w_d.gemm(x_d, b_d, False, True, True)
    ff = wshape[0] // 2
    assert node.shape == list(xshape[:-1]) + [ff]
    assert route in _kernel_of(gpu, node), _kernel_of(gpu, node)
    got = node.resolve().to(Device.CPU).to_f32().reshape(-1, ff)
    full = plain.resolve().to(Device.CPU).to_f32().reshape(-1, 2 * ff)
    want = oracle.silu_mul(full, ACT_NAME[act])
    if act == F16:
        d = _ulps_apart_f16(got, want)
        # a last-bit difference of exp may move the rounded silu by one step, and the rounded product by up to two
        assert d.max() <= 2, f"{(d > 2).sum()} of {d.size} outputs more than two f16 steps from the fold"
        assert (d > 1).mean() <= 1e-5 and (d > 0).mean() <= 5e-3
    else:
        assert oracle.rel_l2(got, want) <= (2e-3 if act == BF16 else 2e-6)
    # f64 truth on a sample of the rows
    rows = np.unique(np.concatenate([[0, got.shape[0] - 1], np.random.default_rng(3).integers(0, got.shape[0], size=24)]))
    xs = x.reshape(-1, wshape[1])[rows]
    truth = oracle.matmul_truth(wv, xs, b, 1, 1, 1, wshape[0], len(rows), wshape[1], False, True, True, 0)
    tr = oracle.silu_mul_truth(truth.reshape(len(rows), 2 * ff))
    # the gate and up roundings both enter the product: twice the single-node bar; bf16 (2^-9 per rounding, three
    # roundings, no reference counterpart) four times
    assert oracle.rel_l2(got[rows], tr) <= (4 if act == BF16 else 2) * TOL[act]


def test_silu_mul_gate_overflow_is_nan_like_the_reference(gpu):
    """exp(v) / (1 + exp(v)) is inf / inf once v passes 88.7 (unary.rs:127): the fused and the two-launch routes
    both give NaN there and nowhere else."""
    ff, K = 64, 128
    w = np.eye(2 * ff, K, dtype=np.float32)               # gate j = x[j], up j = x[ff + j]
    for rows, route in ((2, "gemm_simt"), (300, "paired_tiles")):
        x = np.full((rows, K), 0.5, dtype=np.float32)
        x[0, 3], x[rows - 1, 5], x[0, 7] = 100.0, 89.0, 88.0
        node = Tensor.from_data(w, gpu, F16).gemm(Tensor.from_data(x, gpu, F16), None, False, True, True,
                                                  epilogue=rb.EPILOGUE_SILU_MUL)
        assert route in _kernel_of(gpu, node), _kernel_of(gpu, node)
        y = node.resolve().to(Device.CPU).to_f32().reshape(rows, ff)
        want = np.zeros((rows, ff), dtype=bool)
        want[0, 3] = want[rows - 1, 5] = True
        assert np.array_equal(np.isnan(y), want)
        assert y[0, 7] == np.float32(np.float16(0.5) * np.float16(oracle.silu_f32(np.float32(88.0))))
        assert y[1, 0] == np.float32(np.float16(0.5) * np.float16(oracle.silu_f32(np.float32(0.5))))


# ----------------------------------------------------------------------------- the MLP block as one executable

def _mlp_truth(w1, b1, w2, b2, x2d, act, dt):
    """hidden rounded to the activation dtype between the two nodes, as the reference's graph holds it."""
    n1, k1 = w1.shape
    rows = x2d.shape[0]
    if act == "gelu":
        h = oracle.matmul_truth(w1, x2d, b1, 1, 1, 1, n1, rows, k1, False, True, True, 1).reshape(rows, n1)
    else:
        h = oracle.silu_mul_truth(oracle.matmul_truth(w1, x2d, b1, 1, 1, 1, n1, rows, k1, False, True, True, 0).reshape(rows, n1))
    h_r = oracle.f64_to_f16(h).astype(np.float32) if dt == F16 else h.astype(np.float32)
    n2, k2 = w2.shape
    t = oracle.matmul_truth(w2, h_r, b2, 1, 1, 1, n2, rows, k2, False, True, True, 0).reshape(rows, n2)
    return oracle.f64_to_f16(t).astype(np.float32) if dt == F16 else t.astype(np.float32)


@pytest.mark.parametrize("M", [1, 16, 512])
def test_phi3_mlp_block(gpu, M):
    """Phi-3 mini: gate_up Q8_0H [16384,3072] -> up * silu(gate) -> down Q8_0H [3072,8192], x f16 [1,M,3072]
    (phi3/mlp.rs:31-39), as one executable whose hidden tensor the planner places."""
    w1_t, w1 = make_lhs(Q8H, (16384, 3072), np.random.default_rng(3001), 0.02)
    w2_t, w2 = make_lhs(Q8H, (3072, 8192), np.random.default_rng(3002), 0.02)
    x = round_to(F16, np.random.default_rng(3003 + M).standard_normal((1, M, 3072)).astype(np.float32))
    mlp = MLP(Linear(w1_t.to(gpu)), Linear(w2_t.to(gpu)), act="silu_gate")
    x_d = Tensor.from_data(x, gpu, F16)
    exe, out = mlp.bind(x_d)
    a = exe.arena()
    assert a["arena_bytes"] >= M * 8192 * 2 and a["arena_bytes"] <= a["record_bytes"]
    exe.dispatch()
    gpu.sync()
    assert out.shape == [1, M, 3072]
    got = out.to(Device.CPU).to_f32().reshape(M, 3072)
    rows = np.unique(np.concatenate([[0, M - 1], np.random.default_rng(9).integers(0, M, size=16)]))
    want = _mlp_truth(w1, None, w2, None, x.reshape(M, 3072)[rows], "silu_gate", F16)
    assert oracle.rel_l2(got[rows], want) <= 2e-3
    # a second input through the same executable
    x2 = round_to(F16, np.random.default_rng(3100 + M).standard_normal((1, M, 3072)).astype(np.float32))
    x_d.write(x2.astype(np.float16))
    exe.dispatch()
    gpu.sync()
    got2 = out.to(Device.CPU).to_f32().reshape(M, 3072)
    want2 = _mlp_truth(w1, None, w2, None, x2.reshape(M, 3072)[rows], "silu_gate", F16)
    assert oracle.rel_l2(got2[rows], want2) <= 2e-3


def test_whisper_mlp_block(gpu):
    """Whisper-tiny encoder MLP as one executable: x f16 [1,1500,384] -> Q8_0H [1536,384] + b -> GELU -> Q8_0H
    [384,1536] + b (whisper/mlp.rs:18-22); the same numbers as the two lazily resolved nodes give."""
    w1_t, w1 = make_lhs(Q8H, (1536, 384), np.random.default_rng(1103), 0.02)
    w2_t, w2 = make_lhs(Q8H, (384, 1536), np.random.default_rng(1104), 0.02)
    b1 = round_to(F16, np.random.default_rng(2103).standard_normal(1536) * 0.02)
    b2 = round_to(F16, np.random.default_rng(2104).standard_normal(384) * 0.02)
    x = round_to(F16, np.random.default_rng(103).standard_normal((1, 1500, 384)))
    fc1, fc2 = Linear(w1_t.to(gpu), Tensor.from_data(b1, gpu, F16)), Linear(w2_t.to(gpu), Tensor.from_data(b2, gpu, F16))
    x_d = Tensor.from_data(x, gpu, F16)
    out = MLP(fc1, fc2, act="gelu").schedule(x_d)
    gpu.sync()
    got = out.to(Device.CPU).to_f32().reshape(1500, 384)
    assert oracle.rel_l2(got, _mlp_truth(w1, b1, w2, b2, x.reshape(1500, 384), "gelu", F16)) <= 1e-3
    lazy = Linear(fc2.w, fc2.b).schedule(Linear(fc1.w, fc1.b, epilogue=rb.EPILOGUE_GELU_TANH).schedule(x_d)).resolve()
    assert np.array_equal(lazy.to(Device.CPU).to_numpy().reshape(-1), out.to(Device.CPU).to_numpy().reshape(-1))


def test_bf16_mlp_block_with_rows_beyond_the_f16_range(gpu):
    """A GELU block on bf16 activations against Q8_0H weights as one planned executable: the cast of each node's
    activations (to f16, with a power of two per row) and its factors live in the executable's arena.  Rows of
    magnitude 1e5 and 1e-6 come out as accurately as ordinary ones; the hidden tensor is bf16 between the nodes."""
    rows = 96
    w1_t, w1 = make_lhs(Q8H, (1024, 256), np.random.default_rng(9101), 0.03)
    w2_t, w2 = make_lhs(Q8H, (256, 1024), np.random.default_rng(9102), 0.03)
    b1 = round_to(BF16, np.random.default_rng(9103).standard_normal(1024) * 0.02)  # Linear casts its bias to the input dtype
    b2 = round_to(BF16, np.random.default_rng(9104).standard_normal(256) * 0.02)
    x = np.random.default_rng(9105).standard_normal((1, rows, 256)).astype(np.float32)
    x[0, 0] *= 1e5
    x[0, 1] *= 1e-6
    x = round_to(BF16, x)
    fc1 = Linear(w1_t.to(gpu), Tensor.from_data(b1, gpu, BF16))
    fc2 = Linear(w2_t.to(gpu), Tensor.from_data(b2, gpu, BF16))
    exe, out = MLP(fc1, fc2, act="gelu").bind(Tensor.from_data(x, gpu, BF16))
    assert exe.arena()["arena_bytes"] > 0
    for _ in range(2):  # the second dispatch reuses the arena's cast areas
        exe.dispatch()
    gpu.sync()
    got = out.to(Device.CPU).to_f32().reshape(rows, 256)
    x2 = x.reshape(rows, 256).astype(np.float64)
    with np.errstate(all="ignore"):
        h = oracle.matmul_truth(w1, x2, b1, 1, 1, 1, 1024, rows, 256, False, True, True, 1).reshape(rows, 1024)
        h_r = oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(h)).reshape(rows, 1024)
        t = oracle.matmul_truth(w2, h_r, b2, 1, 1, 1, 256, rows, 1024, False, True, True, 0).reshape(rows, 256)
        want = oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(t)).reshape(rows, 256)
    assert np.all(np.isfinite(got))
    for r in (0, 1, 2, rows - 1):
        # two bf16 roundings in sequence (hidden, output) against a truth with the same two: whole-ulp flips of the hidden
        # tensor carry through, so the bar per row is twice the single node's
        assert oracle.rel_l2(got[r], want[r]) <= 2e-3, r
    assert oracle.rel_l2(got, want) <= 2e-3


def test_phi2_decode_mlp_block_is_the_persistent_gemv_kernel(gpu):
    """Phi-2 decode: x f16 [1,1,2560] -> Q8_0H [10240,2560] + b -> GELU -> Q8_0H [2560,10240] + b
    (phi2/mlp.rs:13-15): the two nodes of the block run as one launch."""
    w1_t, w1 = make_lhs(Q8H, (10240, 2560), np.random.default_rng(5001), 0.02)
    w2_t, w2 = make_lhs(Q8H, (2560, 10240), np.random.default_rng(5002), 0.01)
    b1 = round_to(F16, np.random.default_rng(5003).standard_normal(10240) * 0.02)
    b2 = round_to(F16, np.random.default_rng(5004).standard_normal(2560) * 0.02)
    x = round_to(F16, np.random.default_rng(5005).standard_normal((1, 1, 2560)))
    mlp = MLP(Linear(w1_t.to(gpu), Tensor.from_data(b1, gpu, F16)), Linear(w2_t.to(gpu), Tensor.from_data(b2, gpu, F16)))
    exe, out = mlp.bind(Tensor.from_data(x, gpu, F16))
    assert exe.kernel.startswith("q8_gemv_chain") and exe.launches == 1, exe.kernel
    exe.dispatch()
    gpu.sync()
    got = out.to(Device.CPU).to_f32().reshape(1, 2560)
    assert oracle.rel_l2(got, _mlp_truth(w1, b1, w2, b2, x.reshape(1, 2560), "gelu", F16)) <= 1e-3


def test_mlp_rejects_mismatched_blocks(gpu):
    w1 = Tensor.from_data(np.zeros((64, 32), dtype=np.float16), gpu)
    w2 = Tensor.from_data(np.zeros((16, 48), dtype=np.float16), gpu)   # takes 48, fc1 gives 64
    x = Tensor.from_data(np.zeros((1, 4, 32), dtype=np.float16), gpu)
    with pytest.raises(rb.RatchetError):
        MLP(Linear(w1), Linear(w2)).bind(x)


# ----------------------------------------------------------------------------- planned executables

def _free_bytes():
    import torch
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_planned_executable_places_intermediates_in_one_arena_and_dispatch_allocates_nothing(gpu):
    """Four Linear nodes x -> t0 -> t1 -> t2 -> out with the three intermediates named by id: they share one
    arena by the reference's greedy-by-size rule (allocator.rs:209-271), results match node-by-node launches into
    separate buffers, and 100 dispatches leave the device's free memory where it was."""
    lib = _lib.load()
    rows = 40
    widths = [256, 1024, 512, 768, 128]
    ws, wvals = [], []
    for i in range(4):
        w_t, wv = make_lhs(Q8H if i % 2 == 0 else F16, (widths[i + 1], widths[i]), np.random.default_rng(600 + i), 0.05)
        ws.append(w_t.to(gpu))
        wvals.append(wv)
    x = round_to(F16, np.random.default_rng(610).standard_normal((rows, widths[0])))
    x_d = Tensor.from_data(x, gpu, F16)
    # reference run: the lazy graph, one buffer per node
    h = x_d
    for w in ws:
        h = w.gemm(h, None, False, True, True)
    want = h.resolve().to(Device.CPU).to_numpy().reshape(-1)

    out = Tensor([rows, widths[-1]], F16, gpu, rb.GpuBuffer(gpu, rows * widths[-1] * 2))
    nodes, shape = [], [rows, widths[0]]
    for i, w in enumerate(ws):
        d = _lib.rt_matmul_desc()
        d.lhs_dt, d.rhs_dt = int(w.dt), int(F16)
        d.lhs_shape, d.rhs_shape = _lib.rt_shape.of(w.shape), _lib.rt_shape.of([rows, widths[i]])
        d.trans_rhs = d.trans_out = 1
        nodes.append({"plan": gpu.plan_for(d), "lhs": w.ptr, "rhs": x_d.ptr if i == 0 else ("t", i - 1),
                      "out": out.ptr if i == 3 else ("t", i), "flags": _lib.RT_LAUNCH_LHS_CONSTANT})
    sizes = [rows * widths[i + 1] * 2 for i in range(3)]
    exe = Executable.planned(gpu, nodes, sizes, use_graph=True, keep=[x_d, out] + ws)
    a = exe.arena()
    # t0 (1024 wide) and t2 (768 wide) are never alive together: one object; t1 overlaps both: a second one
    assert a["objects"] >= 2 and a["arena_bytes"] < a["record_bytes"]
    assert exe.tensor_ptr(0) == exe.tensor_ptr(2) != exe.tensor_ptr(1)
    assert exe.tensor_ptr(0) % 256 == 0 and exe.tensor_ptr(3) == 0
    exe.dispatch()
    gpu.sync()
    assert np.array_equal(out.to(Device.CPU).to_numpy().reshape(-1), want)
    before = _free_bytes()
    for _ in range(100):
        exe.dispatch()
    gpu.sync()
    assert _free_bytes() == before
    assert np.array_equal(out.to(Device.CPU).to_numpy().reshape(-1), want)
    # a node that reads an intermediate no earlier node produced
    bad = [dict(nodes[0], rhs=("t", 1))] + nodes[1:]
    with pytest.raises(rb.RatchetError):
        Executable.planned(gpu, bad, sizes, keep=[])
    # an intermediate smaller than its producer's output
    with pytest.raises(rb.RatchetError):
        Executable.planned(gpu, nodes, [sizes[0] - 2] + sizes[1:], keep=[])


def test_executables_own_their_scratch(gpu):
    """Two executables built from the SAME plan (equal descriptions share one, the plan keeps one scratch area)
    dequantise different weights: each has the scratch in its own arena, so replaying them alternately gives each
    its own result.  (Weights not flagged constant: the dequantising pass runs at every dispatch.)"""
    rows, n, k = 64, 512, 256
    x = round_to(F16, np.random.default_rng(701).standard_normal((rows, k)))
    x_d = Tensor.from_data(x, gpu, F16)
    exes, outs, wants = [], [], []
    for i in range(2):
        w_t, wv = make_lhs(Q8H, (n, k), np.random.default_rng(710 + i), 0.05)
        w_d = w_t.to(gpu)
        node = w_d.gemm(x_d, None, False, True, True)
        plan = gpu.plan_for(node.op.desc)
        out = Tensor([rows, n], F16, gpu, rb.GpuBuffer(gpu, rows * n * 2))
        exe = Executable.planned(gpu, [{"plan": plan, "lhs": w_d.ptr, "rhs": x_d.ptr, "out": out.ptr}], [], keep=[w_d, out])
        assert exe.arena()["arena_bytes"] >= n * k * 2
        exes.append(exe)
        outs.append(out)
        wants.append(oracle.f64_to_f16(oracle.matmul_truth(wv, x, None, 1, 1, 1, n, rows, k, False, True, True, 0)).astype(np.float32))
    for _ in range(3):
        for e in exes:
            e.dispatch()
    gpu.sync()
    for out, want in zip(outs, wants):
        assert oracle.rel_l2(out.to(Device.CPU).to_f32().reshape(-1), want) <= TOL[F16]


@pytest.mark.parametrize("seed", range(8))
def test_seeded_planned_chains_match_the_lazy_graph_bit_for_bit(gpu, seed):
    """Chains of three to six Linear nodes of mixed weight formats, with and without bias and GELU, weights flagged
    constant or not, as planned executables (intermediates, dequantising scratch, cast areas and paired rows all placed
    in the one arena): every chain gives exactly what its nodes give when resolved one by one into buffers of their own,
    on the first dispatch and on the third."""
    rng = np.random.default_rng(4200 + seed)
    act = [F16, BF16, F32][seed % 3]
    weights = {F16: [Q8H, Q4K, F16], BF16: [Q8H, Q4K, BF16], F32: [Q8F, F32]}[act]
    rows = int(rng.choice([4, 12, 20, 40, 130]))
    n_nodes = int(rng.integers(3, 7))
    widths = [int(rng.choice([256, 512, 768, 1024])) for _ in range(n_nodes + 1)]
    x = round_to(act, rng.standard_normal((rows, widths[0])).astype(np.float32))
    x_d = Tensor.from_data(x, gpu, act)
    ws, bs, epis, flags = [], [], [], []
    for i in range(n_nodes):
        w_t, _ = make_lhs(weights[int(rng.integers(0, len(weights)))], (widths[i + 1], widths[i]), np.random.default_rng(seed * 100 + i), 0.04)
        ws.append(w_t.to(gpu))
        has_b = bool(rng.integers(0, 2))
        bs.append(Tensor.from_data(round_to(act, rng.standard_normal(widths[i + 1]).astype(np.float32) * 0.05), gpu, act) if has_b else None)
        epis.append(int(rng.integers(0, 2)) if i < n_nodes - 1 else 0)
        flags.append(_lib.RT_LAUNCH_LHS_CONSTANT if rng.integers(0, 2) else 0)
    h = x_d
    for w, b, e in zip(ws, bs, epis):
        h = w.gemm(h, b, False, True, True, epilogue=e)
    want = h.resolve().to(Device.CPU).to_numpy().reshape(-1)

    esz = act.size_of()
    out = Tensor([rows, widths[-1]], act, gpu, rb.GpuBuffer(gpu, rows * widths[-1] * esz))
    nodes = []
    for i, (w, b, e) in enumerate(zip(ws, bs, epis)):
        d = _lib.rt_matmul_desc()
        d.lhs_dt, d.rhs_dt = int(w.dt), int(act)
        d.lhs_shape, d.rhs_shape = _lib.rt_shape.of(w.shape), _lib.rt_shape.of([rows, widths[i]])
        d.trans_rhs = d.trans_out = 1
        d.epilogue = e
        if b is not None:
            d.has_bias, d.bias_dt, d.bias_shape = 1, int(act), _lib.rt_shape.of([widths[i + 1]])
        nodes.append({"plan": gpu.plan_for(d), "lhs": w.ptr, "rhs": x_d.ptr if i == 0 else ("t", i - 1),
                      "bias": b.ptr if b is not None else None,
                      "out": out.ptr if i == n_nodes - 1 else ("t", i), "flags": flags[i]})
    sizes = [rows * widths[i + 1] * esz for i in range(n_nodes - 1)]
    exe = Executable.planned(gpu, nodes, sizes, use_graph=bool(seed & 1), keep=[x_d, out] + ws + [b for b in bs if b is not None])
    for rep in range(3):
        exe.dispatch()
        gpu.sync()
        got = out.to(Device.CPU).to_numpy().reshape(-1)
        assert np.array_equal(got, want, equal_nan=True), (rep, act, [w.dt for w in ws], rows, widths, epis, flags, exe.kernel)
