"""Benchmark of the Matmul hot path: Q8_0 GEMV (decode) at the Phi-2 MLP shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload ("phi2_mlp_q8_0_gemv_decode"): one decode step through the MLPs of Phi-2's 32 layers
reduced to its Matmul nodes: 32 x [fc1: W Q8_0H [10240,2560] . x f16 [2560] -> f16 [10240];
fc2: W Q8_0H [2560,10240] . h f16 [10240] -> f16 [2560]], chained, every layer with its own
weights, each node built as W.gemm(x, None, false, true, true) like nn::Linear.  64 GEMV
launches per step, 27,878,400 algorithmic bytes each (codes + f16 scales + x + y); the weights
(1.78 GB) exceed the 126 MB L2, so every launch streams from HBM.  Synthetic data: weights
N(0, 0.02) (fc2: N(0, 0.01), see make_weights) quantised with sint8_quantize, input N(0, 1), seeded.

A "step" is REPEATS (50) decode steps in a row, so that a run of a few steps is long enough to time.

Legs, all in one JSON line printed by rank 0:
  value         device-timed GB/s, operands resident, one Executable dispatch per decode step
  e2e           the same step through the public host API (Tensor.to / gemm / resolve / to):
                host->device copy of the step's input vector from pinned memory and
                device->host read of the step's output inside the timed region
  roofline      algorithmic bytes per launch / average launch time, against the measured HBM peak
  cpu_baseline  the shader-faithful CPU oracle on all host cores, bounded sample (rank 0, N=1)
  dispatch_forms   the same GEMVs launched one kernel per node, and as two-node fc1 -> fc2 executables
  extras        the other workloads on one GPU (dense f32, Whisper MLP, Q4_K, bf16 prefill), each with its roofline
  sharded       the N-sharded bf16 prefill Linear (at N = 1: the compute-only point of the curve), with a parity check
`--impl reference` times that CPU oracle alone (the reference has no CPU Matmul and its WebGPU
backend cannot run on this box; the oracle is the restated reference arithmetic).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "Q8_0 GEMV effective bandwidth (Phi-2 MLP shapes, decode)"
UNIT = "GB/s"
LAYERS = 32
D_MODEL, D_FF = 2560, 10240
NCU_TRAFFIC_PER_GEMV = 27_900_000     # measured DRAM bytes per GEMV (27.88 MB per node of the chain kernel; 27.89 / 27.91 MB single launches)
REPEATS = 50                          # decode steps per timed "step"
BYTES_PER_GEMV = D_FF * D_MODEL + 2 * (D_FF * D_MODEL // 32) + 2 * D_MODEL + 2 * D_FF  # 27,878,400
WORKLOAD = "phi2_mlp_q8_0_gemv_decode"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20, help="timed steps; one step = %d decode steps" % REPEATS)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS, help="MLP blocks per step (default: Phi-2's 32)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="dispatch node by node instead of one CUDA graph")
    ap.add_argument("--no-lazy", action="store_true", help="skip the node-by-node lazy-graph leg reported beside e2e")
    ap.add_argument("--no-sharded", action="store_true", help="with --gpus > 1: skip the N-sharded prefill GEMM section")
    ap.add_argument("--extras", default="all", help="comma list of the other workloads to time on one GPU and "
                    "report under \"extras\": c1,c3,c4,c5,c5long,mlp, all (default) or none")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


UNIQUE_LAYERS = 4


def make_weights_f32(layers: int, seed: int):
    """Per layer (fc1 [D_FF, D_MODEL], fc2 [D_MODEL, D_FF]) f32 weights.  Four distinct layers are generated and
    repeated: every layer still gets its own device buffer, and bandwidth does not depend on the values.
    fc1 ~ N(0, 0.02); fc2 ~ N(0, 0.01) so that the chained activations keep a constant scale and stay inside the
    f16 range over 32 layers."""
    uniq = []
    for l in range(min(layers, UNIQUE_LAYERS)):
        rng = np.random.default_rng(seed + 1000 + l)
        uniq.append((rng.standard_normal((D_FF, D_MODEL), dtype=np.float32) * np.float32(0.02),
                     rng.standard_normal((D_MODEL, D_FF), dtype=np.float32) * np.float32(0.01)))
    return uniq


def make_weights(layers: int, seed: int):
    """The same as Q8_0H host tensors, built with the library's quantiser (our arm)."""
    import ratchet_b200 as rb
    qz = rb.Quantizer(rb.Quantization.SInt8)
    uniq = [(qz.sint8_quantize(rb.Tensor.from_data(w1), rb.DType.Q8_0H), qz.sint8_quantize(rb.Tensor.from_data(w2), rb.DType.Q8_0H))
            for w1, w2 in make_weights_f32(layers, seed)]
    return [uniq[l % len(uniq)] for l in range(layers)]


def make_weights_oracle(layers: int, seed: int):
    """The same as raw Q8_0H byte buffers, built with the oracle's quantiser: the reference arm's process never
    loads the CUDA library."""
    import oracle
    uniq = [(oracle.q8_quantize_h(w1), oracle.q8_quantize_h(w2)) for w1, w2 in make_weights_f32(layers, seed)]
    return [uniq[l % len(uniq)] for l in range(layers)]


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-i", str(self.index), "-lms", "50"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, smax, reasons = [], [], set()
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        # the sampler also sees the idle moments before and after the timed loops: the upper half of
        # the samples are the ones under load
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": float(np.median(load)) if load else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------- the other configurations

def tensor_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


def time_nodes(gpu, stream, nodes, reps: int, warmup: int = 3):
    """Times a list of resolved Matmul nodes dispatched as one executable (the way a step runs: one CUDA
    graph, weights flagged constant), `reps` dispatches between two events.  Returns microseconds per
    dispatch, the kernels' names and the launches per dispatch."""
    import torch
    import ratchet_b200 as rb
    lib = rb._lib.load()
    for n in nodes:
        n.resolve()
    exe = rb.Executable(gpu, nodes)
    for _ in range(warmup):
        exe.dispatch()
    gpu.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        exe.dispatch()
    e1.record(stream)
    gpu.sync()
    torch.cuda.synchronize()
    kernels = [lib.rt_plan_kernel(gpu.plan_for(n.op.desc)).decode() for n in nodes]
    return e0.elapsed_time(e1) * 1e3 / reps, kernels, exe.launches


def time_node(gpu, stream, make_node, copies: int, iters: int, warmup: int = 3, keep=None):
    """Times one Matmul node: `copies` independent operand sets are rotated inside one executable so
    that a memory-bound node never finds its weights in L2.  Returns microseconds per node.  `keep`, a list, receives
    the first copy's node (its output is what the parity check reads)."""
    nodes = [make_node(i) for i in range(copies)]
    us, kernels, launches = time_nodes(gpu, stream, nodes, max(1, iters // copies), warmup)
    if keep is not None:
        keep.append(nodes[0])
    return us / copies, kernels[0], launches // copies


def mlp_parity(out_t, w1_host, b1_host, w2_host, b2_host, x_host, act, n_rows=6):
    """rel-L2 of sampled rows of an MLP block's f16 output against the fp64 oracle (hidden rounded to f16 between the
    nodes, as the reference's graph holds it); act: "gelu" or "silu_gate"."""
    import oracle
    from ratchet_b200 import Device
    n1, k1 = w1_host.shape
    n2, k2 = w2_host.shape
    xv = x_host.to_f32().reshape(-1, k1)
    rows = np.unique(np.concatenate([[0, xv.shape[0] - 1], np.random.default_rng(7).integers(0, xv.shape[0], size=n_rows)]))
    b1 = b1_host.to_f32().reshape(-1) if b1_host is not None else None
    b2 = b2_host.to_f32().reshape(-1) if b2_host is not None else None
    h = oracle.matmul_truth(w1_host.to_f32().reshape(n1, k1), xv[rows], b1, 1, 1, 1, n1, len(rows), k1, False, True, True,
                            1 if act == "gelu" else 0).reshape(len(rows), n1)
    if act == "silu_gate":
        h = oracle.silu_mul_truth(h)
    h16 = oracle.f64_to_f16(h).astype(np.float32)
    t = oracle.matmul_truth(w2_host.to_f32().reshape(n2, k2), h16, b2, 1, 1, 1, n2, len(rows), k2, False, True, True, 0).reshape(len(rows), n2)
    have = out_t.to(Device.CPU).to_numpy().reshape(-1, n2)[rows].astype(np.float32)
    return oracle.rel_l2(have, oracle.f64_to_f16(t).astype(np.float32))


def linear_parity(node, w_host, x_host, b_host, epilogue, n_rows=8):
    """rel-L2 of sampled rows of a Linear node's output against the fp64 oracle over the weight's exact values (the
    oracle is the checker here, after and outside every timed region)."""
    import oracle
    from ratchet_b200 import Device, DType, Quantizer
    N, K = w_host.shape
    wv = (Quantizer.dequantize_bytes(w_host.to_numpy(), w_host.dt, N * K) if w_host.dt.is_quantized() else w_host.to_f32()).reshape(N, K)
    xv = x_host.to_f32().reshape(-1, K)
    rows = np.unique(np.concatenate([[0, xv.shape[0] - 1], np.random.default_rng(7).integers(0, xv.shape[0], size=n_rows)]))
    bv = b_host.to_f32().reshape(-1) if b_host is not None else None
    truth = oracle.matmul_truth(wv, xv[rows], bv, 1, 1, 1, N, len(rows), K, False, True, True, epilogue).reshape(len(rows), N)
    got = node.to(Device.CPU)
    raw = got.to_numpy().reshape(-1, N)[rows]  # only the sampled rows are converted
    if got.dt == DType.F16:
        want, have = oracle.f64_to_f16(truth).astype(np.float32), raw.astype(np.float32)
    elif got.dt == DType.BF16:
        want = oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(truth)).reshape(truth.shape)
        have = oracle.bf16_bits_to_f32(np.ascontiguousarray(raw).reshape(-1)).reshape(truth.shape)
    else:
        want, have = truth.astype(np.float32), raw.astype(np.float32)
    return oracle.rel_l2(have, want)


# measured DRAM bytes per call (ncu dram__bytes_read.sum + dram__bytes_write.sum, profiles/), where a capture exists
NCU_TRAFFIC = {
    "c1_dense_f32_phi2_fc1_m128": 111.4e6,            # profiles/gemm_umma_tf32x3_dense_f32_c1.md
    "c4_q4_k_phi3_m1": 14.21e6,                       # profiles/q4k_gemv_mma_phi3_decode.md
}


def run_extras(which, gpu, stream):
    """The other workloads on one GPU: time, TFLOP/s or GB/s, roofline object each."""
    import ratchet_b200 as rb
    from ratchet_b200 import DType, Tensor
    hbm, hbm_kind = peaks()
    tf_burst, tf_sust, tf_kind = tensor_peaks()
    qz = rb.Quantizer(rb.Quantization.SInt8)
    out = []

    def weight(shape, dt, seed, std=0.02):
        w = np.random.default_rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(std)
        t = Tensor.from_data(w)
        if dt == DType.Q8_0H:
            return qz.sint8_quantize(t, DType.Q8_0H)
        if dt == DType.Q4_K:
            return rb.Quantizer.q4k_quantize(t)
        return Tensor.from_data(w, dt=dt)

    def act(shape, dt, seed):
        return Tensor.from_data(np.random.default_rng(seed).standard_normal(shape, dtype=np.float32), dt=dt)

    def record(name, us, kernel, launches, flops, nbytes, bound, note="", parity=None):
        tfs, gbs = flops / us / 1e6, nbytes / us / 1e3
        peak = tf_burst if bound == "tensor" else hbm
        ach = tfs if bound == "tensor" else gbs
        out.append({"workload": name, "us_per_call": us, "kernel": kernel, "launches_per_call": launches,
                    "tflops": tfs, "gbs": gbs, "algorithmic_flops": flops, "algorithmic_bytes": nbytes,
                    "roofline": {"bound": bound, "achieved": ach, "peak": peak,
                                 "unit": "TFLOP/s" if bound == "tensor" else "GB/s", "frac": ach / peak,
                                 "peak_kind": f"of {tf_kind if bound == 'tensor' else hbm_kind}",
                                 "traffic": NCU_TRAFFIC.get(name)}, "note": note})
        if parity is not None:
            out[-1]["parity_rel_l2"] = parity

    def linear_node(w_dev, x_dev, b_dev, epilogue=0):
        return w_dev.gemm(x_dev, b_dev, False, True, True, epilogue=epilogue)

    if "c1" in which:
        wh, bh, xh = weight((10240, 2560), DType.F32, 1101), weight((10240,), DType.F32, 2101), act((1, 128, 2560), DType.F32, 101)
        w, b, x = wh.to(gpu), bh.to(gpu), xh.to(gpu)
        kept = []
        us, k, l = time_node(gpu, stream, lambda i: linear_node(w, x, b), 1, 20, keep=kept)
        record("c1_dense_f32_phi2_fc1_m128", us, k, l, 2 * 128 * 10240 * 2560, 111452160, "hbm", "weights L2-resident between calls",
               parity=linear_parity(kept[0], wh, xh, bh, 0))
    if "c3" in which:
        w1h, w2h = weight((1536, 384), DType.Q8_0H, 1103), weight((384, 1536), DType.Q8_0H, 1104)
        b1h, b2h, xh = weight((1536,), DType.F16, 2103), weight((384,), DType.F16, 2104), act((1, 1500, 384), DType.F16, 103)
        w1, w2, b1, b2, x = w1h.to(gpu), w2h.to(gpu), b1h.to(gpu), b2h.to(gpu), xh.to(gpu)
        h = linear_node(w1, x, b1, rb.EPILOGUE_GELU_TANH)
        y = linear_node(w2, h, b2)
        us, ks, l = time_nodes(gpu, stream, [h, y], 200)
        record("c3_whisper_tiny_mlp_q8_0_m1500", us, " + ".join(ks), l, 2 * 1500 * 384 * 1536 * 2, 12777216,
               "tensor", "fc1+GELU then fc2 as one executable; latency-bound (one wave)",
               parity=mlp_parity(y, w1h, b1h, w2h, b2h, xh, "gelu"))
    if "c4" in which:
        hw = weight((8192, 3072), DType.Q4_K, 1104)
        copies = 20  # 20 x 14.2 MB of weights: larger than L2
        ws = [hw.to(gpu) for _ in range(copies)]
        for M in (1, 16, 512):
            xh = act((1, M, 3072), DType.F16, 104)
            x = xh.to(gpu)
            kept = []
            us, k, l = time_node(gpu, stream, lambda i: linear_node(ws[i], x, None), copies, 200 if M < 512 else 60, keep=kept)
            nbytes = 14155776 + 2 * M * 3072 + 2 * M * 8192
            record(f"c4_q4_k_phi3_m{M}", us, k, l, 2 * M * 8192 * 3072, nbytes, "tensor" if M == 512 else "hbm",
                   "rotating 20 weight copies", parity=linear_parity(kept[0], hw, xh, None, 0))
    if "mlp" in which:
        # Phi-3 mini MLP block as ONE executable (rt_mlp_create): gate_up [16384,3072] -> up * silu(gate) -> down [3072,8192]
        copies = 3  # 3 x 80 MB of weights: larger than L2
        host_blocks = [(weight((16384, 3072), DType.Q8_0H, 1201 + c), weight((3072, 8192), DType.Q8_0H, 1301 + c)) for c in range(copies)]
        blocks = [rb.MLP(rb.Linear(a.to(gpu)), rb.Linear(b_.to(gpu)), act="silu_gate") for a, b_ in host_blocks]
        import torch
        for M in (1, 16, 512):
            xh = act((1, M, 3072), DType.F16, 1400 + M)
            x = xh.to(gpu)
            bound = [blk.bind(x) for blk in blocks]
            for exe, _ in bound:
                exe.dispatch()
            gpu.sync()
            reps = 20 if M < 512 else 10
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                for exe, _ in bound:
                    exe.dispatch()
            e1.record(stream)
            gpu.sync()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps / copies
            wbytes = (16384 * 3072 + 3072 * 8192) * 34 // 32
            record(f"mlp_phi3_q8_0_block_m{M}", us, bound[0][0].kernel, bound[0][0].launches,
                   2 * M * (16384 * 3072 + 3072 * 8192), wbytes + 2 * M * (3072 + 3072), "tensor" if M == 512 else "hbm",
                   "gate_up + SiLU*mul + down as one executable, hidden tensor in the executable's arena; rotating 3 weight sets",
                   parity=mlp_parity(bound[0][1], host_blocks[0][0], None, host_blocks[0][1], None, xh, "silu_gate"))
    for name, rows in (("c5", 2048), ("c5long", 8192)):
        if name not in which:
            continue
        wh, bh, xh = weight((10240, 2560), DType.Q8_0H, 1105), weight((10240,), DType.F16, 2105), act((4, rows, 2560), DType.BF16, 105)
        w, b, x = wh.to(gpu), bh.to(gpu), xh.to(gpu)
        kept = []
        us, k, l = time_node(gpu, stream, lambda i: linear_node(w, x, b, rb.EPILOGUE_GELU_TANH), 1, 10, keep=kept)
        record(f"{name}_q8_0_prefill_bf16_4x{rows}", us, k, l, 2 * 4 * rows * 10240 * 2560,
               4 * rows * 2560 * 2 + 27852800 + 4 * rows * 10240 * 2, "tensor", "bias + fused GELU, 1 GPU",
               parity=linear_parity(kept[0], wh, xh, bh, 1))
        del kept, w, x
    return out


def sharded_operands(rows_per_batch):
    """Seeded operands of the sharded prefill Linear: W f32 [10240, 2560] ~ N(0, 0.02), f16 bias, bf16 activations."""
    N, K, rows = 10240, 2560, 4 * rows_per_batch
    w = np.random.default_rng(1105).standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
    b = (np.random.default_rng(2105).standard_normal(N, dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    x = np.random.default_rng(105).standard_normal((rows, K), dtype=np.float32)
    return N, K, rows, w, b, x


def sharded_parity(got_bf16_bits, rows_idx, w_q, b16, x_bf16_f32, N, K):
    """rel-L2 of sampled rows of a gathered bf16 output against the fp64 oracle over the dequantised weights
    (the oracle is the checker here, outside every timed region)."""
    import oracle
    wv = oracle.q8_dequantize_h(w_q, N * K).astype(np.float32).reshape(N, K)
    truth = oracle.matmul_truth(wv, x_bf16_f32[rows_idx], b16.astype(np.float32), 1, 1, 1, N, len(rows_idx), K, False, True, True, 1)
    want = oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(truth)).reshape(len(rows_idx), N)
    got = oracle.bf16_bits_to_f32(got_bf16_bits[rows_idx].reshape(-1)).reshape(len(rows_idx), N)
    return oracle.rel_l2(got, want)


def run_sharded(rank, world, gpu, stream, dist, torch, rows_per_batch=2048, iters=10):
    """The N-sharded bf16 prefill Linear on `world` GPUs: A bf16 [4, rows, 2560] replicated, W Q8_0H [10240, 2560] split
    along N, f16 bias, fused GELU.  Times the local slice alone, slice + NCCL all-gather, and the peer-store epilogue
    (every rank ends with the full [4*rows, 10240]); device events, max over ranks.  After the timed regions a sample of
    rows of every gathered output is compared with the oracle.  With one GPU only the compute leg exists."""
    import ratchet_b200 as rb
    from ratchet_b200 import DType, Device, GpuBuffer, Tensor
    N, K, rows, w32, b16, x32 = sharded_operands(rows_per_batch)
    qz = rb.Quantizer(rb.Quantization.SInt8)
    w = qz.sint8_quantize(Tensor.from_data(w32), DType.Q8_0H)
    b = Tensor.from_data(b16)
    x = Tensor.from_data(x32, gpu, DType.BF16)
    x_vals = rb.bf16_bits_to_f32(rb.f32_to_bf16_bits(x32)).reshape(rows, K)
    sample = np.concatenate([np.random.default_rng(5).choice(rows, size=12, replace=False), [0, rows - 1]])
    lib = rb._lib.load()

    def timed(fn):
        for _ in range(3):
            fn()
        gpu.sync()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        gpu.sync()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        if world > 1:
            t = torch.tensor([ms], device=f"cuda:{gpu.ordinal}", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms * 1e3  # us

    flops = 2.0 * rows * N * K
    res = {"workload": f"c5_q8_0_prefill_bf16_4x{rows_per_batch}_n_sharded", "n_gpus": world, "rows": rows,
           "out_bytes_gathered_per_gpu": rows * N * 2}
    if world == 1:
        node = w.to(gpu).gemm(x, b.to(gpu), False, True, True, epilogue=rb.EPILOGUE_GELU_TANH)
        node.resolve()
        plan = gpu.plan_for(node.op.desc)
        opts = rb._lib.rt_launch_opts()
        opts.flags = rb._lib.RT_LAUNCH_LHS_CONSTANT
        from ctypes import byref
        us = timed(lambda: rb._lib.check(lib.rt_matmul_launch_ex(plan, node.op.lhs.ptr, x.ptr, node.op.bias.ptr, node.ptr, None, byref(opts))))
        got = node.to(Device.CPU).to_numpy().reshape(rows, N)
        res.update({"compute_only_us": us, "tflops_compute_only": flops / us / 1e6, "kernel": lib.rt_plan_kernel(plan).decode(),
                    "parity_rel_l2": sharded_parity(got, sample, w.to_numpy(), b16, x_vals, N, K)})
        return res

    def exchange(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    lin = rb.ShardedLinear(w, b, gpu, rank, world, epilogue=rb.EPILOGUE_GELU_TANH)
    per = N // world
    local = GpuBuffer(gpu, rows * per * 2)
    gathered = GpuBuffer(gpu, rows * N * 2)
    comm = rb.Comm(gpu, rank, world, exchange)
    out_t = lin.bind_outputs(rows, DType.BF16, exchange)
    node = lin._node(x)
    plan = gpu.plan_for(node.op.desc)

    from ctypes import byref
    const_opts = rb._lib.rt_launch_opts()
    const_opts.flags = rb._lib.RT_LAUNCH_LHS_CONSTANT

    def compute_only():
        rb._lib.check(lib.rt_matmul_launch_ex(plan, lin.w.ptr, x.ptr, lin.b.ptr, local.ptr, None, byref(const_opts)))

    us_compute = timed(compute_only)
    us_nccl = timed(lambda: lin.launch_nccl(x, comm, local, gathered))
    us_comm = timed(lambda: comm.all_gather(local.ptr, gathered.ptr, rows * per * 2))  # the all-gather of ready slices alone
    # the NCCL leg gathers [world][rows][N / world]: rank r's column window of row i
    g = Tensor([world, rows, per], DType.BF16, gpu, gathered).to(Device.CPU).to_numpy()
    parity_nccl = sharded_parity(np.ascontiguousarray(np.transpose(g, (1, 0, 2))).reshape(rows, N), sample, w.to_numpy(), b16, x_vals, N, K)
    us_peer = timed(lambda: lin.launch_peer(x))
    gpu.sync()
    dist.barrier()
    full = out_t.to(Device.CPU).to_numpy().reshape(rows, N)
    parity_peer = sharded_parity(full, sample, w.to_numpy(), b16, x_vals, N, K)
    pars = exchange((float(parity_nccl), float(parity_peer)))  # every rank's; the worst is reported
    par = [max(p[0] for p in pars), max(p[1] for p in pars)]
    dist.barrier()
    lin.close_peers()
    comm.close()
    link_bytes = rows * N * 2 * (world - 1) / world  # what every GPU has to receive
    res.update({"compute_only_us": us_compute, "nccl_all_gather_only_us": us_comm, "gemm_plus_nccl_all_gather_us": us_nccl,
                "peer_store_epilogue_us": us_peer,
                # how much of the smaller of the two legs the fused form hides: 1 = the whole of it, 0 = nothing
                "peer_store_overlap": (us_compute + us_comm - us_peer) / max(min(us_compute, us_comm), 1e-3),
                "link_bound_us_at_measured_770_gbs": rows * N * 2 * (world - 1) / world / 770e3,
                "tflops_compute_only": flops / us_compute / 1e6, "tflops_nccl": flops / us_nccl / 1e6, "tflops_peer": flops / us_peer / 1e6,
                "link_ingress_bytes_per_gpu": link_bytes, "link_ingress_gbs_peer": link_bytes / us_peer / 1e3,
                "link_ingress_gbs_nccl": link_bytes / max(us_nccl - us_compute, 1e-3) / 1e3,
                "parity_rel_l2": par[1], "parity_rel_l2_nccl": par[0],
                "kernel": lib.rt_plan_kernel(plan).decode()})
    return res


def cpu_step(weights_raw, x16, layers):
    """One decode step on the CPU oracle (shader-faithful arithmetic, OpenMP)."""
    import oracle
    h = x16
    for l in range(layers):
        w1, w2 = weights_raw[l]
        h = oracle.q8h_gemv_packed(w1, D_FF, D_MODEL, h)
        h = oracle.q8h_gemv_packed(w2, D_MODEL, D_FF, h)
    return h


def time_cpu(weights_raw, x16, budget_s: float, max_layers: int):
    """Times a bounded sample of the workload: whole decode steps (all `max_layers` layers) repeated until about
    `budget_s` seconds of CPU work are done; when one step alone is longer than the budget, as many of its layers as
    fit.  Returns GB/s, the layers per pass, the passes and the seconds."""
    import oracle
    oracle.lib()
    cpu_step(weights_raw, x16, 1)  # warm-up (threads start, pages fault in)
    t0 = time.perf_counter()
    cpu_step(weights_raw, x16, 1)  # cost estimate per layer
    per_layer = time.perf_counter() - t0
    layers = int(max(1, min(max_layers, budget_s / max(per_layer, 1e-6))))
    passes = 0
    t0 = time.perf_counter()
    while True:  # whole passes until the budget is used (the per-layer estimate above is only good for choosing `layers`)
        cpu_step(weights_raw, x16, layers)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or dt + dt / passes > 1.5 * budget_s:
            break
    gbs = passes * layers * 2 * BYTES_PER_GEMV / dt / 1e9
    return gbs, layers, passes, dt


def base_config(layers):
    """The `config` object both arms print: the workload, not how an arm runs it."""
    gemvs = 2 * layers
    return {"workload": WORKLOAD, "layers": layers, "gemv_per_decode_step": gemvs, "decode_steps_per_step": REPEATS,
            "shapes": "W Q8_0H [10240,2560] and [2560,10240], x f16, M=1",
            "l2": f"inputs larger than L2: {gemvs * BYTES_PER_GEMV / 1e6:.0f} MB of distinct weights per decode step vs 126 MB L2"}


def run_reference(args, rank):
    """The reference arm: the restated reference arithmetic on the host cores (rank 0 only).  Everything here,
    the quantiser included, is the oracle's: this process never loads the CUDA library."""
    if rank != 0:
        return
    import oracle
    oracle.use_all_cores()
    raw = make_weights_oracle(args.layers, 102)
    x16 = np.random.default_rng(102).standard_normal(D_MODEL).astype(np.float16)
    t0 = time.perf_counter()
    cpu_step(raw, x16, 1)
    per_layer = time.perf_counter() - t0
    # a bounded sample of the step: as many of one decode step's layers as keep the whole run near two minutes
    layers = int(max(1, min(args.layers, 120.0 / max(args.steps + min(args.warmup, 2), 1) / max(per_layer, 1e-6))))
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_step(raw, x16, layers)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(raw, x16, layers)
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    gbs = layers * 2 * BYTES_PER_GEMV / (dt / args.steps) / 1e9
    sample = (f"{layers} of the {args.layers} layers of ONE decode step per timed step ({2 * layers} GEMVs; our arm's step is "
              f"{REPEATS} decode steps), C oracle with OpenMP")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic", "config": base_config(args.layers),
        "note": "the reference has no CPU Matmul and its WebGPU backend is unavailable on this box; this is the CPU restatement of its shader arithmetic",
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    import ratchet_b200 as rb
    from ratchet_b200 import DType, Device, DeviceRequest, Executable, PinnedArray, Tensor

    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    gpu = Device.request_device(DeviceRequest.GPU, local_rank)
    stream = torch.cuda.ExternalStream(gpu.stream, device=torch.device("cuda", local_rank))
    layers = args.layers

    # ---- operands: weights resident on the device (model state), one pinned input vector, one pinned output
    host_w = make_weights(layers, 102 + 7919 * rank)
    dev_w = [(a.to(gpu), b.to(gpu)) for a, b in host_w]
    rng = np.random.default_rng(102)
    x_pin = PinnedArray((1, 1, D_MODEL), np.float16)
    x_pin.array[...] = rng.standard_normal((1, 1, D_MODEL)).astype(np.float16)
    y_pin = PinnedArray((1, 1, D_MODEL), np.float16)

    def build_graph(x_dev):
        h, nodes = x_dev, []
        for w1, w2 in dev_w:
            h = w1.gemm(h, None, False, True, True)
            nodes.append(h)
            h = w2.gemm(h, None, False, True, True)
            nodes.append(h)
        return h, nodes

    # ---- device-timed leg: buffers bound once, one dispatch per decode step
    x_dev = Tensor.from_data(x_pin.array, gpu)
    y, nodes = build_graph(x_dev)
    y.resolve()
    kernel_names = sorted({rb._lib.load().rt_plan_kernel(gpu.plan_for(t.op.desc)).decode() for t in nodes})
    exe = Executable(gpu, nodes, use_graph=not args.no_graph)
    launches_per_decode = exe.launches

    def barrier():
        gpu.sync()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def device_timed(fn, steps, warmup):
        """`steps` timed steps of REPEATS calls each, between two events on the launching stream."""
        for _ in range(warmup * REPEATS):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps * REPEATS):
            fn()
        e1.record(stream)
        barrier()
        return e0.elapsed_time(e1)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.6)  # nvidia-smi needs a moment before its first sample
    warmup = max(args.warmup, 3)
    dev_ms = device_timed(exe.dispatch, args.steps, warmup)

    # ---- end-to-end leg: the public host API, H2D of the input and D2H of the result every decode step.
    # A decode loop keeps its Executable (the reference's models keep their compiled ops) and feeds it:
    def e2e_step():
        x_dev.write(x_pin.array)                              # H2D from pinned memory into the bound input
        exe.dispatch()                                        # the decode step
        y.to(Device.CPU, out=y_pin.array)                     # D2H of the step's result (waits)

    # the same step with the lazy graph rebuilt and resolved node by node every time (reported beside it)
    def lazy_step():
        xd = Tensor.from_data(x_pin.array, gpu)               # H2D from pinned memory
        out, _ = build_graph(xd)                              # 2*layers lazy Matmul nodes
        out.resolve(sync=False)                               # plan lookup + one launch per node
        out.to(Device.CPU, out=y_pin.array)                   # D2H of the step's result (waits)

    for _ in range(warmup * REPEATS):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev2.record(stream)
    for _ in range(args.steps * REPEATS):
        e2e_step()
    ev3.record(stream)
    barrier()
    e2e_ms = ev2.elapsed_time(ev3)                 # device timeline, host gaps included
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3  # the host's view of the same region
    y_e2e = y_pin.array.reshape(-1).copy()
    lazy_steps = 1 if args.no_lazy else 30
    for _ in range(0 if args.no_lazy else 3):
        lazy_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(lazy_steps):   # at least once: its result is compared with the executable's below
        lazy_step()
    barrier()
    lazy_ms_step = (time.perf_counter() - t0) * 1e3 / lazy_steps
    clocks = sampler.stop() if rank == 0 else None

    # the step's output must be the same through both legs, and finite
    y_dev = y.to(Device.CPU).to_numpy().reshape(-1)
    assert np.all(np.isfinite(y_dev.astype(np.float32))), "non-finite benchmark output"
    assert np.array_equal(y_dev.view(np.uint16), y_e2e.view(np.uint16)), "legs disagree"
    y_lazy = y_pin.array.reshape(-1).astype(np.float64)  # one launch per node: other kernels, another summation order
    rel = float(np.linalg.norm(y_dev.astype(np.float64) - y_lazy) / max(np.linalg.norm(y_lazy), 1e-30))
    # 64 chained GEMVs, each rounding its output to f16: last-digit differences are fed forward and grow
    # with the depth (2e-4 after three nodes, 2e-3 after 64); per-node parity is what the tests check
    assert rel <= 2e-2, f"executable and node-by-node results differ: rel-L2 {rel:.3e}"

    # ---- the same GEMVs in the forms a real graph dispatches them in (rank 0, one GPU): one launch per node, and
    # fc1 -> fc2 pairs (the longest chain of Matmul nodes in the reference's MLPs) as two-node executables
    forms = None
    if world == 1 and rank == 0:
        os.environ["RT_GEMV_CHAIN"] = "0"
        exe_nodes = Executable(gpu, nodes, use_graph=True)
        del os.environ["RT_GEMV_CHAIN"]
        ms_nodes = device_timed(exe_nodes.dispatch, max(2, args.steps // 4), 1)
        n_nodes_steps = max(2, args.steps // 4) * REPEATS
        pairs = []
        for w1, w2 in dev_w:
            h1 = w1.gemm(x_dev, None, False, True, True)
            h2 = w2.gemm(h1, None, False, True, True)
            h2.resolve()
            pairs.append(Executable(gpu, [h1, h2], use_graph=True))

        def all_pairs():
            for p in pairs:
                p.dispatch()
        ms_pairs = device_timed(all_pairs, max(2, args.steps // 4), 1)
        peak_hbm, _ = peaks()
        us_node = ms_nodes * 1e3 / n_nodes_steps / (2 * layers)
        us_pair = ms_pairs * 1e3 / n_nodes_steps / (2 * layers)
        forms = {
            "one_launch_per_node": {"us_per_gemv": us_node, "gbs": BYTES_PER_GEMV / us_node / 1e3, "frac": BYTES_PER_GEMV / us_node / 1e3 / peak_hbm,
                                    "dispatch": exe_nodes.kernel, "kernels": kernel_names},
            "two_node_fc1_fc2_executables": {"us_per_gemv": us_pair, "gbs": BYTES_PER_GEMV / us_pair / 1e3, "frac": BYTES_PER_GEMV / us_pair / 1e3 / peak_hbm,
                                             "dispatch": pairs[0].kernel, "launches_per_pair": pairs[0].launches},
        }
        del exe_nodes, pairs

    sharded = None
    if not args.no_sharded and (world > 1 or args.extras != "none"):
        sharded = [run_sharded(rank, world, gpu, stream, dist, torch, rows_per_batch=r) for r in ((2048, 8192) if world > 1 else (2048,))]
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms, e2e_wall_ms], device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms, e2e_wall_ms = (float(v) for v in t.tolist())

    if rank == 0:
        peak, peak_kind = peaks()
        gemvs = 2 * layers
        decode_bytes = gemvs * BYTES_PER_GEMV
        ms_per_step = dev_ms / args.steps
        ms_per_decode = ms_per_step / REPEATS
        value = world * decode_bytes / (ms_per_decode * 1e-3) / 1e9
        launch_us = ms_per_decode * 1e3 / gemvs
        achieved = BYTES_PER_GEMV / (launch_us * 1e-6) / 1e9
        e2e_ms_step = max(e2e_ms, e2e_wall_ms) / args.steps
        gemv_per_launch = gemvs // max(launches_per_decode, 1)
        config = base_config(layers)
        run_info = {"dispatch": exe.kernel, "kernels": kernel_names,
                    "parallelism": "replicas only (independent decode streams)" if world > 1 else "single GPU"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic", "config": config, "run": run_info,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "kernel": exe.kernel.split("_h_")[0] if exe.kernel.startswith("q8_gemv_") else kernel_names[0],
                         "gemv_per_launch": gemv_per_launch, "launch_us": launch_us * gemv_per_launch,
                         "us_per_gemv": launch_us, "bytes_per_gemv": BYTES_PER_GEMV,
                         "bytes_per_launch": BYTES_PER_GEMV * gemv_per_launch,
                         "traffic": NCU_TRAFFIC_PER_GEMV * gemv_per_launch, "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, "
                         "mean of the two shapes, from the captures summarised in profiles/q8_gemv_chain_phi2_decode.md and profiles/q8_gemv_umma_phi2_decode.md"},
            "e2e": {"value": world * decode_bytes * REPEATS / (e2e_ms_step * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms_step,
                    "h2d_bytes_per_step": int(x_pin.nbytes) * REPEATS, "d2h_bytes_per_step": int(y_pin.nbytes) * REPEATS,
                    "api": "per decode step: Tensor.write(x) + Executable.dispatch() + Tensor.to(CPU)",
                    "lazy_graph_resolve": {"value": world * decode_bytes / (lazy_ms_step * 1e-3) / 1e9, "unit": UNIT,
                                           "ms_per_decode_step": lazy_ms_step, "decode_steps": lazy_steps,
                                           "api": "Tensor.from_data(x) + 64 x gemm() + resolve() + to(CPU), one launch per node"}},
            "gpu_launches": args.steps * REPEATS * launches_per_decode,
            "clocks": clocks,
        }
        if forms is not None:
            line["dispatch_forms"] = forms
        if world == 1 and not args.no_cpu_baseline:
            import oracle
            oracle.use_all_cores()
            raw = [(a.to_numpy(), b.to_numpy()) for a, b in host_w]
            gbs, l_used, passes, dt = time_cpu(raw, x_pin.array.reshape(-1).copy(), budget_s=15.0, max_layers=layers)
            line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                                    "sample": f"{passes} passes over {l_used} of the {layers} layers of one decode step "
                                              f"({passes * 2 * l_used} GEMVs, {dt:.1f} s of CPU work), C oracle with OpenMP"}
        if sharded is not None:
            line["sharded"] = sharded
        if args.extras != "none" and world == 1:
            which = {"c1", "c3", "c4", "c5", "c5long", "mlp"} if args.extras == "all" else set(args.extras.split(","))
            line["extras"] = run_extras(which, gpu, stream)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
