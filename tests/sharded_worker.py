"""One rank of the multi-GPU sharded-Linear test; started by test_sharded_gpu.py under torchrun."""
import ctypes
import os
import sys
import time
from ctypes import byref, c_void_p

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
import ratchet_b200 as rb  # noqa: E402
from ratchet_b200 import DType, Device, DeviceRequest, GpuBuffer, Tensor, _lib  # noqa: E402
from util import make_lhs, round_to  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gpu = Device.request_device(DeviceRequest.GPU, local)

    def exchange(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    N, K, rows = 2048, 768, 300
    for act in (DType.F16, DType.BF16):
        w_cpu, wv = make_lhs(DType.Q8_0H, (N, K), np.random.default_rng(11), 0.02)
        bias = round_to(DType.F16, np.random.default_rng(12).standard_normal(N) * 0.02)
        x = round_to(act, np.random.default_rng(13).standard_normal((rows, K)))
        truth = oracle.matmul_truth(wv, x, bias, 1, 1, 1, N, rows, K, False, True, True, 1)
        truth_r = (oracle.f64_to_f16(truth).astype(np.float32) if act == DType.F16
                   else oracle.bf16_bits_to_f32(oracle.f64_to_bf16_bits(truth))).reshape(rows, N)
        lin = rb.ShardedLinear(w_cpu, Tensor.from_data(bias, dt=DType.F16), gpu, rank, world, epilogue=rb.EPILOGUE_GELU_TANH)
        xd = Tensor.from_data(x, gpu, act)

        # peer mode: every rank ends up with the full [rows, N]
        out = lin.bind_outputs(rows, act, exchange)
        dist.barrier()
        lin.launch_peer(xd)
        gpu.sync()
        dist.barrier()  # every rank's stores have landed
        got = out.to(Device.CPU).to_f32().reshape(rows, N)
        err = oracle.rel_l2(got, truth_r)
        assert err <= 1e-3, ("peer", act, err)
        dist.barrier()
        lin.close_peers()

        # NCCL mode: [world, rows, N/world]
        comm = rb.Comm(gpu, rank, world, exchange, timeout_ms=30000)
        per = N // world
        local_buf = GpuBuffer(gpu, act.nbytes(rows * per))
        gathered = GpuBuffer(gpu, act.nbytes(rows * N))
        lin.launch_nccl(xd, comm, local_buf, gathered)
        gpu.sync()
        g = Tensor([world, rows, per], act, gpu, gathered).to(Device.CPU).to_f32()
        got2 = g.transpose(1, 0, 2).reshape(rows, N)
        err2 = oracle.rel_l2(got2, truth_r)
        assert err2 <= 1e-3, ("nccl", act, err2)
        assert np.array_equal(got, got2), "the two modes disagree"
        comm.close()
        dist.barrier()

    # failure detection on the host: a rank that never joins costs a bounded wait and an error code
    lib = _lib.load()
    if rank == 0:
        uid = (ctypes.c_uint8 * 128)()
        _lib.check(lib.rt_comm_unique_id(uid))
        h = c_void_p()
        t0 = time.time()
        st = lib.rt_comm_init_rank(gpu._h, world, 0, uid, 1500, byref(h))
        dt = time.time() - t0
        assert st == _lib.RT_ERR_COMM_TIMEOUT, (st, lib.rt_last_error())
        assert dt < 20.0, dt
    dist.barrier()
    if rank == 0:
        print("SHARDED_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
