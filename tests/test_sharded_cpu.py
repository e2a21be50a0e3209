"""Host-side logic of the N-sharded Linear with world_size 2 over gloo (CPU only, no GPU).

Checks what does not need a GPU: the slice bounds, that the shards (repacked in each dtype's own
layout) reassemble to the full tensor when the ranks exchange them, and that the two result layouts
of the sharded path ([rows, N] in peer mode, [world, rows, N/world] after the all-gather) reassemble
the oracle's full output from the oracle's per-shard outputs.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import oracle
    import ratchet_b200 as rb
    from ratchet_b200 import DType, Tensor

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, K, rows = 128, 96, 10
        rng = np.random.default_rng(7)  # same data on every rank
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        x = rng.standard_normal((rows, K)).astype(np.float16).astype(np.float32)
        bias = (rng.standard_normal(N) * 0.02).astype(np.float16).astype(np.float32)
        n0, n1 = rb.shard_bounds(N, world, rank)
        assert (n0, n1) == (rank * N // world, (rank + 1) * N // world)
        for dt in (DType.Q8_0H, DType.Q8_0F, DType.Q4_K if K % 256 == 0 else DType.F16, DType.F32):
            full = {DType.Q8_0H: lambda: Tensor.from_quantized(oracle.q8_quantize_h(w), dt, (N, K)),
                    DType.Q8_0F: lambda: Tensor.from_quantized(oracle.q8_quantize_f(w), dt, (N, K)),
                    DType.F16: lambda: Tensor.from_data(w.astype(np.float16)),
                    DType.F32: lambda: Tensor.from_data(w)}[dt]()
            shard = rb.shard_rows(full, n0, n1)
            assert shard.shape == [n1 - n0, K] and shard.nbytes() == dt.nbytes((n1 - n0) * K)
            # exchange the shards' values: together they are the full tensor
            vals = shard.to_f32().reshape(-1)
            got = [None] * world
            dist.all_gather_object(got, vals)
            assert np.array_equal(np.concatenate(got), full.to_f32().reshape(-1)), dt
        # result layouts: per-shard oracle outputs -> full output
        wq = Tensor.from_quantized(oracle.q8_quantize_h(w), DType.Q8_0H, (N, K))
        wv = wq.to_f32()
        truth = oracle.matmul_truth(wv, x, bias, 1, 1, 1, N, rows, K, False, True, True, 1).reshape(rows, N)
        part = oracle.matmul_truth(wv[n0:n1], x, bias[n0:n1], 1, 1, 1, n1 - n0, rows, K, False, True, True, 1).reshape(rows, n1 - n0)
        parts = [None] * world
        dist.all_gather_object(parts, part)
        gathered = np.stack(parts)                       # [world, rows, N/world]  (NCCL mode)
        peer = np.concatenate(parts, axis=1)             # [rows, N]              (peer mode: column offset n0)
        assert np.array_equal(peer, truth)
        assert np.array_equal(gathered.transpose(1, 0, 2).reshape(rows, N), truth)
        # a slice that would break 16-byte stores is refused
        with pytest.raises(rb.RatchetError):
            rb.shard_bounds(100, world, rank)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_sharded_host_logic_world2_gloo():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}
