"""N-sharded nn::Linear for prefill: W split along N over the GPUs of one node, one process per GPU.

The reference is single-device (crates/ratchet-core/src/gpu/device.rs:15-16); this module has no
counterpart in it.  Every rank holds rows [n0, n1) of W (and of the bias) as an ordinary tensor in
the dtype's own layout, the activations are replicated, and each rank computes the node
W_shard.gemm(x, b_shard, false, true, true) -> [rows, n1-n0] with the fused epilogue.  The slices
meet in one of two ways:

  peer   the GEMM's epilogue stores its slice straight into every rank's full-width [rows, N]
         output through CUDA-IPC-mapped pointers (plain stores over NVLink): no collective kernel,
         the transfer overlaps the remaining tiles' math.  Result layout: [rows, N] on every rank.
  nccl   the slice is written locally and ncclAllGather collects them.  Result layout:
         [world, rows, N/world] on every rank (rank-major column blocks).

The control plane (who is rank 0, exchanging the 128-byte NCCL id and the 64-byte IPC handles) is
the caller's: `exchange(obj) -> list of every rank's obj` is any all-gather of small Python objects,
e.g. torch.distributed.all_gather_object.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_void_p
from typing import Callable, List, Optional

import numpy as np

from . import _lib
from ._lib import check
from .tensor import Device, DType, GpuBuffer, RatchetError, Tensor


def shard_bounds(n: int, world: int, rank: int, align: int = 16):
    """Rows [n0, n1) of rank `rank`: equal slices, aligned so that every slice keeps 16-byte stores."""
    if n % (world * align) != 0:
        raise RatchetError(_lib.RT_ERR_SHAPE, "RT_ERR_SHAPE", f"N = {n} does not split into {world} slices of a multiple of {align}")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_rows(t: Tensor, r0: int, r1: int) -> Tensor:
    """Rows [r0, r1) of a CPU tensor [rows, k] (any dtype, block formats included) as a tensor [r1-r0, k]."""
    if t.device.is_gpu() or len(t.shape) != 2:
        raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "shard_rows takes a rank-2 CPU tensor")
    rows, k = t.shape
    src = t.storage if t.dt.is_quantized() else np.ascontiguousarray(t.to_numpy()).view(np.uint8).reshape(-1)
    out = np.empty(t.dt.nbytes((r1 - r0) * k), dtype=np.uint8)
    check(_lib.load().rt_shard_rows(int(t.dt), src.ctypes.data_as(c_void_p), rows, k, r0, r1, out.ctypes.data_as(c_void_p)))
    return Tensor([r1 - r0, k], t.dt, Device.CPU, out)


class Comm:
    """The NCCL communicator of the sharded path (rt_comm_*)."""

    def __init__(self, device: Device, rank: int, world: int, exchange: Callable, timeout_ms: int = 60000):
        lib = _lib.load()
        uid = (ctypes.c_uint8 * 128)()
        if rank == 0:
            check(lib.rt_comm_unique_id(uid))
        ids = exchange(bytes(uid))
        uid0 = (ctypes.c_uint8 * 128).from_buffer_copy(ids[0])
        self._h = c_void_p()
        check(lib.rt_comm_init_rank(device._h, world, rank, uid0, timeout_ms, byref(self._h)))
        self.rank, self.world, self.device = rank, world, device

    def all_gather(self, send_ptr: int, recv_ptr: int, bytes_per_rank: int) -> None:
        check(_lib.load().rt_comm_all_gather(self._h, send_ptr, recv_ptr, bytes_per_rank, None))

    def close(self) -> None:
        if self._h:
            _lib.load().rt_comm_destroy(self._h)
            self._h = None


class ShardedLinear:
    """Column-parallel nn::Linear.  `w` and `b` are the FULL CPU tensors; each rank keeps its slice."""

    def __init__(self, w: Tensor, b: Optional[Tensor], device: Device, rank: int, world: int, epilogue: int = 0):
        self.device, self.rank, self.world, self.epilogue = device, rank, world, epilogue
        self.n, self.k = w.shape
        self.n0, self.n1 = shard_bounds(self.n, world, rank)
        self.w = shard_rows(w, self.n0, self.n1).to(device)
        self.b = None
        if b is not None:
            vals = b.to_numpy().reshape(-1)[self.n0:self.n1]
            self.b = Tensor.from_data(np.ascontiguousarray(vals), device, b.dt)
        self._peer_ptrs: List[int] = []
        self._out: Optional[GpuBuffer] = None
        self._rows = 0
        self._act_dt = None

    # ------------------------------------------------------------------ peer mode
    def bind_outputs(self, rows: int, act_dt: DType, exchange: Callable) -> Tensor:
        """Allocates this rank's full [rows, N] output and maps every rank's copy (collective call)."""
        lib = _lib.load()
        self._rows, self._act_dt = rows, act_dt
        self._out = GpuBuffer(self.device, act_dt.nbytes(rows * self.n))
        handle = (ctypes.c_uint8 * 64)()
        check(lib.rt_ipc_export(self._out._h, handle))
        handles = exchange(bytes(handle))
        self._peer_ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self._peer_ptrs.append(self._out.ptr)
            else:
                p = c_void_p()
                check(lib.rt_ipc_open(self.device._h, (ctypes.c_uint8 * 64).from_buffer_copy(h), byref(p)))
                self._peer_ptrs.append(int(p.value))
        return Tensor([rows, self.n], act_dt, self.device, self._out)

    def _node(self, x: Tensor) -> Tensor:
        return self.w.gemm(x, self.b, False, True, True, epilogue=self.epilogue)

    def launch_peer(self, x: Tensor) -> None:
        """x: [rows, K] on this rank's device.  Enqueues the GEMM; every rank's bound output receives
        this rank's columns.  The caller synchronises all ranks before reading."""
        node = self._node(x)
        plan = self.device.plan_for(node.op.desc)
        opts = _lib.rt_launch_opts()
        opts.flags = _lib.RT_LAUNCH_LHS_CONSTANT
        opts.n_out = self.world
        for r, p in enumerate(self._peer_ptrs):
            opts.outs[r] = p
        opts.out_ld, opts.out_col = self.n, self.n0
        check(_lib.load().rt_matmul_launch_ex(plan, self.w.ptr, x.ptr, self.b.ptr if self.b is not None else None, None,
                                              None, byref(opts)))

    def close_peers(self) -> None:
        lib = _lib.load()
        for r, p in enumerate(self._peer_ptrs):
            if r != self.rank:
                lib.rt_ipc_close(self.device._h, p)
        self._peer_ptrs = []

    # ------------------------------------------------------------------ NCCL mode
    def launch_nccl(self, x: Tensor, comm: Comm, local: GpuBuffer, gathered: GpuBuffer) -> None:
        """local: [rows, N/world]; gathered: [world, rows, N/world].  Enqueues GEMM + all-gather."""
        node = self._node(x)
        plan = self.device.plan_for(node.op.desc)
        opts = _lib.rt_launch_opts()
        opts.flags = _lib.RT_LAUNCH_LHS_CONSTANT
        check(_lib.load().rt_matmul_launch_ex(plan, self.w.ptr, x.ptr, self.b.ptr if self.b is not None else None, local.ptr,
                                              None, byref(opts)))
        comm.all_gather(local.ptr, gathered.ptr, node.nbytes())
