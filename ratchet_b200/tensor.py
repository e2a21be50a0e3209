"""Host-side mirror of ratchet-core's Tensor / Matmul / Quantizer interface for the Matmul path.

Same names, argument meaning and error behaviour as the reference, so that tests read like
the reference's own (crates/ratchet-core/src/ops/matmul.rs:757-926):

    Tensor.gemm / Tensor.matmul      crates/ratchet-core/src/tensor.rs:381-400
    Tensor.resolve / Tensor.to       crates/ratchet-core/src/tensor.rs:738-787, 864-870
    Matmul (LazyOp::Matmul)          crates/ratchet-core/src/ops/matmul.rs:248-282
    Quantizer.sint8_quantize         crates/ratchet-core/src/quant.rs:26-124
    DType.segments                   crates/ratchet-core/src/dtype/mod.rs:85-95

Every rule and every byte of arithmetic lives in libratchet_b200.so; this module only holds
handles, builds descriptors and calls the C ABI.  Invariant violations, which panic in the
reference, raise InvariantError here; shape errors raise ShapeError.
"""
from __future__ import annotations

import ctypes
import enum
import os
from ctypes import byref, c_int32, c_uint64, c_void_p
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import InvariantError, RatchetError, ShapeError, check  # noqa: F401  (re-exported)


class DType(enum.IntEnum):
    F32 = _lib.RT_F32
    F16 = _lib.RT_F16
    BF16 = _lib.RT_BF16
    I32 = _lib.RT_I32
    U32 = _lib.RT_U32
    Q8_0H = _lib.RT_Q8_0H
    Q8_0F = _lib.RT_Q8_0F
    Q4_K = _lib.RT_Q4_K

    def size_of(self) -> int:
        return int(_lib.load().rt_dtype_size(int(self)))

    def is_quantized(self) -> bool:
        return bool(_lib.load().rt_dtype_is_quantized(int(self)))

    def activation_dt(self) -> "DType":
        out = c_int32()
        check(_lib.load().rt_dtype_activation(int(self), byref(out)))
        return DType(out.value)

    def segments(self, numel: int):
        segs = (_lib.rt_segment * 4)()
        n = c_int32(4)
        check(_lib.load().rt_dtype_segments(int(self), int(numel), segs, byref(n)))
        return [(int(segs[i].offset), int(segs[i].size)) for i in range(n.value)]

    def nbytes(self, numel: int) -> int:
        out = c_uint64()
        check(_lib.load().rt_dtype_nbytes(int(self), int(numel), byref(out)))
        return int(out.value)

    def numpy(self):
        return {DType.F32: np.float32, DType.F16: np.float16, DType.BF16: np.uint16,
                DType.I32: np.int32, DType.U32: np.uint32}.get(self, np.uint8)


_NP_TO_DT = {np.dtype(np.float32): DType.F32, np.dtype(np.float16): DType.F16,
             np.dtype(np.int32): DType.I32, np.dtype(np.uint32): DType.U32}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round f32 to bf16 (nearest even); returns the 16-bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7FC0
    return r


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# environment switches that change which kernel a plan takes (the library's cache key holds them too)
_ROUTING_SWITCHES = ("RT_FORCE_KERNEL", "RT_GEMV_UMMA", "RT_Q4K_UMMA", "RT_GEMM_PAIR", "RT_GEMM_PAIR_MIN", "RT_TF32_BN",
                     "RT_TF32_PRESPLIT", "RT_Q4K_WALK_FROM", "RT_KEEP_WEIGHTS")


class DeviceRequest(enum.Enum):
    CPU = "cpu"
    GPU = "gpu"


class Device:
    """Device::CPU holds data only; Device::GPU owns a CUDA device + stream (device.rs:25-80)."""

    CPU: "Device"
    _gpus: dict = {}

    def __init__(self, kind: DeviceRequest, ordinal: int = 0, handle=None):
        self.kind = kind
        self.ordinal = ordinal
        self._h = handle
        self._plans = {}

    @classmethod
    def request_device(cls, req: DeviceRequest, ordinal: Optional[int] = None) -> "Device":
        if req == DeviceRequest.CPU:
            return cls.CPU
        if ordinal is None:
            ordinal = int(os.environ.get("LOCAL_RANK", "0")) if "RT_USE_LOCAL_RANK" in os.environ else 0
        if ordinal not in cls._gpus:
            h = c_void_p()
            check(_lib.load().rt_device_create(ordinal, byref(h)))
            cls._gpus[ordinal] = cls(DeviceRequest.GPU, ordinal, h)
        return cls._gpus[ordinal]

    def is_gpu(self) -> bool:
        return self.kind == DeviceRequest.GPU

    def try_gpu(self) -> "Device":
        if not self.is_gpu():
            raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "DeviceError: expected a GPU device")
        return self

    def sync(self) -> None:
        check(_lib.load().rt_device_sync(self._h))

    @property
    def stream(self) -> int:
        return int(_lib.load().rt_device_stream(self._h) or 0)

    @property
    def sm_count(self) -> int:
        return int(_lib.load().rt_device_sm_count(self._h))

    def plan_for(self, desc: "_lib.rt_matmul_desc"):
        """The compiled-op cache: one plan per distinct node description (the KernelKey's role)."""
        # The library keeps the cache (keyed by the description and by the routing switches of the environment); this
        # memo only saves the two calls per node on the lazy path.  The hold rt_matmul_plan takes goes straight back:
        # the device's own keeps the plan alive as long as the device lives.
        key = (bytes(desc), tuple(os.environ.get(n) for n in _ROUTING_SWITCHES))
        h = self._plans.get(key)
        if h is None:
            h = c_void_p()
            check(_lib.load().rt_matmul_plan(self._h, byref(desc), byref(h)))
            check(_lib.load().rt_plan_destroy(h))
            self._plans[key] = h
        return h

    def __repr__(self):
        return "Device::CPU" if not self.is_gpu() else f"Device::GPU({self.ordinal})"


Device.CPU = Device(DeviceRequest.CPU)


class PinnedArray:
    """Page-locked host memory viewed as a numpy array (for copies that overlap compute)."""

    def __init__(self, shape, dtype):
        self.nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        self._p = c_void_p()
        check(_lib.load().rt_host_alloc(self.nbytes, byref(self._p)))
        buf = (ctypes.c_uint8 * max(self.nbytes, 1)).from_address(self._p.value)
        self.array = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def __del__(self):
        try:
            if self._p:
                _lib.load().rt_host_free(self._p)
                self._p = None
        except Exception:
            pass


class GpuBuffer:
    def __init__(self, device: Device, nbytes: int):
        self.device = device
        self._h = c_void_p()
        check(_lib.load().rt_buffer_alloc(device._h, int(nbytes), byref(self._h)))
        self.ptr = int(_lib.load().rt_buffer_ptr(self._h) or 0)
        self.size = int(_lib.load().rt_buffer_size(self._h))

    @classmethod
    def adopt(cls, device: Device, handle: c_void_p) -> "GpuBuffer":
        """Take ownership of an rt_buffer the library allocated (e.g. rt_gguf_load_tensor)."""
        b = cls.__new__(cls)
        b.device = device
        b._h = handle
        b.ptr = int(_lib.load().rt_buffer_ptr(handle) or 0)
        b.size = int(_lib.load().rt_buffer_size(handle))
        return b

    def __del__(self):
        try:
            if self._h:
                _lib.load().rt_buffer_free(self._h)
                self._h = None
        except Exception:
            pass


class Executable:
    """Executable (executable.rs:13-54): resolved nodes with their buffers bound, dispatched in one
    call.  Built from tensors whose graph has already been resolved once (so every node owns its
    output buffer); re-dispatching recomputes the same buffers in place."""

    def __init__(self, device: Device, nodes: Sequence["Tensor"], use_graph: bool = True):
        self.device = device
        self._keep = list(nodes)
        arr = (_lib.rt_dispatch * len(nodes))()
        for i, t in enumerate(nodes):
            if t.op is None or not isinstance(t.storage, GpuBuffer):
                raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "Executable nodes must be resolved op outputs")
            arr[i].plan = device.plan_for(t.op.desc)
            arr[i].lhs, arr[i].rhs = t.op.lhs.ptr, t.op.rhs.ptr
            arr[i].bias = t.op.bias.ptr if t.op.bias is not None else None
            arr[i].out = t.ptr
            arr[i].opts.flags = _lib.RT_LAUNCH_LHS_CONSTANT if t.op.lhs.op is None else 0
        self._h = c_void_p()
        check(_lib.load().rt_executable_create(device._h, arr, len(nodes), int(use_graph), byref(self._h)))
        self.launches = int(_lib.load().rt_executable_launches(self._h))
        self.kernel = _lib.load().rt_executable_kernel(self._h).decode()

    @classmethod
    def _adopt(cls, device: Device, handle: c_void_p, keep) -> "Executable":
        self = cls.__new__(cls)
        self.device, self._keep, self._h = device, list(keep), handle
        self.launches = int(_lib.load().rt_executable_launches(handle))
        self.kernel = _lib.load().rt_executable_kernel(handle).decode()
        return self

    @classmethod
    def planned(cls, device: Device, nodes: Sequence[dict], tensor_bytes: Sequence[int], use_graph: bool = True,
                keep=()) -> "Executable":
        """An executable whose intermediates the library places in one arena (the reference's
        BufferAllocator::allocate_cfg, allocator.rs:273-340).  Each node is a dict with `plan`
        and, per operand lhs / rhs / bias / out, either a device pointer (int) or ("t", k) naming
        intermediate k; `flags` optional."""
        n = len(nodes)
        arr = (_lib.rt_dispatch * n)()
        ids = (_lib.rt_node_tensors * n)()
        for i, nd in enumerate(nodes):
            arr[i].plan = nd["plan"]
            arr[i].opts.flags = int(nd.get("flags", 0))
            for name in ("lhs", "rhs", "bias", "out"):
                v = nd.get(name)
                if isinstance(v, tuple):
                    setattr(ids[i], name, int(v[1]))
                else:
                    setattr(ids[i], name, -1)
                    setattr(arr[i], name, v)
        sizes = (ctypes.c_uint64 * max(1, len(tensor_bytes)))(*[int(b) for b in tensor_bytes])
        h = c_void_p()
        check(_lib.load().rt_executable_create_planned(device._h, arr, ids, n, sizes, len(tensor_bytes), int(use_graph), byref(h)))
        return cls._adopt(device, h, keep)

    def arena(self) -> dict:
        """Size of the executable's arena, the shared objects in it, and what its records add up to."""
        a, o, r = ctypes.c_uint64(), ctypes.c_int32(), ctypes.c_uint64()
        check(_lib.load().rt_executable_arena(self._h, byref(a), byref(o), byref(r)))
        return {"arena_bytes": int(a.value), "objects": int(o.value), "record_bytes": int(r.value)}

    def tensor_ptr(self, k: int) -> int:
        return int(_lib.load().rt_executable_tensor(self._h, k) or 0)

    def dispatch(self) -> None:
        check(_lib.load().rt_executable_dispatch(self._h, None))

    def __del__(self):
        try:
            if self._h:
                _lib.load().rt_executable_destroy(self._h)
                self._h = None
        except Exception:
            pass


class Matmul:
    """LazyOp::Matmul (ops/matmul.rs:248-282).  `epilogue` is this library's extension."""

    def __init__(self, lhs: "Tensor", rhs: "Tensor", bias: Optional["Tensor"], trans_lhs: bool, trans_rhs: bool,
                 trans_out: bool, epilogue: int = _lib.RT_EPILOGUE_NONE):
        self.lhs, self.rhs, self.bias = lhs, rhs, bias
        self.trans_lhs, self.trans_rhs, self.trans_out = bool(trans_lhs), bool(trans_rhs), bool(trans_out)
        self.epilogue = int(epilogue)
        self.desc = self._desc()
        # Matmul::new guards, check_shapes, check_dtypes: all evaluated by the library
        self.spec = _lib.rt_gemm_spec()
        check(_lib.load().rt_matmul_spec(byref(self.desc), byref(self.spec)))

    def _desc(self) -> "_lib.rt_matmul_desc":
        d = _lib.rt_matmul_desc()
        d.lhs_dt, d.rhs_dt = int(self.lhs.dt), int(self.rhs.dt)
        d.lhs_shape, d.rhs_shape = _lib.rt_shape.of(self.lhs.shape), _lib.rt_shape.of(self.rhs.shape)
        d.has_bias = int(self.bias is not None)
        if self.bias is not None:
            d.bias_dt = int(self.bias.dt)
            d.bias_shape = _lib.rt_shape.of(self.bias.shape)
        d.trans_lhs, d.trans_rhs, d.trans_out = int(self.trans_lhs), int(self.trans_rhs), int(self.trans_out)
        d.epilogue = self.epilogue
        return d

    @staticmethod
    def compute_c_shape(a_shape: Sequence[int], b_shape: Sequence[int], trans_lhs: bool, trans_rhs: bool,
                        trans_out: bool):
        d = _lib.rt_matmul_desc()
        d.lhs_shape, d.rhs_shape = _lib.rt_shape.of(a_shape), _lib.rt_shape.of(b_shape)
        d.trans_lhs, d.trans_rhs, d.trans_out = int(trans_lhs), int(trans_rhs), int(trans_out)
        out = _lib.rt_shape()
        check(_lib.load().rt_matmul_out_shape(byref(d), byref(out)))
        return out.tolist()

    def srcs(self):
        return [self.lhs, self.rhs] + ([self.bias] if self.bias is not None else [])


class Tensor:
    """An immutable, possibly lazy tensor (tensor.rs:40-133)."""

    def __init__(self, shape: Sequence[int], dt: DType, device: Device, storage=None, op: Optional[Matmul] = None):
        self.shape = [int(s) for s in shape]
        self.dt = DType(dt)
        self.device = device
        self.storage = storage  # np.uint8 array (CPU) or GpuBuffer (GPU) or None (unresolved)
        self.op = op

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def from_data(data, device: Device = None, dt: Optional[DType] = None) -> "Tensor":
        """Tensor::from_data.  `dt=DType.BF16` rounds f32 data to bf16."""
        device = device or Device.CPU
        arr = np.ascontiguousarray(data)
        if dt == DType.BF16:
            arr = f32_to_bf16_bits(arr.astype(np.float32)).reshape(arr.shape)
        elif dt is not None:
            arr = arr.astype(DType(dt).numpy(), copy=False)
        else:
            if arr.dtype == np.float64:
                arr = arr.astype(np.float32)
            if arr.dtype not in _NP_TO_DT:
                raise RatchetError(_lib.RT_ERR_DTYPE, "RT_ERR_DTYPE", f"unsupported numpy dtype {arr.dtype}")
            dt = _NP_TO_DT[arr.dtype]
        raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        t = Tensor(arr.shape, dt, Device.CPU, raw)
        return t if not device.is_gpu() else t.to(device)

    @staticmethod
    def randn(shape: Sequence[int], device: Device = None, dt: DType = DType.F32, seed: Optional[int] = None) -> "Tensor":
        """Tensor::randn (tensor.rs:516-532): standard normal, seedable (RATCHET_SEED in the reference)."""
        if seed is None and "RATCHET_SEED" in os.environ:
            seed = int(os.environ["RATCHET_SEED"])
        rng = np.random.default_rng(seed)
        return Tensor.from_data(rng.standard_normal(tuple(shape)).astype(np.float32), device, dt)

    @staticmethod
    def from_quantized(data, dt: DType, shape: Sequence[int], device: Device = None) -> "Tensor":
        """Tensor::from_quantized (tensor.rs:589-599): raw bytes in the dtype's segment layout."""
        device = device or Device.CPU
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        want = DType(dt).nbytes(int(np.prod(shape)))
        if raw.size != want:
            raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", f"{dt.name} tensor of shape {list(shape)} needs {want} bytes, got {raw.size}")
        t = Tensor(shape, dt, Device.CPU, raw)
        return t if not device.is_gpu() else t.to(device)

    # ------------------------------------------------------------------ properties
    def numel(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1

    def rank(self) -> int:
        return len(self.shape)

    def resolved(self) -> bool:
        return self.storage is not None

    def nbytes(self) -> int:
        return self.dt.nbytes(self.numel())

    @property
    def ptr(self) -> int:
        if not isinstance(self.storage, GpuBuffer):
            raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "tensor has no device storage")
        return self.storage.ptr

    # ------------------------------------------------------------------ ops
    def gemm(self, rhs: "Tensor", bias: Optional["Tensor"], trans_lhs: bool, trans_rhs: bool, trans_out: bool,
             epilogue: int = _lib.RT_EPILOGUE_NONE) -> "Tensor":
        """Tensor::gemm (tensor.rs:388-400): self is the lhs."""
        op = Matmul(self, rhs, bias, trans_lhs, trans_rhs, trans_out, epilogue)
        return Tensor(op.spec.out_shape.tolist(), DType(op.spec.out_dt), rhs.device, None, op)

    def matmul(self, rhs: "Tensor", trans_lhs: bool = False, trans_rhs: bool = False) -> "Tensor":
        """Tensor::matmul (tensor.rs:381-386)."""
        return self.gemm(rhs, None, trans_lhs, trans_rhs, False)

    # ------------------------------------------------------------------ execution
    def execution_order(self):
        """Post-order over the op graph (tensor.rs:667-711)."""
        order, seen, stack = [], set(), [(self, False)]
        while stack:
            t, done = stack.pop()
            if done:
                order.append(t)
                continue
            if id(t) in seen:
                continue
            seen.add(id(t))
            stack.append((t, True))
            if t.op is not None and not t.resolved():
                for s in reversed(t.op.srcs()):
                    stack.append((s, False))
        return order

    def resolve(self, sync: bool = True) -> "Tensor":
        """Tensor::resolve (tensor.rs:738-787): plan + dispatch every unresolved node, then wait."""
        device = self.device.try_gpu()
        lib = _lib.load()
        todo = [t for t in self.execution_order() if not t.resolved()]
        for t in todo:
            if t.op is None:
                raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "unresolved tensor without an op")
            for s in t.op.srcs():
                if s.resolved() and (not isinstance(s.storage, GpuBuffer) or s.device is not device):
                    raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG",
                                       f"TensorError: operand on {s.device}, expected {device}")
        for i, t in enumerate(todo):
            op = t.op
            plan = device.plan_for(op.desc)
            out = GpuBuffer(device, t.nbytes())
            opts = _lib.rt_launch_opts()
            # a leaf lhs is a constant of the graph (uploaded weights): nothing in flight writes it
            if op.lhs.op is None:
                opts.flags = _lib.RT_LAUNCH_LHS_CONSTANT
            check(lib.rt_matmul_launch_ex(plan, op.lhs.ptr, op.rhs.ptr, op.bias.ptr if op.bias is not None else None,
                                          out.ptr, None, byref(opts)))
            t.storage = out
        if sync:
            device.sync()
        return self

    def to(self, device: Device, out: Optional[np.ndarray] = None) -> "Tensor":
        """Tensor::to (tensor.rs:864-870).  GPU->CPU may write into `out` (e.g. a pinned array)."""
        lib = _lib.load()
        if device is self.device or (not device.is_gpu() and not self.device.is_gpu()):
            return self
        if not self.resolved():
            raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "TensorError: tensor is not resolved")
        if device.is_gpu() and not self.device.is_gpu():
            buf = GpuBuffer(device, self.nbytes())
            raw = self.storage
            check(lib.rt_upload(device._h, buf._h, 0, raw.ctypes.data_as(c_void_p), raw.size, 1))
            return Tensor(self.shape, self.dt, device, buf)
        if not device.is_gpu() and self.device.is_gpu():
            n = self.nbytes()
            raw = out.view(np.uint8).reshape(-1) if out is not None else np.empty(n, dtype=np.uint8)
            if raw.size < n:
                raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "output array too small")
            check(lib.rt_download(self.device._h, self.storage._h, 0, raw.ctypes.data_as(c_void_p), n, 1))
            return Tensor(self.shape, self.dt, Device.CPU, raw[:n])
        raise RatchetError(_lib.RT_ERR_UNSUPPORTED, "RT_ERR_UNSUPPORTED", "GPU to GPU moves are not part of this path")

    def write(self, data: np.ndarray) -> "Tensor":
        """Overwrites a resolved GPU tensor's bytes from host memory (queue.write_buffer on the tensor's
        own storage): how a caller feeds new input to an Executable whose buffers are bound."""
        if not self.device.is_gpu() or not isinstance(self.storage, GpuBuffer):
            raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "write takes a resolved GPU tensor")
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        if raw.size != self.nbytes():
            raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", f"write: {raw.size} bytes for a tensor of {self.nbytes()}")
        check(_lib.load().rt_upload(self.device._h, self.storage._h, 0, raw.ctypes.data_as(c_void_p), raw.size, 0))
        return self

    # ------------------------------------------------------------------ host views
    def to_numpy(self) -> np.ndarray:
        """CPU tensor -> numpy array (bf16 as uint16 bit patterns, block formats as raw bytes)."""
        if self.device.is_gpu():
            return self.to(Device.CPU).to_numpy()
        if self.dt.is_quantized():
            return self.storage
        n = self.numel()
        return self.storage[: n * self.dt.size_of()].view(self.dt.numpy()).reshape(self.shape)

    def to_f32(self) -> np.ndarray:
        a = self.to_numpy()
        if self.dt == DType.BF16:
            return bf16_bits_to_f32(a).reshape(self.shape)
        if self.dt.is_quantized():
            return Quantizer.dequantize_bytes(a, self.dt, self.numel()).reshape(self.shape)
        return a.astype(np.float32)

    def dequantize_on_device(self) -> np.ndarray:
        """Decode a block-format device tensor with the kernels' own decoder (parity hook)."""
        device = self.device.try_gpu()
        out_dt = DType.F16 if self.dt == DType.Q8_0H else DType.F32
        out = GpuBuffer(device, out_dt.nbytes(self.numel()))
        check(_lib.load().rt_dequantize_device(device._h, int(self.dt), self.numel(), self.ptr, out.ptr, None))
        return Tensor(self.shape, out_dt, device, out).to(Device.CPU).to_numpy()

    def __repr__(self):
        return f"Tensor(shape={self.shape}, dt={self.dt.name}, device={self.device}, resolved={self.resolved()})"


class Quantization(enum.Enum):
    NONE = 0
    SInt8 = 1
    SInt4 = 2


class Quantizer:
    """Quantizer (quant.rs:8-24)."""

    def __init__(self, format: Quantization):
        self.format = format

    def quantize(self, tensor: Tensor) -> Tensor:
        if self.format == Quantization.NONE:
            return tensor
        if self.format == Quantization.SInt8:
            return self.sint8_quantize(tensor)
        raise NotImplementedError("Quantization::SInt4 is todo!() in the reference (quant.rs:21)")

    def sint8_quantize(self, tensor: Tensor, dt: DType = DType.Q8_0F) -> Tensor:
        """f32 CPU tensor -> Q8_0F (quant.rs:26-79); dt=Q8_0H keeps the codes and rounds d to f16."""
        if tensor.dt != DType.F32 or tensor.device.is_gpu():
            raise InvariantError(_lib.RT_ERR_INVARIANT, "RT_ERR_INVARIANT", "sint8_quantize needs an f32 CPU tensor")
        x = tensor.to_numpy().reshape(-1)
        if x.size % 32 != 0:
            raise InvariantError(_lib.RT_ERR_INVARIANT, "RT_ERR_INVARIANT", "numel must be a multiple of 32")
        out = np.empty(dt.nbytes(x.size), dtype=np.uint8)
        check(_lib.load().rt_quantize_q8_0(x.ctypes.data_as(c_void_p), x.size, int(dt), out.ctypes.data_as(c_void_p)))
        return Tensor(tensor.shape, dt, Device.CPU, out)

    def sint8_dequantize(self, quantized: Tensor) -> Tensor:
        """quant.rs:81-124"""
        if quantized.dt not in (DType.Q8_0F, DType.Q8_0H):
            raise InvariantError(_lib.RT_ERR_INVARIANT, "RT_ERR_INVARIANT", "expected a Q8_0 tensor")
        vals = self.dequantize_bytes(quantized.to_numpy(), quantized.dt, quantized.numel())
        return Tensor.from_data(vals.reshape(quantized.shape))

    @staticmethod
    def q4k_quantize(tensor: Tensor) -> Tensor:
        x = tensor.to_numpy().reshape(-1).astype(np.float32)
        out = np.empty(DType.Q4_K.nbytes(x.size), dtype=np.uint8)
        check(_lib.load().rt_quantize_q4_k(x.ctypes.data_as(c_void_p), x.size, out.ctypes.data_as(c_void_p)))
        return Tensor(tensor.shape, DType.Q4_K, Device.CPU, out)

    @staticmethod
    def dequantize_bytes(raw: np.ndarray, dt: DType, numel: int) -> np.ndarray:
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(numel, dtype=np.float32)
        lib = _lib.load()
        if dt == DType.Q4_K:
            check(lib.rt_dequantize_q4_k(raw.ctypes.data_as(c_void_p), numel, out.ctypes.data_as(c_void_p)))
        else:
            check(lib.rt_dequantize_q8_0(raw.ctypes.data_as(c_void_p), numel, int(dt), out.ctypes.data_as(c_void_p)))
        return out


def transcode_gguf_q8_0(blocks: np.ndarray, shape: Sequence[int], dt: DType = DType.Q8_0H, device: Device = None) -> Tensor:
    """GGUFInterop::transcode for Q8_0 (crates/ratchet-loader/src/gguf/dtype.rs:44-110)."""
    raw = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    n_blocks = raw.size // 34
    if raw.size % 34 != 0 or n_blocks * 32 != int(np.prod(shape)):
        raise RatchetError(_lib.RT_ERR_ARG, "RT_ERR_ARG", "block bytes do not match the shape")
    out = np.empty(dt.nbytes(n_blocks * 32), dtype=np.uint8)
    check(_lib.load().rt_transcode_gguf_q8_0(raw.ctypes.data_as(c_void_p), n_blocks, int(dt), out.ctypes.data_as(c_void_p)))
    return Tensor.from_quantized(out, dt, shape, device or Device.CPU)


class Linear:
    """nn::Linear (crates/ratchet-nn/src/linear.rs:10-25): y = x W^T + b as W.gemm(x, b, false, true, true).

    The reference casts the bias to the input dtype with a Cast op on every call; here the cast
    happens once on the host and the device copy is cached per dtype."""

    def __init__(self, w: Tensor, b: Optional[Tensor] = None, epilogue: int = _lib.RT_EPILOGUE_NONE):
        self.w, self.b, self.epilogue = w, b, epilogue
        self._b_cast = {}

    def _bias_for(self, dt: DType, device: Device) -> Optional[Tensor]:
        if self.b is None:
            return None
        if self.b.dt == dt and self.b.device is device:
            return self.b
        key = (dt, id(device))
        if key not in self._b_cast:
            vals = self.b.to(Device.CPU).to_f32()
            self._b_cast[key] = Tensor.from_data(vals, device, dt)
        return self._b_cast[key]

    def schedule(self, input: Tensor) -> Tensor:
        return self.w.gemm(input, self._bias_for(input.dt, input.device), False, True, True, self.epilogue)


class MLP:
    """The MLP block of the reference's models as ONE executable: hidden = act(fc1(x)), out = fc2(hidden).

    `act` "gelu": Phi-2 `l2(l1(x).gelu())` (crates/ratchet-models/src/phi2/mlp.rs:13-15) and Whisper /
    Moondream `fc2(fc1(x).full().gelu().cast())` (whisper/mlp.rs:18-22); `act` "silu_gate": Phi-3
    `down(up * silu(gate.full()).cast())` with fc1 the gate_up projection (phi3/mlp.rs:31-39).
    The hidden tensor is an intermediate of the executable placed by the activation planner."""

    def __init__(self, fc1: Linear, fc2: Linear, act: str = "gelu"):
        if act not in ("gelu", "silu_gate"):
            raise ValueError(act)
        self.fc1, self.fc2, self.act = fc1, fc2, act
        self._exe = {}

    def _desc(self, lin: Linear, x_shape, x_dt: DType, device: Device, epilogue: int) -> "_lib.rt_matmul_desc":
        b = lin._bias_for(x_dt, device)
        d = _lib.rt_matmul_desc()
        d.lhs_dt, d.rhs_dt = int(lin.w.dt), int(x_dt)
        d.lhs_shape, d.rhs_shape = _lib.rt_shape.of(lin.w.shape), _lib.rt_shape.of(x_shape)
        d.has_bias = 0 if b is None else 1
        if b is not None:
            d.bias_dt, d.bias_shape = int(b.dt), _lib.rt_shape.of(b.shape)
        d.trans_lhs, d.trans_rhs, d.trans_out, d.epilogue = 0, 1, 1, epilogue
        return d

    def bind(self, x: Tensor, use_graph: bool = True):
        """(executable, out tensor) for this input tensor; the executable recomputes `out` from the
        current contents of `x` at every dispatch."""
        key = (x.ptr, tuple(x.shape), int(x.dt), use_graph)
        if key in self._exe:
            return self._exe[key]
        dev = x.device
        epi = _lib.RT_EPILOGUE_GELU_TANH if self.act == "gelu" else _lib.RT_EPILOGUE_SILU_MUL
        m = _lib.rt_mlp_desc()
        m.fc1 = self._desc(self.fc1, x.shape, x.dt, dev, epi)
        hid = _lib.rt_shape()
        check(_lib.load().rt_matmul_out_shape(byref(m.fc1), byref(hid)))
        m.fc2 = self._desc(self.fc2, hid.tolist(), x.dt, dev, _lib.RT_EPILOGUE_NONE)
        out_shape = _lib.rt_shape()
        check(_lib.load().rt_matmul_out_shape(byref(m.fc2), byref(out_shape)))
        out = Tensor(out_shape.tolist(), x.dt, dev, GpuBuffer(dev, x.dt.nbytes(int(np.prod(out_shape.tolist())))))
        b1, b2 = self.fc1._bias_for(x.dt, dev), self.fc2._bias_for(x.dt, dev)
        m.w1, m.w2, m.x, m.out = self.fc1.w.ptr, self.fc2.w.ptr, x.ptr, out.ptr
        m.b1 = b1.ptr if b1 is not None else None
        m.b2 = b2.ptr if b2 is not None else None
        h = c_void_p()
        check(_lib.load().rt_mlp_create(dev._h, byref(m), int(use_graph), byref(h)))
        exe = Executable._adopt(dev, h, [x, out, b1, b2, self.fc1.w, self.fc2.w])
        self._exe[key] = (exe, out)
        return exe, out

    def schedule(self, input: Tensor) -> Tensor:
        """Module::schedule + resolve in one: dispatches the block and returns its output tensor."""
        exe, out = self.bind(input)
        exe.dispatch()
        return out
