"""ctypes binding of libratchet_b200.so (the C ABI declared in include/ratchet_b200.h).

The library is the product: if it is missing this module raises, it never substitutes a
CPU or PyTorch implementation.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, byref, c_char_p, c_float, c_int32, c_int64, c_size_t,
                    c_uint64, c_void_p)

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libratchet_b200.so")

RT_MAX_RANK = 8

# rt_status
RT_OK, RT_ERR_SHAPE, RT_ERR_DTYPE, RT_ERR_INVARIANT, RT_ERR_ARG, RT_ERR_CUDA, RT_ERR_UNSUPPORTED, \
    RT_ERR_NOMEM, RT_ERR_COMM, RT_ERR_COMM_TIMEOUT = range(10)

# rt_dtype
RT_F32, RT_F16, RT_BF16, RT_I32, RT_U32, RT_Q8_0H, RT_Q8_0F, RT_Q4_K = range(8)

RT_EPILOGUE_NONE, RT_EPILOGUE_GELU_TANH, RT_EPILOGUE_SILU_MUL = 0, 1, 2
RT_LAUNCH_LHS_CONSTANT = 1


class rt_shape(Structure):
    _fields_ = [("rank", c_int32), ("dims", c_int64 * RT_MAX_RANK)]

    @classmethod
    def of(cls, dims):
        s = cls()
        dims = list(dims)
        if len(dims) > RT_MAX_RANK:
            raise ValueError(f"rank {len(dims)} exceeds {RT_MAX_RANK}")
        s.rank = len(dims)
        for i, d in enumerate(dims):
            s.dims[i] = int(d)
        return s

    def tolist(self):
        return [int(self.dims[i]) for i in range(self.rank)]


class rt_segment(Structure):
    _fields_ = [("offset", c_uint64), ("size", c_uint64)]


class rt_matmul_desc(Structure):
    _fields_ = [("lhs_dt", c_int32), ("rhs_dt", c_int32), ("bias_dt", c_int32),
                ("lhs_shape", rt_shape), ("rhs_shape", rt_shape), ("bias_shape", rt_shape),
                ("has_bias", c_int32), ("trans_lhs", c_int32), ("trans_rhs", c_int32),
                ("trans_out", c_int32), ("epilogue", c_int32)]


class rt_gemm_spec(Structure):
    _fields_ = [("out_shape", rt_shape), ("out_dt", c_int32),
                ("lhs_stack", c_int64), ("rhs_stack", c_int64), ("out_stack", c_int64), ("stacks", c_int64),
                ("dim_lhs_outer", c_int64), ("dim_rhs_outer", c_int64), ("dim_inner", c_int64),
                ("is_gemv", c_int32)]


class rt_launch_opts(Structure):
    _fields_ = [("flags", ctypes.c_uint32), ("n_out", c_int32), ("outs", c_void_p * 8), ("out_ld", c_int64),
                ("out_col", c_int64)]


class rt_dispatch(Structure):
    _fields_ = [("plan", c_void_p), ("lhs", c_void_p), ("rhs", c_void_p), ("bias", c_void_p), ("out", c_void_p),
                ("opts", rt_launch_opts)]


class rt_usage_record(Structure):
    _fields_ = [("size", c_uint64), ("producer", c_int32), ("last_consumer", c_int32)]


class rt_node_tensors(Structure):
    _fields_ = [("lhs", c_int32), ("rhs", c_int32), ("bias", c_int32), ("out", c_int32)]


class rt_mlp_desc(Structure):
    _fields_ = [("fc1", rt_matmul_desc), ("fc2", rt_matmul_desc), ("w1", c_void_p), ("b1", c_void_p),
                ("w2", c_void_p), ("b2", c_void_p), ("x", c_void_p), ("out", c_void_p)]


class rt_gguf_value(Structure):
    _fields_ = [("type", c_int32), ("elem_type", c_int32), ("len", c_uint64), ("u64", c_uint64),
                ("i64", c_int64), ("f64", ctypes.c_double), ("str", c_void_p), ("node", c_void_p)]


class rt_gguf_tensor_info(Structure):
    _fields_ = [("name", c_char_p), ("ggml_type", ctypes.c_uint32), ("shape", rt_shape),
                ("offset", c_uint64), ("nbytes", c_uint64)]


class RatchetError(RuntimeError):
    """A non-OK rt_status.  `.status` is the code, `.status_name` its name."""

    def __init__(self, status: int, name: str, message: str):
        super().__init__(f"{name}: {message}")
        self.status = status
        self.status_name = name
        self.message = message


class ShapeError(RatchetError):
    """Where the reference returns an error from Matmul::compute_c_shape."""


class InvariantError(RatchetError):
    """Where the reference panics (Matmul::new, OpGuards)."""


_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ratchet_b200.build` (nvcc, sm_100a). "
            "ratchet_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    V = c_void_p
    sig = {
        "rt_last_error": (c_char_p, []),
        "rt_status_name": (c_char_p, [c_int32]),
        "rt_version": (c_char_p, []),
        "rt_dtype_size": (c_size_t, [c_int32]),
        "rt_dtype_is_quantized": (c_int32, [c_int32]),
        "rt_dtype_activation": (c_int32, [c_int32, POINTER(c_int32)]),
        "rt_dtype_segments": (c_int32, [c_int32, c_uint64, POINTER(rt_segment), POINTER(c_int32)]),
        "rt_dtype_nbytes": (c_int32, [c_int32, c_uint64, POINTER(c_uint64)]),
        "rt_quantize_q8_0": (c_int32, [V, c_uint64, c_int32, V]),
        "rt_dequantize_q8_0": (c_int32, [V, c_uint64, c_int32, V]),
        "rt_transcode_gguf_q8_0": (c_int32, [V, c_uint64, c_int32, V]),
        "rt_quantize_q4_k": (c_int32, [V, c_uint64, V]),
        "rt_dequantize_q4_k": (c_int32, [V, c_uint64, V]),
        "rt_matmul_spec": (c_int32, [POINTER(rt_matmul_desc), POINTER(rt_gemm_spec)]),
        "rt_matmul_out_shape": (c_int32, [POINTER(rt_matmul_desc), POINTER(rt_shape)]),
        "rt_device_create": (c_int32, [c_int32, POINTER(V)]),
        "rt_device_destroy": (c_int32, [V]),
        "rt_device_sync": (c_int32, [V]),
        "rt_device_stream": (V, [V]),
        "rt_device_sm_count": (c_int32, [V]),
        "rt_device_ordinal": (c_int32, [V]),
        "rt_buffer_alloc": (c_int32, [V, c_uint64, POINTER(V)]),
        "rt_buffer_free": (c_int32, [V]),
        "rt_buffer_ptr": (V, [V]),
        "rt_buffer_size": (c_uint64, [V]),
        "rt_upload": (c_int32, [V, V, c_uint64, V, c_uint64, c_int32]),
        "rt_download": (c_int32, [V, V, c_uint64, V, c_uint64, c_int32]),
        "rt_host_alloc": (c_int32, [c_uint64, POINTER(V)]),
        "rt_host_free": (c_int32, [V]),
        "rt_matmul_plan": (c_int32, [V, POINTER(rt_matmul_desc), POINTER(V)]),
        "rt_plan_destroy": (c_int32, [V]),
        "rt_plan_forget_weights": (c_int32, [V]),
        "rt_abi_layout": (c_int32, [POINTER(c_uint64), c_int32]),
        "rt_plan_spec": (c_int32, [V, POINTER(rt_gemm_spec)]),
        "rt_plan_kernel": (c_char_p, [V]),
        "rt_plan_launches": (c_int32, [V]),
        "rt_matmul_launch": (c_int32, [V, V, V, V, V, V]),
        "rt_matmul_launch_ex": (c_int32, [V, V, V, V, V, V, POINTER(rt_launch_opts)]),
        "rt_executable_create": (c_int32, [V, POINTER(rt_dispatch), c_int32, c_int32, POINTER(V)]),
        "rt_executable_create_planned": (c_int32, [V, POINTER(rt_dispatch), POINTER(rt_node_tensors), c_int32,
                                                   POINTER(c_uint64), c_int32, c_int32, POINTER(V)]),
        "rt_executable_arena": (c_int32, [V, POINTER(c_uint64), POINTER(c_int32), POINTER(c_uint64)]),
        "rt_executable_tensor": (V, [V, c_int32]),
        "rt_mlp_create": (c_int32, [V, POINTER(rt_mlp_desc), c_int32, POINTER(V)]),
        "rt_arena_plan": (c_int32, [POINTER(rt_usage_record), c_int32, c_uint64, POINTER(c_int32), POINTER(c_uint64),
                                    POINTER(c_int32), POINTER(c_uint64)]),
        "rt_executable_dispatch": (c_int32, [V, V]),
        "rt_executable_destroy": (c_int32, [V]),
        "rt_executable_launches": (c_int32, [V]),
        "rt_executable_kernel": (c_char_p, [V]),
        "rt_linear_q8_0_static_scratch": (c_int32, [V, V, V, V, V, c_int64, c_int64, c_int64, c_int32, V]),
        "rt_comm_unique_id": (c_int32, [V]),
        "rt_comm_init_rank": (c_int32, [V, c_int32, c_int32, V, c_int32, POINTER(V)]),
        "rt_comm_all_gather": (c_int32, [V, V, V, c_uint64, V]),
        "rt_comm_destroy": (c_int32, [V]),
        "rt_ipc_export": (c_int32, [V, V]),
        "rt_ipc_open": (c_int32, [V, V, POINTER(V)]),
        "rt_ipc_close": (c_int32, [V, V]),
        "rt_shard_rows": (c_int32, [c_int32, V, c_uint64, c_uint64, c_uint64, c_uint64, V]),
        "rt_dequantize_device": (c_int32, [V, c_int32, c_uint64, V, V, V]),
        "rt_gguf_open": (c_int32, [c_char_p, POINTER(V)]),
        "rt_gguf_close": (c_int32, [V]),
        "rt_gguf_version": (c_int32, [V]),
        "rt_gguf_alignment": (c_uint64, [V]),
        "rt_gguf_tensor_data_offset": (c_uint64, [V]),
        "rt_gguf_tensor_count": (c_uint64, [V]),
        "rt_gguf_metadata_count": (c_uint64, [V]),
        "rt_gguf_metadata_at": (c_int32, [V, c_uint64, POINTER(c_char_p), POINTER(rt_gguf_value)]),
        "rt_gguf_metadata_find": (c_int32, [V, c_char_p, POINTER(rt_gguf_value)]),
        "rt_gguf_array_item": (c_int32, [POINTER(rt_gguf_value), c_uint64, POINTER(rt_gguf_value)]),
        "rt_gguf_tensor_at": (c_int32, [V, c_uint64, POINTER(rt_gguf_tensor_info)]),
        "rt_gguf_tensor_find": (c_int32, [V, c_char_p, POINTER(rt_gguf_tensor_info)]),
        "rt_gguf_tensor_dtype": (c_int32, [V, c_char_p, POINTER(c_int32)]),
        "rt_gguf_read_tensor": (c_int32, [V, c_char_p, c_int32, V, c_uint64]),
        "rt_gguf_tensor_nbytes": (c_int32, [V, c_char_p, c_int32, POINTER(c_uint64)]),
        "rt_gguf_load_tensor": (c_int32, [V, V, c_char_p, c_int32, POINTER(V), POINTER(rt_shape)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status == RT_OK:
        return
    lib = load()
    name = lib.rt_status_name(status).decode()
    msg = (lib.rt_last_error() or b"").decode()
    if status == RT_ERR_SHAPE:
        raise ShapeError(status, name, msg)
    if status in (RT_ERR_INVARIANT, RT_ERR_DTYPE):
        raise InvariantError(status, name, msg)
    raise RatchetError(status, name, msg)
