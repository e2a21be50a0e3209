"""ratchet_b200: B200 (sm_100a) implementation of ratchet-core's Matmul path.

CUDA kernels + C ABI in `csrc/` (built into libratchet_b200.so by `ratchet_b200.build`), and a
host-side mirror of the reference's Tensor / Matmul / Quantizer / Linear interface in
`tensor.py`.  There is no CPU or PyTorch fallback: without the built library, or without an
sm_100 device, the calls raise.
"""
from ._lib import InvariantError, RatchetError, ShapeError
from ._lib import RT_EPILOGUE_GELU_TANH as EPILOGUE_GELU_TANH
from ._lib import RT_EPILOGUE_NONE as EPILOGUE_NONE
from ._lib import RT_EPILOGUE_SILU_MUL as EPILOGUE_SILU_MUL
from .tensor import (Device, DeviceRequest, DType, Executable, GpuBuffer, Linear, Matmul, MLP, PinnedArray, Quantization, Quantizer,
                     Tensor, bf16_bits_to_f32, f32_to_bf16_bits, transcode_gguf_q8_0)

from .sharded import Comm, ShardedLinear, shard_bounds, shard_rows
from .gguf import GGUF, TensorInfo

__all__ = ["GGUF", "TensorInfo", "Comm", "ShardedLinear", "shard_bounds", "shard_rows", "Device", "DeviceRequest", "DType", "Executable", "GpuBuffer", "Linear", "Matmul", "PinnedArray", "Quantization",
           "Quantizer", "Tensor", "RatchetError", "ShapeError", "InvariantError", "EPILOGUE_NONE",
           "EPILOGUE_GELU_TANH", "EPILOGUE_SILU_MUL", "MLP", "bf16_bits_to_f32", "f32_to_bf16_bits", "transcode_gguf_q8_0"]
