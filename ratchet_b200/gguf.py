"""GGUF files: the host-side mirror of the reference loader's `Header`
(crates/ratchet-loader/src/gguf/gguf.rs:158-496) over the library's rt_gguf_* calls.

    with GGUF.open(path) as g:
        g.metadata["general.architecture"]
        g.tensor_infos["blk.0.ffn_up.weight"].shape      # outermost first, as the reference reverses it
        w = g.tensor("blk.0.ffn_up.weight", gpu)         # Header::tensor: read + transcode + upload

Parsing, transcoding and the upload all happen inside the library; this module only walks the
handles.
"""
from __future__ import annotations

from ctypes import byref, c_char_p, c_int32, c_uint64, c_void_p, string_at
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from . import _lib
from ._lib import check, rt_gguf_tensor_info, rt_gguf_value, rt_shape
from .tensor import Device, DType, GpuBuffer, Tensor

# gguf.rs:183-216
U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
# crates/ratchet-loader/src/lib.rs:57-80
GGML_NAMES = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2K",
              11: "Q3K", 12: "Q4K", 13: "Q5K", 14: "Q6K", 15: "Q8K"}


@dataclass(frozen=True)
class TensorInfo:
    """gguf.rs:56-60."""
    name: str
    ggml_type: int
    shape: List[int]
    offset: int
    nbytes: int

    @property
    def ggml_name(self) -> str:
        return GGML_NAMES.get(self.ggml_type, f"?{self.ggml_type}")


def _value(v: rt_gguf_value):
    lib = _lib.load()
    t = v.type
    if t in (U8, U16, U32, U64):
        return int(v.u64)
    if t in (I8, I16, I32, I64):
        return int(v.i64)
    if t in (F32, F64):
        return float(v.f64)
    if t == BOOL:
        return bool(v.u64)
    if t == STRING:
        # String::from_utf8_lossy (gguf.rs:179)
        return string_at(v.str, v.len).decode("utf-8", errors="replace")
    if t == ARRAY:
        out = []
        item = rt_gguf_value()
        for i in range(int(v.len)):
            check(lib.rt_gguf_array_item(byref(v), i, byref(item)))
            out.append(_value(item))
        return out
    raise ValueError(f"value type {t}")


class GGUF:
    def __init__(self, path: str):
        lib = _lib.load()
        self._h = c_void_p()
        check(lib.rt_gguf_open(str(path).encode(), byref(self._h)))
        self.path = str(path)
        self.version = int(lib.rt_gguf_version(self._h))
        self.alignment = int(lib.rt_gguf_alignment(self._h))
        self.tensor_data_offset = int(lib.rt_gguf_tensor_data_offset(self._h))
        self.metadata: Dict[str, object] = {}
        self.metadata_types: Dict[str, int] = {}
        key, val = c_char_p(), rt_gguf_value()
        for i in range(int(lib.rt_gguf_metadata_count(self._h))):
            check(lib.rt_gguf_metadata_at(self._h, i, byref(key), byref(val)))
            k = key.value.decode("utf-8", errors="replace")
            self.metadata[k] = _value(val)
            self.metadata_types[k] = int(val.type)
        self.tensor_infos: Dict[str, TensorInfo] = {}
        info = rt_gguf_tensor_info()
        for i in range(int(lib.rt_gguf_tensor_count(self._h))):
            check(lib.rt_gguf_tensor_at(self._h, i, byref(info)))
            name = info.name.decode("utf-8", errors="replace")
            self.tensor_infos[name] = TensorInfo(name, int(info.ggml_type), info.shape.tolist(), int(info.offset), int(info.nbytes))

    @staticmethod
    def open(path: str) -> "GGUF":
        return GGUF(path)

    def close(self) -> None:
        if self._h:
            _lib.load().rt_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def get(self, key: str):
        """Metadata::get (gguf.rs:149-153): raises on an absent key."""
        v = rt_gguf_value()
        check(_lib.load().rt_gguf_metadata_find(self._h, key.encode(), byref(v)))
        return _value(v)

    def dtype_of(self, name: str) -> DType:
        """The dtype `tensor(name, …)` loads as (ratchet_from_gguf, gguf.rs:113-141)."""
        dt = c_int32()
        check(_lib.load().rt_gguf_tensor_dtype(self._h, name.encode(), byref(dt)))
        return DType(dt.value)

    def tensor(self, name: str, device: Device, dt: Optional[DType] = None) -> Tensor:
        """Header::tensor (gguf.rs:484-496): the named tensor in its device layout, on `device`
        (uploaded by the library) or, for Device.CPU, as host bytes in the same layout."""
        lib = _lib.load()
        dt = DType(dt) if dt is not None else self.dtype_of(name)
        if device.is_gpu():
            buf, shape = c_void_p(), rt_shape()
            check(lib.rt_gguf_load_tensor(self._h, device._h, name.encode(), int(dt), byref(buf), byref(shape)))
            return Tensor(shape.tolist(), dt, device, GpuBuffer.adopt(device, buf))
        info = rt_gguf_tensor_info()
        check(lib.rt_gguf_tensor_find(self._h, name.encode(), byref(info)))
        shape = info.shape.tolist()
        need = c_uint64()
        check(lib.rt_gguf_tensor_nbytes(self._h, name.encode(), int(dt), byref(need)))
        raw = np.zeros(need.value, dtype=np.uint8)
        check(lib.rt_gguf_read_tensor(self._h, name.encode(), int(dt), raw.ctypes.data_as(c_void_p), raw.size))
        return Tensor(shape, dt, Device.CPU, raw)
