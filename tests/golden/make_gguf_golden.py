"""Generates tiny.gguf and tiny_gguf.npz (run once in the build container, outputs committed).

The reference loader (crates/ratchet-loader/src/gguf/gguf.rs) holds no test files of its own.
This fixture is a GGUF v3 file written by the gguf Python package (0.19.0) and what that
package's own reader and decoders return for it, so that the library's reader is pinned without
gguf at test time:

  tiny.gguf        metadata of every value type, a custom alignment of 64, and tensors of
                   ggml types F32, F16, Q8_0 (encoded by gguf.quants.quantize), Q4_K (random
                   super-blocks) and Q4_0 (a type the loader must refuse to load)
  tiny_gguf.npz    per tensor: name, shape (outermost first), ggml type, offset, raw bytes and
                   gguf.quants.dequantize output; data offset; the metadata as JSON

Usage:  python tests/golden/make_gguf_golden.py
"""
import json
import os

import numpy as np
from gguf import GGMLQuantizationType as Q
from gguf import GGUFReader, GGUFValueType, GGUFWriter, quants

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "tiny.gguf")


def main():
    rng = np.random.default_rng(20240611)
    w = GGUFWriter(PATH, "phi2")
    w.add_custom_alignment(64)
    w.add_uint8("t.u8", 200)
    w.add_int8("t.i8", -100)
    w.add_uint16("t.u16", 60000)
    w.add_int16("t.i16", -30000)
    w.add_uint32("t.u32", 4000000000)
    w.add_int32("t.i32", -2000000000)
    w.add_uint64("t.u64", 2 ** 63 + 5)
    w.add_int64("t.i64", -(2 ** 62))
    w.add_float32("t.f32", 0.1)
    w.add_float64("t.f64", 1e-300)
    w.add_bool("t.yes", True)
    w.add_bool("t.no", False)
    w.add_string("t.str", "héllo wörld")
    w.add_array("t.arr_i32", [1, -2, 3, -4])
    w.add_array("t.arr_str", ["a", "", "ccc"])
    w.add_key_value("t.arr_f32", [0.5, -1.25], GGUFValueType.ARRAY, sub_type=GGUFValueType.FLOAT32)

    f32 = rng.standard_normal((3, 5)).astype(np.float32)
    f16 = rng.standard_normal((7, 64)).astype(np.float16)
    vec = rng.standard_normal((2,)).astype(np.float32)          # 8 bytes: shorter than a 16-byte buffer
    wq8 = (rng.standard_normal((48, 128)) * 0.02).astype(np.float32)
    q8 = quants.quantize(wq8, Q.Q8_0)                            # uint8 [48, 128/32*34]
    q4k = rng.integers(0, 256, size=(16, 2 * 144), dtype=np.uint8)  # logical [16, 512]
    blk = q4k.reshape(-1, 144)
    blk[:, 0:2] = rng.uniform(1e-4, 2e-3, size=len(blk)).astype(np.float16).view(np.uint8).reshape(-1, 2)
    blk[:, 2:4] = rng.uniform(1e-4, 2e-3, size=len(blk)).astype(np.float16).view(np.uint8).reshape(-1, 2)
    q4k = blk.reshape(16, 2 * 144)
    q40 = rng.integers(0, 256, size=(4, 2 * 18), dtype=np.uint8)    # logical [4, 64]
    w.add_tensor("dense.f32", f32)
    w.add_tensor("dense.f16", f16)
    w.add_tensor("short.f32", vec)
    w.add_tensor("blk.0.ffn_up.weight", q8, raw_dtype=Q.Q8_0)
    w.add_tensor("blk.0.ffn_down.weight", q4k, raw_dtype=Q.Q4_K)
    w.add_tensor("legacy.q4_0", q40, raw_dtype=Q.Q4_0)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    r = GGUFReader(PATH)
    out = {"data_offset": np.array([r.data_offset], dtype=np.uint64), "alignment": np.array([r.alignment], dtype=np.uint64)}
    names = []
    for i, t in enumerate(r.tensors):
        names.append(t.name)
        out[f"t{i}_shape"] = np.array([int(d) for d in reversed(t.shape)], dtype=np.int64)
        out[f"t{i}_type"] = np.array([int(t.tensor_type)], dtype=np.int64)
        out[f"t{i}_offset"] = np.array([int(t.data_offset) - int(r.data_offset)], dtype=np.uint64)
        raw = np.ascontiguousarray(t.data).view(np.uint8).reshape(-1)
        out[f"t{i}_raw"] = raw
        if t.tensor_type in (Q.F32, Q.F16, Q.Q8_0, Q.Q4_K):
            out[f"t{i}_values"] = quants.dequantize(np.ascontiguousarray(t.data), t.tensor_type).astype(np.float32).reshape(-1)
    meta = {}
    for k, f in r.fields.items():
        if k.startswith("GGUF."):
            continue
        v = f.contents()
        meta[k] = {"type": int(f.types[0]), "value": v}
    out["names"] = np.array(json.dumps(names))
    out["metadata"] = np.array(json.dumps(meta))
    np.savez_compressed(os.path.join(HERE, "tiny_gguf.npz"), **out)
    print("wrote", PATH, os.path.getsize(PATH), "bytes;", len(names), "tensors;", len(meta), "metadata keys")


if __name__ == "__main__":
    main()
