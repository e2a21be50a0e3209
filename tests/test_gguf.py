"""The GGUF reader (rt_gguf_*) against a file written and read back by the gguf Python package
(tests/golden/tiny.gguf + tiny_gguf.npz), hand-written v1/v2/v3 files, and malformed files.
The behaviours checked are those of crates/ratchet-loader/src/gguf/gguf.rs."""
import json
import os
import struct

import numpy as np
import pytest

import oracle
import ratchet_b200 as rb
from ratchet_b200 import DType, Device, RatchetError
from ratchet_b200.gguf import ARRAY, BOOL, F32, GGUF, I32, STRING, U8, U32, U64

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TINY = os.path.join(GOLDEN, "tiny.gguf")


@pytest.fixture(scope="module")
def fx():
    return np.load(os.path.join(GOLDEN, "tiny_gguf.npz"))


def test_header_matches_gguf_py(fx):
    with GGUF.open(TINY) as g:
        assert g.version == 3
        assert g.alignment == int(fx["alignment"][0]) == 64
        assert g.tensor_data_offset == int(fx["data_offset"][0])
        names = json.loads(str(fx["names"]))
        assert list(g.tensor_infos) == names  # file order
        raw_file = open(TINY, "rb").read()
        for i, n in enumerate(names):
            ti = g.tensor_infos[n]
            assert ti.shape == fx[f"t{i}_shape"].tolist()  # reversed: outermost first (gguf.rs:452)
            assert ti.ggml_type == int(fx[f"t{i}_type"][0])
            assert ti.offset == int(fx[f"t{i}_offset"][0])
            raw = fx[f"t{i}_raw"]
            assert ti.nbytes == raw.size  # TensorInfo::size_in_bytes
            start = g.tensor_data_offset + ti.offset
            assert raw_file[start:start + ti.nbytes] == raw.tobytes()  # TensorInfo::byte_range


def test_metadata_matches_gguf_py(fx):
    want = json.loads(str(fx["metadata"]))
    with GGUF.open(TINY) as g:
        assert list(g.metadata) == list(want)
        for k, rec in want.items():
            assert g.metadata_types[k] == rec["type"], k
            got = g.metadata[k]
            assert got == rec["value"] and type(got) is type(rec["value"]), (k, got, rec["value"])
            assert g.get(k) == rec["value"]
        with pytest.raises(RatchetError, match="missing key nope"):
            g.get("nope")


def test_tensors_load_in_the_device_layout(fx):
    names = json.loads(str(fx["names"]))
    with GGUF.open(TINY) as g:
        want_dt = {"dense.f32": DType.F32, "dense.f16": DType.F16, "short.f32": DType.F32,
                   "blk.0.ffn_up.weight": DType.Q8_0H, "blk.0.ffn_down.weight": DType.Q4_K}
        for i, n in enumerate(names):
            if n not in want_dt:
                continue
            assert g.dtype_of(n) == want_dt[n]
            t = g.tensor(n, Device.CPU)
            assert t.shape == fx[f"t{i}_shape"].tolist() and t.dt == want_dt[n]
            assert t.storage.size == t.dt.nbytes(t.numel())
            # the values gguf-py decodes from the same bytes, bit for bit (Q8_0H decodes to the f16
            # product, gemm.rs:400-406; loaded with f32 scales the f32 product itself)
            want = fx[f"t{i}_values"]
            if t.dt == DType.Q8_0H:
                exact = g.tensor(n, Device.CPU, DType.Q8_0F)
                assert np.array_equal(exact.to_f32().reshape(-1).view(np.uint32), want.view(np.uint32)), n
                want = want.astype(np.float16).astype(np.float32)
            assert np.array_equal(t.to_f32().reshape(-1).view(np.uint32), want.view(np.uint32)), n
        # plain tensors shorter than 16 bytes are zero-padded to the minimum buffer (dtype/mod.rs:90)
        short = g.tensor("short.f32", Device.CPU)
        assert short.storage.size == 16 and not short.storage[8:].any()
        # Q8_0: codes | pad | scales, identical to the stand-alone transcode and to the oracle's
        i8 = names.index("blk.0.ffn_up.weight")
        blocks = fx[f"t{i8}_raw"].reshape(-1, 34)
        for dt, sb in ((DType.Q8_0H, 2), (DType.Q8_0F, 4)):
            t = g.tensor("blk.0.ffn_up.weight", Device.CPU, dt)
            assert np.array_equal(t.storage, oracle.q8_transcode_gguf(blocks, sb))
            assert np.array_equal(t.storage, rb.transcode_gguf_q8_0(blocks, t.shape, dt).storage)
        # Q4_K: the raw super-blocks
        i4 = names.index("blk.0.ffn_down.weight")
        assert np.array_equal(g.tensor("blk.0.ffn_down.weight", Device.CPU).storage, fx[f"t{i4}_raw"])


def test_refusals(fx):
    with GGUF.open(TINY) as g:
        with pytest.raises(RatchetError, match="unsupported ggml dtype Q4_0") as e:  # gguf.rs:139
            g.tensor("legacy.q4_0", Device.CPU)
        assert e.value.status_name == "RT_ERR_UNSUPPORTED"
        with pytest.raises(RatchetError, match="cannot find tensor info for nope"):  # gguf.rs:490-493
            g.tensor("nope", Device.CPU)
        with pytest.raises(RatchetError, match="does not load as"):
            g.tensor("dense.f32", Device.CPU, DType.F16)
        with pytest.raises(RatchetError, match="does not load as"):
            g.tensor("dense.f16", Device.CPU, DType.Q8_0H)
    with pytest.raises(RatchetError, match="cannot open"):
        GGUF.open(os.path.join(GOLDEN, "absent.gguf"))


# ------------------------------------------------------------------ hand-written files

def _s(b: bytes, v: int) -> bytes:
    return struct.pack("<I" if v == 1 else "<Q", len(b)) + b


def _n(x: int, v: int) -> bytes:
    return struct.pack("<I" if v == 1 else "<Q", x)


def build(version=3, magic=b"GGUF", kvs=(), tensors=(), data=b"", pad_to=32, counts=None):
    """kvs: (key bytes, type, payload bytes); tensors: (name bytes, dims innermost-first, ggml type, offset)."""
    out = magic + struct.pack("<I", version)
    nt, nk = counts if counts else (len(tensors), len(kvs))
    out += _n(nt, version) + _n(nk, version)
    for k, t, payload in kvs:
        out += _s(k, version) + struct.pack("<I", t) + payload
    for name, dims, gt, off in tensors:
        out += _s(name, version) + struct.pack("<I", len(dims))
        for d in dims:
            out += _n(d, version)
        out += struct.pack("<IQ", gt, off)
    if pad_to:
        out += b"\0" * (-len(out) % pad_to)
    return out + data


def _write(tmp_path, blob, name="x.gguf"):
    p = tmp_path / name
    p.write_bytes(blob)
    return str(p)


@pytest.mark.parametrize("version", [1, 2, 3])
def test_versions_1_to_3(tmp_path, version):
    """v1 holds 32-bit lengths, v2 and v3 64-bit (gguf.rs:412-423, 166-171, 441-451)."""
    vals = np.arange(24, dtype=np.float32)
    kvs = [(b"general.name\0\0", STRING, _s(b"tiny\0", version)),  # trailing NULs dropped (gguf.rs:174-177)
           (b"n", U32, struct.pack("<I", 7)),
           (b"arr", ARRAY, struct.pack("<I", I32) + _n(3, version) + struct.pack("<iii", 1, -2, 3)),
           (b"nest", ARRAY, struct.pack("<I", ARRAY) + _n(2, version)
            + struct.pack("<I", U8) + _n(2, version) + b"\x01\x02"
            + struct.pack("<I", STRING) + _n(1, version) + _s(b"z", version))]
    blob = build(version, kvs=kvs, tensors=[(b"w", [4, 3, 2], 0, 32)], data=b"\xff" * 32 + vals.tobytes())
    with GGUF.open(_write(tmp_path, blob)) as g:
        assert g.version == version and g.alignment == 32  # DEFAULT_ALIGNMENT (gguf.rs:13)
        assert g.metadata == {"general.name": "tiny", "n": 7, "arr": [1, -2, 3], "nest": [[1, 2], ["z"]]}
        assert g.tensor_infos["w"].shape == [2, 3, 4]
        assert g.tensor_data_offset % 32 == 0
        t = g.tensor("w", Device.CPU)
        assert np.array_equal(t.to_numpy(), vals.reshape(2, 3, 4))


def test_byte_swapped_magic_is_accepted(tmp_path):
    """gguf.rs:23-26 accepts 0x46554747 and 0x47475546."""
    with GGUF.open(_write(tmp_path, build(3, magic=b"FUGG"))) as g:
        assert g.version == 3 and not g.tensor_infos and not g.metadata


@pytest.mark.parametrize("ty,payload,expect", [
    (U8, b"\x10", 16), (U32, struct.pack("<I", 128), 128), (I32, struct.pack("<i", 256), 256),
    (I32, struct.pack("<i", -8), 32),      # negative: ignored (gguf.rs:471-473)
    (U64, struct.pack("<Q", 128), 32),     # 64-bit types are not honoured (gguf.rs:466-475)
    (F32, struct.pack("<f", 64.0), 32),
])
def test_alignment_key(tmp_path, ty, payload, expect):
    blob = build(3, kvs=[(b"general.alignment", ty, payload)], tensors=[(b"w", [4], 0, 0)], pad_to=expect,
                 data=np.arange(4, dtype=np.float32).tobytes())
    with GGUF.open(_write(tmp_path, blob)) as g:
        assert g.alignment == expect and g.tensor_data_offset % expect == 0
        assert np.array_equal(g.tensor("w", Device.CPU).to_numpy(), np.arange(4, dtype=np.float32))


@pytest.mark.parametrize("blob,msg", [
    (build(3, magic=b"GGML"), "unknown magic 0x4c4d4747"),
    (build(4), "unsupported magic/version Gguf/4"),
    (build(0), "unsupported magic/version Gguf/0"),
    (build(3, kvs=[(b"k", 13, b"\0" * 8)]), "unrecognized value-type 13"),
    (build(3, kvs=[(b"k", ARRAY, struct.pack("<IQ", 99, 1) + b"\0" * 8)]), "unrecognized value-type 99"),
    (build(3, kvs=[(b"k", BOOL, b"\x02")]), "unexpected bool value 2"),
    (b"GG", "unexpected end of file"),
    (build(3, pad_to=0)[:12], "unexpected end of file"),
    (build(3, kvs=[(b"k", STRING, struct.pack("<Q", 1 << 40) + b"abc")], pad_to=0), "runs past the end of the file"),
    (build(3, kvs=[(b"k", ARRAY, struct.pack("<IQ", U8, 1 << 50))], pad_to=0), "runs past the end of the file"),
    (build(3, counts=(1 << 60, 0)), "counts exceed"),
    (build(3, counts=(0, 3)), "unexpected end of file"),
    (build(3, tensors=[(b"w", [2] * 9, 0, 0)]), "has 9 dimensions"),
    (build(3, tensors=[(b"w", [1 << 39, 1 << 39], 0, 0)]), "too large"),
])
def test_malformed_files_are_errors(tmp_path, blob, msg):
    with pytest.raises(RatchetError, match=msg):
        GGUF.open(_write(tmp_path, blob))


def test_invalid_ggml_type_and_short_data(tmp_path):
    with pytest.raises(RatchetError, match="invalid dtype 4") as e:  # lib.rs:76
        GGUF.open(_write(tmp_path, build(3, tensors=[(b"w", [32], 4, 0)])))
    assert e.value.status_name == "RT_ERR_DTYPE"
    # a Q8_0 tensor whose element count does not divide by 32 (gguf.rs:70-76)
    with GGUF.open(_write(tmp_path, build(3, tensors=[(b"w", [16, 3], 8, 0)], data=b"\0" * 64), "a.gguf")) as g:
        with pytest.raises(rb.ShapeError, match="48 is not divisible by the block size 32"):
            g.tensor("w", Device.CPU)
    # tensor bytes that the file does not hold
    with GGUF.open(_write(tmp_path, build(3, tensors=[(b"w", [64], 0, 0)], data=b"\0" * 100), "b.gguf")) as g:
        with pytest.raises(RatchetError, match="runs past the end of the file"):
            g.tensor("w", Device.CPU)


# ------------------------------------------------------------------ on the device

@pytest.mark.gpu
def test_gguf_weights_feed_the_matmul(fx):
    """Header::tensor on the GPU, then the Linear call W.gemm(x, None, false, true, true) on the loaded
    weights, against the truth computed from the values gguf-py decodes."""
    gpu = Device.request_device(rb.DeviceRequest.GPU, 0)
    names = json.loads(str(fx["names"]))
    rng = np.random.default_rng(7)
    with GGUF.open(TINY) as g:
        for n in ("blk.0.ffn_up.weight", "blk.0.ffn_down.weight", "dense.f16"):
            i = names.index(n)
            w = g.tensor(n, gpu)
            N, K = w.shape
            assert np.array_equal(w.to(Device.CPU).storage, g.tensor(n, Device.CPU).storage)
            vals = fx[f"t{i}_values"].reshape(N, K)
            if w.dt.is_quantized():
                got = w.dequantize_on_device().reshape(-1).astype(np.float32)
                want = vals.reshape(-1).astype(np.float16).astype(np.float32) if w.dt == DType.Q8_0H else vals.reshape(-1)
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), n
            for M in (1, 24):
                x = rng.standard_normal((1, M, K)).astype(np.float16)
                y = w.gemm(rb.Tensor.from_data(x, gpu), None, False, True, True).resolve().to(Device.CPU)
                wv = vals.astype(np.float16).astype(np.float32) if w.dt == DType.Q8_0H else vals
                truth = oracle.matmul_truth(wv, x.astype(np.float32), None, 1, 1, 1, N, M, K, False, True, True)
                err = oracle.rel_l2(y.to_f32().reshape(-1), oracle.f64_to_f16(truth).astype(np.float32))
                assert y.shape == [1, M, N] and err <= 1e-3, (n, M, err)
