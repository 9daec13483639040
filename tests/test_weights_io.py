"""GGUF / NPZ weight files: the from-scratch GGUF reader against files written by the third-party
`gguf` package (CPU), and a loaded block-quantized tensor through the quantized linear on the GPU."""
import struct

import numpy as np
import pytest

from candy_b200 import weights_io as wio
from oracle import oracle_c as oc


def _write_gguf(path, tensors):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_uint32("answer", 42)
    w.add_string("general.name", "tiny")
    w.add_array("some.list", [1.0, 2.0, 3.0])
    raw = {}
    for name, (arr, qt) in tensors.items():
        if qt is None:
            w.add_tensor(name, arr)
            raw[name] = arr
        else:
            q = quants.quantize(arr, qt)
            w.add_tensor(name, q, raw_dtype=qt)
            raw[name] = q
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return raw


def test_reader_matches_a_file_written_by_the_gguf_package(tmp_path):
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(0)
    a = rng.standard_normal((48, 256)).astype(np.float32)
    b = rng.standard_normal((7, 64)).astype(np.float32)
    raw = _write_gguf(tmp_path / "t.gguf", {
        "blk.0.attn_q.weight": (a, gguf.GGMLQuantizationType.Q4_0),
        "blk.0.ffn_up.weight": (a * 3, gguf.GGMLQuantizationType.Q8_0),
        "norm.weight": (b[0], None),
        "half.weight": (b.astype(np.float16), None),
    })
    meta, tensors = wio.read_gguf(tmp_path / "t.gguf")
    assert meta["answer"] == 42 and meta["general.name"] == "tiny" and meta["general.architecture"] == "llama"
    assert list(np.asarray(meta["some.list"])) == [1.0, 2.0, 3.0]
    q4 = tensors["blk.0.attn_q.weight"]
    assert q4.shape == (48, 256) and q4.ggml_type == wio.GGML_Q4_0 and q4.data.size == 48 * 8 * 18
    np.testing.assert_array_equal(q4.data, raw["blk.0.attn_q.weight"].reshape(-1))
    q8 = tensors["blk.0.ffn_up.weight"]
    assert q8.shape == (48, 256) and q8.data.size == 48 * 8 * 34
    np.testing.assert_array_equal(q8.data, raw["blk.0.ffn_up.weight"].reshape(-1))
    np.testing.assert_array_equal(tensors["norm.weight"].to_float32(), b[0])
    np.testing.assert_array_equal(tensors["half.weight"].to_float32(), b.astype(np.float16).astype(np.float32))
    # the block bytes dequantize (split order) to what the package's own codec gives
    from gguf import quants
    want = quants.dequantize(raw["blk.0.attn_q.weight"], gguf.GGMLQuantizationType.Q4_0)
    got = oc.dequantize(oc.Q4_0, 1, np.ascontiguousarray(q4.data)).reshape(48, 256)
    np.testing.assert_array_equal(got, want)


def test_hand_built_minimal_file_and_errors(tmp_path):
    # version 3, one F32 tensor [2, 4] (dims innermost first: 4, 2), alignment 32, no metadata
    name = b"w"
    head = b"GGUF" + struct.pack("<IQQ", 3, 1, 0)
    info = struct.pack("<Q", len(name)) + name + struct.pack("<I", 2) + struct.pack("<QQ", 4, 2) + struct.pack("<IQ", 0, 0)
    body = head + info
    pad = (-len(body)) % 32
    vals = np.arange(8, dtype=np.float32)
    p = tmp_path / "m.gguf"
    p.write_bytes(body + b"\0" * pad + vals.tobytes())
    meta, tensors = wio.read_gguf(p)
    assert meta == {} and tensors["w"].shape == (2, 4)
    np.testing.assert_array_equal(tensors["w"].to_float32(), vals.reshape(2, 4))
    (tmp_path / "bad.gguf").write_bytes(b"GGML" + b"\0" * 40)
    with pytest.raises(wio.GGUFError):
        wio.read_gguf(tmp_path / "bad.gguf")
    (tmp_path / "short.gguf").write_bytes(body + b"\0" * pad + vals.tobytes()[:10])
    with pytest.raises(wio.GGUFError):
        wio.read_gguf(tmp_path / "short.gguf")


def test_npz_round_trip(tmp_path):
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    np.savez(tmp_path / "c.npz", weight=a, bias=a[0])
    got = wio.load_npz(tmp_path / "c.npz")
    np.testing.assert_array_equal(got["weight"], a)
    np.save(tmp_path / "w.npy", a)
    np.testing.assert_array_equal(wio.load_npz(tmp_path / "w.npy")["w"], a)


@pytest.mark.gpu
@pytest.mark.parametrize("qname", ["Q4_0", "Q8_0", "Q4_1", "Q5_0", "Q5_1"])
def test_gguf_tensor_through_the_quantized_linear(device, tmp_path, qname):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from helpers import rel_err
    qt = getattr(gguf.GGMLQuantizationType, qname)
    rng = np.random.default_rng(3)
    n, k = 512, 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    raw = _write_gguf(tmp_path / "l.gguf", {"out.weight": (w, qt)})
    _, tensors = wio.read_gguf(tmp_path / "l.gguf")
    qs = wio.load_linear(device, tensors["out.weight"])
    x = rng.standard_normal((3, k)).astype(np.float32)
    y = device.storage_from_slice(x).matmul(qs, 1, 3, n, k, 0).data().reshape(3, n)
    want = x.astype(np.float64) @ quants.dequantize(raw["out.weight"], qt).astype(np.float64).T
    assert rel_err(y, want) < 1e-4
