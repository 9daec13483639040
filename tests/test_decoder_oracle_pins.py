"""Pins the NumPy decoder oracle (oracle/decoder_np.py) to the known answers gocnn/candy's own unit
tests hold for the same operators (tests/golden/reduce_unary_kats.json, each with its file:line), and
checks the GPU operators against the very same literals.  Tolerance as in the reference tests: 1e-6."""
import json
import math
from pathlib import Path

import numpy as np
import pytest

from oracle import decoder_np as dn

KATS = json.loads((Path(__file__).parent / "golden" / "reduce_unary_kats.json").read_text())
TOL = 1e-6
f32 = np.float32


def rows_of(case):
    src = np.array(case["src"], dtype=f32)
    cols = case["dims"][-1]
    return src.reshape(-1, cols)


@pytest.mark.parametrize("case", KATS["rmsnorm_f32"]["cases"], ids=lambda c: c["name"])
def test_oracle_rmsnorm_matches_reference_literals(case):
    x = rows_of(case)
    alpha = np.ones(x.shape[1], dtype=f32) if case["alpha"] is None else np.array(case["alpha"], dtype=f32)
    got = np.concatenate([dn.rmsnorm(r, alpha, case["eps"]) for r in x])
    assert np.abs(got - np.array(case["want"], dtype=f32)).max() < TOL


@pytest.mark.parametrize("case", KATS["softmax_f32"]["cases"], ids=lambda c: c["name"])
def test_oracle_softmax_matches_reference_literals(case):
    got = np.concatenate([dn.softmax(r) for r in rows_of(case)])
    assert np.abs(got - np.array(case["want"], dtype=f32)).max() < TOL


@pytest.mark.parametrize("case", KATS["argmax_f32"]["cases"], ids=lambda c: c["name"])
def test_oracle_argmax_matches_reference_literals(case):
    assert [dn.argmax(r) for r in rows_of(case)] == case["want"]


@pytest.mark.parametrize("case", KATS["rope_f32"]["cases"], ids=lambda c: c["name"])
def test_oracle_rope_matches_reference_literals(case):
    d, td, bh = case["d"], case["td"], case["bh"]
    src = np.array(case["src"], dtype=f32).reshape(bh, td // d, d)
    cos, sin = np.array(case["cos"], dtype=f32), np.array(case["sin"], dtype=f32)
    out = np.empty_like(src)
    for b in range(bh):
        base = b * case["stride_b"] // 2  # RopeF32 walks the tables by strideB/2 per batch-head (reduce.go:3987-4006)
        for t in range(td // d):
            sl = slice(base + t * (d // 2), base + (t + 1) * (d // 2))
            out[b, t] = dn.rope(src[b, t][None, :], cos[sl], sin[sl])[0]
    assert np.abs(out.reshape(-1) - np.array(case["want"], dtype=f32)).max() < TOL


def silu_want():
    return np.array([0.0, 1 / (1 + math.exp(-1)), -1 / (1 + math.exp(1))], dtype=f32)


def test_oracle_silu_matches_reference_literals():
    case = KATS["silu_f32"]["cases"][0]
    assert np.abs(dn.silu(np.array(case["src"], dtype=f32)) - silu_want()).max() < TOL


# ---- the GPU operators against the same literals ---------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("case", KATS["rmsnorm_f32"]["cases"], ids=lambda c: c["name"])
def test_gpu_rmsnorm_matches_reference_literals(device, case):
    x = rows_of(case)
    lib, ctx = device._lib, device.ctx
    xs, ys = device.storage_from_slice(x), device.alloc(x.size)
    alpha = None if case["alpha"] is None else device.storage_from_slice(np.array(case["alpha"], dtype=f32))
    device._check(lib.cq_rmsnorm(ctx, xs.ptr, alpha.ptr if alpha else None, x.shape[0], x.shape[1], case["eps"], ys.ptr), "rmsnorm")
    device.synchronize()
    assert np.abs(ys.data() - np.array(case["want"], dtype=f32)).max() < TOL


@pytest.mark.gpu
@pytest.mark.parametrize("case", KATS["argmax_f32"]["cases"], ids=lambda c: c["name"])
def test_gpu_argmax_matches_reference_literals(device, case):
    from candy_b200.backend import RawBuffer
    x = rows_of(case)
    lib, ctx = device._lib, device.ctx
    xs, out = device.storage_from_slice(x), RawBuffer(device, 4 * x.shape[0])
    device._check(lib.cq_argmax(ctx, xs.ptr, x.shape[0], x.shape[1], out.ptr), "argmax")
    device.synchronize()
    assert out.data().view(np.uint32).tolist() == case["want"]


@pytest.mark.gpu
def test_gpu_silu_matches_reference_literals(device):
    lib, ctx = device._lib, device.ctx
    gu = np.array([0, 1, -1, 1, 1, 1], dtype=f32)  # gates, then ups of one
    gs, out = device.storage_from_slice(gu), device.alloc(3)
    device._check(lib.cq_silu_mul(ctx, gs.ptr, 1, 3, out.ptr, 3), "silu*mul")
    device.synchronize()
    assert np.abs(out.data() - silu_want()).max() < TOL


@pytest.mark.gpu
def test_gpu_rope_matches_reference_literals(device):
    """Both RopeF32 cases: one q head and one k head of width 4 at positions 0 and 1 of a two-row table."""
    from candy_b200.backend import RawBuffer
    c0, c1 = KATS["rope_f32"]["cases"]
    lib, ctx = device._lib, device.ctx
    cos = device.storage_from_slice(np.array(c1["cos"], dtype=f32))  # rows [1, 0] and [0.5, 0.5]
    sin = device.storage_from_slice(np.array(c1["sin"], dtype=f32))
    kc, vc = device.zeros(2 * 4), device.zeros(2 * 4)
    pos = RawBuffer(device, 4)
    for p, src, want in ((0, c1["src"][:4], c1["want"][:4]), (1, c1["src"][4:], c1["want"][4:]), (0, c0["src"], c0["want"])):
        qkv = device.storage_from_slice(np.array(list(src) * 3, dtype=f32))  # q, k, v all the same vector
        pv = np.array([p], dtype=np.int32)
        device._check(lib.cq_memcpy_h2d(ctx, pos.ptr, pv.ctypes.data, 4), "pos")
        device._check(lib.cq_rope_store_kv(ctx, qkv.ptr, 1, 1, 1, 4, cos.ptr, sin.ptr, pos.ptr, kc.ptr, vc.ptr, 2), "rope")
        device.synchronize()
        got = qkv.data()
        assert np.abs(got[:4] - np.array(want, dtype=f32)).max() < TOL   # q rotated in place
        assert np.abs(got[4:8] - np.array(want, dtype=f32)).max() < TOL  # k too
        assert np.abs(kc.data()[4 * p:4 * p + 4] - np.array(want, dtype=f32)).max() < TOL  # and stored at its position
        assert np.abs(vc.data()[4 * p:4 * p + 4] - np.array(src, dtype=f32)).max() == 0    # v is stored as it is


@pytest.mark.gpu
@pytest.mark.parametrize("case", KATS["softmax_f32"]["cases"][::2], ids=lambda c: c["name"])
def test_gpu_attention_softmax_matches_reference_literals(device, case):
    """The softmax inside decode attention: one head of width 4, q = (2, 0, 0, 0) so that the scaled score of
    key t is its first component, values = unit vectors, hence the output row is the softmax itself."""
    from candy_b200.backend import RawBuffer
    lib, ctx = device._lib, device.ctx
    for row, want in zip(rows_of(case), np.array(case["want"], dtype=f32).reshape(-1, case["dims"][-1])):
        t = len(row)
        assert t <= 4
        k = np.zeros((t, 4), dtype=f32)
        k[:, 0] = row
        v = np.eye(4, dtype=f32)[:t]
        kc, vc = device.storage_from_slice(k), device.storage_from_slice(v)
        qkv = device.storage_from_slice(np.array([2, 0, 0, 0] + [0] * 8, dtype=f32))
        pos = RawBuffer(device, 4)
        pv = np.array([t - 1], dtype=np.int32)
        device._check(lib.cq_memcpy_h2d(ctx, pos.ptr, pv.ctypes.data, 4), "pos")
        scratch = device.alloc(lib.cq_decode_attention_scratch_floats(1, 1, 4, t))
        out = device.alloc(4)
        device._check(lib.cq_decode_attention(ctx, qkv.ptr, 1, 1, 1, 4, pos.ptr, kc.ptr, vc.ptr, t, scratch.ptr, out.ptr), "attention")
        device.synchronize()
        assert np.abs(out.data()[:t] - want).max() < TOL
