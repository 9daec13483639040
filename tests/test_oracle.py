"""CPU tests of the oracle: hand-derived known answers, the C restatement against its NumPy
twin, a third-party GGUF codec, and the committed golden fixtures.

The reference has no test for any function on this path (no quantized_test.go; nothing
mentions DequantizeBlock*, fp16ToFloat32 or NaiveBatchedMatMul*), so the known answers below
are derived by hand from the cited reference lines, in the reference's own table-driven style
(literal inputs, literal expected values)."""
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle_c as oc
from oracle import oracle_np as on

GOLDEN = Path(__file__).resolve().parent / "golden" / "qmatmul_small.npz"


def _u16(b):
    return int(b[0]) | (int(b[1]) << 8)


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


# ---- fp16 decode: tensor/internal/cpu/kernels/quantized.go:149-173 --------------------
FP16_KAT = [
    (0x0000, 0x00000000),  # +0
    (0x8000, 0x80000000),  # -0
    (0x0001, 0x33800000),  # 2^-24, smallest subnormal
    (0x03FF, 0x387FC000),  # 1023 * 2^-24
    (0x0400, 0x38800000),  # 2^-14, smallest normal
    (0x3800, 0x3F000000),  # 0.5
    (0x3C00, 0x3F800000),  # 1
    (0xC000, 0xC0000000),  # -2
    (0x7BFF, 0x477FE000),  # 65504
    (0x7C00, 0x7F800000),  # +inf
    (0xFC00, 0xFF800000),  # -inf
    (0x7E00, 0x7FC00000),  # quiet NaN
    (0x7C01, 0x7F802000),  # signalling NaN: payload kept (mant << 13), not quieted
]


@pytest.mark.parametrize("h,expect", FP16_KAT)
def test_fp16_decode_known_answers(h, expect):
    assert oc.fp16_to_f32_bits(h) == expect
    assert int(on.fp16_bits_to_f32(np.array([h], dtype=np.uint16)).view(np.uint32)[0]) == expect


def test_fp16_decode_all_65536_c_vs_numpy_vs_ieee():
    hs = np.arange(65536, dtype=np.uint16)
    a = on.fp16_bits_to_f32(hs).view(np.uint32)
    b = np.array([oc.fp16_to_f32_bits(int(h)) for h in hs], dtype=np.uint32)
    assert (a == b).all()
    nan = np.isnan(hs.view(np.float16))
    ieee = hs.view(np.float16).astype(np.float32).view(np.uint32)
    assert (a[~nan] == ieee[~nan]).all()
    assert np.isnan(a.view(np.float32)[nan]).all()


def test_f32_to_fp16_round_to_nearest_even():
    rng = np.random.default_rng(7)
    xs = np.concatenate([rng.standard_normal(20000).astype(np.float32) * np.float32(s)
                         for s in (1, 1e-3, 1e-5, 1e-7, 3e-8, 1e4, 7e4)])
    edge = np.array([np.inf, -np.inf, 0.0, -0.0, 65504, 65519.99, 65520, 2.0**-25, 2.0**-25 * 1.0000001,
                     2.0**-24 * 1.5, 2.0**-24 * 2.5, 1 + 2.0**-11, 1 + 3 * 2.0**-11], dtype=np.float32)
    xs = np.concatenate([xs, edge])
    got = np.array([oc.f32_to_fp16(float(x)) for x in xs], dtype=np.uint16)
    assert (got == on.f32_to_fp16_bits(xs)).all()
    # ties: 1 + 2^-11 is halfway between 1 and 1 + 2^-10 -> even (1); 1 + 3*2^-11 -> 1 + 2^-9
    assert oc.f32_to_fp16(1 + 2.0**-11) == 0x3C00
    assert oc.f32_to_fp16(1 + 3 * 2.0**-11) == 0x3C02


# ---- dequantize known answers ----------------------------------------------------------
def _q4_block():
    # D = 0x3800 (0.5); Qs[j] = j | (15 - j) << 4
    qs = np.array([j | ((15 - j) << 4) for j in range(16)], dtype=np.uint8)
    return np.concatenate([np.array([0x00, 0x38], dtype=np.uint8), qs])


def test_dequantize_q4_0_go_order_known_answer():
    # quantized.go:87-92: y[2j] = d*(lo-8) = 0.5*(j-8); y[2j+1] = d*(hi-8) = 0.5*(7-j)
    expect = np.empty(32, dtype=np.float32)
    for j in range(16):
        expect[2 * j] = 0.5 * (j - 8)
        expect[2 * j + 1] = 0.5 * (7 - j)
    for f in (oc.dequantize, on.dequantize):
        assert (bits(f(oc.Q4_0, oc.ORDER_GO, _q4_block())) == bits(expect)).all()
    assert expect[0] == -4.0 and expect[1] == 3.5 and expect[31] == -4.0


def test_dequantize_q4_0_split_order_known_answer():
    # quantized.cu:862-866: y[j] = 0.5*(j-8); y[j+16] = 0.5*(7-j)
    expect = np.array([0.5 * (j - 8) for j in range(16)] + [0.5 * (7 - j) for j in range(16)], dtype=np.float32)
    for f in (oc.dequantize, on.dequantize):
        assert (bits(f(oc.Q4_0, oc.ORDER_SPLIT, _q4_block())) == bits(expect)).all()


def test_dequantize_q8_0_known_answer():
    # D = 0x3C00 (1.0), Qs[i] = i - 16  ->  y[i] = i - 16   (quantized.go:131-136)
    blk = np.concatenate([np.array([0x00, 0x3C], dtype=np.uint8), (np.arange(32) - 16).astype(np.int8).view(np.uint8)])
    expect = (np.arange(32) - 16).astype(np.float32)
    for f in (oc.dequantize, on.dequantize):
        assert (bits(f(oc.Q8_0, 0, blk)) == bits(expect)).all()


def test_dequantize_edge_scales_bit_exact_between_restatements():
    scales = [0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0xFBFF, 0x7C00, 0xFC00, 0x7E00, 0x7C01, 0xFE01]
    rng = np.random.default_rng(3)
    for qt in (oc.Q4_0, oc.Q8_0):
        bb = oc.BLOCK_BYTES[qt]
        blocks = rng.integers(0, 256, size=(len(scales), bb), dtype=np.uint8)
        for i, s in enumerate(scales):
            blocks[i, 0], blocks[i, 1] = s & 0xFF, s >> 8
        for order in (0, 1):
            assert (bits(oc.dequantize(qt, order, blocks)) == bits(on.dequantize(qt, order, blocks))).all()


# ---- quantizers: quantized.metal:4187-4211 (Q4_0), :4129-4145 (Q8_0) -------------------
def test_quantize_q4_0_all_zero_block():
    for order in (0, 1):
        blk = oc.quantize(oc.Q4_0, order, np.zeros(32, dtype=np.float32))
        # max = +0 -> d = 0 / -8 = -0 (stored as 0x8000); id = 0; every q = (int8)(8.5) = 8
        assert blk[0] == 0 and blk[1] == 0x80 and (blk[2:] == 0x88).all()
        assert (oc.dequantize(oc.Q4_0, order, blk) == 0).all()


def test_quantize_q4_0_extremes_and_sign_of_first_max():
    v = np.zeros(32, dtype=np.float32)
    v[5], v[9] = 2.0, -2.0  # equal magnitude: the first one (index 5, positive) gives max = +2
    blk = oc.quantize(oc.Q4_0, oc.ORDER_SPLIT, v)
    assert _u16(blk) == 0xB400  # d = 2 / -8 = -0.25
    deq = oc.dequantize(oc.Q4_0, oc.ORDER_SPLIT, blk)
    assert deq[5] == 2.0  # q = 0 -> -0.25 * -8
    assert deq[9] == -1.75  # q clamps at 15 -> -0.25 * 7
    v[5], v[9] = -2.0, 2.0
    blk = oc.quantize(oc.Q4_0, oc.ORDER_SPLIT, v)
    assert _u16(blk) == 0x3400  # d = +0.25


def test_quantize_q8_0_rounds_half_away_from_zero():
    v = np.zeros(32, dtype=np.float32)
    v[0], v[1], v[2], v[3] = 127.0, 0.5, -0.5, 2.5  # d = 1 exactly
    blk = oc.quantize(oc.Q8_0, 0, v)
    q = blk[2:].view(np.int8)
    assert _u16(blk) == 0x3C00
    assert list(q[:4]) == [127, 1, -1, 3]


@pytest.mark.parametrize("qt", [oc.Q4_0, oc.Q8_0])
@pytest.mark.parametrize("order", [0, 1])
def test_quantize_c_vs_numpy_bytes(qt, order):
    rng = np.random.default_rng(11 + qt + order)
    w = (rng.standard_normal((96, 320)) * 0.02).astype(np.float32)
    w[0, :32] = 0
    w[1, 32:64] = np.float32(1e-8)
    w[2, :] *= np.float32(1e3)
    a, b = oc.quantize(qt, order, w), on.quantize(qt, order, w)
    assert (a == b).all()
    deq = oc.dequantize(qt, order, a).reshape(w.shape)
    step = np.abs(w).reshape(-1, 32).max(axis=1).repeat(32).reshape(w.shape) / (8 if qt == oc.Q4_0 else 127)
    # one quantization step at most (plus the f16 resolution of a scale that underflows)
    assert (np.abs(deq - w) <= step * 1.01 + 8 * 2.0**-24).all()


def test_quantizers_match_gguf_package_in_split_order():
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((64, 512)) * 0.02).astype(np.float32)
    for qt, t in ((oc.Q4_0, gguf.GGMLQuantizationType.Q4_0), (oc.Q8_0, gguf.GGMLQuantizationType.Q8_0)):
        g = quants.quantize(w, t).reshape(-1)
        assert (g == oc.quantize(qt, oc.ORDER_SPLIT, w)).all()
        dg = quants.dequantize(g.reshape(64, -1), t).reshape(-1)
        assert (bits(dg) == bits(oc.dequantize(qt, oc.ORDER_SPLIT, g))).all()


# ---- naive matmul: tensor/internal/cpu/kernels/conv.go:373-389 -------------------------
def test_matmul_strided_known_answer_and_order():
    # [[1,2,3],[4,5,6]] x [[7,8],[9,10],[11,12]] = [[58,64],[139,154]]
    a = np.array([1, 2, 3, 4, 5, 6], dtype=np.float32)
    b = np.array([7, 8, 9, 10, 11, 12], dtype=np.float32)
    c = oc.matmul_strided(a, b, 2, 2, 3, [0, 3, 1], [0, 2, 1])
    assert c.reshape(-1).tolist() == [58, 64, 139, 154]
    # transposed rhs view, strides {0,1,K}: the nn.Linear case (storage.go:893-897)
    bt = np.array([7, 9, 11, 8, 10, 12], dtype=np.float32)  # W[n,k]
    c2 = oc.matmul_strided(a, bt, 2, 2, 3, [0, 3, 1], [0, 1, 3])
    assert c2.reshape(-1).tolist() == [58, 64, 139, 154]
    # summation is strictly left to right in f32: 1e8 + 1 - 1e8 = 0, not 1
    a3 = np.array([1e8, 1.0, -1e8], dtype=np.float32)
    ones = np.ones(3, dtype=np.float32)
    assert oc.matmul_strided(a3, ones, 1, 1, 3, [0, 3, 1], [0, 1, 1]).item() == 0.0


@pytest.mark.parametrize("qt", [oc.Q4_0, oc.Q8_0])
@pytest.mark.parametrize("order", [0, 1])
def test_qmatmul_c_vs_numpy_bit_exact_and_close_to_f64(qt, order):
    rng = np.random.default_rng(5 + qt + order)
    n, k, m = 40, 512, 3
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    blocks = oc.quantize(qt, order, w)
    y = oc.qmatmul(qt, order, x, blocks, n)
    assert (bits(y) == bits(on.qmatmul(qt, order, x, blocks, n))).all()
    assert (bits(y) == bits(oc.qmatmul(qt, order, x, blocks, n, nthreads=4))).all()
    wd = oc.dequantize(qt, order, blocks).reshape(n, k).astype(np.float64)
    ref = x.astype(np.float64) @ wd.T
    assert np.abs(y - ref).max() / np.abs(ref).max() < 1e-5


def test_q4_0_orders_differ_on_the_same_bytes():
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((8, 64)) * 0.02).astype(np.float32)
    x = rng.standard_normal((1, 64)).astype(np.float32)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    y0 = oc.qmatmul(oc.Q4_0, 0, x, blocks, 8)
    y1 = oc.qmatmul(oc.Q4_0, 1, x, blocks, 8)
    assert np.abs(y0 - y1).max() > 1e-3  # same multiset of weights, different positions


# ---- Q8_1 activations: tensor/internal/cuda/kernels/quantized.cu:3521-3558 -------------
def test_quantize_q8_1_known_answer_and_zero_block():
    x = np.zeros(64, dtype=np.float32)
    x[:32] = np.arange(32) - 16  # amax = 16 -> d = 16/127; q = roundf(x / d)
    out = oc.quantize_q8_1(x)
    assert (out == on.quantize_q8_1(x)).all()
    d = np.float32(16) / np.float32(127)
    assert _u16(out) == np.float16(d).view(np.uint16)
    assert _u16(out[2:]) == np.float16(-16.0).view(np.uint16)  # sum of -16..15
    q = out[4:36].view(np.int8)
    assert q[0] == -127 and q[16] == 0 and q[31] == 119  # 15/(16/127) = 119.06
    assert (out[36:] == 0).all()  # zero block: d = 0, sum = 0, q = 0 (amax == 0 branch)


def test_q8_1_matmul_is_close_to_but_not_within_1e3_of_the_cpu_path():
    rng = np.random.default_rng(0)
    n, k = 64, 4096
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((1, k)).astype(np.float32)
    blocks = oc.quantize(oc.Q4_0, 1, w)
    y1 = oc.qmatmul(oc.Q4_0, 1, x, blocks, n)
    y2 = oc.qmatmul(oc.Q4_0, 1, x, blocks, n, q8_1=True)
    err = np.abs(y2 - y1).max() / np.abs(y1).max()
    assert 1e-4 < err < 5e-2  # single-slice int8 activations: percent-level, not 1e-3


# ---- golden fixtures -------------------------------------------------------------------
def test_golden_fixture_reproduced_by_both_restatements():
    g = np.load(GOLDEN)
    w, x = g["w"], g["x"]
    n = w.shape[0]
    for qt, name in ((oc.Q4_0, "q4_0"), (oc.Q8_0, "q8_0")):
        for order in (0, 1):
            tag = f"{name}_o{order}"
            if f"{tag}_blocks" not in g:
                continue
            blocks = g[f"{tag}_blocks"]
            for mod in (oc, on):
                assert (mod.quantize(qt, order, w) == blocks).all()
                assert (bits(mod.dequantize(qt, order, blocks)) == bits(g[f"{tag}_deq"])).all()
                assert (bits(mod.qmatmul(qt, order, x, blocks, n)) == bits(g[f"{tag}_y"])).all()
            assert (bits(oc.qmatmul(qt, order, x, blocks, n, q8_1=True)) == bits(g[f"{tag}_y_q8_1"])).all()
    assert (oc.quantize_q8_1(x) == g["x_q8_1"]).all()
    assert (on.quantize_q8_1(x) == g["x_q8_1"]).all()
