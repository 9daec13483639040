"""Prefill GEMM (m > 8) on the tensor cores, CQ_ACT_F16, through the C ABI.

Two checks per case: (1) against a NumPy emulation of the mode's own arithmetic -- activations and
dequantized weights each rounded once to f16, products summed in f64 -- where only f32 accumulation
order may differ (bound 2e-5); (2) against candy's CPU path (the oracle) under the stated bar,
max|y - y_ref| / max|y_ref| <= 1e-3.  At the BASELINE config-3 sizes the CPU path is evaluated on a
sample of activation rows (the scalar oracle needs ~1e11 operations for all of them)."""
import numpy as np
import pytest

from helpers import REL_TOL, make_case, rel_err
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu
ACT_F16 = 2


def emulate_f16(qt, order, x, blocks, n):
    k = x.shape[1]
    w16 = oc.dequantize(qt, order, blocks).reshape(n, k).astype(np.float16).astype(np.float64)
    x16 = x.astype(np.float16).astype(np.float64)
    return x16 @ w16.T


def run(device, qt, order, x, blocks, n, actmode=ACT_F16):
    from candy_b200.backend import QStorage
    m, k = x.shape
    qs = QStorage.from_blocks(device, qt, order, n, k, blocks)
    xs = device.storage_from_slice(x)
    y = xs.matmul(qs, 1, m, n, k, actmode).data().reshape(m, n)
    device.synchronize()
    return y


@pytest.mark.parametrize("qt,order", [(oc.Q4_0, 0), (oc.Q4_0, 1), (oc.Q8_0, 0)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (16, 300, 512), (130, 257, 96), (9, 40, 32),
                                   (512, 1024, 4096), (300, 700, 1056)])
def test_gemm_f16_small_and_ragged(device, qt, order, m, n, k):
    w, x = make_case(5000 + m + n + k, n, k, m)
    blocks = oc.quantize(qt, order, w)
    got = run(device, qt, order, x, blocks, n)
    assert rel_err(got, emulate_f16(qt, order, x, blocks, n)) < 2e-5
    rows = np.linspace(0, m - 1, num=min(m, 6), dtype=int)
    cpu = oc.qmatmul(qt, order, x[rows], blocks, n, nthreads=8)
    assert rel_err(got[rows], cpu) <= REL_TOL


@pytest.mark.parametrize("qt", [oc.Q4_0, oc.Q8_0])
@pytest.mark.parametrize("m", [16, 128, 512, 2048])
def test_config3_prefill_gemm(device, qt, m):
    n, k = 11008, 4096
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    x = rng.standard_normal((m, k), dtype=np.float32)
    blocks = oc.quantize(qt, 0, w)
    got = run(device, qt, 0, x, blocks, n)
    assert rel_err(got, emulate_f16(qt, 0, x, blocks, n)) < 2e-5
    rows = np.linspace(0, m - 1, num=4, dtype=int)
    cpu = oc.qmatmul(qt, 0, x[rows], blocks, n, nthreads=8)
    err = rel_err(got[rows], cpu)
    assert err <= REL_TOL, f"f16-operand GEMM vs CPU path: {err}"


@pytest.mark.parametrize("actmode", [0, 1])
def test_wide_batches_in_f32_and_q8_1_modes_use_the_decode_kernels(device, actmode):
    w, x = make_case(77, 96, 1024, 19)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    got = run(device, oc.Q4_0, 0, x, blocks, 96, actmode=actmode)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, 96, nthreads=8, q8_1=bool(actmode))
    assert rel_err(got, want) < 1e-4


# ---- narrow batches (8 < m <= 128, Q4_0, k % 256 == 0): blocks dequantized into tensor memory ----
@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (2, 4096, 4096), (8, 11008, 4096), (9, 128, 256), (16, 300, 512), (17, 129, 768), (32, 1000, 1024), (33, 4096, 4096), (64, 257, 2304),
                                   (64, 11008, 4096), (12, 8192, 14336), (100, 300, 512), (128, 1000, 2048), (97, 5000, 4096)])
def test_narrow_batch_gemm_streams_raw_blocks(device, order, m, n, k):
    w, x = make_case(9000 + m + n + k, n, k, m)
    blocks = oc.quantize(oc.Q4_0, order, w)
    got = run(device, oc.Q4_0, order, x, blocks, n)
    assert rel_err(got, emulate_f16(oc.Q4_0, order, x, blocks, n)) < 2e-5
    rows = np.linspace(0, m - 1, num=min(m, 4), dtype=int)
    cpu = oc.qmatmul(oc.Q4_0, order, x[rows], blocks, n, nthreads=8)
    assert rel_err(got[rows], cpu) <= REL_TOL
    # the two-step path (f16 copy of W, then the wide kernel) computes from identical operands
    device.set_option("gemm_variant", 3)
    try:
        two_step = run(device, oc.Q4_0, order, x, blocks, n)
    finally:
        device.set_option("gemm_variant", 0)
    assert rel_err(got, two_step) < 5e-5  # f32 summation order differs (k split, tensor-core internals)


def test_narrow_batch_gemm_edge_scales(device):
    """Blocks whose scale is zero, subnormal or large: the f16 product d*(q-8) must still round once."""
    n, k, m = 256, 512, 16
    rng = np.random.default_rng(5)
    blocks = rng.integers(0, 256, size=(n * k // 32, 18), dtype=np.uint8)
    scales = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0x57FF, 0xD000], dtype=np.uint16)
    d = scales[rng.integers(0, len(scales), size=blocks.shape[0])]
    blocks[:, 0], blocks[:, 1] = d & 0xFF, d >> 8
    x = rng.standard_normal((m, k), dtype=np.float32)
    got = run(device, oc.Q4_0, 0, x, blocks.reshape(-1), n)
    assert rel_err(got, emulate_f16(oc.Q4_0, 0, x, blocks.reshape(-1), n)) < 2e-5


@pytest.mark.parametrize("m,n,k", [(9, 128, 256), (16, 300, 512), (33, 4096, 4096), (64, 257, 2304), (64, 11008, 4096), (12, 8192, 14336),
                                   (16, 11008, 4096), (65, 300, 512), (100, 1024, 2048), (128, 11008, 4096)])  # > 64 rows: two 64-row passes
def test_narrow_batch_gemm_q8_0(device, m, n, k):
    w, x = make_case(9100 + m + n + k, n, k, m)
    blocks = oc.quantize(oc.Q8_0, 0, w)
    got = run(device, oc.Q8_0, 0, x, blocks, n)
    assert rel_err(got, emulate_f16(oc.Q8_0, 0, x, blocks, n)) < 2e-5
    rows = np.linspace(0, m - 1, num=min(m, 4), dtype=int)
    cpu = oc.qmatmul(oc.Q8_0, 0, x[rows], blocks, n, nthreads=8)
    assert rel_err(got[rows], cpu) <= REL_TOL
    device.set_option("gemm_variant", 3)
    try:
        two_step = run(device, oc.Q8_0, 0, x, blocks, n)
    finally:
        device.set_option("gemm_variant", 0)
    assert rel_err(got, two_step) < 5e-5  # f32 summation order differs


def test_narrow_batch_gemm_q8_0_edge_values(device):
    """Every int8 value and scale patterns incl. zero and subnormal scales."""
    n, k, m = 256, 512, 16
    rng = np.random.default_rng(6)
    blocks = rng.integers(0, 256, size=(n * k // 32, 34), dtype=np.uint8)
    blocks[0, 2:] = np.arange(32, dtype=np.uint8) * 8          # 0, 8, ..., 248 (as int8: 0..127, -128..-8)
    blocks[1, 2:] = np.array([0x80, 0x7F, 0xFF, 0x01] * 8, dtype=np.uint8)
    scales = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0x2E00, 0xB000], dtype=np.uint16)
    d = scales[rng.integers(0, len(scales), size=blocks.shape[0])]
    blocks[:, 0], blocks[:, 1] = d & 0xFF, d >> 8
    x = rng.standard_normal((m, k), dtype=np.float32)
    got = run(device, oc.Q8_0, 0, x, blocks.reshape(-1), n)
    assert rel_err(got, emulate_f16(oc.Q8_0, 0, x, blocks.reshape(-1), n)) < 2e-5


@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("m,n,k", [(129, 256, 256), (130, 257, 512), (300, 700, 1024), (512, 1000, 4096), (1000, 2048, 2304)])
def test_wide_gemm_dequantizes_in_the_producer(device, order, m, n, k):
    """m > 128, Q4_0, k % 256 == 0: no f16 copy of W; the raw blocks are dequantized inside the GEMM.  Same f16
    values as the two-step route (exact n - 8, one rounding in the product with the scale), so the two agree to
    summation order; ragged m and n exercise the zero-filled tile edges."""
    w, x = make_case(7000 + m + n + k + order, n, k, m)
    blocks = oc.quantize(oc.Q4_0, order, w)
    device.set_option("gemm_fused_dequant", 2)  # at every batch size, not only where it is the faster route
    try:
        got = run(device, oc.Q4_0, order, x, blocks, n)
        device.set_option("gemm_fused_dequant", 0)
        two_step = run(device, oc.Q4_0, order, x, blocks, n)
    finally:
        device.set_option("gemm_fused_dequant", 1)
    assert rel_err(got, emulate_f16(oc.Q4_0, order, x, blocks, n)) < 2e-5
    assert rel_err(got, two_step) < 2e-5
    rows = np.linspace(0, m - 1, num=4, dtype=int)
    assert rel_err(got[rows], oc.qmatmul(oc.Q4_0, order, x[rows], blocks, n, nthreads=8)) <= REL_TOL


def test_wide_gemm_edge_scales(device):
    """Zero, negative-zero, subnormal, large and negative scales through the in-producer dequantizer."""
    n, k, m = 512, 512, 160
    rng = np.random.default_rng(6)
    blocks = rng.integers(0, 256, size=(n * k // 32, 18), dtype=np.uint8)
    scales = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0x57FF, 0xD000], dtype=np.uint16)
    d = scales[rng.integers(0, len(scales), size=blocks.shape[0])]
    blocks[:, 0], blocks[:, 1] = d & 0xFF, d >> 8
    x = rng.standard_normal((m, k), dtype=np.float32)
    got = run(device, oc.Q4_0, 0, x, blocks.reshape(-1), n)
    assert rel_err(got, emulate_f16(oc.Q4_0, 0, x, blocks.reshape(-1), n)) < 2e-5


@pytest.mark.parametrize("qt", [oc.Q4_0, oc.Q8_0])
@pytest.mark.parametrize("m,n,k", [(400, 700, 1056), (513, 1300, 2048), (1024, 4096, 4096)])
def test_wide_gemm_on_cta_pairs_and_on_single_ctas(device, qt, m, n, k):
    """m > 384: the f16 GEMM runs 256 x 256 tiles on CTA pairs (one MMA of M = 256 across two SMs); with the
    option off it runs 128 x 256 tiles per CTA.  Both against the mode's own arithmetic, ragged edges included."""
    w, x = make_case(8000 + m + n + k + qt, n, k, m)
    blocks = oc.quantize(qt, 0, w)
    want = emulate_f16(qt, 0, x, blocks, n)
    got_pair = run(device, qt, 0, x, blocks, n)
    device.set_option("gemm_pair", 0)
    try:
        got_single = run(device, qt, 0, x, blocks, n)
    finally:
        device.set_option("gemm_pair", 1)
    assert rel_err(got_pair, want) < 2e-5
    assert rel_err(got_single, want) < 2e-5
