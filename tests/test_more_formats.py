"""Q4_1 / Q5_0 / Q5_1: the oracle against hand-derived answers and a third-party GGUF codec (CPU),
then the CUDA library through its C ABI against the oracle (GPU): bytes and dequantized values
bit for bit, matmul outputs under the 1e-3 bar."""
import numpy as np
import pytest

from helpers import REL_TOL, make_case, rel_err
from oracle import oracle_c as oc

FORMATS = [(oc.Q4_1, 0), (oc.Q4_1, 1), (oc.Q5_0, 1), (oc.Q5_1, 1)]


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def f16(v):
    return np.array([v], dtype=np.float16).view(np.uint8)


def edge_blocks(qt, rng, nblocks=64):
    """Random block bytes with finite scales of every magnitude (subnormal f16 scales included)."""
    bb = oc.BLOCK_BYTES[qt]
    raw = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    scales = np.concatenate([[0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0xFBFF],
                             rng.integers(0, 0x7C00, size=nblocks - 8)]).astype(np.uint16)
    raw[:, 0:2] = scales.view(np.uint8).reshape(-1, 2)
    if qt in (oc.Q4_1, oc.Q5_1):
        mins = rng.integers(0, 0x7C00, size=nblocks).astype(np.uint16) | (rng.integers(0, 2, size=nblocks).astype(np.uint16) << 15)
        raw[:, 2:4] = mins.view(np.uint8).reshape(-1, 2)
    return raw.reshape(-1)


# ---- CPU: the oracle itself ----------------------------------------------------------------
def test_known_answers_by_hand():
    # Q4_1, d = 0.5, m = -1: byte j = j | (15-j) << 4
    qs = np.array([j | ((15 - j) << 4) for j in range(16)], dtype=np.uint8)
    blk = np.concatenate([f16(0.5), f16(-1.0), qs])
    go = oc.dequantize(oc.Q4_1, 0, blk)
    assert go[0] == -1.0 and go[1] == 0.5 * 15 - 1 and go[2] == -0.5 and go[31] == -1.0
    split = oc.dequantize(oc.Q4_1, 1, blk)
    assert (split[:16] == 0.5 * np.arange(16) - 1).all() and (split[16:] == 0.5 * (15 - np.arange(16)) - 1).all()
    # Q5_0, d = 1: nibbles 0, fifth bits set for values 0..15 only -> 0 for those, -16 for the rest
    blk = np.concatenate([f16(1.0), np.array([0xFF, 0xFF, 0, 0], dtype=np.uint8), np.zeros(16, dtype=np.uint8)])
    y = oc.dequantize(oc.Q5_0, 1, blk)
    assert (y[:16] == 0).all() and (y[16:] == -16).all()
    # Q5_1, d = 0.25, m = 2: value j = j (fifth bit for j >= 16 comes from the high half of qh)
    qs = np.array([j | (j << 4) for j in range(16)], dtype=np.uint8)
    blk = np.concatenate([f16(0.25), f16(2.0), np.array([0, 0, 0xFF, 0xFF], dtype=np.uint8), qs])
    y = oc.dequantize(oc.Q5_1, 1, blk)
    assert (y == 0.25 * np.arange(32) + 2).all()


@pytest.mark.parametrize("qt,name", [(oc.Q4_1, "Q4_1"), (oc.Q5_0, "Q5_0"), (oc.Q5_1, "Q5_1")])
def test_oracle_agrees_with_the_gguf_codec(qt, name):
    gguf = pytest.importorskip("gguf")
    t = getattr(gguf.GGMLQuantizationType, name)
    rng = np.random.default_rng(qt)
    w = (rng.standard_normal((48, 512)) * 0.05).astype(np.float32)
    w[0, :32] = 0            # an all-zero block
    w[1, :32] = 0.125        # a constant block: d = 0 for the min/max formats
    w[2, 5] = 30.0           # one dominant value
    blocks = oc.quantize(qt, 1, w)
    assert (blocks == gguf.quants.quantize(w, t).reshape(-1)).all()
    raw = edge_blocks(qt, rng)
    want = gguf.quants.dequantize(raw.reshape(1, -1), t).astype(np.float32).reshape(-1)
    assert (bits(oc.dequantize(qt, 1, raw)) == bits(want)).all()


def test_q4_1_orders_are_permutations_of_each_other():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((4, 64)).astype(np.float32)
    a = oc.dequantize(oc.Q4_1, 0, oc.quantize(oc.Q4_1, 0, w))
    b = oc.dequantize(oc.Q4_1, 1, oc.quantize(oc.Q4_1, 1, w))
    assert (bits(a) == bits(b)).all()  # each quantizer/dequantizer pair returns source order
    assert np.abs(a - w.reshape(-1)).max() < (w.max() - w.min()) / 15


# ---- GPU: the library against the oracle ----------------------------------------------------
def gpu_qmatmul(device, qt, order, x, blocks, n, actmode=0):
    from candy_b200.backend import QStorage
    m, k = x.shape
    qs = QStorage.from_blocks(device, qt, order, n, k, blocks)
    y = device.storage_from_slice(x).matmul(qs, 1, m, n, k, actmode).data().reshape(m, n)
    device.synchronize()
    return y


@pytest.mark.gpu
@pytest.mark.parametrize("qt,order", FORMATS)
def test_quantize_and_dequantize_bit_exact(device, qt, order):
    from candy_b200.backend import QStorage
    rng = np.random.default_rng(10 * qt + order)
    w = (rng.standard_normal((37, 1024)) * 0.03).astype(np.float32)
    w[0, :32] = 0
    w[1, 32:64] = -0.5
    w[2, 70] = 1e4
    w[3] *= 1e-6
    got = QStorage.quantize(device, qt, order, w).data()
    assert (got == oc.quantize(qt, order, w)).all()
    raw = edge_blocks(qt, rng, 256)
    qs = QStorage.from_blocks(device, qt, order, 1, 256 * 32, raw)
    assert (bits(qs.dequantize().data()) == bits(oc.dequantize(qt, order, raw))).all()


@pytest.mark.gpu
@pytest.mark.parametrize("qt,order", FORMATS)
@pytest.mark.parametrize("m,n,k", [(1, 300, 4096), (1, 33, 96), (3, 130, 1024), (8, 64, 11008), (1, 4096, 4096), (11, 70, 512)])
def test_gemv_f32_matches_cpu_path(device, qt, order, m, n, k):
    w, x = make_case(500 + m + n + k, n, k, m)
    w += 0.01  # a non-zero mean exercises the block minimum
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=8)
    err = rel_err(gpu_qmatmul(device, qt, order, x, blocks, n), want)
    # k % 256 == 0: streaming kernel, 16-bit block fixed-point activations (near 1e-5); else the plain f32 kernel
    assert err <= REL_TOL and err < (1e-4 if k % 256 == 0 else 2e-5), err
    device.set_option("gemv_force_simple", 1)
    try:
        err = rel_err(gpu_qmatmul(device, qt, order, x, blocks, n), want)
    finally:
        device.set_option("gemv_force_simple", 0)
    assert err < 2e-5, err


@pytest.mark.gpu
@pytest.mark.parametrize("qt,order", FORMATS)
@pytest.mark.parametrize("m,n,k", [(16, 512, 1024), (130, 300, 4096), (64, 256, 256)])
def test_gemm_f16_matches_cpu_path(device, qt, order, m, n, k):
    w, x = make_case(900 + m + n, n, k, m)
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=8)
    # emulation of the tensor-core path: f16 activations and f16 weights, products summed in f32
    w16 = oc.dequantize(qt, order, blocks).reshape(n, k).astype(np.float16).astype(np.float32)
    emu = x.astype(np.float16).astype(np.float32) @ w16.T
    got = gpu_qmatmul(device, qt, order, x, blocks, n, actmode=2)
    assert rel_err(got, emu) < 2e-5
    assert rel_err(got, want) <= REL_TOL


@pytest.mark.gpu
def test_unsupported_combinations_answer_cleanly(device):
    from candy_b200 import abi
    lib, ctx = device._lib, device.ctx
    w, x = make_case(1, 64, 256, 1)
    blocks = oc.quantize(oc.Q5_0, 1, w)
    from candy_b200.backend import QStorage
    qs = QStorage.from_blocks(device, oc.Q5_0, 1, 64, 256, blocks)
    xs = device.storage_from_slice(x)
    y = device.alloc(64)
    assert lib.cq_qmatmul(ctx, oc.Q5_0, 0, 0, xs.ptr, 1, 256, 256, qs.buf.ptr, 64, y.ptr, 64) == abi.CQ_ERR_UNSUPPORTED  # no interleaved Q5
    assert lib.cq_qmatmul(ctx, oc.Q5_0, 1, 1, xs.ptr, 1, 256, 256, qs.buf.ptr, 64, y.ptr, 64) == abi.CQ_ERR_UNSUPPORTED  # no Q8_1 activations
    assert lib.cq_qlinear_fused(ctx, oc.Q5_0, 1, xs.ptr, None, None, 1e-5, None, 1, 256, qs.buf.ptr, 64, 0, y.ptr, 64) == abi.CQ_ERR_UNSUPPORTED
    assert lib.cq_qmatmul(ctx, 5, 1, 0, xs.ptr, 1, 256, 256, qs.buf.ptr, 64, y.ptr, 64) == abi.CQ_ERR_INVALID_ARG
    assert lib.cq_blocks_bytes(oc.Q4_1, 2, 64) == 80 and lib.cq_blocks_bytes(oc.Q5_0, 2, 64) == 88 and lib.cq_blocks_bytes(oc.Q5_1, 2, 64) == 96
