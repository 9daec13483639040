"""The K super-block formats (Q2_K .. Q6_K, 256 values per block).  The reference defines them only through its
CUDA dequantizers (tensor/internal/cuda/kernels/quantized.cu:899-1147) and holds no test or fixture for them;
the CPU oracle restates those kernels and is pinned bit for bit to the third-party gguf package's
dequantizers on random block bytes (CPU tests), and the GPU kernels must reproduce the oracle's bits and, for
matmuls, stay within the 1e-3 bar of dequantize-then-naive-matmul (GPU tests)."""
import numpy as np
import pytest

from helpers import rel_err
from oracle import oracle_c as oc

K_TYPES = [oc.Q2_K, oc.Q3_K, oc.Q4_K, oc.Q5_K, oc.Q6_K]
SCALE_OFFSETS = {oc.Q2_K: [80, 82], oc.Q3_K: [108], oc.Q4_K: [0, 2], oc.Q5_K: [0, 2], oc.Q6_K: [208]}
GGUF_NAMES = {oc.Q2_K: "Q2_K", oc.Q3_K: "Q3_K", oc.Q4_K: "Q4_K", oc.Q5_K: "Q5_K", oc.Q6_K: "Q6_K"}


def random_blocks(qt, nblocks, seed, small=False):
    """Random bits in every field, finite f16 super-block scales (subnormal, normal, both signs, zero)."""
    rng = np.random.default_rng(seed)
    bb = oc.K_BLOCK_BYTES[qt]
    blocks = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    for off in SCALE_OFFSETS[qt]:
        if small:  # weights of ordinary size for matmul tests
            h = (rng.uniform(0.0005, 0.004, size=nblocks).astype(np.float16)).view(np.uint16)
        else:
            h = rng.integers(0, 0x7C00, size=nblocks).astype(np.uint16) | (rng.integers(0, 2, size=nblocks).astype(np.uint16) << 15)
            h[:4] = [0x0000, 0x8000, 0x0001, 0x7BFF]
        blocks[:, off] = h & 0xFF
        blocks[:, off + 1] = h >> 8
    return blocks.reshape(-1)


@pytest.mark.parametrize("qt", K_TYPES)
def test_oracle_dequantize_equals_gguf_bit_for_bit(qt):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    blocks = random_blocks(qt, 700, 40 + qt)
    mine = oc.dequantize_k(qt, blocks)
    ref = quants.dequantize(blocks.reshape(700, -1), getattr(gguf.GGMLQuantizationType, GGUF_NAMES[qt])).reshape(-1).astype(np.float32)
    assert (mine.view(np.uint32) == ref.view(np.uint32)).all()


def test_q4_k_hand_derived_block():
    """d = 1, dmin = 0.5, every 6-bit scale = 2 and min = 3, every nibble byte 0x21: low values 2*1 - 1.5, high 2*2 - 1.5."""
    b = np.zeros(144, dtype=np.uint8)
    b[0:2] = [0x00, 0x3C]  # 1.0
    b[2:4] = [0x00, 0x38]  # 0.5
    b[4:8] = 2             # scales 0..3
    b[8:12] = 3            # mins 0..3
    b[12:16] = 2 | (3 << 4)  # scales 4..7 (low nibble) and mins 4..7 (high nibble); their top bits (in bytes 0..7 >> 6) are 0
    b[16:] = 0x21
    y = oc.dequantize_k(oc.Q4_K, b).reshape(4, 2, 32)
    assert (y[:, 0] == 0.5).all() and (y[:, 1] == 2.5).all()


@pytest.mark.gpu
@pytest.mark.parametrize("qt", K_TYPES)
def test_gpu_dequantize_bit_exact(device, qt):
    from candy_b200.backend import QStorage
    nb = 301
    blocks = random_blocks(qt, nb, 50 + qt)
    qs = QStorage.from_blocks(device, qt, 1, 1, nb * 256, blocks)
    got = qs.dequantize().data()
    want = oc.dequantize_k(qt, blocks)
    assert (got.view(np.uint32) == want.view(np.uint32)).all()


@pytest.mark.gpu
@pytest.mark.parametrize("qt", K_TYPES)
@pytest.mark.parametrize("m,n,k", [(1, 300, 1024), (3, 129, 512), (8, 64, 4096)])
def test_gpu_gemv_matches_dequantize_then_matmul(device, qt, m, n, k):
    from candy_b200.backend import QStorage
    blocks = random_blocks(qt, n * (k // 256), 60 + qt + m, small=True)
    x = np.random.default_rng(m + n).standard_normal((m, k)).astype(np.float32)
    qs = QStorage.from_blocks(device, qt, 1, n, k, blocks)
    y = device.storage_from_slice(x).matmul(qs, 1, m, n, k, 0).data().reshape(m, n)
    device.synchronize()
    assert rel_err(y, oc.qmatmul_k(qt, x, blocks, n, nthreads=8)) < 2e-5


@pytest.mark.gpu
@pytest.mark.parametrize("qt", [oc.Q4_K, oc.Q6_K])
def test_gpu_gemm_f16_route(device, qt):
    from candy_b200.backend import QStorage
    m, n, k = 40, 384, 1024
    blocks = random_blocks(qt, n * (k // 256), 70 + qt, small=True)
    x = np.random.default_rng(7).standard_normal((m, k)).astype(np.float32)
    qs = QStorage.from_blocks(device, qt, 1, n, k, blocks)
    y = device.storage_from_slice(x).matmul(qs, 1, m, n, k, 2).data().reshape(m, n)
    device.synchronize()
    assert rel_err(y, oc.qmatmul_k(qt, x, blocks, n, nthreads=8)) < 1e-3


@pytest.mark.gpu
def test_k_formats_refuse_what_is_not_built(device):
    from candy_b200 import abi
    lib, ctx = device._lib, device.ctx
    buf = device.alloc(1 << 16)
    p = buf.ptr
    assert lib.cq_quantize_rows(ctx, abi.Q4_K, 1, p, 1, 256, p) == abi.ERR_UNSUPPORTED
    assert lib.cq_qmatmul(ctx, abi.Q4_K, 0, 0, p, 1, 256, 256, p, 4, p, 4) == abi.ERR_UNSUPPORTED   # interleaved order does not exist
    assert lib.cq_qmatmul(ctx, abi.Q4_K, 1, 0, p, 1, 128, 128, p, 4, p, 4) == abi.ERR_INVALID_ARG   # k % 256
    assert lib.cq_qmatmul(ctx, abi.Q4_K, 1, 1, p, 1, 256, 256, p, 4, p, 4) == abi.ERR_UNSUPPORTED   # Q8_1 activations
    assert lib.cq_blocks_bytes(abi.Q6_K, 3, 512) == 3 * 2 * 210
    device.synchronize()
