"""Small batches (2..8 activation rows) against Q4_0 in one launch: the streaming kernel whose block dots run on
mma.sync (gemv_mma_kernel), in CQ_ACT_F32 and in CQ_ACT_Q8_1.  Checked against the CPU oracle over every batch
size, both element orders, row counts that leave ragged last stages, k values that need 1, 2, 4 and 8 k slices
per cluster, row strides, a bias, adversarial scales, and against the int8 tensor-core GEMM, which computes the
same integers and the same per-block terms."""
import numpy as np
import pytest

from helpers import make_case, rel_err
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _route(device):
    device.set_option("gemv_mma", 2)
    yield
    device.set_option("gemv_mma", 3)


def run(device, order, x, blocks, n, ldx=None, ldy=None, bias=None, act=0):
    from candy_b200.backend import QStorage
    m, k = x.shape
    ldx, ldy = ldx or k, ldy or n
    lib, ctx = device._lib, device.ctx
    qs = QStorage.from_blocks(device, oc.Q4_0, order, n, k, blocks)
    xp = np.zeros((m, ldx), dtype=np.float32)
    xp[:, :k] = x
    xs, ys = device.storage_from_slice(xp), device.zeros(m * ldy)
    if bias is None:
        st = lib.cq_qmatmul(ctx, oc.Q4_0, order, act, xs.ptr, m, k, ldx, qs.buf.ptr, n, ys.ptr, ldy)
    else:
        bs = device.storage_from_slice(bias)
        st = lib.cq_qlinear(ctx, oc.Q4_0, order, act, xs.ptr, m, k, ldx, qs.buf.ptr, n, bs.ptr, ys.ptr, ldy)
    assert st == 0, lib.cq_last_error(ctx)
    device.synchronize()
    out = ys.data().reshape(m, ldy)
    assert (out[:, n:] == 0).all()  # nothing written between the rows
    return out[:, :n]


@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("m", [2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("n,k", [(600, 4096), (4100, 11008), (96, 256), (5000, 2048), (2500, 8192), (700, 28672), (148 * 16 + 5, 512)])
def test_small_batch_matches_cpu_path(device, order, m, n, k):
    w, x = make_case(9500 + m + n + k, n, k, m)
    x[m - 1, :32] *= 1e-4
    x[0, 64:96] = 0.0  # an all-zero activation block
    blocks = oc.quantize(oc.Q4_0, order, w)
    want = oc.qmatmul(oc.Q4_0, order, x, blocks, n, nthreads=8)
    got = run(device, order, x, blocks, n)
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("m", [2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("n,k", [(600, 4096), (4100, 11008), (96, 256), (2500, 8192), (700, 28672), (148 * 16 + 5, 512), (300, 1536)])
def test_small_batch_q8_1_mode_matches_reference_cuda_arithmetic(device, order, m, n, k):
    w, x = make_case(9800 + m + n + k, n, k, m)
    x[m - 1, :32] *= 1e-4
    x[0, 64:96] = 0.0  # an all-zero activation block: d = 0, every q = 0
    blocks = oc.quantize(oc.Q4_0, order, w)
    want = oc.qmatmul(oc.Q4_0, order, x, blocks, n, nthreads=8, q8_1=True)
    got = run(device, order, x, blocks, n, act=1)
    assert rel_err(got, want) < 2e-5


@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("m", [3, 8])
def test_small_batch_agrees_with_the_int8_gemm(device, m, act):
    """Both kernels form the same 15-bit integers and the same per-block terms; only the order of the f32 sums differs."""
    n, k = 1500, 4096
    w, x = make_case(9600 + m, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    got = run(device, 0, x, blocks, n, act=act)
    device.set_option("gemv_mma", 0)
    other = run(device, 0, x, blocks, n, act=act)
    assert rel_err(got, other) < 2e-6


def test_small_batch_with_row_strides_and_bias(device):
    m, n, k = 5, 520, 1024
    w, x = make_case(9700, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    bias = np.random.default_rng(1).standard_normal(n).astype(np.float32)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8)
    assert rel_err(run(device, 0, x, blocks, n, ldx=k + 64, ldy=n + 8), want) < 1e-4
    assert rel_err(run(device, 0, x, blocks, n, bias=bias), want + bias) < 1e-4
    want81 = oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8, q8_1=True)
    assert rel_err(run(device, 0, x, blocks, n, ldx=k + 64, ldy=n + 8, act=1), want81) < 2e-5
    assert rel_err(run(device, 0, x, blocks, n, bias=bias, act=1), want81 + bias) < 2e-5
    k = 11008  # four k slices: the bias is added once, by the cluster's final sum
    w, x = make_case(9701, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8)
    assert rel_err(run(device, 0, x, blocks, n, bias=bias), want + bias) < 1e-4


def test_small_batch_q8_1_tiny_and_tied_activations(device):
    """Blocks whose scale is subnormal, and values that sit exactly on rounding ties of x / d (d = amax / 127 with
    amax = 127 makes d = 1, so x = n + 0.5 are ties): the quantizer must still round as the reference does."""
    m, n, k = 4, 200, 512
    w, x = make_case(9900, n, k, m)
    x[0, :32] = 1e-41
    x[0, 5] = -3e-41
    x[1, 32:64] = (np.arange(32) - 16) + 0.5
    x[1, 32] = 127.0
    x[2, 64:96] = 0.0
    blocks = oc.quantize(oc.Q4_0, 0, w)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8, q8_1=True)
    got = run(device, 0, x, blocks, n, act=1)
    assert rel_err(got, want) < 2e-5
    device.set_option("gemv_mma", 0)
    other = run(device, 0, x, blocks, n, act=1)
    assert rel_err(got, other) < 2e-6


def test_small_batch_extreme_nibbles_and_activations(device):
    """Every nibble 0 or 15 against activations at the ends of the 15-bit range: the largest block sums the
    float-bits conversion has to carry (|T| = 8 * 16383 * 32)."""
    m, n, k = 8, 64, 512
    rng = np.random.default_rng(5)
    raw = np.zeros((n * (k // 32), 18), dtype=np.uint8)
    raw[:, 0:2] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
    raw[0::2, 2:] = 0xFF
    raw[1::2, 2:] = 0x00
    x = np.where(rng.random((m, k)) < 0.5, -3.0, 3.0).astype(np.float32)
    x[0] = 3.0
    x[1] = -3.0
    blocks = raw.reshape(-1)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8)
    got = run(device, 0, x, blocks, n)
    assert rel_err(got, want) < 1e-5
