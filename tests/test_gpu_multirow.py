"""Decode GEMV with m = 2..8 activation rows: one pass over the weights serves every row
(gemv_stream_mr_kernel).  Checked against the CPU oracle in both activation modes, against the
one-launch-per-row route (option gemv_multirow = 0, same arithmetic per row), with a row stride, with a
bias, and for batches beyond eight rows in the non-tensor-core modes (eight rows a pass)."""
import numpy as np
import pytest

from helpers import make_case, rel_err
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu
QT_ORDERS = [(oc.Q4_0, 0), (oc.Q4_0, 1), (oc.Q8_0, 0)]


@pytest.fixture(autouse=True)
def _decode_kernels_only(device):
    """These tests are about the multi-row streaming GEMV: keep the tensor-core kernels out of the way."""
    device.set_option("gemm_int8", 0)
    device.set_option("gemv_mma", 0)
    yield
    device.set_option("gemm_int8", 1)
    device.set_option("gemv_mma", 3)


def run(device, qt, order, x, blocks, n, actmode, ldx=None, ldy=None, bias=None):
    from candy_b200.backend import QStorage
    m, k = x.shape
    ldx, ldy = ldx or k, ldy or n
    lib, ctx = device._lib, device.ctx
    qs = QStorage.from_blocks(device, qt, order, n, k, blocks)
    xp = np.zeros((m, ldx), dtype=np.float32)
    xp[:, :k] = x
    xs, ys = device.storage_from_slice(xp), device.zeros(m * ldy)
    if bias is None:
        st = lib.cq_qmatmul(ctx, qt, order, actmode, xs.ptr, m, k, ldx, qs.buf.ptr, n, ys.ptr, ldy)
    else:
        bs = device.storage_from_slice(bias)
        st = lib.cq_qlinear(ctx, qt, order, actmode, xs.ptr, m, k, ldx, qs.buf.ptr, n, bs.ptr, ys.ptr, ldy)
    assert st == 0, lib.cq_last_error(ctx)
    device.synchronize()
    out = ys.data().reshape(m, ldy)
    assert (out[:, n:] == 0).all()  # nothing written between the rows
    return out[:, :n]


@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("m", [2, 3, 4, 5, 7, 8])
@pytest.mark.parametrize("n,k", [(600, 4096), (257, 11008), (96, 256), (130, 2048)])
def test_multirow_f32_mode_matches_cpu_path(device, qt, order, m, n, k):
    w, x = make_case(9000 + m + n + k, n, k, m)
    x[m - 1, :32] *= 1e-4
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=8)
    got = run(device, qt, order, x, blocks, n, 0)
    assert rel_err(got, want) < 1e-4
    device.set_option("gemv_multirow", 0)
    try:
        per_row = run(device, qt, order, x, blocks, n, 0)
    finally:
        device.set_option("gemv_multirow", 1)
    assert rel_err(got, per_row) < 2e-6  # the same integers, summed in a different order


@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("m", [2, 4, 6, 8])
@pytest.mark.parametrize("n,k", [(600, 4096), (257, 11008), (96, 256)])
def test_multirow_q8_1_mode_matches_reference_cuda_arithmetic(device, qt, order, m, n, k):
    w, x = make_case(9100 + m + n + k, n, k, m)
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=8, q8_1=True)
    assert rel_err(run(device, qt, order, x, blocks, n, 1), want) < 2e-5


@pytest.mark.parametrize("actmode,bound", [(0, 1e-4), (1, 2e-5)])
def test_multirow_with_row_strides_and_bias(device, actmode, bound):
    m, n, k = 5, 520, 1024
    w, x = make_case(9200, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    bias = np.random.default_rng(1).standard_normal(n).astype(np.float32)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8, q8_1=bool(actmode))
    assert rel_err(run(device, oc.Q4_0, 0, x, blocks, n, actmode, ldx=k + 64, ldy=n + 8), want) < bound
    assert rel_err(run(device, oc.Q4_0, 0, x, blocks, n, actmode, bias=bias), want + bias) < bound
    assert rel_err(run(device, oc.Q4_0, 0, x[:1], blocks, n, actmode, bias=bias), want[:1] + bias) < bound  # one row: bias in the one-row kernel


@pytest.mark.parametrize("m,n,k", [(8, 11008, 4096), (4, 4096, 11008), (8, 4096, 4096), (2, 32000, 4096)])
def test_multirow_at_the_decode_shapes(device, m, n, k):
    w, x = make_case(9300 + m, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=16)
    assert rel_err(run(device, oc.Q4_0, 0, x, blocks, n, 0), want) < 1e-4


def test_batches_beyond_eight_rows_without_tensor_cores(device):
    m, n, k = 19, 300, 1024
    w, x = make_case(9400, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    assert rel_err(run(device, oc.Q4_0, 0, x, blocks, n, 0), oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8)) < 1e-4


def test_bias_on_the_tensor_core_route(device):
    m, n, k = 40, 512, 1024
    w, x = make_case(9500, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    bias = np.random.default_rng(2).standard_normal(n).astype(np.float32)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8) + bias
    assert rel_err(run(device, oc.Q4_0, 0, x, blocks, n, 2, bias=bias), want) < 1e-3


@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("n,k", [(600, 4096), (257, 11008), (96, 256)])
def test_q8_1_activations_quantized_inside_the_gemv_give_the_same_bits(device, qt, order, m, n, k):
    """One and two rows in CQ_ACT_Q8_1: the quantizer runs in the GEMV's set-up.  Its integers, scales and block sums
    must be those of the separate quantize launch bit for bit, so the results are equal, including on rounding ties
    (x / d = n + 0.5 exactly), all-zero blocks and subnormal scales."""
    w, x = make_case(9300 + m + n + k, n, k, m)
    x[0, :32] = (np.arange(32) - 16) + 0.5
    x[0, 0] = 127.0
    x[0, 32:64] = 0.0
    x[m - 1, 64:96] = 1e-41
    x[m - 1, 70] = -3e-41
    blocks = oc.quantize(qt, order, w)
    got = run(device, qt, order, x, blocks, n, 1)
    device.set_option("gemv_q81_inline", 0)
    try:
        two_launches = run(device, qt, order, x, blocks, n, 1)
    finally:
        device.set_option("gemv_q81_inline", 1)
    assert np.array_equal(got, two_launches)
    assert rel_err(got, oc.qmatmul(qt, order, x, blocks, n, nthreads=8, q8_1=True)) < 2e-5
