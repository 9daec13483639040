"""The int8 tensor-core kernel (tcgen05.mma kind::i8, one MMA per quant block, per-block scaling in the
epilogue): CQ_ACT_Q8_1 batches against the oracle of the reference's CUDA arithmetic (O2: quantize_q8_1 +
vec_dot_q4_0_q8_1 / vec_dot_q8_0_q8_1), CQ_ACT_F32 batches (15-bit block fixed-point planes) against
candy's CPU path (O1).  Bars: 1e-3; asserted tighter: 2e-5 vs O2, 1e-4 vs O1."""
import ctypes as C

import numpy as np
import pytest

from helpers import make_case, rel_err
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu
QT_ORDERS = [(oc.Q4_0, 0), (oc.Q4_0, 1), (oc.Q8_0, 0)]


def run(device, qt, order, x, blocks, n, actmode, ldy=None):
    from candy_b200.backend import QStorage
    m, k = x.shape
    ldy = ldy or n
    lib, ctx = device._lib, device.ctx
    qs = QStorage.from_blocks(device, qt, order, n, k, blocks)
    xs, ys = device.storage_from_slice(x), device.zeros(m * ldy)
    st = lib.cq_qmatmul(ctx, qt, order, actmode, xs.ptr, m, k, k, qs.buf.ptr, n, ys.ptr, ldy)
    assert st == 0, lib.cq_last_error(ctx)
    device.synchronize()
    return ys.data().reshape(m, ldy)[:, :n]


@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("m,n,k", [(2, 300, 256), (5, 128, 512), (16, 1000, 1024), (17, 129, 2048), (40, 2048, 4096), (128, 640, 768),
                                   (130, 257, 512), (300, 96, 256)])
def test_q8_1_batches_match_reference_cuda_arithmetic(device, qt, order, m, n, k):
    w, x = make_case(7000 + m + n + k, n, k, m)
    x[0, :32] = 0.0          # an all-zero activation block
    x[m - 1, 32:64] *= 1e3   # and a loud one
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=16, q8_1=True)
    got = run(device, qt, order, x, blocks, n, 1)
    assert rel_err(got, want) < 2e-5
    assert rel_err(got, oc.qmatmul(qt, order, x, blocks, n, nthreads=16)) < 2e-2  # and it is the same product: ~5e-3 from the f32-activation path


@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("m,n,k", [(3, 300, 256), (4, 4096, 4096), (8, 257, 11008), (9, 640, 1024), (33, 129, 512), (64, 512, 2048), (70, 96, 256)])
def test_f32_mode_batches_match_cpu_path(device, qt, order, m, n, k):
    w, x = make_case(7100 + m + n + k, n, k, m)
    x[0, :32] = 0.0
    x[m - 1, 32:64] *= 1e3
    x[1, 5] = -x[1, :32].__abs__().max() * 3  # the block's extreme is negative: the most negative fixed-point value
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=16)
    assert rel_err(run(device, qt, order, x, blocks, n, 0), want) < 1e-4


def test_row_stride_of_y_and_repeatability(device):
    m, n, k = 6, 700, 1024
    w, x = make_case(7200, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    a = run(device, oc.Q4_0, 0, x, blocks, n, 1, ldy=n + 12)
    b = run(device, oc.Q4_0, 0, x, blocks, n, 1)
    assert (a == b).all()  # partial tiles are summed in a fixed order: bit-identical from run to run
    assert rel_err(a, oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=8, q8_1=True)) < 2e-5


@pytest.mark.parametrize("m", [16, 128, 512, 2048])
def test_config3_prefill_q8_1_on_sampled_rows(device, m):
    """BASELINE config 3 at full size (N 11008, K 4096, Q4_0) in the reference CUDA kernels' numerics; the CPU
    oracle checks eight activation rows (rows of Y are independent of each other)."""
    n, k = 11008, 4096
    w, x = make_case(1, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    got = run(device, oc.Q4_0, 0, x, blocks, n, 1)
    rows = np.unique(np.linspace(0, m - 1, 8).astype(int))
    want = oc.qmatmul(oc.Q4_0, 0, x[rows], blocks, n, nthreads=16, q8_1=True)
    assert rel_err(got[rows], want) < 2e-5
    o1 = oc.qmatmul(oc.Q4_0, 0, x[rows[:2]], blocks, n, nthreads=16)
    print(f"m={m}: distance of the Q8_1 numerics from the CPU path (O1): {rel_err(got[rows[:2]], o1):.2e}")


def test_int8_tensor_pipe_probe(device):
    tops = C.c_double()
    st = device._lib.cq_measure_i8_mma_peak(device.ctx, 2000, C.byref(tops))
    assert st == 0, device._lib.cq_last_error(device.ctx)
    print(f"int8 tcgen05 issue peak: {tops.value:.0f} TOPS")
    assert 500 < tops.value < 6000
