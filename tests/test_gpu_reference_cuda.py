"""Pins the oracle against code the reference itself ships: its CUDA kernels for this path,
compiled from the checkout (oracle/_ref, built by oracle/build_oracle.py) and run here on the GPU.
Covers what exists in the reference as executable arithmetic: split-order dequantize, the Q8_1
activation quantizer, the Q8_1 integer-dot GEMV and the f32-activation GEMV.  (The Go CPU code and
the Metal weight quantizers cannot be executed in this environment.)"""
import numpy as np
import pytest

from helpers import make_case, rel_err
from oracle import oracle_c as oc
from oracle import ref_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(device):
    if not ref_cuda.CUBIN.exists():
        pytest.skip("oracle/_ref/quantized_sm100a.cubin not built (needs a reference checkout at build time)")
    return ref_cuda.RefKernels(device.ordinal)


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("qt,qname", [(oc.Q4_0, "q4_0"), (oc.Q8_0, "q8_0")])
def test_reference_dequantize_kernels_equal_the_oracle(device, ref, qt, qname):
    rng = np.random.default_rng(21 + qt)
    nb = 1003
    blocks = rng.integers(0, 256, size=(nb, oc.BLOCK_BYTES[qt]), dtype=np.uint8)
    hi = blocks[:, 1]
    hi[(hi & 0x7C) == 0x7C] &= 0xBF  # finite scales
    buf = device.upload_bytes(blocks)
    y = device.zeros(nb * 32)
    device.synchronize()
    ref.dequantize(qname, buf.ptr.value, y.ptr.value, nb)
    got = y.data()
    want = oc.dequantize(qt, oc.ORDER_SPLIT, blocks.reshape(-1))
    # The reference's own two dequantizers differ in the sign of zero: the CUDA kernel computes
    # d*q + (-8d), which cancels to +0 for q = 8, the Go loop computes d*(q-8) = d*0, which is -0
    # for a negative scale.  The oracle (and the library) follow the Go form; every non-zero value
    # must match bit for bit and zeros must be zeros.
    nz = want != 0
    assert (bits(got)[nz] == bits(want)[nz]).all()
    assert (got[~nz] == 0).all()
    from candy_b200.backend import QStorage
    mine = QStorage.from_blocks(device, qt, oc.ORDER_SPLIT, 1, nb * 32, blocks.reshape(-1)).dequantize().data()
    assert (bits(mine) == bits(want)).all()


def test_reference_quantize_q8_1_equals_the_oracle(device, ref):
    from candy_b200.backend import RawBuffer
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 2048)).astype(np.float32)
    x[1, 64:96] = 0
    x[2] *= 100
    xs = device.storage_from_slice(x)
    out = RawBuffer(device, 3 * 64 * 36)
    device.synchronize()
    ref.quantize_q8_1(xs.ptr.value, out.ptr.value, 2048, 3)
    assert (out.data() == oc.quantize_q8_1(x)).all()


@pytest.mark.parametrize("qt,qname", [(oc.Q4_0, "q4_0"), (oc.Q8_0, "q8_0")])
def test_reference_gemv_kernels_against_oracle_and_library(device, ref, qt, qname):
    from candy_b200.backend import QStorage, RawBuffer
    n, k = 300, 4096
    w, x = make_case(91 + qt, n, k, 1)
    blocks = oc.quantize(qt, oc.ORDER_SPLIT, w)
    qs = QStorage.from_blocks(device, qt, oc.ORDER_SPLIT, n, k, blocks)
    xs = device.storage_from_slice(x)
    act = RawBuffer(device, (k // 32) * 36)
    dst = device.zeros(n)
    device.synchronize()
    # the reference's integer-dot path: its quantizer, then its GEMV
    ref.quantize_q8_1(xs.ptr.value, act.ptr.value, k, 1)
    ref.mul_mat_vec_q8_1(qname, qs.buf.ptr.value, act.ptr.value, dst.ptr.value, k, n)
    y_ref_q8 = dst.data()
    assert rel_err(y_ref_q8, oc.qmatmul(qt, oc.ORDER_SPLIT, x, blocks, n, q8_1=True)[0]) < 2e-5
    mine = xs.matmul(qs, 1, 1, n, k, actmode=1).data()
    assert rel_err(mine, y_ref_q8) < 2e-5
    # the reference's f32-activation path
    ref.dequantize_mul_mat_vec(qname, qs.buf.ptr.value, xs.ptr.value, dst.ptr.value, k, n)
    y_ref_f32 = dst.data()
    assert rel_err(y_ref_f32, oc.qmatmul(qt, oc.ORDER_SPLIT, x, blocks, n)[0]) < 2e-5
    mine32 = xs.matmul(qs, 1, 1, n, k, actmode=0).data()
    assert rel_err(mine32, y_ref_f32) < 1e-4
