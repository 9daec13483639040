"""Batches of up to eight activation rows in CQ_ACT_F16 against Q4_0 in one launch (gemv_mma_f16_kernel; 9 and more
rows in the same tests take the narrow GEMM, so the hand-over between the two is covered): against a
NumPy emulation of the mode's arithmetic (operands rounded once to f16, exact products: bound 2e-5, only the f32
summation order may differ), against candy's CPU path under the stated bar, against the narrow tensor-memory GEMM
that serves the same batches when this kernel is off, with row strides, a bias, and edge scales."""
import ctypes as C

import numpy as np
import pytest

from helpers import REL_TOL, make_case, rel_err
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu
ACT_F16 = 2


def emulate_f16(order, x, blocks, n):
    k = x.shape[1]
    w16 = oc.dequantize(oc.Q4_0, order, blocks).reshape(n, k).astype(np.float16).astype(np.float64)
    return x.astype(np.float16).astype(np.float64) @ w16.T


def run(device, order, x, blocks, n, ldx=None, ldy=None, bias=None):
    from candy_b200.backend import QStorage
    m, k = x.shape
    ldx, ldy = ldx or k, ldy or n
    lib, ctx = device._lib, device.ctx
    qs = QStorage.from_blocks(device, oc.Q4_0, order, n, k, blocks)
    xp = np.zeros((m, ldx), dtype=np.float32)
    xp[:, :k] = x
    xs, ys = device.storage_from_slice(xp), device.zeros(m * ldy)
    if bias is None:
        st = lib.cq_qmatmul(ctx, oc.Q4_0, order, ACT_F16, xs.ptr, m, k, ldx, qs.buf.ptr, n, ys.ptr, ldy)
    else:
        bs = device.storage_from_slice(bias)
        st = lib.cq_qlinear(ctx, oc.Q4_0, order, ACT_F16, xs.ptr, m, k, ldx, qs.buf.ptr, n, bs.ptr, ys.ptr, ldy)
    assert st == 0, lib.cq_last_error(ctx)
    device.synchronize()
    out = ys.data().reshape(m, ldy)
    assert (out[:, n:] == 0).all()  # nothing written between the rows
    return out[:, :n]


@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 12, 16])
@pytest.mark.parametrize("n,k", [(600, 4096), (4100, 11008), (96, 256), (2500, 8192), (148 * 16 + 5, 512), (300, 1536)])
def test_small_batch_f16_matches_its_arithmetic_and_the_cpu_path(device, order, m, n, k):
    w, x = make_case(9950 + m + n + k, n, k, m)
    x[m - 1, :32] *= 1e-4
    blocks = oc.quantize(oc.Q4_0, order, w)
    got = run(device, order, x, blocks, n)
    assert rel_err(got, emulate_f16(order, x, blocks, n)) < 2e-5
    assert rel_err(got, oc.qmatmul(oc.Q4_0, order, x, blocks, n, nthreads=8)) <= REL_TOL


@pytest.mark.parametrize("m", [1, 4, 8])
def test_small_batch_f16_agrees_with_the_narrow_gemm(device, m):
    n, k = 1500, 4096
    w, x = make_case(9960 + m, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    got = run(device, 0, x, blocks, n)
    device.set_option("gemv_mma", 0)
    try:
        other = run(device, 0, x, blocks, n)
    finally:
        device.set_option("gemv_mma", 3)
    assert rel_err(got, other) < 5e-5  # identical f16 operands, other order of the f32 sums


def test_small_batch_f16_strides_bias_and_edge_scales(device):
    m, n, k = 7, 520, 1024
    w, x = make_case(9970, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    bias = np.random.default_rng(1).standard_normal(n).astype(np.float32)
    want = emulate_f16(0, x, blocks, n)
    assert rel_err(run(device, 0, x, blocks, n, ldx=k + 64, ldy=n + 8), want) < 2e-5
    assert rel_err(run(device, 0, x, blocks, n, bias=bias), want + bias) < 2e-5
    # scales that are zero, negative zero, subnormal, large: d * (n - 8) must still round once
    rng = np.random.default_rng(5)
    raw = rng.integers(0, 256, size=(n * k // 32, 18), dtype=np.uint8)
    scales = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0x57FF, 0xD000], dtype=np.uint16)
    d = scales[rng.integers(0, len(scales), size=raw.shape[0])]
    raw[:, 0], raw[:, 1] = d & 0xFF, d >> 8
    got = run(device, 0, x, raw.reshape(-1), n)
    assert rel_err(got, emulate_f16(0, x, raw.reshape(-1), n)) < 2e-5
