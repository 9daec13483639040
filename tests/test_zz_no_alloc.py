"""The allocation-free entry point, cq_qmatmul_q8_1_static.

Some hosts cannot let a library allocate device memory: a server that sized its own arena at
start-up and left nothing for cudaMalloc, or a cgo/JNI layer that must not call the CUDA
allocator.  For them the library keeps the quantized activations of the Q8_1 GEMV in a fixed
array inside its own image.  This file checks, through the C ABI, that the entry point gives
the same numbers as the regular one, twice in a row (the array is reused between calls), and
that it refuses problems that do not fit.  It is named to be collected last, so a run that
stops at the first failure has already been through every other test.
"""
import numpy as np
import pytest

from helpers import make_case, rel_err
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu


def _run_both(device, qt, order, seed, m, n, k):
    from candy_b200.backend import QStorage
    lib, ctx = device._lib, device.ctx
    w, x = make_case(seed, n, k, m)
    blocks = oc.quantize(qt, order, w)
    qs = QStorage.from_blocks(device, qt, order, n, k, blocks)
    xs = device.storage_from_slice(x)
    y_static = device.zeros(m * n)
    st = lib.cq_qmatmul_q8_1_static(ctx, qt, order, xs.ptr, m, k, k, qs.buf.ptr, n, y_static.ptr, n)
    assert st == 0, lib.cq_last_error(ctx)
    y_regular = xs.matmul(qs, 1, m, n, k, actmode=1)
    device.synchronize()
    a, b = y_static.data().reshape(m, n), y_regular.data().reshape(m, n)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=4, q8_1=True)
    return a, b, want


def test_static_scratch_matches_regular_entry_twice_in_a_row(device):
    # two calls back to back with different shapes: the second must not see the first's blocks
    for seed, qt, order, m, n, k in [(11, oc.Q4_0, 0, 3, 200, 4096), (12, oc.Q4_0, 1, 1, 96, 1024),
                                     (13, oc.Q8_0, 0, 8, 64, 2048), (14, oc.Q4_0, 0, 1, 130, 32768)]:
        a, b, want = _run_both(device, qt, order, seed, m, n, k)
        assert rel_err(a, b) < 2e-5  # same arithmetic, same routes
        assert rel_err(a, want) < 2e-5  # and the reference CUDA arithmetic of the oracle


def test_static_scratch_rejects_what_does_not_fit(device):
    from candy_b200 import abi
    lib, ctx = device._lib, device.ctx
    buf = device.alloc(1 << 16)
    p = buf.ptr
    assert lib.cq_qmatmul_q8_1_static(ctx, 2, 0, p, 9, 64, 64, p, 4, p, 4) == abi.ERR_TOO_LARGE  # m > 8
    assert lib.cq_qmatmul_q8_1_static(ctx, 2, 0, p, 1, 32800, 32800, p, 1, p, 1) == abi.ERR_TOO_LARGE  # k > 32768
    assert b"32768" in lib.cq_last_error(ctx)
    assert lib.cq_qmatmul_q8_1_static(ctx, 2, 0, p, 1, 48, 48, p, 4, p, 4) == abi.ERR_INVALID_ARG
    assert lib.cq_qmatmul_q8_1_static(ctx, 2, 0, None, 1, 64, 64, p, 4, p, 4) == abi.ERR_INVALID_ARG
    device.synchronize()
