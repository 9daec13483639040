"""The fused exchange (cq_qmatmul_push + cq_add_rmsnorm_reduce) on ONE GPU.

world = 1: a push lands in this rank's own slot and the reducing norm adds it to the residual, so the
pair must equal oracle matmul + residual add + RMSNorm.  world = 2 in the single-process stand-in mode
(cq_comm_connect with no handles): the second rank's data never arrives, the reducing norm's bounded
wait runs out -- by design, no fault and no unbounded spin -- and the give-up must surface as
CQ_ERR_TIMEOUT at cq_synchronize within moments, leaving the context usable.
"""
import ctypes as C
import time

import numpy as np
import pytest

from helpers import make_case, rel_err
from oracle import decoder_np as dn
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu


def _comm(dev, rank, world, max_floats, connect=True):
    from candy_b200 import abi
    comm, handle = C.c_void_p(), (C.c_char * 64)()
    abi.check(dev.ctx, dev._lib.cq_comm_create(dev.ctx, rank, world, max_floats, C.byref(comm), handle), "comm create")
    if connect:
        abi.check(dev.ctx, dev._lib.cq_comm_connect(dev.ctx, comm, None), "comm connect (stand-in)")
    return comm


@pytest.mark.parametrize("m,n,k", [(1, 4096, 1024), (3, 2048, 512), (8, 8192, 256), (2, 520, 256)])
def test_push_and_reducing_norm_match_oracle_world_one(m, n, k):
    from candy_b200.backend import CudaDevice, QStorage
    dev = CudaDevice(0)
    lib, ctx = dev._lib, dev.ctx
    w, x = make_case(500 + m + n, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    qs = QStorage.from_blocks(dev, oc.Q4_0, 0, n, k, blocks)
    rng = np.random.default_rng(3)
    resid = rng.standard_normal((m, n)).astype(np.float32)
    alpha = rng.standard_normal(n).astype(np.float32)
    comm = _comm(dev, 0, 1, m * n)
    xs, rs, als, ys = dev.storage_from_slice(x), dev.storage_from_slice(resid), dev.storage_from_slice(alpha), dev.alloc(m * n)
    want_x = resid + oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=4)
    want_y = np.stack([dn.rmsnorm(r, alpha, 1e-5) for r in want_x])
    for rep in range(2):  # twice: the tag advances on the device and the second exchange must see only its own data
        for st in (lib.cq_qmatmul_push(ctx, comm, rep & 1, oc.Q4_0, 0, xs.ptr, m, k, k, qs.buf.ptr, n),
                   lib.cq_add_rmsnorm_reduce(ctx, comm, rep & 1, rs.ptr, als.ptr, m, n, 1e-5, ys.ptr)):
            assert st == 0, lib.cq_last_error(ctx)
        dev.synchronize()
        assert rel_err(rs.data().reshape(m, n), want_x) < 1e-4
        assert rel_err(ys.data().reshape(m, n), want_y) < 1e-4
        dev._check(lib.cq_memcpy_h2d(ctx, rs.ptr, resid.ctypes.data_as(C.c_void_p), resid.nbytes), "reset residual")
    # a second push into a set whose data nobody consumed is refused on the host
    assert lib.cq_qmatmul_push(ctx, comm, 0, oc.Q4_0, 0, xs.ptr, m, k, k, qs.buf.ptr, n) == 0
    assert lib.cq_qmatmul_push(ctx, comm, 0, oc.Q4_0, 0, xs.ptr, m, k, k, qs.buf.ptr, n) == -1
    assert lib.cq_add_rmsnorm_reduce(ctx, comm, 0, rs.ptr, als.ptr, m, n, 1e-5, ys.ptr) == 0
    dev.synchronize()
    lib.cq_comm_destroy(ctx, comm)
    dev.close()


def test_missing_peer_times_out_and_context_stays_usable():
    from candy_b200 import abi
    from candy_b200.backend import CudaDevice, QStorage
    dev = CudaDevice(0)
    lib, ctx = dev._lib, dev.ctx
    m, n, k = 1, 4096, 256
    w, x = make_case(77, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    qs = QStorage.from_blocks(dev, oc.Q4_0, 0, n, k, blocks)
    xs, rs, ys = dev.storage_from_slice(x), dev.zeros(m * n), dev.alloc(m * n)
    comm = _comm(dev, 0, 2, m * n)  # rank 1 exists only on paper: its slot is never written
    dev.set_option("comm_poll_limit", 2000)  # about a millisecond of polling instead of a second
    assert lib.cq_qmatmul_push(ctx, comm, 0, oc.Q4_0, 0, xs.ptr, m, k, k, qs.buf.ptr, n) == 0
    assert lib.cq_add_rmsnorm_reduce(ctx, comm, 0, rs.ptr, None, m, n, 1e-5, ys.ptr) == 0
    t0 = time.perf_counter()
    st = lib.cq_synchronize(ctx)
    waited = time.perf_counter() - t0
    assert st == abi.ERR_TIMEOUT, (st, lib.cq_last_error(ctx))
    assert b"bounded wait" in lib.cq_last_error(ctx)
    assert waited < 2.0
    dev.set_option("comm_poll_limit", 0)
    # the context is intact: the next synchronize is clean and an ordinary matmul is still right
    assert lib.cq_synchronize(ctx) == 0
    y = xs.matmul(qs, 1, m, n, k).data().reshape(m, n)
    dev.synchronize()
    assert rel_err(y, oc.qmatmul(oc.Q4_0, 0, x, blocks, n, nthreads=4)) < 1e-4
    lib.cq_comm_destroy(ctx, comm)
    dev.close()
