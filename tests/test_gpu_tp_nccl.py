"""The NCCL all-reduce behind the C ABI (cq_tp_*).  One GPU: a world of one (identity), also recorded into a
graph.  Two GPUs (skipped with fewer): the sum across two processes, then a rank that stops taking part --
it simply does not issue the next all-reduce, nothing faults -- so that the other rank's bounded host wait
(cq_tp_wait) runs out, aborts the communicator and returns CQ_ERR_TIMEOUT with its context still usable."""
import ctypes as C
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def test_world_of_one_allreduce_plain_and_captured(device):
    from candy_b200 import abi
    lib, ctx = device._lib, device.ctx
    ident = (C.c_char * 128)()
    st = lib.cq_tp_unique_id(ctx, ident)
    if st == abi.ERR_UNSUPPORTED:
        pytest.skip("no NCCL library on this machine: " + lib.cq_last_error(ctx).decode())
    assert st == 0, lib.cq_last_error(ctx)
    tp = C.c_void_p()
    assert lib.cq_tp_init(ctx, 0, 1, ident, 128, C.byref(tp)) == 0, lib.cq_last_error(ctx)
    x = np.arange(1000, dtype=np.float32)
    buf = device.storage_from_slice(x)
    assert lib.cq_allreduce_sum_f32(ctx, tp, buf.ptr, x.size) == 0, lib.cq_last_error(ctx)
    assert lib.cq_tp_wait(ctx, tp, 10000) == 0, lib.cq_last_error(ctx)
    assert (buf.data() == x).all()
    g = C.c_void_p()
    assert lib.cq_capture_begin(ctx) == 0
    assert lib.cq_allreduce_sum_f32(ctx, tp, buf.ptr, x.size) == 0, lib.cq_last_error(ctx)
    assert lib.cq_capture_end(ctx, C.byref(g)) == 0, lib.cq_last_error(ctx)
    for _ in range(3):
        assert lib.cq_graph_launch(ctx, g) == 0
    assert lib.cq_tp_wait(ctx, tp, 10000) == 0, lib.cq_last_error(ctx)
    assert (buf.data() == x).all()
    lib.cq_graph_destroy(ctx, g)
    assert lib.cq_tp_destroy(ctx, tp) == 0


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["NCCL_NVLS_ENABLE"] = "0"  # a rank that goes quiet must not hold NVLink multicast bindings
    import torch.distributed as dist
    from candy_b200 import abi
    from candy_b200.backend import CudaDevice
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # host-side rendezvous only
    dev = CudaDevice(rank)
    lib, ctx = dev._lib, dev.ctx
    ident = (C.c_char * 128)()
    if rank == 0:
        abi.check(ctx, lib.cq_tp_unique_id(ctx, ident), "unique id")
    ids = [bytes(ident.raw)]
    dist.broadcast_object_list(ids, src=0)
    tp = C.c_void_p()
    abi.check(ctx, lib.cq_tp_init(ctx, rank, world, ids[0], 128, C.byref(tp)), "tp init")
    x = (np.arange(4096, dtype=np.float32) + 1000.0 * rank)
    buf = dev.storage_from_slice(x)
    abi.check(ctx, lib.cq_allreduce_sum_f32(ctx, tp, buf.ptr, x.size), "allreduce")
    abi.check(ctx, lib.cq_tp_wait(ctx, tp, 20000), "wait")
    want = 2 * np.arange(4096, dtype=np.float32) + 1000.0
    ok_sum = bool((buf.data() == want).all())
    dist.barrier()
    # between steps, with nothing in flight, rank 1 stops taking part in the exchange
    status, usable = 0, True
    if rank == 0:
        abi.check(ctx, lib.cq_allreduce_sum_f32(ctx, tp, buf.ptr, x.size), "allreduce without a partner")
        status = lib.cq_tp_wait(ctx, tp, 1500)
        y = dev.storage_from_slice(np.ones(8, dtype=np.float32))  # the context still answers
        usable = bool((y.data() == 1).all()) and lib.cq_synchronize(ctx) == 0
    np.save(Path(out_dir) / f"res{rank}.npy", np.array([int(ok_sum), status, int(usable)]))
    dist.barrier()
    lib.cq_tp_destroy(ctx, tp)
    dist.destroy_process_group()


def test_two_ranks_sum_then_late_rank_times_out(tmp_path):
    from candy_b200 import abi
    if abi.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "res0.npy"), np.load(tmp_path / "res1.npy")
    assert r0[0] == 1 and r1[0] == 1          # the sum was right on both ranks
    assert r0[1] == abi.ERR_TIMEOUT           # the waiting rank gave up with a status, not a hang
    assert r0[2] == 1                         # and its context kept working
