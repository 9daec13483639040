"""Two-GPU test of the fused tensor-parallel exchange (cq_qmatmul_push + cq_add_rmsnorm_reduce):
two processes, one per GPU, run a two-layer sharded stack twice -- once with the fused exchange over
peer memory, once summing the partials through the host (gloo) -- and must end in the same state.
Skipped on machines with fewer than two GPUs."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import ctypes as C
    import torch
    import torch.distributed as dist
    from candy_b200 import abi
    from candy_b200.backend import CudaDevice
    from candy_b200.decoder import DecoderConfig, QuantDecoder
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = CudaDevice(rank)
    lib, ctx = dev._lib, dev.ctx
    cfg = DecoderConfig(n_layers=2, dim=1024, n_heads=8, n_kv_heads=2, head_dim=128, ffn=1024, vocab=0, max_ctx=8, with_head=False)
    batch = 2

    def host_allreduce(buf, count):  # reference exchange: through the host, summed in rank order by gloo
        dev.synchronize()
        t = torch.from_numpy(buf.data()[:count].copy())
        dist.all_reduce(t)
        a = t.numpy()
        abi.check(ctx, lib.cq_memcpy_h2d(ctx, buf.ptr, a.ctypes.data_as(C.c_void_p), a.nbytes), "upload")

    comm = C.c_void_p()
    handle = (C.c_char * 64)()
    abi.check(ctx, lib.cq_comm_create(ctx, rank, world, batch * cfg.dim, C.byref(comm), handle), "comm create")
    handles = [None] * world
    dist.all_gather_object(handles, bytes(handle.raw))
    abi.check(ctx, lib.cq_comm_connect(ctx, comm, b"".join(handles)), "comm connect")
    dist.barrier()
    states = []
    for mode in ("host", "fused"):  # host first: every other kernel is loaded and warm before ranks wait on each other
        model = QuantDecoder(dev, cfg, seed=9, batch=batch, rank=rank, world=world,
                             allreduce=host_allreduce if mode == "host" else None, comm=comm if mode == "fused" else None,
                             fuse=False)  # separate norm / SiLU kernels in both modes: only the exchange differs
        abi.check(ctx, lib.cq_rand_normal(ctx, model.x.ptr, batch * cfg.dim, 0.0, 1.0, 77), "x")
        model.set_state(np.zeros(batch, dtype=np.uint32), 0)
        for _ in range(3):
            model.step()
            dev.synchronize()
        if mode == "fused":  # fold in the last down projection, as the next step's first norm would
            abi.check(ctx, lib.cq_add_rmsnorm_reduce(ctx, comm, 1, model.x.ptr, model.layers[0]["attn_norm"].ptr, batch, cfg.dim, cfg.eps,
                                                     model.xn.ptr), "final reduce")
        else:
            abi.check(ctx, lib.cq_add_rmsnorm(ctx, model.x.ptr, model.d.ptr, model.layers[0]["attn_norm"].ptr, batch, cfg.dim, cfg.eps,
                                              model.xn.ptr), "final add")
        dev.synchronize()
        states.append((model.x.data().copy(), model.xn.data().copy()))
        del model
        dist.barrier()
    (xh, nh), (xf, nf) = states
    err = max(float(np.abs(xf - xh).max() / np.abs(xh).max()), float(np.abs(nf - nh).max() / np.abs(nh).max()))
    np.save(Path(out_dir) / f"err{rank}.npy", np.array([err]))
    dist.barrier()
    lib.cq_comm_destroy(ctx, comm)
    dist.destroy_process_group()


def test_fused_exchange_matches_host_allreduce_on_two_gpus(tmp_path):
    from candy_b200 import abi
    if abi.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert float(np.load(tmp_path / f"err{r}.npy")[0]) < 1e-5
