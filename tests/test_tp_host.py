"""Host-side tensor-parallel logic on CPU: two gloo ranks shard a quantized MLP the way the
decoder does (gate/up by rows, down by columns + all-reduce) with the CPU oracle standing in for
the GPU kernels, and must reproduce the unsharded result.  Covers shard_sizes, the zero-padded k
of row-parallel shards and the sum-of-partials identity the NCCL path relies on."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from candy_b200.decoder import DecoderConfig, shard_sizes
    from oracle import oracle_c as oc
    from oracle.decoder_np import silu
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = DecoderConfig(n_layers=1, dim=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=320, vocab=0, max_ctx=8, with_head=False)
    nq, nkv, ffn = shard_sizes(cfg, world)
    assert (nq, nkv, ffn) == (2, 1, 160)
    rng = np.random.default_rng(7)  # same stream on every rank: the full weights, then slices
    wg = (rng.standard_normal((cfg.ffn, cfg.dim)) * 0.02).astype(np.float32)
    wu = (rng.standard_normal((cfg.ffn, cfg.dim)) * 0.02).astype(np.float32)
    wd = (rng.standard_normal((cfg.dim, cfg.ffn)) * 0.02).astype(np.float32)
    x = rng.standard_normal((1, cfg.dim)).astype(np.float32)
    sl = slice(rank * ffn, (rank + 1) * ffn)
    gu_blocks = oc.quantize(oc.Q4_0, 0, np.concatenate([wg[sl], wu[sl]]))
    ffn_pad = -(-ffn // 256) * 256
    wd_shard = np.zeros((cfg.dim, ffn_pad), dtype=np.float32)
    wd_shard[:, :ffn] = wd[:, sl]
    wd_blocks = oc.quantize(oc.Q4_0, 0, wd_shard)
    gu = oc.qmatmul(oc.Q4_0, 0, x, gu_blocks, 2 * ffn)[0]
    h = np.zeros((1, ffn_pad), dtype=np.float32)
    h[0, :ffn] = silu(gu[:ffn]) * gu[ffn:]
    part = torch.from_numpy(oc.qmatmul(oc.Q4_0, 0, h, wd_blocks, cfg.dim))
    dist.all_reduce(part)  # the exchange step of a row-parallel linear
    if rank == 0:
        # unsharded reference: blocks never straddle a shard boundary (ffn/world % 32 == 0), so the
        # per-shard quantization equals the quantization of the full matrices
        gu_full = oc.qmatmul(oc.Q4_0, 0, x, oc.quantize(oc.Q4_0, 0, np.concatenate([wg, wu])), 2 * cfg.ffn)[0]
        hf = (silu(gu_full[: cfg.ffn]) * gu_full[cfg.ffn:]).reshape(1, -1)
        want = oc.qmatmul(oc.Q4_0, 0, hf, oc.quantize(oc.Q4_0, 0, wd), cfg.dim)
        err = float(np.abs(part.numpy() - want).max() / np.abs(want).max())
        np.save(Path(out_dir) / "err.npy", np.array([err]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_row_parallel_sum_equals_unsharded(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    err = float(np.load(tmp_path / "err.npy")[0])
    assert err < 1e-5  # only the grouping of the f32 sums differs


def test_shard_sizes_rejects_bad_degrees():
    from candy_b200.decoder import DecoderConfig, shard_sizes
    cfg = DecoderConfig(n_layers=1, dim=8192, n_heads=64, n_kv_heads=8, head_dim=128, ffn=28672)
    assert shard_sizes(cfg, 8) == (8, 1, 3584)
    assert shard_sizes(cfg, 1) == (64, 8, 28672)
    with pytest.raises(ValueError):
        shard_sizes(cfg, 16)  # 8 kv heads do not split 16 ways
    with pytest.raises(ValueError):
        shard_sizes(DecoderConfig(n_heads=32, n_kv_heads=32, ffn=11008), 3)
