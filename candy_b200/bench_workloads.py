"""Secondary workloads of bench.py: the 7B-shape greedy decode (BASELINE config 4) and the
70B-shape tensor-parallel layer stack (config 5).  Both drive candy_b200.decoder.QuantDecoder;
timing is CUDA-event time on the launching stream, graph-replayed.
"""
from __future__ import annotations

import ctypes as C
import time

import numpy as np

from .decoder import DecoderConfig, QuantDecoder


def decode_7b(dev, peak_gbs: float, prompt: int = 128, decode: int = 256, seed: int = 2, n_layers: int = 32, persistent: bool = False):
    """32 layers, d=4096, 32 heads x 128, SwiGLU 11008, vocab 32000, Q4_0, batch 1: the `prompt` uniform-random ids
    run as ONE pass (QuantDecoder.prefill: tensor-core linears over all positions, cq_rope_prefill, cq_flash_attention;
    timed separately as `prompt_ms`), then `decode` greedy tokens are timed as replays of a one-step CUDA graph.
    persistent: the step is ONE cooperative kernel (cq_decoder_step); otherwise one launch per operator (~195 per token)."""
    cfg = DecoderConfig(n_layers=n_layers, dim=4096, n_heads=32, n_kv_heads=32, head_dim=128, ffn=11008, vocab=32000,
                        max_ctx=prompt + decode)
    t0 = time.perf_counter()
    model = QuantDecoder(dev, cfg, seed=seed)
    build_s = time.perf_counter() - t0
    lib, ctx = dev._lib, dev.ctx
    is_persistent = bool(persistent) and model.enable_persistent()
    ids = np.random.default_rng(seed).integers(0, cfg.vocab, size=prompt)
    model.set_state(np.array([ids[0]], dtype=np.uint32), 0)
    model.step()  # first launches outside any capture
    dev.synchronize()
    model.set_state(np.array([ids[0]], dtype=np.uint32), 0)
    model.prefill(ids)  # first pass: buffers and kernel attributes
    dev.synchronize()
    model.set_state(np.array([ids[0]], dtype=np.uint32), 0)
    pms = C.c_float()
    lib.cq_timer_start(ctx)
    prompt_launches = model.prefill(ids)
    lib.cq_timer_stop(ctx, C.byref(pms))
    dev.synchronize()
    model.set_state(model.read_ids(), prompt)  # continue from the model's own prediction
    g = model.capture(1)
    ms = C.c_float()
    dev.synchronize()
    lib.cq_timer_start(ctx)
    model.replay(g, decode)
    lib.cq_timer_stop(ctx, C.byref(ms))
    dev.synchronize()
    lib.cq_graph_destroy(ctx, g)
    tok_s = decode / (ms.value * 1e-3)
    wbytes = model.weight_bytes_per_step()
    kv_bytes_mid = cfg.n_layers * 2 * (prompt + decode // 2) * cfg.n_heads * cfg.head_dim * 4
    return {
        "tok_s": round(tok_s, 1), "ms_per_token": round(ms.value / decode, 4), "prompt_tokens": prompt, "decode_tokens": decode,
        "n_layers": n_layers, "weight_bytes_per_token": wbytes, "kv_bytes_per_token_mid": kv_bytes_mid,
        "weight_gbs": round(wbytes * tok_s / 1e9, 1), "frac_of_peak": round(wbytes * tok_s / 1e9 / peak_gbs, 4),
        "roofline_tok_s": round(peak_gbs * 1e9 / wbytes, 1), "launches_per_token": model.launches_per_step(),
        "path": "one persistent cooperative kernel per token (cq_decoder_step)" if is_persistent else "one launch per operator",
        "prompt_ms": round(pms.value, 3), "prompt_tok_s": round(prompt / (pms.value * 1e-3), 1), "prompt_launches": prompt_launches,
        "prompt_path": "one pass: f16-operand tensor-core linears (m = prompt), rotary step for all positions, tcgen05 causal attention",
        "build_seconds": round(build_s, 1),
    }


def prefill_gemm(dev, peak_gbs: float, peak_tflops: float, ms_rows=(16, 128, 256, 512, 2048), n: int = 11008, k: int = 4096, seed: int = 1,
                 calls: int = 16):
    """BASELINE config 3: Y = X . W^T for M in {16,128,512,2048} (and 256, where the in-producer dequantization is the route), N=11008, K=4096, Q4_0 and Q8_0, in two
    numerics: CQ_ACT_F16 (f16 operands, f32 accumulate, tcgen05 kind::f16) and CQ_ACT_Q8_1 (the reference CUDA
    kernels' integer dots: Q8_1 activations, tcgen05 kind::i8, one MMA per quant block, per-block scaling on the
    CUDA cores).  Each figure is the whole cq_qmatmul call (activation pre-pass, any weight conversion, GEMM,
    partial-sum kernel) timed as replays of a CUDA graph of `calls` calls that cycle through eight copies of the
    weights (more than L2).  `frac_of_roofline` = max(algorithmic bytes / measured copy peak, operations /
    measured tensor peak) / measured time; the tensor peak is the measured bf16 burst figure for the f16 mode and
    the int8 MMA issue peak measured here (cq_measure_i8_mma_peak) for the Q8_1 mode."""
    from .backend import QStorage
    lib, ctx = dev._lib, dev.ctx
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    out = []
    tops = C.c_double()
    dev._check(lib.cq_measure_i8_mma_peak(ctx, 4000, C.byref(tops)), "int8 peak")
    int8_peak = float(tops.value)
    for qt, name, bb in ((2, "q4_0", 18), (8, "q8_0", 34)):
        first = QStorage.quantize(dev, qt, 0, w)
        ring = [first]
        for _ in range(7):
            c = RawCopy(dev, first)
            ring.append(c)
        for act, actname in ((2, "f16"), (1, "q8_1")):
          for m in ms_rows:
              x = dev.storage_from_slice(rng.standard_normal((m, k), dtype=np.float32))
              y = dev.alloc(m * n)
              cursor = [0]

              def call():
                  q = ring[cursor[0] % len(ring)]
                  cursor[0] += 1
                  dev._check(lib.cq_qmatmul(ctx, qt, 0, act, x.ptr, m, k, k, q.ptr if isinstance(q, RawCopy) else q.buf.ptr, n, y.ptr, n), "qmatmul")

              call()
              dev.synchronize()
              lib.cq_capture_begin(ctx)
              for _ in range(calls):
                  call()
              g = C.c_void_p()
              dev._check(lib.cq_capture_end(ctx, C.byref(g)), "capture end")
              for _ in range(2):
                  dev._check(lib.cq_graph_launch(ctx, g), "graph launch")
              dev.synchronize()
              ms = C.c_float()
              reps = 5
              lib.cq_timer_start(ctx)
              for _ in range(reps):
                  dev._check(lib.cq_graph_launch(ctx, g), "graph launch")
              lib.cq_timer_stop(ctx, C.byref(ms))
              dev.synchronize()
              lib.cq_graph_destroy(ctx, g)
              t = ms.value * 1e-3 / (reps * calls)
              flops = 2.0 * m * n * k
              nbytes = n * (k // 32) * bb + 4 * m * k + 4 * m * n
              tensor_peak = peak_tflops if act == 2 else int8_peak
              t_hbm, t_tensor = nbytes / (peak_gbs * 1e9), flops / (tensor_peak * 1e12)
              out.append({"qtype": name, "actmode": actname, "m": m, "us": round(t * 1e6, 2), "tflops": round(flops / t / 1e12, 1),
                          "algorithmic_gbs": round(nbytes / t / 1e9, 1), "bound": "hbm" if t_hbm >= t_tensor else "tensor",
                          "roofline_us": round(max(t_hbm, t_tensor) * 1e6, 2), "frac_of_roofline": round(max(t_hbm, t_tensor) / t, 4),
                          "tensor_peak_used": round(tensor_peak, 1),
                          "path": "int8 tcgen05 (kind::i8), one MMA per quant block, per-block scaling in the epilogue" if act == 1 else (
                              ("raw blocks dequantized into tensor memory" + (" (two 64-row passes)" if qt != 2 and m > 64 else "")) if m <= 128
                              else ("raw Q4_0 blocks dequantized inside the tcgen05 GEMM's producer (no f16 copy of W)" if qt == 2 and m <= 384
                                    else "f16 copy of W, then f16 tcgen05 GEMM on CTA pairs (cta_group::2, 256 x 256 tiles)"))})
              del x, y
        del ring, first
    return {"n": n, "k": k, "peak_gbs": peak_gbs, "peak_tflops": peak_tflops, "int8_peak_measured": round(int8_peak, 1),
            "int8_peak_note": "tcgen05.mma kind::i8 s8 x s8 -> s32, M128 N256 K32 back to back on every SM, operands in shared memory; nominal dense 4500",
            "l2_defeat": "ring of 8 weight copies", "cases": out}


def small_batch(dev, peak_gbs: float, ms_rows=(1, 2, 4, 8), n: int = 11008, k: int = 4096, seed: int = 3, calls: int = 40):
    """Decode-side batches (m = 1 .. 8 activation rows against one Q4_0 weight, n = 11008, k = 4096) in the two
    decode numerics, CQ_ACT_F32 and CQ_ACT_Q8_1, and in CQ_ACT_F16: the whole cq_qmatmul call, timed as replays of a CUDA graph of
    `calls` calls that cycle through eight copies of the weight.  One pass over the weights serves every row:
    m = 1 the streaming GEMV, m = 2 its two-row form; m = 3..8 the single-launch kernel with mma.sync block dots
    (plane or Q8_1 columns)."""
    from .backend import QStorage
    lib, ctx = dev._lib, dev.ctx
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    first = QStorage.quantize(dev, 2, 0, w)
    ring = [first] + [RawCopy(dev, first) for _ in range(7)]
    out = []
    for act, actname in ((0, "f32"), (1, "q8_1"), (2, "f16")):
        for m in ms_rows:
            x = dev.storage_from_slice(rng.standard_normal((m, k), dtype=np.float32))
            y = dev.alloc(m * n)
            cursor = [0]

            def call():
                q = ring[cursor[0] % len(ring)]
                cursor[0] += 1
                dev._check(lib.cq_qmatmul(ctx, 2, 0, act, x.ptr, m, k, k, q.ptr if isinstance(q, RawCopy) else q.buf.ptr, n, y.ptr, n), "qmatmul")

            call()
            dev.synchronize()
            lib.cq_capture_begin(ctx)
            for _ in range(calls):
                call()
            g = C.c_void_p()
            dev._check(lib.cq_capture_end(ctx, C.byref(g)), "capture end")
            for _ in range(2):
                dev._check(lib.cq_graph_launch(ctx, g), "graph launch")
            dev.synchronize()
            ms = C.c_float()
            reps = 10
            lib.cq_timer_start(ctx)
            for _ in range(reps):
                dev._check(lib.cq_graph_launch(ctx, g), "graph launch")
            lib.cq_timer_stop(ctx, C.byref(ms))
            dev.synchronize()
            lib.cq_graph_destroy(ctx, g)
            t = ms.value * 1e-3 / (reps * calls)
            nbytes = n * (k // 32) * 18 + 4 * m * k + 4 * m * n
            out.append({"actmode": actname, "m": m, "us": round(t * 1e6, 2), "algorithmic_gbs": round(nbytes / t / 1e9, 1),
                        "frac_of_hbm_peak": round(nbytes / t / 1e9 / peak_gbs, 4),
                        "path": ("streaming kernel with mma.sync f16 operands dequantized in registers, one launch" if m <= 8 and k % 256 == 0
                                 else "narrow tensor-memory GEMM") if act == 2 else "streaming GEMV" if m == 1 else (
                            "streaming kernel with mma.sync block dots, one launch" if m <= 8 and k % 256 == 0 and (
                                m >= 3 or (n * k >= 40 << 20 if act == 0 else (k >= 8192 or n * k >= 100 << 20)))
                            else ("two-row streaming GEMV" if m == 2 else "int8 tcgen05 kernel"))})
            del x, y
    del ring, first
    return {"n": n, "k": k, "qtype": "q4_0", "peak_gbs": peak_gbs, "l2_defeat": "ring of 8 weight copies", "cases": out}


def prefill_attention(dev, peak_tflops: float, cases=((1, 32, 32, 128), (1, 32, 32, 2048), (2, 64, 8, 4096)), d: int = 128, reps: int = 10):
    """The prompt-phase attention (cq_flash_attention, causal, f16, head dimension 128) at the 7B prompt of BASELINE
    config 4 (128 tokens, 32 heads) and at two longer contexts (7B heads at 2048 tokens, the 70B shape's 64 / 8 grouped
    heads at 4096).  flops = 4 * seq^2 * heads * d / 2 (causal); fraction of the measured bf16-class burst peak."""
    from .backend import RawBuffer
    lib, ctx = dev._lib, dev.ctx
    out = []
    for b, h, hk, s in cases:
        nq, nkv = b * s * h * d, b * s * hk * d
        q, k, v, o = RawBuffer(dev, 2 * nq), RawBuffer(dev, 2 * nkv), RawBuffer(dev, 2 * nkv), RawBuffer(dev, 2 * nq)
        lib.cq_memset(ctx, q.ptr, 0x3C, 2 * nq)  # constant fills (every f16 = 0x3C3C = 1.06 ...): the kernel's time does not depend on the values
        lib.cq_memset(ctx, k.ptr, 0x2C, 2 * nkv)
        lib.cq_memset(ctx, v.ptr, 0x34, 2 * nkv)
        args = [q.ptr, k.ptr, v.ptr, o.ptr, None, None, None, None, s * h * d, s * hk * d, s * hk * d, s * h * d, 0, h * d, hk * d, hk * d, h * d, d, d, d, d,
                b, h, hk, d, d, float(1.0 / np.sqrt(d)), s, s, s, s, 0, 1, 0, -1, -1, 0.0]
        dev._check(lib.cq_flash_attention(ctx, *args), "flash attention")
        dev.synchronize()
        ms = C.c_float()
        lib.cq_timer_start(ctx)
        for _ in range(reps):
            dev._check(lib.cq_flash_attention(ctx, *args), "flash attention")
        lib.cq_timer_stop(ctx, C.byref(ms))
        dev.synchronize()
        t = ms.value * 1e-3 / reps
        flops = 4.0 * s * s * h * d * b / 2
        out.append({"batch": b, "heads": h, "kv_heads": hk, "seq": s, "head_dim": d, "causal": True, "dtype": "f16", "us": round(t * 1e6, 1),
                    "tflops": round(flops / t / 1e12, 1), "frac_of_tensor_peak": round(flops / t / 1e12 / peak_tflops, 4),
                    "includes": "the whole cq_flash_attention call: one persistent kernel, V tiles read in place"})
    return {"peak_tflops": peak_tflops, "cases": out}


def independent_gemvs(dev, peak_gbs: float, shapes=((4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)), sweeps: int = 50, reps: int = 10):
    """The headline sweep once more with the caller's promise that consecutive GEMVs do not depend on one another
    (option gemv_independent: a decoder's q / k / v, or gate / up, projections of one x are such launches).  The
    kernels then skip the wait on the previous launch, whose last rows overlap the next launch's set-up.  Reported
    next to the default, dependent, figures; results are the same bits (checked).  Weights cycle through eight copies
    per shape, the results alternate between two buffers."""
    from .backend import RawBuffer
    lib, ctx = dev._lib, dev.ctx
    rng = np.random.default_rng(11)
    rings, xs, ys = [], [], []

    def device_copy(src):
        dst = RawBuffer(dev, src.nbytes)
        dev._check(lib.cq_memcpy_d2d(ctx, dst.ptr, src.ptr, src.nbytes), "copy")
        return dst

    for n, k in shapes:
        raw = rng.integers(0, 256, size=(n * (k // 32), 18), dtype=np.uint8)
        raw[:, 1] = (raw[:, 1] & 0x3F) | 0x20  # finite f16 scales of moderate size
        first = dev.upload_bytes(raw.reshape(-1))
        rings.append([first] + [device_copy(first) for _ in range(7)])
        xs.append(dev.storage_from_slice(rng.standard_normal((1, k), dtype=np.float32)))
        ys.append([dev.alloc(n), dev.alloc(n)])

    def timed(which):
        cur = [0]

        def sweep():
            for i in which:
                n, k = shapes[i]
                dev._check(lib.cq_qmatmul(ctx, 2, 0, 0, xs[i].ptr, 1, k, k, rings[i][cur[0] % 8].ptr, n, ys[i][cur[0] & 1].ptr, n), "qmatmul")
            cur[0] += 1

        sweep()
        dev.synchronize()
        lib.cq_capture_begin(ctx)
        for _ in range(sweeps):
            sweep()
        g = C.c_void_p()
        dev._check(lib.cq_capture_end(ctx, C.byref(g)), "capture end")
        for _ in range(2):
            dev._check(lib.cq_graph_launch(ctx, g), "graph launch")
        dev.synchronize()
        ms = C.c_float()
        lib.cq_timer_start(ctx)
        for _ in range(reps):
            dev._check(lib.cq_graph_launch(ctx, g), "graph launch")
        lib.cq_timer_stop(ctx, C.byref(ms))
        dev.synchronize()
        lib.cq_graph_destroy(ctx, g)
        us = ms.value * 1e3 / (reps * sweeps)
        nbytes = sum(shapes[i][0] * (shapes[i][1] // 32) * 18 + 4 * shapes[i][1] + 4 * shapes[i][0] for i in which)
        return us, nbytes / us / 1e3

    dom = max(range(len(shapes)), key=lambda i: shapes[i][0] * shapes[i][1])
    out = {"shapes": [list(s) for s in shapes], "l2_defeat": "ring of 8 weight copies per shape"}
    results = {}
    for opt in (0, 1):
        dev.set_option("gemv_independent", opt)
        try:
            us_sweep, gbs_sweep = timed(range(len(shapes)))
            us_dom, gbs_dom = timed([dom])
            results[opt] = ys[dom][0].data().copy()
        finally:
            dev.set_option("gemv_independent", 0)
        out["independent" if opt else "dependent"] = {
            "sweep_us": round(us_sweep, 2), "sweep_gbs": round(gbs_sweep, 1), "dominant_shape_us": round(us_dom, 2),
            "dominant_shape_gbs": round(gbs_dom, 1), "dominant_shape_frac_of_hbm_peak": round(gbs_dom / peak_gbs, 4)}
    out["same_bits"] = bool(np.array_equal(results[0], results[1]))
    return out


class RawCopy:
    """A device copy of a QStorage's blocks (ring element)."""

    def __init__(self, dev, q):
        from .backend import RawBuffer
        self.buf = RawBuffer(dev, q.buf.nbytes)
        dev._check(dev._lib.cq_memcpy_d2d(dev.ctx, self.buf.ptr, q.buf.ptr, q.buf.nbytes), "copy")
        self.ptr = self.buf.ptr


def tp_connect(dev, dist, rank: int, world: int):
    """The library's own NCCL communicator (cq_tp_*): rank 0 makes the id, torch.distributed only carries it."""
    from . import abi
    lib, ctx = dev._lib, dev.ctx
    ident = (C.c_char * 128)()
    if rank == 0:
        abi.check(ctx, lib.cq_tp_unique_id(ctx, ident), "tp unique id")
    ids = [bytes(ident.raw)]
    dist.broadcast_object_list(ids, src=0)
    tp = C.c_void_p()
    abi.check(ctx, lib.cq_tp_init(ctx, rank, world, ids[0], 128, C.byref(tp)), "tp init")
    return tp


def tp_layer_70b(dev, dist, rank: int, world: int, local_rank: int, peak_gbs: float, batches=(1, 32), ctx_len: int = 2048,
                 n_layers: int = 8, reps: int = 30, seed: int = 3, tp=None):
    """8 layers of d=8192, 64 q / 8 kv heads x 128, ffn 28672, Q4_0; QKV/gate/up split by rows,
    o/down by columns with an exchange after each: the fused peer-store exchange (batch <= 8) or the
    library's NCCL all-reduce (cq_allreduce_sum_f32; torch.distributed is used for rendezvous only); decode at
    a fixed context of `ctx_len` keys (caches pre-filled with noise).  Returns per-batch step times."""
    cfg = DecoderConfig(n_layers=n_layers, dim=8192, n_heads=64, n_kv_heads=8, head_dim=128, ffn=28672, vocab=0,
                        max_ctx=ctx_len, with_head=False)
    lib, ctx = dev._lib, dev.ctx
    out = {"world": world, "n_layers": n_layers, "ctx": ctx_len}
    torch = None
    if world > 1:
        import torch
    for batch in batches:
        # 8 < batch <= 64 runs the narrow tensor-core GEMM that streams the raw blocks; wider batches the
        # f16 GEMM, whose f16 weight copies are then kept across steps (weights are static in a decode
        # loop), trading 4x the Q4_0 bytes of device memory for no per-step conversion
        dev.set_option("gemm_cache_weights", 1 if batch > 64 else 0)

        def allreduce(buf, count):
            dev._check(lib.cq_allreduce_sum_f32(ctx, tp, buf.ptr, count), "allreduce")

        fused = world > 1 and batch <= 8
        comm = None
        if fused:  # exchange fused into the GEMV epilogue / residual-norm kernel over peer memory
            comm = C.c_void_p()
            handle = (C.c_char * 64)()
            model_check = lambda st, what: __import__("candy_b200").abi.check(ctx, st, what)
            model_check(lib.cq_comm_create(ctx, rank, world, batch * cfg.dim, C.byref(comm), handle), "comm create")
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw))
            model_check(lib.cq_comm_connect(ctx, comm, b"".join(handles)), "comm connect")
            dist.barrier()
        model = QuantDecoder(dev, cfg, seed=seed, batch=batch, rank=rank, world=world,
                             allreduce=allreduce if (world > 1 and not fused) else None, actmode=0 if batch <= 8 else 2, comm=comm)
        for L in model.layers:  # noise in the caches, as if ctx_len tokens had been decoded
            n = batch * cfg.max_ctx * model.kv_dim
            lib.cq_rand_normal(ctx, L["k"].ptr, n, 0.0, 1.0, seed + 101)
            lib.cq_rand_normal(ctx, L["v"].ptr, n, 0.0, 1.0, seed + 202)
        lib.cq_rand_normal(ctx, model.x.ptr, batch * cfg.dim, 0.0, 1.0, seed + 303)
        model.set_state(np.zeros(batch, dtype=np.uint32), ctx_len - 1)
        dev.synchronize()

        def time_own_graph():
            model.step(advance=False)
            model.step(advance=False)
            dev.synchronize()
            lib.cq_capture_begin(ctx)
            model.step(advance=False)
            g = C.c_void_p()
            model._check(lib.cq_capture_end(ctx, C.byref(g)), "capture end")
            if dist is not None:
                dist.barrier()
            model.replay(g, 3)
            ms = C.c_float()
            dev.synchronize()
            if dist is not None:
                dist.barrier()
            lib.cq_timer_start(ctx)
            model.replay(g, reps)
            lib.cq_timer_stop(ctx, C.byref(ms))
            dev.synchronize()
            lib.cq_graph_destroy(ctx, g)
            return ms.value / reps

        def max_over_ranks(v):
            if dist is None:
                return v
            t = torch.tensor([v], dtype=torch.float64, device=torch.device("cuda", local_rank))
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        nccl_ms = None
        step_ms = max_over_ranks(time_own_graph())
        if fused:  # the same stack with NCCL all-reduces, for comparison
            model.comm, model.allreduce = None, allreduce
            nccl_ms = max_over_ranks(time_own_graph())
        wbytes_all = model.weight_bytes_per_step() * world
        out[f"batch{batch}"] = {
            "ms_per_step": round(step_ms, 4), "layers_per_s": round(n_layers / (step_ms * 1e-3), 1),
            "tokens_per_s": round(batch / (step_ms * 1e-3), 1), "weight_bytes_per_step_all_ranks": wbytes_all,
            "weight_gbs_all_ranks": round(wbytes_all / (step_ms * 1e-3) / 1e9, 1),
            "frac_of_peak_per_gpu": round(wbytes_all / world / (step_ms * 1e-3) / 1e9 / peak_gbs, 4),
            "allreduce": "none" if world == 1 else ("fused: tagged peer stores from the GEMV epilogue, summed inside the following residual+RMSNorm kernel"
                                                    if fused else f"NCCL sum of [{batch},8192] f32 (cq_allreduce_sum_f32), twice per layer"),
            "nccl_ms_per_step": None if nccl_ms is None else round(nccl_ms, 4),
            "linear_mode": "f32 activations (decode GEMV)" if batch <= 8 else (
                "f16 operands, raw blocks dequantized into tensor memory (narrow-batch tcgen05 GEMM)" if batch <= 64
                else "f16 operands (tensor-core GEMM), f16 weight copies cached"),
        }
        del model
        dev.synchronize()
        if comm is not None:
            dist.barrier()
            lib.cq_comm_destroy(ctx, comm)
    return out
