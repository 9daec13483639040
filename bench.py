#!/usr/bin/env python
"""Benchmark of the block-quantized matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): BASELINE config 2, the Q4_0 decode-GEMV sweep with M = 1 over
(N,K) in {(4096,4096),(11008,4096),(4096,11008),(32000,4096)}, W ~ N(0,0.02) quantized to
Q4_0 by the library's GPU quantizer, x ~ N(0,1), seed 0.  One *step* is 400 passes over the
four shapes (1600 kernel launches, about 16 ms), so that the driver's 20 steps make a timed region
of a third of a second.  Every shape cycles through a ring of distinct copies of its weight matrix
(>= 512 MiB per shape, four times the L2), so no launch finds its weights in cache.  Sweeps are
recorded once into a CUDA graph and replayed; time is CUDA-event time on the launching stream.

Printed line: metric = aggregate algorithmic GB/s of the sweep (weight blocks + x + y bytes
per launch, divided by device time); `roofline` is the dominant kernel (the 32000x4096 GEMV)
timed alone; `e2e` is the same sweep through cq_qmatmul_host with pinned HOST x and y (copies
inside the timed region); `cpu_baseline` is the CPU oracle (a C port of candy's dequantize +
naive f32 matmul, one thread as in candy) on a bounded sample.

With N > 1 (torchrun) every rank runs the same sweep on its own GPU over its own row shard of
an N-times taller layer (column-parallel linear: no exchange), weak scaling; the time is the
max over ranks.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]  # (N, K), M = 1
RING_BYTES = 512 << 20
SWEEPS_PER_STEP = 400   # one step = this many passes over the four shapes (1600 kernel launches, about 16 ms of device time)
GRAPH_SWEEPS = 100      # sweeps recorded per CUDA graph; a step replays it SWEEPS_PER_STEP / GRAPH_SWEEPS times
Q4_0, Q8_0 = 2, 8
ORDER = 0  # the Go CPU path's element order
WORKLOAD = ("BASELINE config 2: Q4_0 decode GEMV sweep, M=1, (N,K) in {(4096,4096),(11008,4096),(4096,11008),(32000,4096)}, "
            "W~N(0,0.02)->Q4_0, x~N(0,1), seed 0")


def gemv_bytes(n, k, m=1, bb=18):
    return n * (k // 32) * bb + 4 * m * k + 4 * m * n


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_peak_tflops():
    """Dense bf16-class tensor peak for a kernel timed alone (burst figure), else the pool's earlier measurement."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"])
        except Exception:
            pass
    return 1590.0


class ClockSampler:
    """Samples SM clock, power and clock-event reasons through NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self.index, self.period = index, period_s
        self._stop = threading.Event()
        self._thread = None
        self.error = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # no NVML: report it, do not guess
            self.nv, self.error = None, repr(e)

    def _once(self):
        nv = self.nv
        mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
        try:
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        self.samples.append(mhz)
        names = {
            "sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20,
            "hw_thermal_slowdown": 0x40, "hw_power_brake_slowdown": 0x80, "applications_clocks_setting": 0x2,
        }
        for name, bit in names.items():
            if r & bit:
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._once()
            except Exception as e:
                self.error = repr(e)
                return
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()
        if self.nv and not self.samples:
            try:
                self._once()
            except Exception as e:
                self.error = repr(e)

    def summary(self):
        out = {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.error:
            out["error"] = self.error
        return out


class Workload:
    def __init__(self, dev, shapes, seed=0, ring_bytes=RING_BYTES, rank=0):
        from candy_b200.backend import QStorage, RawBuffer
        self.dev = dev
        self.shapes = shapes
        self.rings, self.xs, self.ys, self.qs0 = [], [], [], []
        rng = np.random.default_rng(seed + 1000 * rank)
        for (n, k) in shapes:
            w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
            x = rng.standard_normal((1, k), dtype=np.float32)
            q = QStorage.quantize(dev, Q4_0, ORDER, w)
            del w
            nbytes = q.buf.nbytes
            copies = max(2, -(-ring_bytes // nbytes))
            ring = [q.buf]
            for _ in range(copies - 1):
                b = RawBuffer(dev, nbytes)
                dev._check(dev._lib.cq_memcpy_d2d(dev.ctx, b.ptr, q.buf.ptr, nbytes), "ring copy")
                ring.append(b)
            self.rings.append(ring)
            self.qs0.append(q)
            self.xs.append(dev.storage_from_slice(x))
            self.ys.append(dev.alloc(n))
        dev.synchronize()
        self.cursor = [0] * len(shapes)

    def launch(self, i):
        dev = self.dev
        n, k = self.shapes[i]
        ring = self.rings[i]
        w = ring[self.cursor[i] % len(ring)]
        self.cursor[i] += 1
        dev._check(dev._lib.cq_qmatmul(dev.ctx, Q4_0, ORDER, 0, self.xs[i].ptr, 1, k, k, w.ptr, n, self.ys[i].ptr, n), "qmatmul")

    def capture(self, steps, which=None):
        """Records `steps` steps (or `steps` launches of shape `which`) into a CUDA graph."""
        dev = self.dev
        g = C.c_void_p()
        dev._check(dev._lib.cq_capture_begin(dev.ctx), "capture begin")
        for _ in range(steps):
            for i in (range(len(self.shapes)) if which is None else [which]):
                self.launch(i)
        dev._check(dev._lib.cq_capture_end(dev.ctx, C.byref(g)), "capture end")
        return g

    def run_graph(self, g, times=1):
        dev = self.dev
        for _ in range(times):
            dev._check(dev._lib.cq_graph_launch(dev.ctx, g), "graph launch")

    def timed(self, fn):
        """CUDA-event time of fn() on the context's stream, synchronised on both sides.  An untimed
        filler kernel (a 64 MiB random fill, which also sweeps L2) runs just before the start event, so
        that the host has enqueued fn()'s launches by the time the GPU reaches the event: the timed region
        then holds the GPU work only, not the host's launch latency after an idle GPU."""
        dev = self.dev
        ms = C.c_float()
        if not hasattr(self, "_gate"):
            self._gate = dev.alloc(16 << 20)
        dev.synchronize()
        dev._check(dev._lib.cq_rand_uniform(dev.ctx, self._gate.ptr, 16 << 20, 0.0, 1.0, 1), "gate")
        dev._check(dev._lib.cq_timer_start(dev.ctx), "timer start")
        fn()
        dev._check(dev._lib.cq_timer_stop(dev.ctx, C.byref(ms)), "timer stop")
        dev.synchronize()
        return ms.value


def dist_setup(world, local_rank):
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return dist


def dist_max(dist, value, local_rank):
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=torch.device("cuda", local_rank))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def dist_barrier(dist):
    if dist is not None:
        import torch
        dist.barrier()
        torch.cuda.synchronize()


def cpu_baseline(blocks_by_shape, xs, budget_s=12.0, threads=1):
    """Times the CPU oracle (C port of candy's dequantize + naive matmul) on the sweep."""
    from oracle import oracle_c as oc
    oc.lib()
    total_bytes, reps = sum(gemv_bytes(n, k) for n, k in SHAPES), 0
    t0 = time.perf_counter()
    while True:
        for (n, k), blocks, x in zip(SHAPES, blocks_by_shape, xs):
            oc.qmatmul(Q4_0, ORDER, x, blocks, n, nthreads=threads)
        reps += 1
        el = time.perf_counter() - t0
        if el >= budget_s or reps >= 20:
            break
    return {"value": total_bytes * reps / el / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{reps} full passes over the 4-shape Q4_0 M=1 sweep ({el:.1f} s); C port of candy's "
                      f"dequantize + sequential f32 matmul, {threads} thread(s)",
            "seconds_per_sweep": el / reps}


def tp_layer_parity(dev, dist, rank, world, local_rank, ctx_len=32, seed=3, tp=None):
    """Checker for BASELINE config 5, run before its timing: ONE reduced step -- one layer with the 70B
    shard shapes (d 8192, 64 q / 8 kv heads x 128, ffn 28672, Q4_0), context of `ctx_len` keys -- on every
    rank, through the fused exchange (batch 1), through NCCL all-reduces (batch 1 and 32) or, on one GPU,
    with no exchange.  Rank 0 gathers every rank's weight blocks and caches and compares its residual stream
    after the layer with the CPU oracle of the UNSHARDED layer (oracle/decoder_np.sharded_layer_step: candy's
    CPU arithmetic, row-parallel partials summed in rank order).  The oracle is only the checker here; at
    batch 32 it checks the first and the last sequence (each costs 0.86 G scalar multiply-adds)."""
    import ctypes as C
    from candy_b200 import abi
    from candy_b200.decoder import DecoderConfig, QuantDecoder, rope_tables
    cfg = DecoderConfig(n_layers=1, dim=8192, n_heads=64, n_kv_heads=8, head_dim=128, ffn=28672, vocab=0, max_ctx=ctx_len, with_head=False)
    lib, ctx = dev._lib, dev.ctx
    cos, sin = rope_tables(cfg)
    torch = None
    if world > 1:
        import torch
    cases = [(1, "single"), (32, "single")] if world == 1 else [(1, "fused"), (1, "nccl"), (32, "nccl")]
    out = {"bar": 1e-3, "ranks": world, "layer": "d 8192, 64/8 heads, ffn 28672, Q4_0", "ctx": ctx_len, "cases": []}
    worst = 0.0
    for batch, mode in cases:
        def allreduce(buf, count):  # the library's NCCL all-reduce
            abi.check(ctx, lib.cq_allreduce_sum_f32(ctx, tp, buf.ptr, count), "allreduce")

        comm = None
        if mode == "fused":
            comm, handle = C.c_void_p(), (C.c_char * 64)()
            abi.check(ctx, lib.cq_comm_create(ctx, rank, world, batch * cfg.dim, C.byref(comm), handle), "comm create")
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw))
            abi.check(ctx, lib.cq_comm_connect(ctx, comm, b"".join(handles)), "comm connect")
            dist.barrier()
        model = QuantDecoder(dev, cfg, seed=seed, batch=batch, rank=rank, world=world, allreduce=allreduce if mode == "nccl" else None,
                             actmode=0 if batch <= 8 else 2, comm=comm)
        L = model.layers[0]
        nkv_floats = batch * cfg.max_ctx * model.kv_dim
        lib.cq_rand_normal(ctx, L["k"].ptr, nkv_floats, 0.0, 1.0, seed + 101 + rank)
        lib.cq_rand_normal(ctx, L["v"].ptr, nkv_floats, 0.0, 1.0, seed + 202 + rank)
        lib.cq_rand_normal(ctx, model.x.ptr, batch * cfg.dim, 0.0, 1.0, seed + 303)  # the same on every rank
        pos = ctx_len - 1
        model.set_state(np.zeros(batch, dtype=np.uint32), pos)
        dev.synchronize()
        x0 = model.x.data().reshape(batch, cfg.dim).copy()
        kc = L["k"].data().reshape(batch, cfg.max_ctx, model.nkv, cfg.head_dim).copy()
        vc = L["v"].data().reshape(batch, cfg.max_ctx, model.nkv, cfg.head_dim).copy()
        if dist is not None:
            torch.cuda.synchronize()
            dist.barrier()
        model.step(advance=False)
        if mode == "fused":  # fold in the down projection's partials, as the next layer's first norm would
            abi.check(ctx, lib.cq_add_rmsnorm_reduce(ctx, comm, 1, model.x.ptr, L["attn_norm"].ptr, batch, cfg.dim, cfg.eps, model.xn.ptr), "final reduce")
        if dist is not None:
            torch.cuda.synchronize()
        dev.synchronize()
        x2 = model.x.data().reshape(batch, cfg.dim)
        if mode != "fused":
            x2 = x2 + model.d.data().reshape(batch, cfg.dim)
        rows = sorted({0, batch - 1})
        shard = {"wqkv": L["wqkv"].data(), "wo": L["wo"].data(), "wgu": L["wgu"].data(), "wdown": L["wdown"].data(),
                 "k": kc[rows], "v": vc[rows], "nq": model.nq, "nkv": model.nkv, "ffn": model.ffn}
        shards = [shard]
        if dist is not None:
            shards = [None] * world
            dist.all_gather_object(shards, shard)
        err = None
        if rank == 0:
            from oracle import decoder_np as dn  # the checker
            err = 0.0
            for i, b in enumerate(rows):
                per_rank = [dict(s, k=s["k"][i], v=s["v"][i]) for s in shards]
                want = dn.sharded_layer_step(cfg, model.qtype, model.order, per_rank, x0[b], pos, cos, sin)
                err = max(err, float(np.abs(x2[b] - want).max() / np.abs(want).max()))
            worst = max(worst, err)
            out["cases"].append({"batch": batch, "exchange": mode, "rows_checked": rows, "max_rel_err": err,
                                 "linear_mode": "f32 activations" if batch <= 8 else "f16 operands (tensor cores)"})
        del model, shards, shard
        dev.synchronize()
        if comm is not None:
            dist.barrier()
            lib.cq_comm_destroy(ctx, comm)
    out["max_rel_err"] = worst
    out["pass"] = bool(worst <= out["bar"])
    return out


def reference_cuda_baseline(dev, wl, reps=40):
    """A GPU-side anchor beside the CPU baseline: the reference's OWN decode kernels
    (tensor/internal/cuda/kernels/quantized.cu compiled unchanged for sm_100a into oracle/_ref by
    oracle/build_oracle.py) timed on the same box, same config-2 shapes, same rings of weight copies, with the
    launch shapes the parity tests validated (oracle/ref_cuda.py): dequantize_mul_mat_vec_q4_0_cuda (f32
    activations) and quantize_q8_1 + mul_mat_vec_q4_0_q8_1_cuda1.  The reference never launches them itself."""
    from oracle import ref_cuda
    if not ref_cuda.CUBIN.exists():
        return {"unavailable": "oracle/_ref/quantized_sm100a.cubin not built (no reference checkout at build time)"}
    from candy_b200.backend import RawBuffer
    rk = ref_cuda.RefKernels(dev.ordinal)
    out = {"kernels": "the reference's quantized.cu, unchanged, sm_100a", "shapes": []}
    tot = {"dmmv": 0.0, "mmvq": 0.0}
    for i, (n, k) in enumerate(wl.shapes):
        ring = [b.ptr.value for b in wl.rings[i]]
        x, y = wl.xs[i].ptr.value, wl.ys[i].ptr.value
        act = RawBuffer(dev, (k // 32) * 36)
        cur = [0]

        def dmmv():
            for _ in range(reps):
                rk.dequantize_mul_mat_vec("q4_0", ring[cur[0] % len(ring)], x, y, k, n, sync=False)
                cur[0] += 1

        def mmvq():
            for _ in range(reps):
                rk.quantize_q8_1(x, act.ptr.value, k, 1, sync=False)
                rk.mul_mat_vec_q8_1("q4_0", ring[cur[0] % len(ring)], act.ptr.value, y, k, n, sync=False)
                cur[0] += 1

        dev.synchronize()
        dmmv()
        t_d = rk.timed_ms(dmmv) / reps * 1e3
        mmvq()
        t_q = rk.timed_ms(mmvq) / reps * 1e3
        tot["dmmv"] += t_d
        tot["mmvq"] += t_q
        out["shapes"].append({"n": n, "k": k, "dmmv_us": round(t_d, 2), "dmmv_gbs": round(gemv_bytes(n, k) / t_d / 1e3, 1),
                              "q8_1_mmvq_us": round(t_q, 2), "q8_1_mmvq_gbs": round(gemv_bytes(n, k) / t_q / 1e3, 1)})
    sweep = sum(gemv_bytes(n, k) for n, k in wl.shapes)
    out["sweep_gbs_dmmv"] = round(sweep / tot["dmmv"] / 1e3, 1)
    out["sweep_gbs_q8_1_mmvq"] = round(sweep / tot["mmvq"] / 1e3, 1)
    return out


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    from candy_b200.backend import CudaDevice
    dist = dist_setup(world, local_rank)
    dev = CudaDevice(local_rank)
    wl = Workload(dev, SHAPES, seed=0, rank=rank)
    lib, ctx = dev._lib, dev.ctx
    K, W = args.steps, args.warmup
    for i in range(len(SHAPES)):  # first launches outside any capture (one-time kernel attribute setup)
        wl.launch(i)
    dev.synchronize()

    g_main = wl.capture(GRAPH_SWEEPS)
    replays_per_step = SWEEPS_PER_STEP // GRAPH_SWEEPS

    def timed_region():
        wl.run_graph(g_main, K * replays_per_step)

    wl.run_graph(g_main, W * replays_per_step)  # W untimed warm-up steps
    dev.synchronize()
    dist_barrier(dist)
    with ClockSampler(local_rank) as clocks:
        ms = wl.timed(timed_region)
    dist_barrier(dist)
    ms = dist_max(dist, ms, local_rank)
    sweep_bytes = sum(gemv_bytes(n, k) for n, k in SHAPES)
    value = world * sweep_bytes * K * SWEEPS_PER_STEP / (ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak_gbs()

    # ---- per-kernel timing: each shape alone, same ring discipline ------------------------
    per_shape = []
    launches = 2000
    for i, (n, k) in enumerate(SHAPES):
        g = wl.capture(100, which=i)
        wl.run_graph(g, 2)
        t = wl.timed(lambda: wl.run_graph(g, launches // 100))
        us = t * 1e3 / (launches // 100 * 100)
        gbs = gemv_bytes(n, k) / (us * 1e-6) / 1e9
        per_shape.append({"n": n, "k": k, "bytes": gemv_bytes(n, k), "us": round(us, 3), "gbs": round(gbs, 1),
                          "frac_of_" + peak_kind: round(gbs / peak, 4), "frac_of_8000": round(gbs / 8000.0, 4),
                          "ring_copies": len(wl.rings[i])})
        lib.cq_graph_destroy(ctx, g)
    dom = max(range(len(SHAPES)), key=lambda i: per_shape[i]["us"])
    roofline = {"bound": "hbm", "kernel": f"gemv_stream_kernel<Q4_0> n={SHAPES[dom][0]} k={SHAPES[dom][1]} m=1",
                "achieved": per_shape[dom]["gbs"], "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": round(per_shape[dom]["gbs"] / peak, 4), "traffic": NCU_TRAFFIC_BYTES,
                "algorithmic_bytes": per_shape[dom]["bytes"]}

    # ---- end to end through the host-buffer entry point -----------------------------------
    e2e_steps = 200  # host-buffer sweeps (a sweep = the four shapes once)
    hx, hy = [], []
    for (n, k) in SHAPES:
        px, py = C.c_void_p(), C.c_void_p()
        dev._check(lib.cq_malloc_host(ctx, 4 * k, C.byref(px)), "pinned x")
        dev._check(lib.cq_malloc_host(ctx, 4 * n, C.byref(py)), "pinned y")
        C.memmove(px, np.random.default_rng(1).standard_normal(k, dtype=np.float32).ctypes.data, 4 * k)
        hx.append(px)
        hy.append(py)

    def e2e_step():
        for i, (n, k) in enumerate(SHAPES):
            ring = wl.rings[i]
            w = ring[wl.cursor[i] % len(ring)]
            wl.cursor[i] += 1
            dev._check(lib.cq_qmatmul_host(ctx, Q4_0, ORDER, 0, hx[i], 1, k, w.ptr, n, hy[i]), "qmatmul_host")

    for _ in range(3):
        e2e_step()
    dist_barrier(dist)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    e2e_s = dist_max(dist, e2e_s, local_rank)
    # The pinned result buffers are written by the kernel itself (no copy back): the same call into a pageable buffer,
    # which does copy back, must give the same bits.
    for i, (n, k) in enumerate(SHAPES):
        w = wl.rings[i][0]
        dev._check(lib.cq_qmatmul_host(ctx, Q4_0, ORDER, 0, hx[i], 1, k, w.ptr, n, hy[i]), "qmatmul_host")
        pageable = np.empty(n, dtype=np.float32)
        dev._check(lib.cq_qmatmul_host(ctx, Q4_0, ORDER, 0, hx[i], 1, k, w.ptr, n, pageable.ctypes.data_as(C.c_void_p)),
                   "qmatmul_host")
        pinned = np.ctypeslib.as_array(C.cast(hy[i], C.POINTER(C.c_float)), shape=(n,))
        if not np.array_equal(pinned, pageable) or not np.isfinite(pinned).all():
            raise SystemExit(f"host entry point: the in-place result differs from the copied one at shape {n}x{k}")
    e2e = {"value": round(world * sweep_bytes * e2e_steps / e2e_s / 1e9, 2), "unit": "GB/s",
           "h2d_bytes_per_step": sum(4 * k for _, k in SHAPES), "d2h_bytes_per_step": sum(4 * n for n, _ in SHAPES),
           "steps": e2e_steps, "us_per_step": round(e2e_s / e2e_steps * 1e6, 1),
           "d2h_route": "kernel stores into the pinned result buffer (checked against the copied result)"}

    line = {
        "metric": "q4_0_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "element_order": "go_interleaved", "actmode": "f32",
                   "step": f"{SWEEPS_PER_STEP} passes over the four shapes ({SWEEPS_PER_STEP * len(SHAPES)} launches); the driver's 20 steps time about a third of a second",
                   "l2_defeat": f"inputs larger than L2: each shape cycles a ring of weight copies >= {RING_BYTES >> 20} MiB",
                   "sharding": "none" if world == 1 else f"rows of an {world}x taller layer, one shard per GPU, no collective"},
        "frac_of_peak": round(value / world / peak, 4), "frac_of_8000": round(value / world / 8000.0, 4),
        "roofline": roofline, "per_shape": per_shape, "e2e": e2e, "gpu_launches": K * SWEEPS_PER_STEP * len(SHAPES),
        "clocks": clocks.summary(),
    }
    cpu_inputs = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu_inputs = ([q.data() for q in wl.qs0], [x.data().reshape(1, -1) for x in wl.xs])
        try:  # the reference's own CUDA kernels on the same box: a baseline leg like cpu_baseline, never the product path
            line["ref_cuda_baseline"] = reference_cuda_baseline(dev, wl)
        except Exception as e:  # noqa: BLE001
            line["ref_cuda_baseline"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    lib.cq_graph_destroy(ctx, g_main)
    del wl  # free the rings before the secondary workloads
    if not args.skip_extras:
        from candy_b200 import bench_workloads as bw
        # the secondary workloads never take the headline line down with them
        def extra(key, fn):
            try:
                line[key] = fn()
            except Exception as e:  # noqa: BLE001 - reported in the line itself
                line[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
        if world == 1:
            extra("small_batch", lambda: bw.small_batch(dev, peak))
            extra("independent_gemvs", lambda: bw.independent_gemvs(dev, peak))
            extra("prefill_gemm", lambda: bw.prefill_gemm(dev, peak, measured_peak_tflops()))
            extra("prefill_attention", lambda: bw.prefill_attention(dev, measured_peak_tflops()))
            extra("decode_7b", lambda: bw.decode_7b(dev, peak))
            extra("decode_7b_persistent_kernel", lambda: bw.decode_7b(dev, peak, persistent=True))
        tp = None
        if world > 1:
            try:
                tp = bw.tp_connect(dev, dist, rank, world)
            except Exception as e:  # noqa: BLE001
                line["tp_connect_error"] = f"{type(e).__name__}: {e}"[:300]
        if not args.no_cpu:  # parity of the config-5 layer against the CPU oracle, checked before it is timed
            extra("tp_layer_70b_parity", lambda: tp_layer_parity(dev, dist, rank, world, local_rank, tp=tp))
        extra("tp_layer_70b", lambda: bw.tp_layer_70b(dev, dist, rank, world, local_rank, peak, tp=tp))
        if isinstance(line.get("tp_layer_70b"), dict) and "tp_layer_70b_parity" in line:
            line["tp_layer_70b"]["parity"] = line.pop("tp_layer_70b_parity")
    if cpu_inputs is not None:
        blocks, xs = cpu_inputs
        line["cpu_baseline"] = cpu_baseline(blocks, xs, threads=1)
    elif rank == 0:
        line["cpu_baseline"] = None
    if rank == 0:
        args.emit(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernel
# (n=32000, k=4096) from an `ncu --set full -k regex:gemv_stream_kernel` capture of
# `bench.py --kernel-only 32000x4096`: 73.81 MB read + 0.85 MB written.
NCU_TRAFFIC_BYTES = 73805824 + 853248


def run_reference(args):
    """Reference arm: candy's CPU algorithm for the same sweep (the C port in oracle/, since
    the Go original cannot be built without a Go toolchain), on host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle_c as oc
    oc.lib()
    # candy's kernels start no goroutines (one core is all its own path uses); this arm nevertheless
    # spreads the rows over every host core with OpenMP, the most the same algorithm could use, and
    # reports the faithful single-thread figure beside it
    threads = max(1, os.cpu_count() or 1)
    rng = np.random.default_rng(0)
    # bounded sample: the first `rows` rows of every shape, sized from a calibration pass so
    # that steps + warmup finish in about two minutes
    data = []
    for (n, k) in SHAPES:
        rows = min(n, 512)
        w = rng.standard_normal((rows, k), dtype=np.float32) * np.float32(0.02)
        x = rng.standard_normal((1, k), dtype=np.float32)
        data.append((rows, k, oc.quantize(Q4_0, ORDER, w), x))
    t0 = time.perf_counter()
    for rows, k, blocks, x in data:
        oc.qmatmul(Q4_0, ORDER, x, blocks, rows, nthreads=threads)
    per_row_s = (time.perf_counter() - t0) / sum(d[0] for d in data)
    total_steps = args.steps + args.warmup
    frac = min(1.0, (120.0 / total_steps) / (per_row_s * sum(n for n, _ in SHAPES)))
    sample = []
    for (n, k) in SHAPES:
        rows = max(32, int(n * frac))
        w = rng.standard_normal((rows, k), dtype=np.float32) * np.float32(0.02)
        x = rng.standard_normal((1, k), dtype=np.float32)
        sample.append((rows, k, oc.quantize(Q4_0, ORDER, w), x))
    step_bytes = sum(gemv_bytes(rows, k) for rows, k, _, _ in sample)

    def step():
        for rows, k, blocks, x in sample:
            oc.qmatmul(Q4_0, ORDER, x, blocks, rows, nthreads=threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    el = time.perf_counter() - t0
    value = step_bytes * args.steps / el / 1e9
    t0 = time.perf_counter()
    for rows, k, blocks, x in sample[:2]:
        oc.qmatmul(Q4_0, ORDER, x, blocks, rows, nthreads=1)
    single = sum(gemv_bytes(rows, k) for rows, k, _, _ in sample[:2]) / (time.perf_counter() - t0) / 1e9
    desc = (f"first {frac:.4f} of the rows of each of the 4 shapes per step "
            f"({', '.join(str(s[0]) for s in sample)} rows); C port of candy's dequantize + sequential f32 matmul, rows spread over {threads} OpenMP thread(s)")
    line = {
        "impl": "reference", "metric": "q4_0_gemv_hbm_gbs", "value": round(value, 4), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "element_order": "go_interleaved", "actmode": "f32",
                   "step": "one pass over the four shapes" + ("" if frac >= 1.0 else f", first {frac:.4f} of each shape's rows")},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "host_cores_available": os.cpu_count(),
        "single_thread_gbs": round(single, 4),  # what candy's own single-goroutine kernel reaches
    }
    print(json.dumps(line), flush=True)


def run_kernel_only(args):
    """A few plain launches of one GEMV shape over a small ring: the case ncu captures."""
    from candy_b200.backend import CudaDevice
    n, k = (int(v) for v in args.kernel_only.lower().split("x"))
    dev = CudaDevice(int(os.environ.get("LOCAL_RANK", "0")))
    nbytes = n * (k // 32) * 18
    for kv in args.option:
        key, val = kv.split("=")
        dev.set_option(key, int(val))
    if args.qtype != 2 or args.actmode != 0:
        # another block format (3 = Q4_1, 6 = Q5_0, 7 = Q5_1, 8 = Q8_0) or activation mode (1 = Q8_1): same ring idea
        import numpy as np
        from candy_b200.backend import QStorage
        from candy_b200.bench_workloads import RawCopy
        rng = np.random.default_rng(0)
        w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
        order = 1 if args.qtype in (6, 7) else 0
        first = QStorage.quantize(dev, args.qtype, order, w)
        copies = max(2, (160 << 20) // first.buf.nbytes + 1)
        ring = [first.buf.ptr] + [RawCopy(dev, first) for _ in range(copies - 1)]
        x = dev.storage_from_slice(rng.standard_normal((1, k), dtype=np.float32))
        y = dev.alloc(n)
        for i in range(args.launches):
            q = ring[i % copies]
            dev._check(dev._lib.cq_qmatmul(dev.ctx, args.qtype, order, args.actmode, x.ptr, 1, k, k, q if i % copies == 0 else q.ptr, n, y.ptr, n), "qmatmul")
        dev.synchronize()
        print(json.dumps({"kernel_only": [n, k], "qtype": args.qtype, "actmode": args.actmode, "launches": args.launches, "ring_copies": copies}))
        return
    wl = Workload(dev, [(n, k)], seed=0, ring_bytes=max(2 * nbytes, 160 << 20))
    for _ in range(args.launches):
        wl.launch(0)
    dev.synchronize()
    print(json.dumps({"kernel_only": [n, k], "launches": args.launches, "ring_copies": len(wl.rings[0])}))


def run_attn_only(args):
    """A few plain launches of the prefill attention (f16, causal, head dimension 128) on one shape: the case ncu captures."""
    from candy_b200.backend import CudaDevice, RawBuffer
    b, h, hk, s = (int(v) for v in args.attn_only.lower().split("x"))
    d = 128
    dev = CudaDevice(int(os.environ.get("LOCAL_RANK", "0")))
    lib, ctx = dev._lib, dev.ctx
    q, k, v, o = (RawBuffer(dev, 2 * b * s * hh * d) for hh in (h, hk, hk, h))
    for buf, byte in ((q, 0x3C), (k, 0x2C), (v, 0x34)):
        lib.cq_memset(ctx, buf.ptr, byte, buf.nbytes)
    a = [q.ptr, k.ptr, v.ptr, o.ptr, None, None, None, None, s * h * d, s * hk * d, s * hk * d, s * h * d, 0, h * d, hk * d, hk * d, h * d, d, d, d, d,
         b, h, hk, d, d, float(1.0 / np.sqrt(d)), s, s, s, s, 0, 1, 0, -1, -1, 0.0]
    for _ in range(args.launches):
        dev._check(lib.cq_flash_attention(ctx, *a), "flash attention")
    dev.synchronize()
    print(json.dumps({"attn_only": [b, h, hk, s], "launches": args.launches}))


def run_gemm_only(args):
    """A few plain launches of the prefill GEMM on one shape (--actmode 2: f16 operands, 1: Q8_1 / int8, 0: f32 mode): the case ncu captures."""
    from candy_b200.backend import CudaDevice, QStorage
    m, n, k = (int(v) for v in args.gemm_only.lower().split("x"))
    dev = CudaDevice(int(os.environ.get("LOCAL_RANK", "0")))
    rng = np.random.default_rng(1)
    q = QStorage.quantize(dev, Q4_0, ORDER, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    x = dev.storage_from_slice(rng.standard_normal((m, k), dtype=np.float32))
    y = dev.alloc(m * n)
    for _ in range(args.launches):
        dev._check(dev._lib.cq_qmatmul(dev.ctx, Q4_0, ORDER, args.gemm_actmode, x.ptr, m, k, k, q.buf.ptr, n, y.ptr, n), "qmatmul")
    dev.synchronize()
    print(json.dumps({"gemm_only": [m, n, k], "actmode": args.gemm_actmode, "launches": args.launches}))


def run_decode_only(args):
    """A few un-captured decode steps of a shallow 7B-width model: the case ncu lists kernel by kernel."""
    from candy_b200.backend import CudaDevice
    from candy_b200.decoder import DecoderConfig, QuantDecoder
    dev = CudaDevice(int(os.environ.get("LOCAL_RANK", "0")))
    for kv in args.option:
        key, val = kv.split("=")
        dev.set_option(key, int(val))
    cfg = DecoderConfig(n_layers=args.decode_only, dim=4096, n_heads=32, n_kv_heads=32, head_dim=128, ffn=11008, vocab=32000, max_ctx=384)
    model = QuantDecoder(dev, cfg, seed=2)
    model.set_state(np.array([1], dtype=np.uint32), 255)
    for _ in range(args.launches):
        model.step(advance=False)
    dev.synchronize()
    print(json.dumps({"decode_only_layers": args.decode_only, "steps": args.launches, "launches_per_step": model.launches_per_step()}))


class _QuietStdout:
    """Everything libraries print to file descriptor 1 while the benchmark runs (NCCL announces its version
    there) goes to stderr; the JSON line is written to the real stdout at the end, alone."""

    def __enter__(self):
        sys.stdout.flush()
        self.real = os.dup(1)
        os.dup2(2, 1)
        return self

    def emit(self, text: str):
        os.write(self.real, (text + "\n").encode())

    def __exit__(self, *a):
        sys.stdout.flush()
        os.dup2(self.real, 1)
        os.close(self.real)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg (profiling runs)")
    ap.add_argument("--skip-extras", action="store_true", help="skip the 7B decode and 70B tensor-parallel layer workloads")
    ap.add_argument("--kernel-only", default=None, metavar="NxK", help="profiling aid: launch one GEMV shape a few times")
    ap.add_argument("--gemm-only", default=None, metavar="MxNxK", help="profiling aid: launch the prefill GEMM a few times")
    ap.add_argument("--gemm-actmode", type=int, default=2, help="gemm-only mode: 2 f16 operands, 1 Q8_1 activations (int8 tensor cores), 0 f32 mode")
    ap.add_argument("--attn-only", default=None, metavar="BxHxHKxS", help="profiling aid: launch the prefill attention a few times")
    ap.add_argument("--decode-only", type=int, default=0, metavar="LAYERS", help="profiling aid: a few plain decode steps of a shallow 7B-width model")
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--qtype", type=int, default=2, help="kernel-only mode: block format id (2 Q4_0, 3 Q4_1, 6 Q5_0, 7 Q5_1, 8 Q8_0)")
    ap.add_argument("--actmode", type=int, default=0, help="kernel-only mode: 0 f32 activations, 1 Q8_1 activations")
    ap.add_argument("--option", action="append", default=[], metavar="KEY=INT", help="library tuning option (kernel-only mode)")
    args = ap.parse_args()
    if args.kernel_only:
        run_kernel_only(args)
        return
    if args.gemm_only:
        run_gemm_only(args)
        return
    if args.attn_only:
        run_attn_only(args)
        return
    if args.decode_only:
        run_decode_only(args)
        return
    if args.impl == "reference":
        args.steps = 20 if args.steps is None else args.steps
        args.warmup = 3 if args.warmup is None else max(args.warmup, 0)
        run_reference(args)
    else:
        args.steps = 50 if args.steps is None else args.steps
        args.warmup = 3 if args.warmup is None else max(args.warmup, 3)
        with _QuietStdout() as out:
            args.emit = out.emit
            run_ours(args)


if __name__ == "__main__":
    main()
