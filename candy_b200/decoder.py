"""A Llama-shape decoder step built only from libcandyq calls: the caller of the quantized
linear that BASELINE configs 4 and 5 measure (tokens/s of greedy decode; tensor-parallel layers).

candy itself has no LLM code (llm/ holds a README and a FlashAttention binding), so this module
is the host-side loop a candy user would write against the backend API: embedding gather, then
per layer RMSNorm -> fused QKV linear -> RoPE + KV-cache write -> decode attention -> o linear ->
residual + RMSNorm -> fused gate/up linear -> SiLU*mul -> down linear, then final norm, output
linear and argmax.  Every operator is a kernel of the library; positions and token ids stay on
the device, so one step can be captured into a CUDA graph and replayed once per token.

Tensor parallelism (world > 1): QKV / gate / up are split by output rows (whole heads), o / down
by input columns, and `allreduce` (supplied by the caller, e.g. NCCL through torch.distributed)
sums the two row-parallel outputs of each layer.  Each rank creates only its own shards.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np

from . import abi
from .backend import CudaDevice, QStorage, RawBuffer, Q4_0, ORDER_GO_INTERLEAVED, ACT_F32, ACT_F16


@dataclass
class DecoderConfig:
    n_layers: int = 32
    dim: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    vocab: int = 32000
    max_ctx: int = 384
    eps: float = 1e-5
    rope_theta: float = 10000.0
    with_head: bool = True  # embedding + output linear + argmax (a bare layer stack otherwise)


def shard_sizes(cfg: DecoderConfig, world: int):
    """Per-rank sizes under tensor parallelism; raises if heads or ffn do not divide."""
    if cfg.n_heads % world or cfg.n_kv_heads % world or cfg.ffn % world:
        raise ValueError(f"tensor parallel degree {world} must divide heads ({cfg.n_heads}), kv heads ({cfg.n_kv_heads}) and ffn ({cfg.ffn})")
    nq, nkv, ffn = cfg.n_heads // world, cfg.n_kv_heads // world, cfg.ffn // world
    if (nq * cfg.head_dim) % 32 or ffn % 32:
        raise ValueError("row-parallel shards must keep k a multiple of 32 so no block is cut")
    return nq, nkv, ffn


def rope_tables(cfg: DecoderConfig):
    """cos/sin [max_ctx, head_dim/2] in f32 from f64 angles (the tables RopeF32 takes as inputs)."""
    half = cfg.head_dim // 2
    inv = 1.0 / (cfg.rope_theta ** (np.arange(half, dtype=np.float64) * 2.0 / cfg.head_dim))
    ang = np.arange(cfg.max_ctx, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


class PositionGuard:
    """Host-side shadow of the device-resident decode position.

    The position is advanced on the device (inside captured graphs), where the host cannot see it, so
    the runner keeps its own count and refuses any step, replay or state that would index a KV cache
    or rotary table at or beyond ``max_ctx``.  (The kernels clamp and flag such a position as well;
    this check fails earlier and with the offending numbers.)"""

    def __init__(self, max_ctx: int):
        self.max_ctx = int(max_ctx)
        self.pos = 0

    def set(self, pos: int) -> None:
        if not 0 <= int(pos) < self.max_ctx:
            raise ValueError(f"decoder: position {pos} outside [0, {self.max_ctx})")
        self.pos = int(pos)

    def need(self, steps: int, what: str = "step") -> None:
        """Raises unless `steps` more advancing steps fit: the last of them runs at pos + steps - 1."""
        if steps > 0 and self.pos + steps > self.max_ctx:
            raise ValueError(f"decoder: {what} of {steps} position(s) from {self.pos} runs past max_ctx {self.max_ctx}")

    def advance(self, steps: int) -> None:
        self.need(steps)
        self.pos += int(steps)


class QuantDecoder:
    def __init__(self, dev: CudaDevice, cfg: DecoderConfig, seed: int = 0, batch: int = 1, qtype: int = Q4_0,
                 order: int = ORDER_GO_INTERLEAVED, rank: int = 0, world: int = 1,
                 allreduce: Optional[Callable[[object, int], None]] = None, actmode: Optional[int] = None, comm=None, fuse: bool = True):
        self.dev, self.cfg, self.batch, self.qtype, self.order = dev, cfg, batch, qtype, order
        # actmode None: f32-activation GEMVs (one weight pass per row) up to two rows, the tensor-core
        # kernel (f16 activations, one weight pass for the batch) for wider batches without a communicator
        if actmode is None:
            actmode = ACT_F32 if (batch <= 2 or comm is not None) else ACT_F16
        self.rank, self.world, self.allreduce, self.actmode = rank, world, allreduce, actmode
        # comm: a connected cq_comm handle -> the two all-reduces of a layer are fused into the GEMV
        # before them and the residual+norm after them (batch <= 8 only); else `allreduce` is called
        self.comm = comm
        # fuse: residual add + RMSNorm ride in the prologue of the QKV / gate-up / output GEMVs and
        # SiLU(gate)*up in the gate-up GEMV's epilogue (cq_qlinear_fused); f32 activation mode, batch <= 8, no communicator
        self.fuse = bool(fuse) and comm is None and batch <= 8 and actmode == ACT_F32
        self._pending = [False, False]  # a push into set i awaits its reducing norm
        if world > 1 and allreduce is None and comm is None:
            raise ValueError("tensor parallel decoder needs an allreduce callback or a communicator")
        if comm is not None and (batch > 8 or cfg.with_head):
            raise ValueError("the fused exchange serves bare layer stacks with batch <= 8")
        self.nq, self.nkv, self.ffn = shard_sizes(cfg, world)
        self.lib, self.ctx = dev._lib, dev.ctx
        hd, dim = cfg.head_dim, cfg.dim
        self.qkv_rows = (self.nq + 2 * self.nkv) * hd
        self.kv_dim = self.nkv * hd
        # The down projection's k (this rank's slice of the feed-forward width) is padded to a
        # multiple of 256 so its rows stay 16-byte aligned for the streaming kernel; the padded
        # activations are zero, so whatever the padded weight columns hold contributes nothing.
        self.ffn_pad = -(-self.ffn // 256) * 256
        # ---- weights: generated and quantized on the device, shard by shard ------------------
        biggest = max(self.qkv_rows * dim, dim * self.nq * hd, 2 * self.ffn * dim, dim * self.ffn_pad,
                      (cfg.vocab * dim) if cfg.with_head else 0)
        tmp = dev.alloc(biggest)
        self.layers = []
        for l in range(cfg.n_layers):
            s = (seed * 1000003 + l) * 16 + rank * 4099
            self.layers.append({
                "wqkv": self._rand_q(tmp, self.qkv_rows, dim, s + 1),
                "wo": self._rand_q(tmp, dim, self.nq * hd, s + 2),
                "wgu": self._rand_q(tmp, 2 * self.ffn, dim, s + 3),
                "wdown": self._rand_q(tmp, dim, self.ffn_pad, s + 4),
                "attn_norm": dev.storage_from_slice(np.ones(dim, dtype=np.float32)),
                "ffn_norm": dev.storage_from_slice(np.ones(dim, dtype=np.float32)),
                "k": dev.zeros(batch * cfg.max_ctx * self.kv_dim),
                "v": dev.zeros(batch * cfg.max_ctx * self.kv_dim),
            })
        if cfg.with_head:
            self.embed = dev.alloc(cfg.vocab * dim)
            self._check(self.lib.cq_rand_normal(self.ctx, self.embed.ptr, cfg.vocab * dim, 0.0, 0.02, seed * 7919 + 11), "rand")
            self.wout = self._rand_q(tmp, cfg.vocab, dim, seed * 7919 + 13)
            self.final_norm = dev.storage_from_slice(np.ones(dim, dtype=np.float32))
            self.logits = dev.alloc(batch * cfg.vocab)
        del tmp
        cos, sin = rope_tables(cfg)
        self.cos, self.sin = dev.storage_from_slice(cos), dev.storage_from_slice(sin)
        # ---- activations --------------------------------------------------------------------
        self.x = dev.zeros(batch * dim)
        self.x2 = dev.zeros(batch * dim)  # the residual stream alternates between x and x2 when norms are fused
        self.xn = dev.alloc(batch * dim)
        self.qkv = dev.alloc(batch * self.qkv_rows)
        self.att = dev.alloc(batch * self.nq * hd)
        self.o = dev.alloc(batch * dim)
        self.gu = dev.alloc(batch * 2 * self.ffn)
        self.h = dev.zeros(batch * self.ffn_pad)
        self.d = dev.zeros(batch * dim)
        self.att_scratch = dev.alloc(self.lib.cq_decode_attention_scratch_floats(batch, self.nq, hd, cfg.max_ctx))
        self.ids = RawBuffer(dev, 4 * batch)
        self.pos = RawBuffer(dev, 4)
        self.guard = PositionGuard(cfg.max_ctx)
        self._capturing = False
        self._graph_steps = {}  # graph handle -> advancing steps recorded in it
        self.set_state(np.zeros(batch, dtype=np.uint32), 0)
        dev.synchronize()

    # ---- helpers ----------------------------------------------------------------------------
    def _check(self, st, where):
        abi.check(self.ctx, st, where)

    def _rand_q(self, tmp, n, k, seed) -> QStorage:
        self._check(self.lib.cq_rand_normal(self.ctx, tmp.ptr, n * k, 0.0, 0.02, seed), "rand normal")
        buf = RawBuffer(self.dev, n * (k // 32) * abi.BLOCK_BYTES[self.qtype])
        self._check(self.lib.cq_quantize_rows(self.ctx, self.qtype, self.order, tmp.ptr, n, k, buf.ptr), "quantize")
        return QStorage(self.dev, self.qtype, self.order, n, k, buf)

    def _linear(self, w: QStorage, x, y):
        self._check(self.lib.cq_qmatmul(self.ctx, w.qtype, w.order, self.actmode, x.ptr, self.batch, w.k, w.k, w.buf.ptr, w.n,
                                        y.ptr, w.n), "qmatmul")

    def set_state(self, ids: np.ndarray, pos: int):
        self.guard.set(pos)
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        p = np.array([pos], dtype=np.int32)
        self._check(self.lib.cq_memcpy_h2d(self.ctx, self.ids.ptr, ids.ctypes.data_as(C.c_void_p), ids.nbytes), "ids")
        self._check(self.lib.cq_memcpy_h2d(self.ctx, self.pos.ptr, p.ctypes.data_as(C.c_void_p), 4), "pos")

    def weight_bytes_per_step(self) -> int:
        """Quantized weight bytes one decode step streams on this rank."""
        per_layer = sum(self.layers[0][k].buf.nbytes for k in ("wqkv", "wo", "wgu", "wdown"))
        return per_layer * self.cfg.n_layers + (self.wout.buf.nbytes if self.cfg.with_head else 0)

    def launches_per_step(self) -> int:
        if getattr(self, "_pdec", None):
            return 1
        # fused: QKV(+norm), attention (+rotary step; one cluster launch for contexts up to 1024 without grouped heads, else
        # partial + combine), o, gate-up(+norm, +SiLU*mul), down
        one_launch_attention = self.cfg.max_ctx <= 1024 and self.cfg.head_dim <= 128 and self.nq == self.nkv
        per_layer = (5 if one_launch_attention else 6) if self.fuse else (9 if one_launch_attention else 10)
        return self.cfg.n_layers * per_layer + ((3 if self.fuse else 5) if self.cfg.with_head else 0)

    # ---- the whole step as one persistent kernel (batch 1, one GPU, with embedding and output linear) -------
    def enable_persistent(self) -> bool:
        """Switches step() to cq_decoder_step: one cooperative launch per token instead of ~200 small ones.
        Returns False (and changes nothing) when the library has no persistent kernel for this model's shape."""
        cfg = self.cfg
        if self.batch != 1 or self.world != 1 or not cfg.with_head or self.comm is not None:
            return False
        n = cfg.n_layers

        def arr(key):
            return (C.c_void_p * n)(*[(L[key].buf.ptr.value if hasattr(L[key], "buf") else L[key].ptr.value) for L in self.layers])

        self._pd_arrays = {k: arr(k) for k in ("wqkv", "wo", "wgu", "wdown", "attn_norm", "ffn_norm", "k", "v")}
        d = abi.DecoderDesc()
        d.n_layers, d.dim, d.n_heads, d.n_kv_heads, d.head_dim = n, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        d.ffn, d.ffn_pad, d.vocab, d.max_ctx, d.eps, d.qtype, d.order = cfg.ffn, self.ffn_pad, cfg.vocab, cfg.max_ctx, cfg.eps, self.qtype, self.order
        for field, key in (("wqkv", "wqkv"), ("wo", "wo"), ("wgu", "wgu"), ("wdown", "wdown"), ("attn_norm", "attn_norm"), ("ffn_norm", "ffn_norm"),
                           ("k_cache", "k"), ("v_cache", "v")):
            setattr(d, field, C.cast(self._pd_arrays[key], C.POINTER(C.c_void_p)))
        d.embed, d.wout, d.final_norm = self.embed.ptr.value, self.wout.buf.ptr.value, self.final_norm.ptr.value
        d.cos_table, d.sin_table = self.cos.ptr.value, self.sin.ptr.value
        handle = C.c_void_p()
        st = self.lib.cq_decoder_create(self.ctx, C.byref(d), C.byref(handle))
        if st == abi.CQ_ERR_UNSUPPORTED:
            return False
        self._check(st, "decoder create")
        self._pdec = handle
        return True

    def _step_persistent(self, advance: bool):
        if not advance:
            raise ValueError("the persistent step always advances the position")
        self._check(self.lib.cq_decoder_step(self.ctx, self._pdec, self.ids.ptr, self.pos.ptr), "decoder step")
        if not self._capturing:
            self.guard.advance(1)

    # ---- one decode step, enqueued on the context's stream -----------------------------------
    def step(self, advance: bool = True):
        if getattr(self, "_pdec", None):
            if not self._capturing:
                self.guard.need(1)
            return self._step_persistent(advance)
        # A decode step is a chain of GEMVs with small kernels in between: the library's planner then prefers one CTA
        # of twelve warps per SM over two of eight (single-GPU, batch-1 step: +3 %; the sharded layers of a tensor-parallel
        # step were measured slightly slower with it, 0.706 against 0.693 ms on two GPUs, and keep the default).
        chain = self.world == 1 and self.batch == 1
        if chain:
            self._check(self.lib.cq_ctx_set_option(self.ctx, b"gemv_chain", 1), "set option")
        try:
            return self._step_launches(advance)
        finally:
            if chain:
                self._check(self.lib.cq_ctx_set_option(self.ctx, b"gemv_chain", 0), "set option")

    def _step_launches(self, advance: bool = True):
        lib, ctx, cfg, B = self.lib, self.ctx, self.cfg, self.batch
        hd, dim = cfg.head_dim, cfg.dim
        if not self._capturing:  # a recorded step runs at replay time: replay() accounts for it
            self.guard.need(1)
        if cfg.with_head:
            self._check(lib.cq_embedding(ctx, self.embed.ptr, cfg.vocab, dim, self.ids.ptr, B, self.x.ptr), "embedding")
        first = True
        fused = self.comm is not None
        xc, xo = self.x, self.x2  # residual stream: current / next buffer (fused norms ping-pong them)

        def fused_linear(w, delta, alpha, y, ld_y, epilogue=0, keep=True):
            """y = epilogue(rmsnorm(xc + delta) . W^T); the sum xc + delta goes to xo, which becomes xc.  False if the shape is not taken."""
            nonlocal xc, xo
            st = lib.cq_qlinear_fused(ctx, w.qtype, w.order, xc.ptr, delta.ptr if delta is not None else None, alpha.ptr, cfg.eps,
                                      xo.ptr if keep else None, B, dim, w.buf.ptr, w.n, epilogue, y.ptr, ld_y)
            if st == abi.CQ_ERR_UNSUPPORTED:
                return False
            self._check(st, "fused linear")
            if keep:
                xc, xo = xo, xc
            return True

        for L in self.layers:
            delta = None if (first and cfg.with_head) else self.d  # previous feed-forward output (zeros before the first step)
            done = False
            if self.fuse:
                done = fused_linear(L["wqkv"], delta, L["attn_norm"], self.qkv, self.qkv_rows)
            if not done:
                if first and cfg.with_head:  # x was just gathered from the embedding table
                    self._check(lib.cq_rmsnorm(ctx, xc.ptr, L["attn_norm"].ptr, B, dim, cfg.eps, self.xn.ptr), "rmsnorm")
                elif fused and self._pending[1]:  # the down projection's partials are summed inside this norm
                    self._check(lib.cq_add_rmsnorm_reduce(ctx, self.comm, 1, xc.ptr, L["attn_norm"].ptr, B, dim, cfg.eps, self.xn.ptr), "reduce+rmsnorm")
                    self._pending[1] = False
                elif fused:  # very first step of a fused stack: nothing has been pushed yet
                    self._check(lib.cq_rmsnorm(ctx, xc.ptr, L["attn_norm"].ptr, B, dim, cfg.eps, self.xn.ptr), "rmsnorm")
                else:  # residual of the previous feed-forward (previous layer, or previous step of a bare stack), then the norm
                    self._check(lib.cq_add_rmsnorm(ctx, xc.ptr, self.d.ptr, L["attn_norm"].ptr, B, dim, cfg.eps, self.xn.ptr), "add+rmsnorm")
                self._linear(L["wqkv"], self.xn, self.qkv)
            first = False
            if self.fuse:  # rotary step and cache write inside the attention kernels
                self._check(lib.cq_decode_attention_rope(ctx, self.qkv.ptr, B, self.nq, self.nkv, hd, self.cos.ptr, self.sin.ptr, self.pos.ptr,
                                                         L["k"].ptr, L["v"].ptr, cfg.max_ctx, self.att_scratch.ptr, self.att.ptr), "rope+attention")
            else:
                self._check(lib.cq_rope_store_kv(ctx, self.qkv.ptr, B, self.nq, self.nkv, hd, self.cos.ptr, self.sin.ptr, self.pos.ptr,
                                                 L["k"].ptr, L["v"].ptr, cfg.max_ctx), "rope")
                self._check(lib.cq_decode_attention(ctx, self.qkv.ptr, B, self.nq, self.nkv, hd, self.pos.ptr, L["k"].ptr, L["v"].ptr,
                                                    cfg.max_ctx, self.att_scratch.ptr, self.att.ptr), "attention")
            done = False
            if fused:
                w = L["wo"]
                self._check(lib.cq_qmatmul_push(ctx, self.comm, 0, w.qtype, w.order, self.att.ptr, B, w.k, w.k, w.buf.ptr, w.n), "push o")
                self._check(lib.cq_add_rmsnorm_reduce(ctx, self.comm, 0, xc.ptr, L["ffn_norm"].ptr, B, dim, cfg.eps, self.xn.ptr), "reduce+rmsnorm")
            else:
                self._linear(L["wo"], self.att, self.o)
                if self.world > 1:
                    self.allreduce(self.o, B * dim)
                if self.fuse:  # gate and up rows are interleaved, so the epilogue can pair them
                    done = fused_linear(L["wgu"], self.o, L["ffn_norm"], self.h, self.ffn_pad, epilogue=1)
                if not done:
                    self._check(lib.cq_add_rmsnorm(ctx, xc.ptr, self.o.ptr, L["ffn_norm"].ptr, B, dim, cfg.eps, self.xn.ptr), "add+rmsnorm")
            # (fusing only the epilogue when the prologue is refused measured no gain: 133.0 vs 131.5 us per 70B-shape layer)
            if not done:
                self._linear(L["wgu"], self.xn, self.gu)
                self._check(lib.cq_silu_mul_pairs(ctx, self.gu.ptr, B, self.ffn, self.h.ptr, self.ffn_pad), "silu*mul")
            if fused:
                w = L["wdown"]
                self._check(lib.cq_qmatmul_push(ctx, self.comm, 1, w.qtype, w.order, self.h.ptr, B, w.k, w.k, w.buf.ptr, w.n), "push down")
                self._pending[1] = True
            else:
                self._linear(L["wdown"], self.h, self.d)
                if self.world > 1:
                    self.allreduce(self.d, B * dim)
        if cfg.with_head:
            done = self.fuse and fused_linear(self.wout, self.d, self.final_norm, self.logits, cfg.vocab, keep=False)
            if not done:
                self._check(lib.cq_add_rmsnorm(ctx, xc.ptr, self.d.ptr, self.final_norm.ptr, B, dim, cfg.eps, self.xn.ptr), "final norm")
                self._linear(self.wout, self.xn, self.logits)
            self._check(lib.cq_argmax(ctx, self.logits.ptr, B, cfg.vocab, self.ids.ptr), "argmax")
        if xc is not self.x:  # an odd number of fused norms ran (one fell back): bring the stream home
            self._check(lib.cq_memcpy_d2d(ctx, self.x.ptr, xc.ptr, 4 * B * dim), "residual home")
        if advance:
            self._check(lib.cq_add_int(ctx, self.pos.ptr, 1), "advance")
            if not self._capturing:
                self.guard.advance(1)


    # ---- the prompt as one pass (batch 1, one GPU, with embedding and output linear) ---------------------------
    def prefill(self, tokens, actmode: int = ACT_F16, bf16: bool = False):
        """Runs the whole prompt through the model in ONE pass instead of one decode step per token: the linears see
        all positions at once (cq_qmatmul with m = len(tokens): tensor-core GEMMs in CQ_ACT_F16, the default here),
        the rotary step and the KV-cache writes cover every position (cq_rope_prefill) and the causal attention of
        the prompt runs on the tensor cores (cq_flash_attention, f16 operands).  Afterwards the caches, the position
        and the next token are exactly where len(tokens) calls of step() would have left them (the token up to the
        arg-max of logits that differ by the f16 roundings of this path), so step() / replay() continue from there.
        bf16: the attention operands are bf16 instead of f16.  The pass may continue a sequence (a second prompt after
        some decoding): the cached keys and values of the earlier positions are then cast to 16 bits for the attention.
        Returns the number of kernel launches of the pass."""
        cfg, lib, ctx, dev = self.cfg, self.lib, self.ctx, self.dev
        if self.batch != 1 or self.world != 1 or not cfg.with_head or self.comm is not None:
            raise ValueError("prefill serves a single sequence on one GPU with embedding and output linear")
        if cfg.head_dim not in (64, 128):
            raise ValueError("prefill attention is built for head dimensions 64 and 128")
        toks = np.ascontiguousarray(tokens, dtype=np.uint32).reshape(-1)
        T = int(toks.size)
        if T < 1:
            raise ValueError("prefill needs at least one token")
        pos0 = int(self.guard.pos)
        self.guard.need(T, "prefill")
        hd, dim, nq, nkv = cfg.head_dim, cfg.dim, self.nq, self.nkv
        ctx_len = pos0 + T  # keys the prompt's queries may see
        bufs = getattr(self, "_prefill_bufs", None)
        if bufs is None or bufs["T"] < T or bufs["C"] < ctx_len:
            bufs = {"T": T, "C": ctx_len, "ids": RawBuffer(dev, 4 * T), "x": dev.alloc(T * dim), "xn": dev.alloc(T * dim), "qkv": dev.alloc(T * self.qkv_rows),
                    "q16": RawBuffer(dev, 2 * T * nq * hd), "k16": RawBuffer(dev, 2 * ctx_len * nkv * hd), "v16": RawBuffer(dev, 2 * ctx_len * nkv * hd),
                    "o16": RawBuffer(dev, 2 * T * nq * hd), "att": dev.alloc(T * nq * hd), "o": dev.alloc(T * dim), "gu": dev.alloc(T * 2 * self.ffn),
                    "h": dev.zeros(T * self.ffn_pad), "d": dev.alloc(T * dim), "lse": dev.alloc(nq * ((T + 127) // 128 * 128))}
            self._prefill_bufs = bufs
        P = bufs
        self._check(lib.cq_memcpy_h2d(ctx, P["ids"].ptr, toks.ctypes.data_as(C.c_void_p), toks.nbytes), "prompt ids")
        launches = 0

        def linear(w, x, y):
            self._check(lib.cq_qmatmul(ctx, w.qtype, w.order, actmode, x.ptr, T, w.k, w.k, w.buf.ptr, w.n, y.ptr, w.n), "prefill qmatmul")

        self._check(lib.cq_embedding(ctx, self.embed.ptr, cfg.vocab, dim, P["ids"].ptr, T, P["x"].ptr), "embedding")
        scale = 1.0 / float(np.sqrt(hd))
        for li, L in enumerate(self.layers):
            if li == 0:
                self._check(lib.cq_rmsnorm(ctx, P["x"].ptr, L["attn_norm"].ptr, T, dim, cfg.eps, P["xn"].ptr), "rmsnorm")
            else:
                self._check(lib.cq_add_rmsnorm(ctx, P["x"].ptr, P["d"].ptr, L["attn_norm"].ptr, T, dim, cfg.eps, P["xn"].ptr), "add+rmsnorm")
            linear(L["wqkv"], P["xn"], P["qkv"])
            if pos0 > 0:  # the earlier positions' keys and values, as the attention wants them
                self._check(lib.cq_cast_f32_to_16(ctx, L["k"].ptr, pos0 * nkv * hd, 1 if bf16 else 0, P["k16"].ptr), "cast k")
                self._check(lib.cq_cast_f32_to_16(ctx, L["v"].ptr, pos0 * nkv * hd, 1 if bf16 else 0, P["v16"].ptr), "cast v")
            new16 = 2 * pos0 * nkv * hd  # this prompt's rows follow them
            self._check(lib.cq_rope_prefill(ctx, P["qkv"].ptr, T, nq, nkv, hd, self.cos.ptr, self.sin.ptr, pos0, L["k"].ptr, L["v"].ptr, cfg.max_ctx,
                                            P["q16"].ptr, C.c_void_p(P["k16"].ptr.value + new16), C.c_void_p(P["v16"].ptr.value + new16),
                                            1 if bf16 else 0), "rope prefill")
            self._check(lib.cq_flash_attention(ctx, P["q16"].ptr, P["k16"].ptr, P["v16"].ptr, P["o16"].ptr, P["lse"].ptr, None, None, None,
                                               T * nq * hd, ctx_len * nkv * hd, ctx_len * nkv * hd, T * nq * hd, 0, nq * hd, nkv * hd, nkv * hd, nq * hd, hd, hd, hd, hd,
                                               1, nq, nkv, hd, hd, scale, T, ctx_len, (T + 127) // 128 * 128, (ctx_len + 127) // 128 * 128, 1 if bf16 else 0, 1, 0, -1, -1, 0.0),
                        "prefill attention")
            self._check(lib.cq_cast16_to_f32(ctx, P["o16"].ptr, T * nq * hd, 1 if bf16 else 0, P["att"].ptr), "cast")
            linear(L["wo"], P["att"], P["o"])
            self._check(lib.cq_add_rmsnorm(ctx, P["x"].ptr, P["o"].ptr, L["ffn_norm"].ptr, T, dim, cfg.eps, P["xn"].ptr), "add+rmsnorm")
            linear(L["wgu"], P["xn"], P["gu"])
            self._check(lib.cq_silu_mul_pairs(ctx, P["gu"].ptr, T, self.ffn, P["h"].ptr, self.ffn_pad), "silu*mul")
            linear(L["wdown"], P["h"], P["d"])
            launches += 11
        # the last position's row only: final norm, output linear (a GEMV), arg-max
        last = 4 * (T - 1) * dim
        x_last, d_last = C.c_void_p(P["x"].ptr.value + last), C.c_void_p(P["d"].ptr.value + last)
        self._check(lib.cq_add_rmsnorm(ctx, x_last, d_last, self.final_norm.ptr, 1, dim, cfg.eps, self.xn.ptr), "final norm")
        w = self.wout
        self._check(lib.cq_qmatmul(ctx, w.qtype, w.order, ACT_F32, self.xn.ptr, 1, w.k, w.k, w.buf.ptr, w.n, self.logits.ptr, w.n), "output linear")
        self._check(lib.cq_argmax(ctx, self.logits.ptr, 1, cfg.vocab, self.ids.ptr), "argmax")
        pos = np.array([ctx_len], dtype=np.int32)
        self._check(lib.cq_memcpy_h2d(ctx, self.pos.ptr, pos.ctypes.data_as(C.c_void_p), 4), "pos")
        self.guard.pos = ctx_len
        return launches + 5

    def capture(self, steps: int = 1):
        g = C.c_void_p()
        self._check(self.lib.cq_capture_begin(self.ctx), "capture begin")
        self._capturing = True
        try:
            for _ in range(steps):
                self.step()
        finally:
            self._capturing = False
            self._check(self.lib.cq_capture_end(self.ctx, C.byref(g)), "capture end")
        self._graph_steps[g.value] = steps
        return g

    def replay(self, g, times: int = 1):
        """Launches a captured graph `times` times; refused when that would run past max_ctx."""
        self.guard.advance(self._graph_steps.get(g.value, 0) * times)
        for _ in range(times):
            self._check(self.lib.cq_graph_launch(self.ctx, g), "graph launch")

    def read_logits(self) -> np.ndarray:
        if getattr(self, "_pdec", None):
            out = np.empty((1, self.cfg.vocab), dtype=np.float32)
            src = self.lib.cq_decoder_logits(self._pdec)
            self._check(self.lib.cq_memcpy_d2h(self.ctx, out.ctypes.data_as(C.c_void_p), src, out.nbytes), "logits")
            return out
        return self.logits.data().reshape(self.batch, self.cfg.vocab)

    def __del__(self):
        try:
            if getattr(self, "_pdec", None):
                self.lib.cq_decoder_destroy(self.ctx, self._pdec)
                self._pdec = None
        except Exception:
            pass

    def read_ids(self) -> np.ndarray:
        return self.ids.data().view(np.uint32).copy()
