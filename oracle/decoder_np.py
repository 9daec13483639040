"""NumPy restatement of one decoder step with candy's CPU arithmetic (test infrastructure).

Linears go through the C oracle (dequantize + sequential f32 matmul); the operators between them
follow the CPU kernels in tensor/internal/cpu/kernels/: FastRmsNormF32 (reduce.go:3071-3092),
RopeF32 (reduce.go:3987-4006), FastSoftmaxF32 (reduce.go:2855-2879), USiluF32 (unary.go:3353-3365,
f64 inside), FastArgmaxF32 (reduce.go:846-862).  Sums over a row are taken with np.float32
accumulation; their order differs from the sequential Go loops by rounding only.
Pinned by tests/test_decoder_oracle_pins.py to the known answers of the reference's own unit tests
(reduce_test.go, unary_test.go; the literals are in tests/golden/reduce_unary_kats.json).
"""
from __future__ import annotations

import numpy as np

from . import oracle_c as oc

f32 = np.float32


def rmsnorm(x, alpha, eps):
    mean = (x.astype(f32) ** 2).sum(dtype=f32) / f32(x.size)
    scale = f32(1.0) / f32(np.sqrt(np.float64(mean + f32(eps))))
    return (scale * x * alpha).astype(f32)


def rope(v, cos, sin):
    """v: [heads, head_dim]; pairs (i, i + d/2)."""
    half = v.shape[1] // 2
    a, b = v[:, :half].copy(), v[:, half:].copy()
    out = np.empty_like(v)
    out[:, :half] = a * cos - b * sin
    out[:, half:] = a * sin + b * cos
    return out


def softmax(s):
    m = s.max()
    e = np.exp((s - m).astype(np.float64)).astype(f32)
    return (e * (f32(1.0) / e.sum(dtype=f32))).astype(f32)


def argmax(x):
    """FastArgmaxF32 (reduce.go:846-862): strict '>', so the lowest index among equal maxima."""
    best, bi = x[0], 0
    for i in range(1, len(x)):
        if x[i] > best:
            best, bi = x[i], i
    return bi


def silu(x):
    x64 = x.astype(np.float64)
    return (x64 / (1.0 + np.exp(-x64))).astype(f32)


class OracleDecoder:
    """Single sequence.  `layers` is a list of dicts with the Q-blocks (uint8) of wqkv, wo, wgu, wdown."""

    def __init__(self, cfg, qtype, order, layers, embed=None, wout=None, cos=None, sin=None, nq=None, nkv=None, ffn=None, gu_interleaved=True):
        self.cfg, self.qt, self.order, self.layers = cfg, qtype, order, layers
        self.embed, self.wout, self.cos, self.sin = embed, wout, cos, sin
        self.nq = nq or cfg.n_heads
        self.nkv = nkv or cfg.n_kv_heads
        self.ffn = ffn or cfg.ffn
        self.gu_interleaved = gu_interleaved  # rows of wgu: (gate_0, up_0, gate_1, up_1, ...) instead of all gates, then all ups
        self.k = [np.zeros((cfg.max_ctx, self.nkv, cfg.head_dim), dtype=f32) for _ in layers]
        self.v = [np.zeros((cfg.max_ctx, self.nkv, cfg.head_dim), dtype=f32) for _ in layers]

    def lin(self, x, blocks, n):
        return oc.qmatmul(self.qt, self.order, x.reshape(1, -1), blocks, n, nthreads=8)[0]

    def step(self, token: int, pos: int):
        cfg = self.cfg
        hd, dim = cfg.head_dim, cfg.dim
        x = self.embed[token].astype(f32).copy()
        ones = np.ones(dim, dtype=f32)
        for li, L in enumerate(self.layers):
            xn = rmsnorm(x, ones, cfg.eps)
            qkv = self.lin(xn, L["wqkv"], (self.nq + 2 * self.nkv) * hd)
            q = rope(qkv[: self.nq * hd].reshape(self.nq, hd), self.cos[pos], self.sin[pos])
            k = rope(qkv[self.nq * hd:(self.nq + self.nkv) * hd].reshape(self.nkv, hd), self.cos[pos], self.sin[pos])
            v = qkv[(self.nq + self.nkv) * hd:].reshape(self.nkv, hd)
            self.k[li][pos], self.v[li][pos] = k, v
            att = np.empty((self.nq, hd), dtype=f32)
            group = self.nq // self.nkv
            for h in range(self.nq):
                kh = self.k[li][: pos + 1, h // group]
                s = (kh @ q[h]).astype(f32) * f32(1.0 / np.sqrt(hd))
                p = softmax(s)
                att[h] = (p[:, None] * self.v[li][: pos + 1, h // group]).sum(axis=0, dtype=f32)
            x = x + self.lin(att.reshape(-1), L["wo"], dim)
            xn = rmsnorm(x, ones, cfg.eps)
            gu = self.lin(xn, L["wgu"], 2 * self.ffn)
            h_ = silu(gu[0::2]) * gu[1::2] if self.gu_interleaved else silu(gu[: self.ffn]) * gu[self.ffn:]
            kpad = L["wdown"].size // dim // oc.BLOCK_BYTES[self.qt] * 32  # rows may be zero-padded in k
            hp = np.zeros(kpad, dtype=f32)
            hp[: self.ffn] = h_
            x = x + self.lin(hp, L["wdown"], dim)
        xn = rmsnorm(x, ones, cfg.eps)
        logits = self.lin(xn, self.wout, cfg.vocab)
        return logits


def sharded_layer_step(cfg, qtype, order, shards, x, pos, cos, sin):
    """One decoder layer for one sequence, computed from tensor-parallel SHARDS of its weights: the
    unsharded layer's arithmetic with the row-parallel outputs summed in rank order, which is what an
    all-reduce over the ranks yields.  `shards`: per rank a dict with the Q-blocks `wqkv` ([q heads; k heads;
    v heads] of that rank), `wo`, `wgu` (gate/up rows interleaved), `wdown` (k zero-padded to a multiple of
    256), the rank's key / value cache `k`, `v` as [ctx, nkv, head_dim] holding positions < pos, and its
    `nq`, `nkv`, `ffn`.  Returns the residual stream after the layer (x + attention + feed-forward)."""
    hd, dim = cfg.head_dim, cfg.dim
    ones = np.ones(dim, dtype=f32)

    def lin(v, blocks, n):
        return oc.qmatmul(qtype, order, v.reshape(1, -1), blocks, n, nthreads=16)[0]

    xn = rmsnorm(x.astype(f32), ones, cfg.eps)
    o = None
    for s in shards:
        nq, nkv = s["nq"], s["nkv"]
        qkv = lin(xn, s["wqkv"], (nq + 2 * nkv) * hd)
        q = rope(qkv[: nq * hd].reshape(nq, hd), cos[pos], sin[pos])
        k = rope(qkv[nq * hd:(nq + nkv) * hd].reshape(nkv, hd), cos[pos], sin[pos])
        v = qkv[(nq + nkv) * hd:].reshape(nkv, hd)
        K = np.concatenate([s["k"][:pos], k[None]], axis=0)
        V = np.concatenate([s["v"][:pos], v[None]], axis=0)
        att = np.empty((nq, hd), dtype=f32)
        group = nq // nkv
        for h in range(nq):
            sc = (K[:, h // group] @ q[h]).astype(f32) * f32(1.0 / np.sqrt(hd))
            p = softmax(sc)
            att[h] = (p[:, None] * V[:, h // group]).sum(axis=0, dtype=f32)
        part = lin(att.reshape(-1), s["wo"], dim)
        o = part if o is None else (o + part).astype(f32)
    x1 = (x + o).astype(f32)
    xn = rmsnorm(x1, ones, cfg.eps)
    d = None
    for s in shards:
        gu = lin(xn, s["wgu"], 2 * s["ffn"])
        h_ = silu(gu[0::2]) * gu[1::2]
        kpad = s["wdown"].size // dim // oc.BLOCK_BYTES[qtype] * 32
        hp = np.zeros(kpad, dtype=f32)
        hp[: s["ffn"]] = h_
        part = lin(hp, s["wdown"], dim)
        d = part if d is None else (d + part).astype(f32)
    return (x1 + d).astype(f32)
