"""CPU restatement of scaled-dot-product attention with the contract of the reference's FlashAttention
binding (test infrastructure; never used by the library).

Arithmetic: scores = q . k * softmax_scale; softmax as candy's FastSoftmax (tensor/internal/cpu/kernels/
reduce.go:2855-2879: subtract the row maximum, exponentiate, divide by the sum), here in float64; output =
probabilities . v.  Contract of llm/internal/flashattn (kernels/flash_api.cu:13-147): grouped-query heads
(query head i reads kv head i // (h / h_k)), causal mask aligned to the bottom right (kernels/mask.h:61-62:
key j is visible to row i iff j < i + 1 + seqlen_k - seqlen_q), softmax_lse = max * scale + log(sum)
(kernels/softmax.h:206; +inf and a zero output row when no key is visible).

The reference's own library cannot be built here (its CUTLASS submodule is not in the checkout) and holds no
golden vectors for attention, so this oracle is pinned by hand-derived answers in tests/test_oracle_attention.py.
"""
from __future__ import annotations

import numpy as np


def mha_forward(q, k, v, softmax_scale, causal):
    """q [b, sq, h, d], k / v [b, sk, h_k, d] (any float type) -> out [b, sq, h, d] float64, lse [b, h, sq] float64."""
    q, k, v = (np.asarray(a, dtype=np.float64) for a in (q, k, v))
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    group = h // hk
    out = np.zeros((b, sq, h, d))
    lse = np.full((b, h, sq), np.inf)
    rows = np.arange(sq)[:, None]
    cols = np.arange(sk)[None, :]
    visible = (cols < rows + 1 + sk - sq) if causal else np.ones((sq, sk), dtype=bool)
    for bi in range(b):
        for hi in range(h):
            s = (q[bi, :, hi, :] @ k[bi, :, hi // group, :].T) * softmax_scale
            s = np.where(visible, s, -np.inf)
            m = s.max(axis=1)
            alive = np.isfinite(m)
            e = np.exp(s - np.where(alive, m, 0.0)[:, None])
            tot = e.sum(axis=1)
            p = e / np.where(tot > 0, tot, 1.0)[:, None]
            out[bi, :, hi, :] = p @ v[bi, :, hi // group, :]
            lse[bi, hi, alive] = m[alive] * 1.0 + np.log(tot[alive])
    return out, lse


def to_bf16_bits(a):
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
