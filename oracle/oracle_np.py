"""NumPy twin of ``candy_oracle.c`` (test infrastructure).

Written independently of the C file, in vectorised form, so that the two restatements
check each other: every function here must agree with its C counterpart bit for bit.
Citations are paths inside a gocnn/candy checkout.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0 = 2, 8
ORDER_GO, ORDER_SPLIT = 0, 1
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34}
f32 = np.float32


def _round_half_away(x: np.ndarray) -> np.ndarray:
    """C roundf: nearest, ties away from zero (the +0.5 is done in f64 so it is exact)."""
    x64 = np.asarray(x, dtype=np.float64)
    return np.sign(x64) * np.floor(np.abs(x64) + 0.5)


def fp16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    """tensor/internal/cpu/kernels/quantized.go:149-173, vectorised.  NaN payloads are
    kept (mantissa << 13) exactly as the Go code does, which numpy's own float16 cast
    does not promise, hence the bit arithmetic."""
    h = np.asarray(h, dtype=np.uint16).astype(np.uint32)
    sign = (h & 0x8000) << 16
    exp = (h >> 10) & 0x1F
    mant = h & 0x3FF
    out = np.empty(h.shape, dtype=np.uint32)
    infnan = exp == 31
    zero = (exp == 0) & (mant == 0)
    sub = (exp == 0) & (mant != 0)
    norm = ~(infnan | zero | sub)
    out[infnan] = sign[infnan] | 0x7F800000 | (mant[infnan] << 13)
    out[zero] = sign[zero]
    out[norm] = sign[norm] | ((exp[norm] + 112) << 23) | (mant[norm] << 13)
    if sub.any():
        m = mant[sub].astype(np.int64)
        nbits = np.floor(np.log2(m)).astype(np.int64)  # position of the leading one, 0..9
        shift = 10 - nbits
        e32 = (113 - shift).astype(np.uint32)
        frac = ((m << shift) & 0x3FF).astype(np.uint32)
        out[sub] = sign[sub] | (e32 << 23) | (frac << 13)
    return out.view(np.float32)


def f32_to_fp16_bits(x: np.ndarray) -> np.ndarray:
    """IEEE round-to-nearest-even f32 -> binary16 (what ``half = float`` does in
    tensor/internal/metal/kernels/quantized.metal:4132,4198)."""
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def dequantize(qtype: int, order: int, blocks: np.ndarray) -> np.ndarray:
    bb = BLOCK_BYTES[qtype]
    blk = np.asarray(blocks, dtype=np.uint8).reshape(-1, bb)
    d = fp16_bits_to_f32(blk[:, 0].astype(np.uint16) | (blk[:, 1].astype(np.uint16) << 8))[:, None]
    if qtype == Q8_0:  # quantized.go:131-136
        return (d * blk[:, 2:].view(np.int8).astype(f32)).reshape(-1)
    qs = blk[:, 2:]
    lo = (qs & 0xF).astype(f32) - f32(8)
    hi = (qs >> 4).astype(f32) - f32(8)
    y = np.empty((blk.shape[0], 32), dtype=f32)
    if order == ORDER_GO:  # quantized.go:85-93
        y[:, 0::2] = d * lo
        y[:, 1::2] = d * hi
    else:  # tensor/internal/cuda/kernels/quantized.cu:838-867
        y[:, :16] = d * lo
        y[:, 16:] = d * hi
    return y.reshape(-1)


def quantize(qtype: int, order: int, w: np.ndarray) -> np.ndarray:
    v = np.asarray(w, dtype=f32).reshape(-1, 32)
    nb = v.shape[0]
    out = np.empty((nb, BLOCK_BYTES[qtype]), dtype=np.uint8)
    a = np.abs(v)
    with np.errstate(divide="ignore", invalid="ignore"):
        if qtype == Q8_0:  # quantized.metal:4129-4145
            d = a.max(axis=1) / f32(127)
            idv = np.where(d != 0, f32(1) / d, f32(0)).astype(f32)
            x0 = v * idv[:, None]
            q = _round_half_away(x0).astype(np.int8)
            out[:, 2:] = q.view(np.uint8)
        else:  # quantized.metal:4187-4211
            first = a.argmax(axis=1)  # first index of the largest |v| (strict < in the shader)
            mx = v[np.arange(nb), first]
            d = mx / f32(-8)
            idv = np.where(d != 0, f32(1) / d, f32(0)).astype(f32)
            t = (v * idv[:, None]).astype(f32) + f32(8.5)
            q = np.minimum(np.trunc(t).astype(np.int32), 15).astype(np.uint8)
            if order == ORDER_GO:
                out[:, 2:] = q[:, 0::2] | (q[:, 1::2] << 4)
            else:
                out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    hb = f32_to_fp16_bits(d.astype(f32))
    out[:, 0] = hb & 0xFF
    out[:, 1] = hb >> 8
    return out.reshape(-1)


def qmatmul(qtype: int, order: int, x: np.ndarray, wblocks: np.ndarray, n: int) -> np.ndarray:
    """dequantize (quantized.go:85-93 / :131-136) then the strided naive matmul of
    tensor/internal/cpu/kernels/conv.go:373-389: per output, products and the running
    sum each rounded to f32, l = 0..k-1 in order.  Vectorised over outputs only."""
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    w = dequantize(qtype, order, wblocks).reshape(n, k)
    y = np.zeros((m, n), dtype=f32)
    for i in range(m):
        s = np.zeros(n, dtype=f32)
        for l in range(k):
            s = s + x[i, l] * w[:, l]
        y[i] = s
    return y


def quantize_q8_1(x: np.ndarray) -> np.ndarray:
    """tensor/internal/cuda/kernels/quantized.cu:3521-3558; sum reduced with the
    xor-butterfly pairing of quantized.cu:22-46."""
    v = np.asarray(x, dtype=f32).reshape(-1, 32)
    nb = v.shape[0]
    amax = np.abs(v).max(axis=1)
    s = v.copy()
    idx = np.arange(32)
    for mask in (16, 8, 4, 2, 1):
        s = s + s[:, idx ^ mask]
    d = amax / f32(127)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = (v / d[:, None]).astype(f32)
    q = np.where(amax[:, None] == 0, 0.0, _round_half_away(np.nan_to_num(r)))
    out = np.empty((nb, 36), dtype=np.uint8)
    hd = f32_to_fp16_bits(d)
    hs = f32_to_fp16_bits(s[:, 0])
    out[:, 0], out[:, 1] = hd & 0xFF, hd >> 8
    out[:, 2], out[:, 3] = hs & 0xFF, hs >> 8
    out[:, 4:] = np.nan_to_num(q).astype(np.int8).view(np.uint8)
    return out.reshape(-1)
