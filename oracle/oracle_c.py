"""ctypes front end of ``candy_oracle.c`` (test infrastructure; see that file's header).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_oracle as _b

Q4_0, Q4_1, Q5_0, Q5_1, Q8_0 = 2, 3, 6, 7, 8
ORDER_GO, ORDER_SPLIT = 0, 1
BLOCK_BYTES = {Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34}
Q8_1_BYTES = 36
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 10, 11, 12, 13, 14
K_BLOCK_BYTES = {Q2_K: 84, Q3_K: 110, Q4_K: 144, Q5_K: 176, Q6_K: 210}  # per 256 values

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(_b.build_oracle()))
        i64, p = C.c_int64, C.c_void_p
        _lib.co_fp16_to_f32_bits.restype = C.c_uint32
        _lib.co_fp16_to_f32_bits.argtypes = [C.c_uint16]
        _lib.co_f32_to_fp16.restype = C.c_uint16
        _lib.co_f32_to_fp16.argtypes = [C.c_float]
        _lib.co_dequantize_q4_0.argtypes = [p, i64, C.c_int, p]
        _lib.co_dequantize_q8_0.argtypes = [p, i64, p]
        _lib.co_quantize_q4_0.argtypes = [p, i64, C.c_int, p]
        _lib.co_quantize_q8_0.argtypes = [p, i64, p]
        _lib.co_quantize_q8_1.argtypes = [p, i64, p]
        _lib.co_dequantize_q4_1.argtypes = [p, i64, C.c_int, p]
        _lib.co_dequantize_q5.argtypes = [C.c_int, p, i64, p]
        _lib.co_quantize_more.argtypes = [C.c_int, p, i64, C.c_int, p]
        _lib.co_matmul_strided_f32.argtypes = [i64, i64, i64, i64, p, p, p, p, p, p]
        _lib.co_dequantize_k.argtypes = [C.c_int, p, i64, p]
        _lib.co_qmatmul_k.restype = C.c_int
        _lib.co_qmatmul_k.argtypes = [C.c_int, p, i64, i64, i64, p, i64, p, i64, C.c_int]
        for f in (_lib.co_qmatmul, _lib.co_qmatmul_q8_1):
            f.restype = C.c_int
            f.argtypes = [C.c_int, C.c_int, p, i64, i64, i64, p, i64, p, i64, C.c_int]
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def fp16_to_f32_bits(h: int) -> int:
    return int(lib().co_fp16_to_f32_bits(h))


def f32_to_fp16(f: float) -> int:
    return int(lib().co_f32_to_fp16(C.c_float(f)))


def dequantize(qtype: int, order: int, blocks: np.ndarray) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    nb = blocks.size // BLOCK_BYTES[qtype]
    y = np.empty(nb * 32, dtype=np.float32)
    if qtype == Q4_0:
        lib().co_dequantize_q4_0(_ptr(blocks), nb, order, _ptr(y))
    elif qtype == Q4_1:
        lib().co_dequantize_q4_1(_ptr(blocks), nb, order, _ptr(y))
    elif qtype in (Q5_0, Q5_1):
        assert order == ORDER_SPLIT, "the 5-bit formats exist in the split order only"
        lib().co_dequantize_q5(qtype, _ptr(blocks), nb, _ptr(y))
    else:
        lib().co_dequantize_q8_0(_ptr(blocks), nb, _ptr(y))
    return y


def dequantize_k(qtype: int, blocks: np.ndarray) -> np.ndarray:
    """K super-block formats (256 values per block) -> f32."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    nb = blocks.size // K_BLOCK_BYTES[qtype]
    y = np.empty(nb * 256, dtype=np.float32)
    lib().co_dequantize_k(qtype, _ptr(blocks), nb, _ptr(y))
    return y


def qmatmul_k(qtype, x, wblocks, n, nthreads=1) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    wblocks = np.ascontiguousarray(wblocks, dtype=np.uint8).reshape(-1)
    assert wblocks.size == n * (k // 256) * K_BLOCK_BYTES[qtype]
    y = np.empty((m, n), dtype=np.float32)
    rc = lib().co_qmatmul_k(qtype, _ptr(x), m, k, k, _ptr(wblocks), n, _ptr(y), n, nthreads)
    if rc != 0:
        raise ValueError(f"oracle qmatmul_k rejected its arguments (rc={rc})")
    return y


def quantize(qtype: int, order: int, w: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    assert w.size % 32 == 0
    nb = w.size // 32
    out = np.empty(nb * BLOCK_BYTES[qtype], dtype=np.uint8)
    if qtype == Q4_0:
        lib().co_quantize_q4_0(_ptr(w), nb, order, _ptr(out))
    elif qtype in (Q4_1, Q5_0, Q5_1):
        assert qtype == Q4_1 or order == ORDER_SPLIT, "the 5-bit formats exist in the split order only"
        lib().co_quantize_more(qtype, _ptr(w), nb, order, _ptr(out))
    else:
        lib().co_quantize_q8_0(_ptr(w), nb, _ptr(out))
    return out


def quantize_q8_1(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    nb = x.size // 32
    out = np.empty(nb * Q8_1_BYTES, dtype=np.uint8)
    lib().co_quantize_q8_1(_ptr(x), nb, _ptr(out))
    return out


def matmul_strided(a, b, m, n, k, a_strides, b_strides, bsize=1):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    c = np.empty(bsize * m * n, dtype=np.float32)
    as_ = np.asarray(a_strides, dtype=np.int64)
    bs_ = np.asarray(b_strides, dtype=np.int64)
    cs_ = np.asarray([m * n, n, 1], dtype=np.int64)
    lib().co_matmul_strided_f32(bsize, m, n, k, _ptr(a), _ptr(b), _ptr(c), _ptr(as_), _ptr(bs_), _ptr(cs_))
    return c.reshape(bsize, m, n)


def qmatmul(qtype, order, x, wblocks, n, nthreads=1, q8_1=False) -> np.ndarray:
    """y[m,n] = x[m,k] . W[n,k]^T with candy's CPU arithmetic (or, with ``q8_1``, the
    reference CUDA kernels' quantized-activation arithmetic)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    wblocks = np.ascontiguousarray(wblocks, dtype=np.uint8).reshape(-1)
    assert wblocks.size == n * (k // 32) * BLOCK_BYTES[qtype]
    y = np.empty((m, n), dtype=np.float32)
    f = lib().co_qmatmul_q8_1 if q8_1 else lib().co_qmatmul
    rc = f(qtype, order, _ptr(x), m, k, k, _ptr(wblocks), n, _ptr(y), n, nthreads)
    if rc != 0:
        raise ValueError(f"oracle qmatmul rejected its arguments (rc={rc})")
    return y
