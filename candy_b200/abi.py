"""ctypes binding of ``libcandyq.so`` -- one Python function per C entry point.

This is the same surface a cgo file binds (see ``include/candyq.h``); it adds nothing but
argument marshalling and turning a non-zero status into :class:`CandyqError`.  If the
shared library is missing the import of this module fails: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# CANDYQ_LIBRARY points the binding at another build of the same library (profiling builds).
LIB_PATH = Path(os.environ.get("CANDYQ_LIBRARY") or Path(__file__).resolve().parent / "libcandyq.so")

OK = 0
ERR_INVALID_ARG, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_NOMEM, ERR_TOO_LARGE = -1, -2, -3, -4, -5, -6
Q4_0, Q4_1, Q5_0, Q5_1, Q8_0 = 2, 3, 6, 7, 8
ORDER_GO_INTERLEAVED, ORDER_GGML_SPLIT = 0, 1
ACT_F32, ACT_Q8_1, ACT_F16 = 0, 1, 2
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 10, 11, 12, 13, 14
BLOCK_BYTES = {Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34}
K_BLOCK_BYTES = {Q2_K: 84, Q3_K: 110, Q4_K: 144, Q5_K: 176, Q6_K: 210}  # per 256 values
Q8_1_BYTES = 36


class CandyqError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        text = lib().cq_status_string(status).decode()
        super().__init__(f"{where}: {text}" + (f": {detail}" if detail else ""))


_lib = None

CQ_OK, CQ_ERR_INVALID_ARG, CQ_ERR_CUDA, CQ_ERR_UNSUPPORTED, CQ_ERR_TIMEOUT, CQ_ERR_NOMEM, CQ_ERR_TOO_LARGE = 0, -1, -2, -3, -4, -5, -6
_vp, _i64, _int, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t

# name -> argtypes (every entry returns cq_status unless listed in _OTHER_RESTYPE)
SIGNATURES = {
    "cq_device_count": [C.POINTER(C.c_int)],
    "cq_ctx_create": [_int, C.POINTER(_vp)],
    "cq_ctx_destroy": [_vp],
    "cq_ctx_set_stream": [_vp, _vp],
    "cq_ctx_set_option": [_vp, C.c_char_p, _i64],
    "cq_reserve": [_vp, _sz],
    "cq_invalidate_weight_cache": [_vp, _vp, _sz],
    "cq_malloc": [_vp, _sz, C.POINTER(_vp)],
    "cq_free": [_vp, _vp],
    "cq_malloc_host": [_vp, _sz, C.POINTER(_vp)],
    "cq_free_host": [_vp, _vp],
    "cq_memset": [_vp, _vp, _int, _sz],
    "cq_memcpy_h2d": [_vp, _vp, _vp, _sz],
    "cq_memcpy_d2h": [_vp, _vp, _vp, _sz],
    "cq_memcpy_d2d": [_vp, _vp, _vp, _sz],
    "cq_synchronize": [_vp],
    "cq_quantize_rows": [_vp, _int, _int, _vp, _i64, _i64, _vp],
    "cq_dequantize": [_vp, _int, _int, _vp, _i64, _vp],
    "cq_quantize_q8_1": [_vp, _vp, _i64, _i64, _i64, _vp],
    "cq_qmatmul": [_vp, _int, _int, _int, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64],
    "cq_qlinear": [_vp, _int, _int, _int, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _i64],
    "cq_qmatmul_host": [_vp, _int, _int, _int, _vp, _i64, _i64, _vp, _i64, _vp],
    "cq_qmatmul_q8_1_static": [_vp, _int, _int, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64],
    "cq_rand_normal": [_vp, _vp, _i64, C.c_float, C.c_float, C.c_uint64],
    "cq_rand_uniform": [_vp, _vp, _i64, C.c_float, C.c_float, C.c_uint64],
    "cq_rmsnorm": [_vp, _vp, _vp, _i64, _i64, C.c_float, _vp],
    "cq_add_rmsnorm": [_vp, _vp, _vp, _vp, _i64, _i64, C.c_float, _vp],
    "cq_rope_store_kv": [_vp, _vp, _i64, _int, _int, _int, _vp, _vp, _vp, _vp, _vp, _int],
    "cq_rope_prefill": [_vp, _vp, _i64, _int, _int, _int, _vp, _vp, _int, _vp, _vp, _int, _vp, _vp, _vp, _int],
    "cq_cast16_to_f32": [_vp, _vp, _i64, _int, _vp],
    "cq_cast_f32_to_16": [_vp, _vp, _i64, _int, _vp],
    "cq_decode_attention": [_vp, _vp, _i64, _int, _int, _int, _vp, _vp, _vp, _int, _vp, _vp],
    "cq_decode_attention_rope": [_vp, _vp, _i64, _int, _int, _int, _vp, _vp, _vp, _vp, _vp, _int, _vp, _vp],
    "cq_silu_mul": [_vp, _vp, _i64, _i64, _vp, _i64],
    "cq_silu_mul_pairs": [_vp, _vp, _i64, _i64, _vp, _i64],
    "cq_argmax": [_vp, _vp, _i64, _i64, _vp],
    "cq_embedding": [_vp, _vp, _i64, _i64, _vp, _i64, _vp],
    "cq_add_int": [_vp, _vp, _int],
    "cq_comm_create": [_vp, _int, _int, _i64, C.POINTER(_vp), _vp],
    "cq_comm_connect": [_vp, _vp, _vp],
    "cq_comm_destroy": [_vp, _vp],
    "cq_qmatmul_push": [_vp, _vp, _int, _int, _int, _vp, _i64, _i64, _i64, _vp, _i64],
    "cq_qlinear_fused": [_vp, _int, _int, _vp, _vp, _vp, C.c_float, _vp, _i64, _i64, _vp, _i64, _int, _vp, _i64],
    "cq_add_rmsnorm_reduce": [_vp, _vp, _int, _vp, _vp, _i64, _i64, C.c_float, _vp],
    "cq_decoder_create": [_vp, _vp, C.POINTER(_vp)],
    "cq_decoder_step": [_vp, _vp, _vp, _vp],
    "cq_decoder_destroy": [_vp, _vp],
    "cq_flash_attention": [_vp] + [_vp] * 8 + [C.c_uint32] * 18 + [C.c_float] + [C.c_uint32] * 4 + [_int] * 5 + [C.c_float],
    "cq_tp_unique_id": [_vp, _vp],
    "cq_tp_init": [_vp, _int, _int, _vp, _sz, C.POINTER(_vp)],
    "cq_tp_destroy": [_vp, _vp],
    "cq_allreduce_sum_f32": [_vp, _vp, _vp, _i64],
    "cq_tp_wait": [_vp, _vp, _int],
    "cq_capture_begin": [_vp],
    "cq_capture_end": [_vp, C.POINTER(_vp)],
    "cq_graph_launch": [_vp, _vp],
    "cq_graph_destroy": [_vp, _vp],
    "cq_measure_i8_mma_peak": [_vp, _int, C.POINTER(C.c_double)],
    "cq_timer_start": [_vp],
    "cq_timer_stop": [_vp, C.POINTER(C.c_float)],
}
_OTHER_RESTYPE = {
    "run_mha": (None, [_vp] * 8 + [C.c_uint32] * 18 + [C.c_float] + [C.c_uint32] * 4 + [_int] * 5 + [C.c_float]),
    "cq_run_mha_last_status": (C.c_int32, []),
    "cq_decoder_logits": (_vp, [_vp]),
    "cq_status_string": (C.c_char_p, [C.c_int32]),
    "cq_last_error": (C.c_char_p, [_vp]),
    "cq_version": (C.c_char_p, []),
    "cq_blocks_bytes": (_sz, [_int, _i64, _i64]),
    "cq_decode_attention_scratch_floats": (_sz, [_i64, _int, _int, _int]),
}


class DecoderDesc(C.Structure):
    """cq_decoder_desc of include/candyq.h."""
    _fields_ = [(n, C.c_int) for n in ("n_layers", "dim", "n_heads", "n_kv_heads", "head_dim", "ffn", "ffn_pad", "vocab", "max_ctx")] + \
               [("eps", C.c_float), ("qtype", C.c_int), ("order", C.c_int)] + \
               [(n, C.POINTER(C.c_void_p)) for n in ("wqkv", "wo", "wgu", "wdown", "attn_norm", "ffn_norm", "k_cache", "v_cache")] + \
               [(n, C.c_void_p) for n in ("embed", "wout", "final_norm", "cos_table", "sin_table")]


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m candy_b200.build` (needs nvcc). "
                "candy_b200 has no CPU or eager fallback.")
        handle = C.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here means header and library disagree
            fn.restype = C.c_int32
            fn.argtypes = argtypes
        for name, (restype, argtypes) in _OTHER_RESTYPE.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(ctx, status: int, where: str) -> None:
    if status != OK:
        detail = lib().cq_last_error(ctx).decode() if ctx else ""
        raise CandyqError(status, where, detail)


def version() -> str:
    return lib().cq_version().decode()


def device_count() -> int:
    n = C.c_int(0)
    lib().cq_device_count(C.byref(n))
    return n.value
