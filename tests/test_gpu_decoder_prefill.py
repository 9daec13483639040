"""The prompt as one pass (QuantDecoder.prefill: tensor-core linears over all positions, cq_rope_prefill,
cq_flash_attention) against the same prompt fed token by token through the decode path and against the CPU oracle.

The decode path is the tighter statement (1e-3 vs the oracle, tested elsewhere); the one-pass prompt adds the f16
roundings of its attention operands and, in CQ_ACT_F16, of its linears, so its logits are held to 5e-3 of the
oracle's and the KV caches it leaves behind to 2e-3 of the decode path's (bit-equal in the rotary arithmetic itself:
the differences come from the inputs of later layers).  Decoding continues from the state it leaves."""
import numpy as np
import pytest

from helpers import rel_err
from oracle import oracle_c as oc
from oracle.decoder_np import OracleDecoder

pytestmark = pytest.mark.gpu


def build(device, cfg, seed):
    from candy_b200.decoder import QuantDecoder, rope_tables
    model = QuantDecoder(device, cfg, seed=seed, batch=1, qtype=oc.Q4_0, order=0)
    layers = [{k: L[k].data() for k in ("wqkv", "wo", "wgu", "wdown")} for L in model.layers]
    cos, sin = rope_tables(cfg)
    embed = model.embed.data().reshape(cfg.vocab, cfg.dim)
    ref = OracleDecoder(cfg, oc.Q4_0, 0, layers, embed=embed, wout=model.wout.data(), cos=cos, sin=sin)
    return model, ref


@pytest.mark.parametrize("actmode,bar", [(2, 5e-3), (0, 3e-3)])  # CQ_ACT_F16 linears / CQ_ACT_F32 linears (int8 plane kernel)
@pytest.mark.parametrize("T", [1, 37, 140])
def test_prompt_in_one_pass(device, T, actmode, bar):
    from candy_b200.decoder import DecoderConfig
    cfg = DecoderConfig(n_layers=2, dim=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=1000, max_ctx=160)
    model, ref = build(device, cfg, seed=5)
    rng = np.random.default_rng(T)
    tokens = rng.integers(0, cfg.vocab, size=T)
    # token by token through the decode path: logits of the last position, caches of every position
    for pos, tok in enumerate(tokens):
        model.set_state(np.array([tok], dtype=np.uint32), pos)
        model.step()
        want = ref.step(int(tok), pos)
    device.synchronize()
    step_logits = model.read_logits()[0].copy()
    kv = cfg.n_kv_heads * cfg.head_dim
    step_k = [L["k"].data().reshape(cfg.max_ctx, kv)[:T].copy() for L in model.layers]
    step_v = [L["v"].data().reshape(cfg.max_ctx, kv)[:T].copy() for L in model.layers]
    assert rel_err(step_logits, want) <= 1e-3
    # the same prompt in one pass, on a fresh sequence of the same model
    for L in model.layers:
        device._check(device._lib.cq_memset(device.ctx, L["k"].ptr, 0, 4 * cfg.max_ctx * kv), "clear")
        device._check(device._lib.cq_memset(device.ctx, L["v"].ptr, 0, 4 * cfg.max_ctx * kv), "clear")
    model.set_state(np.array([0], dtype=np.uint32), 0)
    model.prefill(tokens, actmode=actmode)
    device.synchronize()
    got = model.read_logits()[0]
    assert rel_err(got, want) <= bar, rel_err(got, want)
    assert rel_err(got, step_logits) <= bar
    for l, L in enumerate(model.layers):
        k = L["k"].data().reshape(cfg.max_ctx, kv)
        v = L["v"].data().reshape(cfg.max_ctx, kv)
        if l == 0 and actmode == 0:  # first layer, same linear arithmetic: only the batch route of the linear differs
            assert rel_err(k[:T], step_k[0]) <= 1e-4 and rel_err(v[:T], step_v[0]) <= 1e-4
        assert rel_err(k[:T], step_k[l]) <= 2e-3 and rel_err(v[:T], step_v[l]) <= 2e-3
        assert not k[T:].any() and not v[T:].any()  # nothing beyond the prompt was written
    # decoding continues from the state the pass left: position T, next token = arg-max of its logits
    assert model.guard.pos == T
    assert int(model.read_ids()[0]) == int(np.argmax(got))
    if T < cfg.max_ctx - 1:
        nxt = int(model.read_ids()[0])
        model.step()
        device.synchronize()
        want_next = ref.step(nxt, T)
        assert rel_err(model.read_logits()[0], want_next) <= bar


def test_prompt_in_one_pass_bf16_attention(device):
    """bf16 attention operands (8 mantissa bits): the logits stay within 2e-2 of the oracle's."""
    from candy_b200.decoder import DecoderConfig
    cfg = DecoderConfig(n_layers=2, dim=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=1000, max_ctx=160)
    model, ref = build(device, cfg, seed=6)
    tokens = np.random.default_rng(9).integers(0, cfg.vocab, size=75)
    for pos, tok in enumerate(tokens):
        want = ref.step(int(tok), pos)
    model.prefill(tokens, bf16=True)
    device.synchronize()
    assert rel_err(model.read_logits()[0], want) <= 2e-2


def test_second_prompt_continues_the_sequence(device):
    """A prompt, a few decoded tokens, then another prompt in one pass: the second pass attends to the cached keys and
    values of everything before it (cast to f16) and leaves the state a token-by-token run would have."""
    from candy_b200.decoder import DecoderConfig
    cfg = DecoderConfig(n_layers=2, dim=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=1000, max_ctx=200)
    model, ref = build(device, cfg, seed=7)
    rng = np.random.default_rng(3)
    first, second = rng.integers(0, cfg.vocab, size=50), rng.integers(0, cfg.vocab, size=90)
    pos = 0
    for tok in first:
        ref.step(int(tok), pos)
        pos += 1
    model.prefill(first)
    forced = rng.integers(0, cfg.vocab, size=5)
    for tok in forced:  # a few decode steps, teacher-forced
        model.set_state(np.array([tok], dtype=np.uint32), pos)
        model.step()
        ref.step(int(tok), pos)
        pos += 1
    for tok in second:
        want = ref.step(int(tok), pos)
        pos += 1
    model.prefill(second)
    device.synchronize()
    assert model.guard.pos == pos
    assert rel_err(model.read_logits()[0], want) <= 5e-3


def test_prefill_refuses_what_it_does_not_serve(device):
    from candy_b200.decoder import DecoderConfig
    cfg = DecoderConfig(n_layers=1, dim=256, n_heads=2, n_kv_heads=1, head_dim=128, ffn=512, vocab=100, max_ctx=16)
    model, _ = build(device, cfg, seed=1)
    with pytest.raises(ValueError):
        model.prefill(np.arange(17))  # runs past max_ctx
    model.set_state(np.array([1], dtype=np.uint32), 14)
    with pytest.raises(ValueError):
        model.prefill(np.arange(4))  # 14 + 4 positions do not fit in 16
    with pytest.raises(ValueError):
        model.prefill(np.array([], dtype=np.uint32))


@pytest.mark.parametrize("bf16", [False, True])
def test_rope_prefill_equals_the_decode_rotary_step_position_by_position(device, bf16):
    """cq_rope_prefill writes, for every prompt position, exactly the cache rows cq_rope_store_kv writes for that
    position (bit for bit), and its 16-bit copies are the round-to-nearest-even images of the rotated f32 values."""
    import ctypes as C
    from candy_b200.backend import RawBuffer
    from candy_b200.decoder import DecoderConfig, rope_tables
    from oracle import attention_np as an
    lib, ctx = device._lib, device.ctx
    T, nq, nkv, hd, max_ctx, pos0 = 19, 4, 2, 128, 64, 7
    cfg = DecoderConfig(n_layers=1, dim=nq * hd, n_heads=nq, n_kv_heads=nkv, head_dim=hd, ffn=256, vocab=10, max_ctx=max_ctx)
    cos, sin = rope_tables(cfg)
    dcos, dsin = device.storage_from_slice(cos), device.storage_from_slice(sin)
    rng = np.random.default_rng(17)
    row = (nq + 2 * nkv) * hd
    qkv = rng.standard_normal((T, row)).astype(np.float32)
    dqkv = device.storage_from_slice(qkv)
    kc, vc = device.zeros(max_ctx * nkv * hd), device.zeros(max_ctx * nkv * hd)
    q16, k16, v16 = RawBuffer(device, 2 * T * nq * hd), RawBuffer(device, 2 * T * nkv * hd), RawBuffer(device, 2 * T * nkv * hd)
    assert lib.cq_rope_prefill(ctx, dqkv.ptr, T, nq, nkv, hd, dcos.ptr, dsin.ptr, pos0, kc.ptr, vc.ptr, max_ctx, q16.ptr, k16.ptr, v16.ptr,
                               1 if bf16 else 0) == 0
    device.synchronize()
    got_k, got_v = kc.data().reshape(max_ctx, nkv * hd), vc.data().reshape(max_ctx, nkv * hd)
    # the decode entry, one position at a time, on a copy
    kc2, vc2 = device.zeros(max_ctx * nkv * hd), device.zeros(max_ctx * nkv * hd)
    pos = RawBuffer(device, 4)
    rot_q = np.empty((T, nq * hd), dtype=np.float32)
    for t in range(T):
        one = device.storage_from_slice(qkv[t])
        p = np.array([pos0 + t], dtype=np.int32)
        assert lib.cq_memcpy_h2d(ctx, pos.ptr, p.ctypes.data_as(C.c_void_p), 4) == 0
        assert lib.cq_rope_store_kv(ctx, one.ptr, 1, nq, nkv, hd, dcos.ptr, dsin.ptr, pos.ptr, kc2.ptr, vc2.ptr, max_ctx) == 0
        device.synchronize()
        rot_q[t] = one.data()[: nq * hd]
    want_k, want_v = kc2.data().reshape(max_ctx, nkv * hd), vc2.data().reshape(max_ctx, nkv * hd)
    assert np.array_equal(got_k.view(np.uint32), want_k.view(np.uint32))
    assert np.array_equal(got_v.view(np.uint32), want_v.view(np.uint32))

    def bits16(a):
        return an.to_bf16_bits(a) if bf16 else a.astype(np.float16).view(np.uint16)

    assert np.array_equal(q16.data().view(np.uint16).reshape(T, nq * hd), bits16(rot_q))
    assert np.array_equal(k16.data().view(np.uint16).reshape(T, nkv * hd), bits16(want_k[pos0:pos0 + T]))
    assert np.array_equal(v16.data().view(np.uint16).reshape(T, nkv * hd), bits16(want_v[pos0:pos0 + T]))
    # the casts: 16 -> 32 exact, 32 -> 16 round to nearest even
    back = device.alloc(T * nkv * hd)
    assert lib.cq_cast16_to_f32(ctx, k16.ptr, T * nkv * hd, 1 if bf16 else 0, back.ptr) == 0
    again = RawBuffer(device, 2 * T * nkv * hd)
    assert lib.cq_cast_f32_to_16(ctx, kc.ptr.value + 4 * pos0 * nkv * hd, T * nkv * hd, 1 if bf16 else 0, again.ptr) == 0
    device.synchronize()
    k_bits = k16.data().view(np.uint16)
    want_back = an.from_bf16_bits(k_bits) if bf16 else k_bits.view(np.float16).astype(np.float32)
    assert np.array_equal(back.data().view(np.uint32), want_back.view(np.uint32))
    assert np.array_equal(again.data().view(np.uint16), k_bits)
    # positions outside the cache are refused on the host
    assert lib.cq_rope_prefill(ctx, dqkv.ptr, T, nq, nkv, hd, dcos.ptr, dsin.ptr, max_ctx - T + 1, kc.ptr, vc.ptr, max_ctx, q16.ptr, k16.ptr, v16.ptr, 0) != 0
