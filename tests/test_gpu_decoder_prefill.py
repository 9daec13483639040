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
