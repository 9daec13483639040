"""The decoder step (embedding, RMSNorm, quantized linears, RoPE, KV cache, decode attention,
SiLU*mul, argmax) against the NumPy/C oracle of candy's CPU arithmetic, teacher-forced so that a
near-tie in the flat logits of a random-init model cannot fork the two token streams: the logits
of every position are compared under the 1e-3 bar, token agreement is reported on top."""
import numpy as np
import pytest

from helpers import REL_TOL, rel_err
from oracle import oracle_c as oc
from oracle.decoder_np import OracleDecoder

pytestmark = pytest.mark.gpu


def build(device, cfg, seed, qtype=oc.Q4_0, order=0):
    from candy_b200.decoder import QuantDecoder, rope_tables
    model = QuantDecoder(device, cfg, seed=seed, batch=1, qtype=qtype, order=order)
    layers = [{k: L[k].data() for k in ("wqkv", "wo", "wgu", "wdown")} for L in model.layers]
    cos, sin = rope_tables(cfg)
    embed = model.embed.data().reshape(cfg.vocab, cfg.dim)
    ref = OracleDecoder(cfg, qtype, order, layers, embed=embed, wout=model.wout.data(), cos=cos, sin=sin)
    return model, ref


@pytest.mark.parametrize("qtype,order", [(oc.Q4_0, 0), (oc.Q4_0, 1), (oc.Q8_0, 0)])
def test_small_decoder_logits_teacher_forced(device, qtype, order):
    from candy_b200.decoder import DecoderConfig
    cfg = DecoderConfig(n_layers=2, dim=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=1000, max_ctx=160)
    model, ref = build(device, cfg, seed=2, qtype=qtype, order=order)
    rng = np.random.default_rng(2)
    tokens = rng.integers(0, cfg.vocab, size=140)  # crosses the 128-key chunk boundary of the attention kernel
    agree = 0
    for pos, tok in enumerate(tokens):
        model.set_state(np.array([tok], dtype=np.uint32), pos)
        model.step()
        device.synchronize()
        if pos in (0, 1, 2, 3, 7, 31, 127, 128, 129, 139):
            want = ref.step(int(tok), pos)
            got = model.read_logits()[0]
            assert rel_err(got, want) <= REL_TOL, f"position {pos}"
            agree += int(model.read_ids()[0] == int(np.argmax(want)))
        else:
            ref.step(int(tok), pos)
    assert agree >= 8  # greedy tokens agree except where the two top logits are within rounding


def test_batch_of_four_rows_takes_the_tensor_core_linears(device):
    """A batch of four sequences: the linears run as one narrow tensor-core launch each (f16
    activations); every row's logits stay under the 1e-3 bar against its own oracle stream."""
    from candy_b200.decoder import DecoderConfig, QuantDecoder, rope_tables
    cfg = DecoderConfig(n_layers=2, dim=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=1000, max_ctx=48)
    batch = 4
    model = QuantDecoder(device, cfg, seed=3, batch=batch)
    assert not model.fuse and model.actmode == 2
    layers = [{k: L[k].data() for k in ("wqkv", "wo", "wgu", "wdown")} for L in model.layers]
    cos, sin = rope_tables(cfg)
    embed = model.embed.data().reshape(cfg.vocab, cfg.dim)
    refs = [OracleDecoder(cfg, oc.Q4_0, 0, layers, embed=embed, wout=model.wout.data(), cos=cos, sin=sin) for _ in range(batch)]
    rng = np.random.default_rng(4)
    tokens = rng.integers(0, cfg.vocab, size=(40, batch))
    for pos in range(tokens.shape[0]):
        model.set_state(tokens[pos].astype(np.uint32), pos)
        model.step()
        device.synchronize()
        got = model.read_logits()
        for b in range(batch):
            want = refs[b].step(int(tokens[pos, b]), pos)
            if pos in (0, 1, 5, 33, 39):
                assert rel_err(got[b], want) <= REL_TOL, f"row {b} position {pos}"


def test_greedy_decode_graph_replay_matches_stepwise(device):
    """The captured one-step graph (token id and position on the device) replayed n times gives
    the same token stream as n individual steps."""
    from candy_b200.decoder import DecoderConfig, QuantDecoder
    cfg = DecoderConfig(n_layers=2, dim=512, n_heads=4, n_kv_heads=4, head_dim=128, ffn=1024, vocab=777, max_ctx=64)
    model = QuantDecoder(device, cfg, seed=5)
    model.set_state(np.array([3], dtype=np.uint32), 0)
    a = []
    for _ in range(20):
        model.step()
        device.synchronize()
        a.append(int(model.read_ids()[0]))
    model.set_state(np.array([3], dtype=np.uint32), 0)
    model.step()  # first launch outside capture
    device.synchronize()
    model.set_state(np.array([3], dtype=np.uint32), 0)
    g = model.capture(1)
    b = []
    for _ in range(20):
        model.replay(g)
        device.synchronize()
        b.append(int(model.read_ids()[0]))
    assert a == b


def test_7b_width_two_layers(device):
    from candy_b200.decoder import DecoderConfig
    cfg = DecoderConfig(n_layers=2, dim=4096, n_heads=32, n_kv_heads=32, head_dim=128, ffn=11008, vocab=32000, max_ctx=16)
    model, ref = build(device, cfg, seed=2)
    tokens = [11, 31999, 5, 1234]
    for pos, tok in enumerate(tokens):
        model.set_state(np.array([tok], dtype=np.uint32), pos)
        model.step()
        device.synchronize()
        want = ref.step(tok, pos)
        assert rel_err(model.read_logits()[0], want) <= REL_TOL


# ---- decode attention, operator level: every kernel route against the softmax(q.K^T/sqrt(d)).V of
# candy's CPU path (reduce.go:2855-2879 restated in oracle.decoder_np.softmax) --------------------------
@pytest.mark.parametrize("batch,nq,nkv,hd,max_ctx,pos", [
    (1, 8, 8, 128, 96, 40),       # one query head per kv head: chunk kernel
    (2, 16, 2, 128, 300, 257),    # groups of eight: split-context kernel, ragged last chunk
    (3, 8, 4, 128, 64, 0),        # a single key
    (2, 6, 3, 64, 80, 79),        # head_dim != 128: generic kernel
    (1, 64, 8, 128, 2048, 2047),  # the 70B-shape group at full context
])
def test_decode_attention_routes(device, batch, nq, nkv, hd, max_ctx, pos):
    import ctypes as C
    from candy_b200 import abi
    from oracle.decoder_np import softmax
    lib, ctx = device._lib, device.ctx
    rng = np.random.default_rng(batch * 1000 + nq + pos)
    qkv = rng.standard_normal((batch, (nq + 2 * nkv) * hd), dtype=np.float32)
    kc = rng.standard_normal((batch, max_ctx, nkv, hd), dtype=np.float32)
    vc = rng.standard_normal((batch, max_ctx, nkv, hd), dtype=np.float32)
    want = np.zeros((batch, nq, hd), dtype=np.float32)
    G = nq // nkv
    for b in range(batch):
        for h in range(nq):
            q = qkv[b, h * hd:(h + 1) * hd]
            s = (kc[b, :pos + 1, h // G, :] @ q) / np.float32(np.sqrt(hd))
            want[b, h] = softmax(s.astype(np.float32)) @ vc[b, :pos + 1, h // G, :]
    d_qkv, d_k, d_v = device.storage_from_slice(qkv), device.storage_from_slice(kc), device.storage_from_slice(vc)
    d_pos = device.upload_bytes(np.array([pos], dtype=np.int32))
    scratch = device.alloc(lib.cq_decode_attention_scratch_floats(batch, nq, hd, max_ctx))
    out = device.alloc(batch * nq * hd)
    for variant in (0, 1):
        device.set_option("attn_variant", variant)
        try:
            abi.check(ctx, lib.cq_decode_attention(ctx, d_qkv.ptr, batch, nq, nkv, hd, d_pos.ptr, d_k.ptr, d_v.ptr, max_ctx, scratch.ptr, out.ptr), "attention")
            got = out.data().reshape(batch, nq, hd)
        finally:
            device.set_option("attn_variant", 0)
        assert rel_err(got, want) < 2e-5, f"variant {variant}"


# ---- one decode linear with its neighbours fused in (cq_qlinear_fused) -----------------------------------
@pytest.mark.parametrize("m,k,n,epilogue,with_delta,with_norm", [
    (1, 4096, 12288, 0, True, True),     # QKV-like
    (1, 4096, 22016, 1, True, True),     # gate/up with the pairing epilogue
    (3, 4096, 512, 1, True, True),       # several rows, few output rows
    (1, 8192, 7168, 1, True, True),      # 70B-shape shard: the prologue would crowd the ring -> refused, caller falls back
    (1, 8192, 7168, 1, False, False),    # ... and fuses only the epilogue
    (1, 11008, 4096, 0, True, True),     # k = 11008: the per-thread activation set-up
    (2, 1024, 2048, 0, False, True),     # norm without the residual add
    (1, 4096, 4096, 0, True, False),     # add only
])
def test_fused_linear_matches_separate_operators_and_oracle(device, m, k, n, epilogue, with_delta, with_norm):
    import ctypes as C
    from candy_b200 import abi
    from candy_b200.backend import QStorage
    from oracle.decoder_np import silu
    lib, ctx = device._lib, device.ctx
    rng = np.random.default_rng(m + k + n + epilogue)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    x = rng.standard_normal((m, k), dtype=np.float32)
    delta = rng.standard_normal((m, k), dtype=np.float32) * np.float32(0.3)
    alpha = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    eps = 1e-5
    blocks = oc.quantize(oc.Q4_0, 0, w)
    qs = QStorage.from_blocks(device, oc.Q4_0, 0, n, k, blocks)
    d_x, d_delta, d_alpha = device.storage_from_slice(x), device.storage_from_slice(delta), device.storage_from_slice(alpha)
    d_xout = device.alloc(m * k)
    n_out = n // 2 if epilogue else n
    d_y = device.alloc(m * n_out)
    st = lib.cq_qlinear_fused(ctx, oc.Q4_0, 0, d_x.ptr, d_delta.ptr if with_delta else None, d_alpha.ptr if with_norm else None, eps,
                              d_xout.ptr if (with_delta or with_norm) else None, m, k, qs.buf.ptr, n, epilogue, d_y.ptr, n_out)
    if k == 8192 and (with_delta or with_norm):
        assert st == abi.CQ_ERR_UNSUPPORTED  # documented: the caller issues the separate operators
        return
    abi.check(ctx, st, "fused linear")
    got = d_y.data().reshape(m, n_out)
    xs = x + delta if with_delta else x
    if with_delta or with_norm:
        np.testing.assert_array_equal(d_xout.data().reshape(m, k), xs.astype(np.float32))
    xn = xs
    if with_norm:
        ms = (xs.astype(np.float64) ** 2).mean(axis=1, keepdims=True)
        xn = (xs / np.sqrt(ms + eps) * alpha).astype(np.float32)
    t = oc.qmatmul(oc.Q4_0, 0, xn, blocks, n, nthreads=8)
    want = (silu(t[:, 0::2]) * t[:, 1::2]) if epilogue else t
    assert rel_err(got, want) < 1e-4
    assert rel_err(got, want) <= REL_TOL


def test_decoder_fused_and_unfused_agree(device):
    """The same model stepped with fused linears and with the separate operators: same logits (norm sums differ in order only)."""
    from candy_b200.decoder import DecoderConfig, QuantDecoder
    cfg = DecoderConfig(n_layers=2, dim=1024, n_heads=8, n_kv_heads=4, head_dim=128, ffn=2816, vocab=2000, max_ctx=32)
    outs = []
    for fuse in (True, False):
        model = QuantDecoder(device, cfg, seed=5, fuse=fuse)
        assert model.fuse == fuse
        ids = [3, 77, 1999, 5, 1024]
        logits = []
        for pos, tok in enumerate(ids):
            model.set_state(np.array([tok], dtype=np.uint32), pos)
            model.step()
            logits.append(model.read_logits().copy())
        outs.append(np.stack(logits))
        del model
    assert rel_err(outs[0], outs[1]) < 5e-5


@pytest.mark.parametrize("batch,nq,nkv,hd,max_ctx,pos", [
    (1, 8, 8, 128, 96, 40), (2, 16, 2, 128, 300, 257), (3, 8, 4, 128, 64, 0), (2, 6, 3, 64, 80, 79), (1, 8, 8, 128, 64, 31), (2, 16, 2, 128, 128, 63),
])
def test_attention_with_fused_rotary_step_equals_the_two_operators(device, batch, nq, nkv, hd, max_ctx, pos):
    """cq_decode_attention_rope against cq_rope_store_kv + cq_decode_attention: same output, same cache rows."""
    from candy_b200 import abi
    lib, ctx = device._lib, device.ctx
    rng = np.random.default_rng(7 * batch + nq + pos)
    qkv = rng.standard_normal((batch, (nq + 2 * nkv) * hd), dtype=np.float32)
    kc = rng.standard_normal((batch, max_ctx, nkv, hd), dtype=np.float32)
    vc = rng.standard_normal((batch, max_ctx, nkv, hd), dtype=np.float32)
    ang = rng.uniform(0, 6.28, size=(max_ctx, hd // 2))
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    d_cos, d_sin = device.storage_from_slice(cos), device.storage_from_slice(sin)
    d_pos = device.upload_bytes(np.array([pos], dtype=np.int32))
    scratch = device.alloc(lib.cq_decode_attention_scratch_floats(batch, nq, hd, max_ctx))
    results = []
    for fused in (False, True):
        for variant in (0, 1):
            d_qkv, d_k, d_v = device.storage_from_slice(qkv), device.storage_from_slice(kc), device.storage_from_slice(vc)
            out = device.alloc(batch * nq * hd)
            device.set_option("attn_variant", variant)
            try:
                if fused:
                    abi.check(ctx, lib.cq_decode_attention_rope(ctx, d_qkv.ptr, batch, nq, nkv, hd, d_cos.ptr, d_sin.ptr, d_pos.ptr, d_k.ptr, d_v.ptr,
                                                                max_ctx, scratch.ptr, out.ptr), "rope+attention")
                else:
                    abi.check(ctx, lib.cq_rope_store_kv(ctx, d_qkv.ptr, batch, nq, nkv, hd, d_cos.ptr, d_sin.ptr, d_pos.ptr, d_k.ptr, d_v.ptr, max_ctx), "rope")
                    abi.check(ctx, lib.cq_decode_attention(ctx, d_qkv.ptr, batch, nq, nkv, hd, d_pos.ptr, d_k.ptr, d_v.ptr, max_ctx, scratch.ptr,
                                                           out.ptr), "attention")
            finally:
                device.set_option("attn_variant", 0)
            results.append((out.data().copy(), d_k.data().reshape(kc.shape)[:, pos].copy(), d_v.data().reshape(vc.shape)[:, pos].copy()))
    ref = results[0]
    for got in results[1:]:
        assert rel_err(got[0], ref[0]) < 2e-6
        np.testing.assert_allclose(got[1], ref[1], rtol=0, atol=1e-6)
        np.testing.assert_array_equal(got[2], ref[2])


def test_7b_full_depth_three_positions(device):
    """BASELINE config 4's model at its full 32 layers (d 4096, 32 heads x 128, SwiGLU 11008, vocab 32000,
    Q4_0): logits of three teacher-forced positions against the CPU oracle, under the 1e-3 bar."""
    from candy_b200.decoder import DecoderConfig
    cfg = DecoderConfig(n_layers=32, dim=4096, n_heads=32, n_kv_heads=32, head_dim=128, ffn=11008, vocab=32000, max_ctx=8)
    model, ref = build(device, cfg, seed=2)
    assert model.fuse  # the fused norm / SiLU linears are the route a 7B decode takes
    for pos, tok in enumerate([17, 31999, 4242]):
        model.set_state(np.array([tok], dtype=np.uint32), pos)
        model.step()
        device.synchronize()
        want = ref.step(tok, pos)
        assert rel_err(model.read_logits()[0], want) <= REL_TOL, f"position {pos}"


@pytest.mark.parametrize("batch", [1, 3, 12])
def test_70b_shape_single_layer(device, batch):
    """One layer of BASELINE config 5's shape (d 8192, 64 q / 8 kv heads x 128, ffn 28672, Q4_0), unsharded,
    at a position inside a noise-filled cache: the residual stream after the layer against the CPU oracle.
    Batch 1 runs the f32-activation GEMVs, batches 3 and 12 the narrow tensor-core linears (f16 operands),
    as the decoder routes them."""
    from candy_b200.decoder import DecoderConfig, QuantDecoder, rope_tables
    from oracle.decoder_np import sharded_layer_step
    cfg = DecoderConfig(n_layers=1, dim=8192, n_heads=64, n_kv_heads=8, head_dim=128, ffn=28672, vocab=0, max_ctx=24, with_head=False)
    lib, ctx = device._lib, device.ctx
    model = QuantDecoder(device, cfg, seed=3, batch=batch)
    L = model.layers[0]
    nkv_floats = batch * cfg.max_ctx * model.kv_dim
    lib.cq_rand_normal(ctx, L["k"].ptr, nkv_floats, 0.0, 1.0, 11)
    lib.cq_rand_normal(ctx, L["v"].ptr, nkv_floats, 0.0, 1.0, 12)
    lib.cq_rand_normal(ctx, model.x.ptr, batch * cfg.dim, 0.0, 1.0, 13)
    pos = 20
    model.set_state(np.zeros(batch, dtype=np.uint32), pos)
    device.synchronize()
    x0 = model.x.data().reshape(batch, cfg.dim).copy()
    kc = L["k"].data().reshape(batch, cfg.max_ctx, model.nkv, cfg.head_dim).copy()
    vc = L["v"].data().reshape(batch, cfg.max_ctx, model.nkv, cfg.head_dim).copy()
    model.step(advance=False)
    device.synchronize()
    got = model.x.data().reshape(batch, cfg.dim) + model.d.data().reshape(batch, cfg.dim)
    cos, sin = rope_tables(cfg)
    blocks = {k: L[k].data() for k in ("wqkv", "wo", "wgu", "wdown")}
    for b in sorted({0, batch - 1}):
        shard = dict(blocks, k=kc[b], v=vc[b], nq=model.nq, nkv=model.nkv, ffn=model.ffn)
        want = sharded_layer_step(cfg, model.qtype, model.order, [shard], x0[b], pos, cos, sin)
        assert rel_err(got[b], want) <= REL_TOL, f"row {b}"


def test_position_outside_the_cache_is_clamped_and_reported(device):
    """A device-resident position at or beyond max_ctx must not index outside the caches: the kernels clamp
    it, flag it, and cq_synchronize answers CQ_ERR_INVALID_ARG; the next call is clean again."""
    from candy_b200 import abi
    from candy_b200.backend import CudaDevice, RawBuffer
    dev = CudaDevice(0)  # its own context: the error word of the shared test device stays untouched
    lib, ctx = dev._lib, dev.ctx
    nq, nkv, hd, max_ctx = 2, 1, 128, 4
    qkv = dev.storage_from_slice(np.ones((nq + 2 * nkv) * hd, dtype=np.float32))
    cos, sin = dev.storage_from_slice(np.ones(max_ctx * hd // 2, dtype=np.float32)), dev.zeros(max_ctx * hd // 2)
    kc, vc = dev.zeros(max_ctx * nkv * hd), dev.zeros(max_ctx * nkv * hd)
    scratch = dev.alloc(lib.cq_decode_attention_scratch_floats(1, nq, hd, max_ctx))
    out = dev.alloc(nq * hd)
    pos = RawBuffer(dev, 4)
    for bad in (max_ctx, 1000000, -3):
        pv = np.array([bad], dtype=np.int32)
        dev._check(lib.cq_memcpy_h2d(ctx, pos.ptr, pv.ctypes.data, 4), "pos")
        assert lib.cq_rope_store_kv(ctx, qkv.ptr, 1, nq, nkv, hd, cos.ptr, sin.ptr, pos.ptr, kc.ptr, vc.ptr, max_ctx) == 0
        assert lib.cq_synchronize(ctx) == abi.ERR_INVALID_ARG
        assert b"max_ctx" in lib.cq_last_error(ctx)
        assert lib.cq_decode_attention_rope(ctx, qkv.ptr, 1, nq, nkv, hd, cos.ptr, sin.ptr, pos.ptr, kc.ptr, vc.ptr, max_ctx, scratch.ptr, out.ptr) == 0
        assert lib.cq_synchronize(ctx) == abi.ERR_INVALID_ARG
    pv = np.array([max_ctx - 1], dtype=np.int32)
    dev._check(lib.cq_memcpy_h2d(ctx, pos.ptr, pv.ctypes.data, 4), "pos")
    assert lib.cq_rope_store_kv(ctx, qkv.ptr, 1, nq, nkv, hd, cos.ptr, sin.ptr, pos.ptr, kc.ptr, vc.ptr, max_ctx) == 0
    assert lib.cq_synchronize(ctx) == 0
    dev.close()
