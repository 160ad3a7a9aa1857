"""CPU checks: the oracle's known answers read off the reference sources, and the product's host-side
logic (quantiser, RoPE tables, synthetic checkpoints) against the oracle."""
import numpy as np
import pytest
import torch

from oracle import llama_np
from oracle import ops_np as O


def test_int4_lut_matches_reference_table():
    """custom_ops/int4_to_half_custom_op.cpp:139-166: table[2i] = float(char(i) >> 4), table[2i+1] = float(char(i << 4) >> 4)."""
    w = np.arange(256, dtype=np.uint8).view(np.int8).reshape(256, 1)
    out = O.int4_to_half(w, np.ones(256, np.float16), axis=1)         # [2, 256]
    assert out[0, 0x7F] == 7 and out[1, 0x7F] == -1
    assert out[0, 0x80] == -8 and out[1, 0x80] == 0
    assert out[0, 0xF8] == -1 and out[1, 0xF8] == -8
    assert out[0, 0x12] == 1 and out[1, 0x12] == 2
    rt = O.int4_unpack(O.int4_pack(np.arange(-8, 8).reshape(1, 16)))
    assert np.array_equal(rt, np.arange(-8, 8).reshape(1, 16))


def test_kv_cache_fp8_storage_is_the_fp16_cache_of_the_rounded_values():
    """fp8 storage = the fp16 op applied to values that were rounded to E4M3 once, on the way in (kv_cache.cpp:100-104, :183-185)."""
    r = np.random.default_rng(3)
    st8, st16 = O.KVCacheState(), O.KVCacheState()
    p8, p16 = O.KVCachePipelineState(), O.KVCachePipelineState()
    for step in [0, 1, 2, 3, 4, 5, 0, 1]:
        kv = (r.standard_normal((2, 3, 1, 8)) * 2).astype(np.float16)
        rounded = O.f16(O.e4m3_decode(O.cast_fp8(kv, 0.25)) * np.float32(0.25))
        assert np.array_equal(O.kv_cache(st8, step, kv, 4, 2, 1, fp8=True, fp8_scale=0.25), O.kv_cache(st16, step, rounded, 4, 2, 1))
        assert st8.cache.dtype == np.uint8
        assert np.array_equal(O.kv_cache_pipeline(p8, step, kv, 4, 2, 2, 1, fp8=True, fp8_scale=0.25),
                              O.kv_cache_pipeline(p16, step, rounded, 4, 2, 2, 1))


def test_kv_cache_is_shift_right_newest_first():
    st = O.KVCacheState()
    for step in range(5):
        kv = np.full((1, 1, 2), step + 1, np.float16)
        c = O.kv_cache(st, step, kv, 4, 1, 1)
    assert c[0, :, 0].tolist() == [5, 4, 3, 2]       # newest at index 0, oldest dropped at max_len
    c = O.kv_cache(st, 0, np.full((1, 1, 2), 9, np.float16), 4, 1, 1)
    assert c[0, :, 0].tolist() == [9, 0, 0, 0]       # step 0 zeroes the clone (kv_cache.cpp:118-124)


def test_softmax_v3_unstable_equals_stable_in_safe_range():
    x = (np.random.default_rng(0).standard_normal((4, 64)) * 2).astype(np.float32)
    a, b = O.softmax_v3(x, False), O.softmax_v3(x, True)
    np.testing.assert_allclose(a, b, rtol=1e-5)
    np.testing.assert_allclose(a.sum(-1), 1.0, rtol=1e-5)


def test_masked_positions_contribute_exactly_zero():
    """Skipping masked cache slots equals the reference's additive -10000 over a zero tail (Q6)."""
    r = np.random.default_rng(1)
    B, N, L, H, step = 1, 2, 16, 8, 5
    q = r.standard_normal((B, N, 1, H)).astype(np.float16)
    K = np.zeros((B, N, L, H), np.float16); V = np.zeros((B, N, L, H), np.float16)
    K[:, :, : step + 1] = r.standard_normal((B, N, step + 1, H)); V[:, :, : step + 1] = r.standard_normal((B, N, step + 1, H))
    full = O.attention_decode(q, K, V, O.decode_mask(B, L, step), H, "float32")
    short = O.attention_decode(q, K[:, :, : step + 1], V[:, :, : step + 1], np.zeros((B, step + 1), np.float16), H, "float32")
    assert np.array_equal(full, short)
    full16 = O.attention_decode(q, K, V, O.decode_mask(B, L, step), H, "float16")
    short16 = O.attention_decode(q, K[:, :, : step + 1], V[:, :, : step + 1], np.zeros((B, step + 1), np.float16), H, "float16")
    assert np.array_equal(full16, short16)


def test_e4m3_roundtrip_and_saturation():
    t = O.E4M3_TABLE
    finite = np.array([b for b in range(256) if not np.isnan(t[b])], dtype=np.uint8)
    enc = O.e4m3_encode(t[finite])
    assert np.array_equal(t[enc], t[finite])                     # every representable value encodes to itself (-0 -> -0)
    assert t[O.e4m3_encode(np.array([1e6, -1e6], np.float32))].tolist() == [448.0, -448.0]
    # ties to even: 17 is halfway between 16 and 18 (spacing 2) -> 16; 19 -> 20
    assert t[O.e4m3_encode(np.array([17.0, 19.0], np.float32))].tolist() == [16.0, 20.0]
    # agrees with torch's e4m3fn conversion inside the finite range
    x = np.random.default_rng(2).standard_normal(10000).astype(np.float32) * 50
    x = np.clip(x, -448, 448)
    tb = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(x), tb)


def test_beam_search_first_step_and_parent_rule():
    r = np.random.default_rng(3)
    B, beam, V = 2, 3, 50
    logits = r.standard_normal((B, beam, V)).astype(np.float32)
    hyp = np.zeros((B, 6, beam), np.int32); prob = np.zeros((B, beam), np.float32)
    nid, gid, hyp, prob = O.beam_search_step(logits, hyp, prob, 0, beam)
    assert np.array_equal(nid, np.argsort(-logits[:, 0], axis=-1, kind="stable")[:, :beam])
    assert np.array_equal(hyp[:, 0], nid)
    logits2 = r.standard_normal((B, beam, V)).astype(np.float32)
    nid2, gid2, hyp2, prob2 = O.beam_search_step(logits2, hyp, prob, 1, beam)
    for b in range(B):
        for k in range(beam):
            par = gid2[b, k] // beam
            assert hyp2[b, 0, k] == hyp[b, 0, par] and hyp2[b, 1, k] == nid2[b, k]
            assert np.isclose(prob2[b, k], prob[b, par] + logits2[b, par, nid2[b, k]])


def test_norm_ce_single_row_and_multi_row_paths_differ_only_in_statistics():
    r = np.random.default_rng(4)
    x = r.standard_normal((2, 768)).astype(np.float16)
    g = np.ones(768, np.float16); b = np.zeros(768, np.float16)
    multi = O.norm_ce(x, g, b, 1e-5)
    single = np.stack([O.norm_ce(x[i:i + 1], g, b, 1e-5)[0] for i in range(2)])
    assert np.abs(multi.astype(np.float32) - single.astype(np.float32)).max() < 4e-3
    np.testing.assert_allclose(multi.astype(np.float32).std(axis=1), 1.0, atol=2e-2)


def test_product_quantiser_and_tables_match_oracle():
    from poptransformer_b200 import quant
    from poptransformer_b200.llama import rope_tables
    w = torch.randn(32, 512, generator=torch.Generator().manual_seed(0)) * 0.02
    for group in (128, 512):
        p, s = quant.quantize_int4(w, group)
        po, so = O.quantize_int4(w.numpy(), group)
        assert np.array_equal(p.numpy(), po) and np.array_equal(s.numpy().view(np.uint16), so.view(np.uint16))
    sin, cos = rope_tables(768, 128, "cpu")
    so, co = O.llama_rope_tables(768, 128)
    assert np.array_equal(sin.numpy().view(np.uint16), so.view(np.uint16)) and np.array_equal(cos.numpy().view(np.uint16), co.view(np.uint16))
    q8, sc = quant.quantize_fp8(w)
    assert np.array_equal(q8.numpy(), O.e4m3_encode(w.numpy() / np.float32(sc)))


def test_llama_oracle_tp_equals_single_rank_within_tolerance():
    from poptransformer_b200 import synth
    cfgd = dict(n_layer=2, d_model=256, n_head=2, ffn=512, vocab=1000)
    sd = {k: v.numpy() for k, v in synth.llama_state_dict(**cfgd, seed=0, device="cpu", int4_group=0).items()}
    cfg = llama_np.LlamaConfig(**cfgd, max_len=16)
    ids = synth.prompt_ids(1, 4, 16, 1000, 999, seed=0).numpy()
    a = llama_np.LlamaOracle(cfg, sd, 1, tp=1).generate(ids, 10, 999)
    b = llama_np.LlamaOracle(cfg, sd, 1, tp=2).generate(ids, 10, 999)
    assert np.array_equal(a[:, :4], ids[:, :4])
    assert (a == b).mean() > 0.8


def test_c_restatement_matches_numpy_oracle():
    """oracle/c/decode_ref.c (timed CPU baseline) against oracle/llama_np.py on the same weights: the two
    differ only in float32 summation order."""
    from oracle import c_ref
    from poptransformer_b200 import synth
    cfgd = dict(n_layer=2, d_model=256, n_head=2, ffn=512, vocab=1000)
    for group in (128, 0):
        sd = {k: v.numpy() for k, v in synth.llama_state_dict(**cfgd, seed=1, device="cpu", int4_group=group).items()}
        cfg = llama_np.LlamaConfig(**cfgd, max_len=24, group=group)
        ids = synth.prompt_ids(2, 24, 24, 1000, 999, seed=3).numpy()
        a = llama_np.LlamaOracle(cfg, sd, 2)
        b = c_ref.LlamaOracleC(cfg, sd, 2)
        for step in range(24):
            la, _ = a.logits(ids[:, step], step)
            lb, nb = b.logits(ids[:, step], step)
            np.testing.assert_allclose(la.astype(np.float32), lb.astype(np.float32), rtol=1e-2, atol=5e-3, err_msg=f"step {step}")
        ka, kb = a.kv[0][0].cache[0], b.kcache(0)        # layer-0 K cache: same values up to fp16 rounding flips of the matmul sums
        assert (ka.view(np.uint16) == kb.view(np.uint16)).mean() > 0.97
        np.testing.assert_allclose(ka.astype(np.float32), kb.astype(np.float32), rtol=4e-3, atol=1e-3)


def test_gpt2_oracle_matches_plain_fp32_transformer():
    """The step-by-step fp16 restatement of the reference's GPT-2 decode graph (shift-right KV cache, additive mask, NormCE,
    pre-scaled query, tied head) against a plain float32 causal transformer over the whole sequence."""
    import math
    from oracle import gpt2_np
    from poptransformer_b200 import synth
    dims = dict(n_layer=2, d_model=128, n_head=2, vocab=300, n_positions=32)
    T = 12
    sd = {k: v.numpy() for k, v in synth.gpt2_state_dict(**dims, seed=4).items()}
    orc = gpt2_np.GPT2Oracle(gpt2_np.GPT2Config(**dims, max_len=T), sd, 1)
    ids = synth.prompt_ids(1, T, T, dims["vocab"], dims["vocab"] - 1, seed=5).numpy()
    got = np.stack([orc.logits(ids[:, t], t)[0][0].astype(np.float32) for t in range(T)])

    f = lambda k: sd[k].astype(np.float32)
    d, nh = dims["d_model"], dims["n_head"]
    hs = d // nh

    def ln(x, p):
        mu, var = x.mean(-1, keepdims=True), x.var(-1, keepdims=True)
        return (x - mu) / np.sqrt(var + 1e-5) * f(p + ".weight") + f(p + ".bias")

    x = f("transformer.wte.weight")[ids[0]] + f("transformer.wpe.weight")[:T]
    causal = np.triu(np.full((T, T), -np.inf, np.float32), 1)
    for i in range(dims["n_layer"]):
        p = f"transformer.h.{i}."
        qkv = ln(x, p + "ln_1") @ f(p + "attn.c_attn.weight").T + f(p + "attn.c_attn.bias")
        q, k, v = (qkv[:, j * d:(j + 1) * d].reshape(T, nh, hs).transpose(1, 0, 2) for j in range(3))
        s = q @ k.transpose(0, 2, 1) + causal                       # the 1/sqrt(hs) is already in the query weights
        pr = np.exp(s - s.max(-1, keepdims=True))
        pr /= pr.sum(-1, keepdims=True)
        a = (pr @ v).transpose(1, 0, 2).reshape(T, d)
        x = x + a @ f(p + "attn.c_proj.weight").T + f(p + "attn.c_proj.bias")
        h = ln(x, p + "ln_2") @ f(p + "mlp.c_fc.weight").T + f(p + "mlp.c_fc.bias")
        h = 0.5 * h * (1 + np.vectorize(math.erf)(h / math.sqrt(2.0)))
        x = x + h @ f(p + "mlp.c_proj.weight").T + f(p + "mlp.c_proj.bias")
    exp = ln(x, "transformer.ln_f") @ f("transformer.wte.weight").T
    np.testing.assert_allclose(got, exp, rtol=3e-2, atol=3e-2)


def test_chatglm2_rope_is_a_rotation_of_interleaved_pairs():
    """chatglm2/attention.py:98-151 restated: pair i of the first half of a head turns by angle pos * 10000^(-2i/(H/2))."""
    r = np.random.default_rng(31)
    H, L = 128, 50
    sin_t, cos_t = O.chatglm2_rope_tables(L, H)
    x = r.standard_normal((3, 2, 1, H)).astype(np.float16)
    for pos in (0, 1, 17, 49):
        y = O.chatglm2_rope_apply(x, sin_t[pos], cos_t[pos]).astype(np.float32)
        ang = pos * np.array([1.0 / (10000 ** (i / (H // 2))) for i in range(0, H // 2, 2)])
        xe, xo = x[..., 0:H // 2:2].astype(np.float64), x[..., 1:H // 2:2].astype(np.float64)
        np.testing.assert_allclose(y[..., 0:H // 2:2], xe * np.cos(ang) - xo * np.sin(ang), atol=2e-2)
        np.testing.assert_allclose(y[..., 1:H // 2:2], xo * np.cos(ang) + xe * np.sin(ang), atol=2e-2)
        assert np.array_equal(y[..., H // 2:], x[..., H // 2:].astype(np.float32))


def test_chatglm2_oracle_matches_plain_fp32_transformer():
    """The step-by-step fp16 restatement of the reference's ChatGLM2 decode graph (multi-query groups, interleaved RoPE on half of
    each head, RMSNorm, SwiGLU) against a plain float32 causal transformer over the whole sequence."""
    from oracle import chatglm2_np
    from poptransformer_b200 import synth
    dims = dict(n_layer=2, d_model=256, n_head=4, n_group=2, ffn=384, vocab=300)
    T = 10
    sd = {k: (v.numpy() if hasattr(v, "numpy") else v) for k, v in synth.chatglm2_state_dict(**dims, seed=6).items()}
    orc = chatglm2_np.ChatGLM2Oracle(chatglm2_np.ChatGLM2Config(**dims, max_len=T), sd, 1)
    ids = synth.prompt_ids(1, T, T, dims["vocab"], dims["vocab"] - 1, seed=7).numpy()
    got = np.stack([orc.logits(ids[:, t], t)[0][0].astype(np.float32) for t in range(T)])

    f = lambda k: sd[k].astype(np.float32)
    d, N, G = dims["d_model"], dims["n_head"], dims["n_group"]
    hs = d // N
    rms = lambda x, k: x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * f(k)
    ang = np.arange(T)[:, None] * np.array([1.0 / (10000 ** (i / (hs // 2))) for i in range(0, hs // 2, 2)])[None, :]   # [T, hs/4]

    def rope(x):                                   # x [T, heads, hs]
        y = x.copy()
        xe, xo = x[..., 0:hs // 2:2], x[..., 1:hs // 2:2]
        c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        y[..., 0:hs // 2:2], y[..., 1:hs // 2:2] = xe * c - xo * s, xo * c + xe * s
        return y

    x = f("transformer.embedding.word_embeddings.weight")[ids[0]]
    causal = np.triu(np.full((T, T), -np.inf, np.float32), 1)
    for i in range(dims["n_layer"]):
        p = f"transformer.encoder.layers.{i}."
        h = rms(x, p + "input_layernorm.weight")
        q = (h @ f(p + "self_attention.query.weight").T + f(p + "self_attention.query.bias")).reshape(T, N, hs)
        kv = h @ f(p + "self_attention.key_value.weight").T + f(p + "self_attention.key_value.bias")
        k, v = kv[:, : G * hs].reshape(T, G, hs), kv[:, G * hs:].reshape(T, G, hs)
        q, k = rope(q), rope(k)
        k, v = np.repeat(k, N // G, axis=1), np.repeat(v, N // G, axis=1)
        s = np.einsum("tnh,unh->ntu", q, k) / np.sqrt(hs) + causal
        pr = np.exp(s - s.max(-1, keepdims=True))
        pr /= pr.sum(-1, keepdims=True)
        a = np.einsum("ntu,unh->tnh", pr, v).reshape(T, d)
        x = x + a @ f(p + "self_attention.dense.weight").T
        h = rms(x, p + "post_attention_layernorm.weight")
        g = h @ f(p + "mlp.dense_h_to_4h_1.weight").T
        u = h @ f(p + "mlp.dense_h_to_4h_2.weight").T
        x = x + (u * g / (1 + np.exp(-g))) @ f(p + "mlp.dense_4h_to_h.weight").T
    exp = rms(x, "transformer.encoder.final_layernorm.weight") @ f("transformer.output_layer.weight").T
    np.testing.assert_allclose(got, exp, rtol=3e-2, atol=3e-2)


def test_rwkv_oracle_matches_plain_float_recurrence():
    """The fp16 restatement of the reference's RWKV decode graph (token shift, max-shifted WKV states, rescale) against the
    textbook float64 RWKV-4 recurrence with explicit exponential sums."""
    from oracle import rwkv_np
    from poptransformer_b200 import synth
    dims = dict(n_layer=2, d_model=64, ffn=128, vocab=200, rescale_every=1)
    T = 8
    sd = {k: v.numpy() for k, v in synth.rwkv_state_dict(**dims, seed=8).items()}
    orc = rwkv_np.RWKVOracle(rwkv_np.RWKVConfig(**dims, max_len=T), sd, 1)
    ids = synth.prompt_ids(1, T, T, dims["vocab"], dims["vocab"] - 1, seed=9).numpy()
    got = np.stack([orc.logits(ids[:, t])[0][0].astype(np.float64) for t in range(T)])

    f = lambda k: sd[k].astype(np.float64).reshape(sd[k].shape[-2:] if sd[k].ndim > 2 else sd[k].shape)
    d = dims["d_model"]

    def ln(x, p):
        return (x - x.mean()) / np.sqrt(x.var() + 1e-5) * f(p + ".weight") + f(p + ".bias")

    sig = lambda z: 1 / (1 + np.exp(-z))
    prev_a = [np.zeros(d) for _ in range(2)]
    prev_f = [np.zeros(d) for _ in range(2)]
    hist = [[] for _ in range(2)]          # (k, v) history per layer: wkv_t = sum_{i<t} e^{-(t-1-i) w + k_i} v_i + e^{u + k_t} v_t over the same with v = 1
    exp = []
    for t in range(T):
        x = f("rwkv.embeddings.weight")[ids[0, t]]
        for i in range(2):
            p = f"rwkv.blocks.{i}."
            if i == 0:
                x = ln(x, p + "pre_ln")
            h = ln(x, p + "ln1")
            a = p + "attention."
            mix = lambda nm, prev: h * f(a + nm).reshape(-1) + (1 - f(a + nm).reshape(-1)) * prev
            k = f(a + "key.weight") @ mix("time_mix_key", prev_a[i])
            v = f(a + "value.weight") @ mix("time_mix_value", prev_a[i])
            r = sig(f(a + "receptance.weight") @ mix("time_mix_receptance", prev_a[i]))
            prev_a[i] = h
            w, u = np.exp(f(a + "time_decay")), f(a + "time_first")
            num = sum(np.exp(-(len(hist[i]) - 1 - j) * w + kj) * vj for j, (kj, vj) in enumerate(hist[i])) + np.exp(u + k) * v
            den = sum(np.exp(-(len(hist[i]) - 1 - j) * w + kj) for j, (kj, vj) in enumerate(hist[i])) + np.exp(u + k)
            hist[i].append((k, v))
            x = x + f(a + "output.weight") @ (r * num / den)
            h = ln(x, p + "ln2")
            m = p + "feed_forward."
            kk = np.maximum(f(m + "key.weight") @ (h * f(m + "time_mix_key").reshape(-1) + (1 - f(m + "time_mix_key").reshape(-1)) * prev_f[i]), 0) ** 2
            rr = sig(f(m + "receptance.weight") @ (h * f(m + "time_mix_receptance").reshape(-1) + (1 - f(m + "time_mix_receptance").reshape(-1)) * prev_f[i]))
            prev_f[i] = h
            x = x + rr * (f(m + "value.weight") @ kk)
            x = x / 2                      # rescale_every = 1
        exp.append(f("head.weight") @ ln(x, "rwkv.ln_out"))
    np.testing.assert_allclose(got, np.stack(exp), rtol=3e-2, atol=3e-2)


def test_gpt2_beam_oracle_width_one_is_greedy_and_scores_are_sorted():
    """Beam decode composed from the BeamSearch op: width 1 reproduces the greedy stream; for width 3 the running scores stay
    sorted (the op's global top-k is sorted)."""
    from oracle import gpt2_np
    from poptransformer_b200 import synth
    dims = dict(n_layer=2, d_model=128, n_head=2, vocab=301, n_positions=64)
    sd = {k: v.numpy() for k, v in synth.gpt2_state_dict(**dims, seed=3).items()}
    prompt = np.random.default_rng(0).integers(0, 300, (2, 5)).astype(np.int32)
    one = gpt2_np.GPT2Oracle(gpt2_np.GPT2Config(**dims, max_len=24), sd, 2)
    h1, _ = one.generate_beam(prompt, 8, 1)
    ids = np.full((2, 24), 300, np.int32)
    ids[:, :5] = prompt
    greedy = one.generate(ids, 12, 300)
    assert np.array_equal(h1[:, :, 0], greedy[:, 5:13])
    three = gpt2_np.GPT2Oracle(gpt2_np.GPT2Config(**dims, max_len=24), sd, 6)
    hyp, prob = three.generate_beam(prompt, 8, 3)
    assert hyp.shape == (2, 8, 3) and (np.diff(prob.astype(np.float32), axis=1) <= 0).all()


def test_multi_stream_loop_serves_streams_in_turn():
    """MultiStreamLoop on a stand-in decoder (no GPU): global iteration s goes to stream s % max_bps at that stream's own step
    s // max_bps (GetStepBps, custom_ops/kv_cache_codelet.cpp:18-36), a stream that has finished takes the next waiting request, and
    every request gets exactly max_loop iterations."""
    import torch
    from poptransformer_b200 import loop

    order = []

    class Fake(loop.DecodeLoop):
        graph = object()                      # "already captured"

        def __init__(self, sid=0, family=None):
            self.sid, self.family = sid, family if family is not None else [self]
            self.cfg = type("C", (), {"max_len": 8})()
            self.ids = torch.zeros((1, 8), dtype=torch.int32)
            self.step_t = torch.zeros(1, dtype=torch.int32)
            self.error_flag = torch.zeros(1, dtype=torch.int32)
            self._init_loop("cpu", False)

        def new_stream(self):
            s = Fake(len(self.family), self.family)
            self.family.append(s)
            return s

        def reset(self, ids):
            self.ids.copy_(torch.as_tensor(ids, dtype=torch.int32))
            self.step_t.zero_()

        def step(self):
            order.append((self.sid, int(self.step_t.item()), int(self.ids[0, 0])))
            self.ids[0, 1 + int(self.step_t.item())] = 100 * int(self.ids[0, 0]) + int(self.step_t.item())
            self.step_t += 1

    ms = loop.MultiStreamLoop(Fake(), 2, capture=False)
    reqs = [np.full((1, 8), 0, np.int32) for _ in range(3)]
    for i, r in enumerate(reqs):
        r[0, 0] = i + 1                                     # request tag
    outs = ms.run(reqs, max_loop=3)
    # streams alternate; stream 0 finishes request 1 after three turns and picks up request 3 while stream 1 is still on request 2
    assert order[:6] == [(0, 0, 1), (1, 0, 2), (0, 1, 1), (1, 1, 2), (0, 2, 1), (1, 2, 2)]
    assert [o for o in order[6:]] == [(0, 0, 3), (0, 1, 3), (0, 2, 3)]
    for i, o in enumerate(outs):
        tag = i + 1
        assert int(o["Loop:1"][0]) == 3 and o["Loop:0"][0, 1:4].tolist() == [100 * tag, 100 * tag + 1, 100 * tag + 2]
    with pytest.raises(loop.PtError, match="new_stream"):
        loop.MultiStreamLoop(object(), 2)
