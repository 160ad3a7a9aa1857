"""One-pass prompt ingestion (the work of the reference's first stage, models/base_model.py:358-494) against the token-by-token
loop and the restatements: the causal attention op against numpy with the reference's roundings (llama2/attention.py:28-56,
:97-114 with stable_mode = True), and the decoder's `prefill()` + decode against the C restatement of the loop run from step 0."""
import math

import numpy as np
import pytest
import torch

from oracle import c_ref, llama_np
from oracle import ops_np as O

pytestmark = pytest.mark.gpu
F16 = np.float16


def _attn_reference(qkv, sin, cos, B, P, start, n_head, past_k=None, past_v=None):
    """numpy: RoPE, K/V of positions 0 .. start + P - 1 (oldest first), causal softmax(fp32, max-subtracted) . V, fp16 at the
    reference's tensor boundaries."""
    H = 128
    q, k, v = (qkv.reshape(B, P, 3, n_head, H)[:, :, i].transpose(0, 2, 1, 3) for i in range(3))      # [B, N, P, H]
    pos = np.arange(start, start + P)
    qr = np.stack([O.llama_rope_apply(q[:, :, t], sin[pos[t]], cos[pos[t]]) for t in range(P)], axis=2)
    kr = np.stack([O.llama_rope_apply(k[:, :, t], sin[pos[t]], cos[pos[t]]) for t in range(P)], axis=2)
    K = kr if past_k is None else np.concatenate([past_k, kr], axis=2)
    V = v if past_v is None else np.concatenate([past_v, v], axis=2)
    s = O.matmul_f16(qr, np.swapaxes(K, -1, -2))                                                      # [B, N, P, start + P]
    s = O.mul_f16(s, np.array([1 / math.sqrt(H)]).astype(F16))
    mask = np.where(np.arange(start + P)[None, :] <= pos[:, None], 0.0, -10000.0).astype(F16)
    s = O.add_f16(s, mask[None, None])
    p = O.softmax_v3(O.f32(s), stable_mode=True).astype(F16)
    o = O.matmul_f16(p, V)                                                                            # [B, N, P, H]
    return np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(B * P, n_head * H), K, V


@pytest.mark.parametrize("B,P,n_head", [(2, 70, 2), (1, 16, 1), (3, 129, 2)])
def test_prefill_attn_matches_numpy(cuda, B, P, n_head):
    from poptransformer_b200 import llama, ops
    H, max_len = 128, 256
    rng = np.random.default_rng(3)
    qkv = (rng.standard_normal((B * P, 3 * n_head * H)) * 0.7).astype(F16)
    sin_t, cos_t = llama.rope_tables(max_len, H, cuda)
    sin, cos = sin_t.cpu().numpy(), cos_t.cpu().numpy()
    cache = ops.PagedKVCache(B, n_head, H, max_len, 64, cuda)
    scale = float(F16(1 / math.sqrt(H)))
    exp, K, V = _attn_reference(qkv, sin, cos, B, P, 0, n_head)
    got = ops.prefill_attn(torch.from_numpy(qkv).to(cuda), cache, B, P, 0, n_head, scale, sin_t, cos_t).cpu().numpy()
    np.testing.assert_allclose(got.astype(np.float32), exp.astype(np.float32), rtol=2e-3, atol=2e-3)
    # the cache holds the rotated keys and the values bit for bit (export: newest first)
    last = torch.full((1,), P - 1, dtype=torch.int32, device=cuda)
    dense = cache.export(last, max_len).cpu().numpy()                 # [2, B, N, max_len, H]
    np.testing.assert_array_equal(dense[0][:, :, :P][:, :, ::-1], K)
    np.testing.assert_array_equal(dense[1][:, :, :P][:, :, ::-1], V)
    assert not dense[:, :, :, P:].any()

    # a second chunk on top of the first: positions P .. P + 39
    P2 = 40
    qkv2 = (rng.standard_normal((B * P2, 3 * n_head * H)) * 0.7).astype(F16)
    exp2, _, _ = _attn_reference(qkv2, sin, cos, B, P2, P, n_head, K, V)
    got2 = ops.prefill_attn(torch.from_numpy(qkv2).to(cuda), cache, B, P2, P, n_head, scale, sin_t, cos_t).cpu().numpy()
    np.testing.assert_allclose(got2.astype(np.float32), exp2.astype(np.float32), rtol=2e-3, atol=2e-3)


def test_prefill_attn_rejects_bad_arguments(cuda):
    from poptransformer_b200 import llama, ops
    sin_t, cos_t = llama.rope_tables(128, 128, cuda)
    cache = ops.PagedKVCache(1, 1, 128, 128, 64, cuda)
    qkv = torch.zeros((100, 384), dtype=torch.float16, device=cuda)
    with pytest.raises(ops.PtError):
        ops.prefill_attn(qkv, cache, 1, 100, 64, 1, 1.0, sin_t, cos_t)        # positions 64 .. 163 exceed max_len 128
    with pytest.raises(ops.PtError):
        ops.prefill_attn(qkv, cache, 1, 50, 0, 1, 1.0, sin_t, cos_t)          # shape mismatch


DIMS = dict(n_layer=3, d_model=256, n_head=2, ffn=512, vocab=640)
GROUP, MAX_LEN = 128, 192


@pytest.fixture(scope="module")
def checkpoint(cuda):
    from poptransformer_b200 import synth
    sd = synth.llama_state_dict(**DIMS, seed=21, device=cuda, int4_group=GROUP)
    return sd, {k: v.cpu().numpy() for k, v in sd.items()}


@pytest.mark.parametrize("batch,persistent,chunk", [(2, True, 1024), (2, False, 48), (5, False, 1024)])
def test_prefill_then_decode_matches_the_loop(cuda, checkpoint, batch, persistent, chunk):
    """Teacher-forced: the restatement runs the loop token by token from step 0; the decoder ingests N positions in one pass
    (optionally in chunks) and then steps.  Logits of the following steps within rtol/atol 2e-2, ids equal or tied within it,
    the ingested K/V rows of every block within 1e-2 of the restatement's."""
    from poptransformer_b200 import llama, synth
    sd, sd_np = checkpoint
    N, STEPS = 133, 6
    dec = llama.LlamaDecoder(llama.LlamaConfig(**DIMS, max_len=MAX_LEN, int4_group=GROUP), sd, batch, device=cuda, persistent=persistent,
                             prefill=True)
    assert dec.persistent == persistent
    orc = c_ref.LlamaOracleC(llama_np.LlamaConfig(**DIMS, max_len=MAX_LEN, group=GROUP), sd_np, batch)
    ids = synth.prompt_ids(batch, MAX_LEN, MAX_LEN, DIMS["vocab"], dec.pad_id, seed=8)      # all prompt: every step is forced
    for s in range(N):
        orc.logits(ids[:, s].numpy(), s)
    dec.reset(ids)
    assert dec.prefill(N, chunk=chunk) == N
    assert dec.step_t.item() == N
    at = torch.full((1,), N - 1, dtype=torch.int32, device=cuda)
    for li in (0, DIMS["n_layer"] - 1):
        dense = dec.caches[li].export(at, MAX_LEN).cpu().numpy().astype(np.float32)     # newest first
        np.testing.assert_allclose(dense[0][:, :, :N], orc.kcache(li)[:, :, :N].astype(np.float32), rtol=1e-2, atol=1e-2)
        np.testing.assert_allclose(dense[1][:, :, :N], orc.vcache(li)[:, :, :N].astype(np.float32), rtol=1e-2, atol=1e-2)
    for i in range(STEPS):
        step = N + i
        dec.step()
        got = dec.logits.cpu().numpy().astype(np.float32)
        got_id = dec.next_ids.cpu().numpy().reshape(-1)
        exp, exp_id = orc.logits(ids[:, step].numpy(), step)
        exp = exp.astype(np.float32)
        np.testing.assert_allclose(got, exp, rtol=2e-2, atol=2e-2)
        for b in range(batch):
            if got_id[b] != exp_id[b]:
                assert exp[b].max() - exp[b][got_id[b]] <= 2e-2
    assert dec.error_flag.item() == 0


def test_run_with_prefill_returns_the_loop_anchors(cuda, checkpoint):
    """Ragged prompts through `run(..., prefill=True)`: the ingested length is one less than the shortest prompt, the longer
    prompts' remaining tokens are consumed by the loop's own rule, and the id container and step come back as from the
    token-by-token run (ids equal wherever the two runs' logits are not tied)."""
    from poptransformer_b200 import llama, synth
    sd, _ = checkpoint
    cfg = llama.LlamaConfig(**DIMS, max_len=MAX_LEN, int4_group=GROUP)
    ids = synth.prompt_ids(2, 90, MAX_LEN, DIMS["vocab"], DIMS["vocab"] - 1, seed=9)
    ids[0, 70:] = DIMS["vocab"] - 1                                    # prompt lengths 70 and 90
    dec = llama.LlamaDecoder(cfg, sd, 2, device=cuda, prefill=True)
    a = dec.run(ids, max_loop=100)
    b = dec.run(ids, max_loop=100, prefill=True)
    assert int(a["Loop:1"][0]) == int(b["Loop:1"][0]) == 100
    given = ids.numpy() != DIMS["vocab"] - 1
    np.testing.assert_array_equal(b["Loop:0"][given], ids.numpy()[given])
    assert (b["Loop:0"][:, :101] != DIMS["vocab"] - 1).all()
    same = (a["Loop:0"] == b["Loop:0"]).mean()
    assert same >= 0.9, f"only {same:.2f} of the container agrees between the two runs"
    dec.reset(ids)
    assert dec.prefill() == 69


def test_prefill_needs_the_flag(cuda, checkpoint):
    from poptransformer_b200 import llama, ops
    sd, _ = checkpoint
    dec = llama.LlamaDecoder(llama.LlamaConfig(**DIMS, max_len=MAX_LEN, int4_group=GROUP), sd, 1, device=cuda)
    with pytest.raises(ops.PtError):
        dec.prefill(4)
