"""GPU parity of the GPT-2 decode loop (per-op kernels: NormCE, biased linears, GELU, tied LM head, attention without RoPE and
with the fp16 softmax) against the numpy restatement of the reference model (oracle/gpt2_np.py)."""
import numpy as np
import pytest

from oracle import gpt2_np

pytestmark = pytest.mark.gpu

SMALL = dict(n_layer=2, d_model=256, n_head=4, vocab=1000, n_positions=128)    # head size 64, like GPT-2


def _setup(cuda, batch, max_len, seed=0):
    from poptransformer_b200 import gpt2, synth
    sd = synth.gpt2_state_dict(**SMALL, seed=seed, device="cpu")
    dec = gpt2.GPT2Decoder(gpt2.GPT2Config(**SMALL, max_len=max_len), sd, batch, device=cuda)
    orc = gpt2_np.GPT2Oracle(gpt2_np.GPT2Config(**SMALL, max_len=max_len), {k: v.numpy() for k, v in sd.items()}, batch)
    return dec, orc


@pytest.mark.parametrize("batch", [1, 4])
def test_gpt2_logits_teacher_forced(cuda, batch):
    from poptransformer_b200 import synth
    max_len = 72
    dec, orc = _setup(cuda, batch, max_len)
    ids = synth.prompt_ids(batch, max_len, max_len, SMALL["vocab"], dec.pad_id, seed=1)
    dec.reset(ids)
    orc.reset()
    for step in range(max_len):
        dec.step()
        exp, _ = orc.logits(ids[:, step].numpy(), step)
        np.testing.assert_allclose(dec.logits.cpu().numpy().astype(np.float32), exp.astype(np.float32), rtol=2e-2, atol=2e-2, err_msg=f"step {step}")
    assert dec.error_flag.item() == 0


@pytest.mark.parametrize("use_graph", [False, True])
def test_gpt2_greedy_stream(cuda, use_graph):
    from poptransformer_b200 import synth
    batch, max_len, prompt = 2, 40, 6
    dec, orc = _setup(cuda, batch, max_len, seed=2)
    ids = synth.prompt_ids(batch, prompt, max_len, SMALL["vocab"], dec.pad_id, seed=3)
    if use_graph:
        dec.capture()
    got = dec.run(ids, max_loop=max_len)["Loop:0"]
    exp, logits = orc.generate(ids.numpy(), max_len, dec.pad_id, return_logits=True)
    for b in range(batch):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            t = int(diff[0])
            top2 = np.sort(logits[t - 1][b].astype(np.float32))[-2:]
            assert top2[1] - top2[0] <= 2e-2, f"row {b}: streams diverge at {t} without a numerical tie"
    assert (got == exp).mean() > 0.9


@pytest.mark.parametrize("page_size", [8, 64])
def test_gpt2_beam_decode(cuda, page_size):
    """BeamSearch on top of the GPT-2 step with the beam reorder of the paged cache (batch 2 x beam 4, like the GPT-2 XL beam
    configuration in small).  Per generated position:
      * the op's outputs (next ids, global-best ids, parents, hypothesis and score containers) are bit-identical to the oracle's
        BeamSearch applied to the SAME logits (the GPU's);
      * the GPU logits agree (rtol / atol 2e-2) with the oracle model that is fed the GPU's tokens and whose dense caches are
        reordered with the GPU's parents, which checks the page-table reorder through the attention that reads it.
    Page size 8 makes the position cross several page boundaries."""
    import torch
    from oracle import ops_np as O
    from poptransformer_b200 import gpt2, synth
    n, beam, P, new = 2, 4, 7, 22
    max_len = P + new
    sd = synth.gpt2_state_dict(**SMALL, seed=5, device="cpu")
    dec = gpt2.GPT2BeamDecoder(gpt2.GPT2Config(**SMALL, max_len=max_len), sd, n, beam, new, device=cuda, page_size=page_size)
    orc = gpt2_np.GPT2Oracle(gpt2_np.GPT2Config(**SMALL, max_len=max_len), {k: v.numpy() for k, v in sd.items()}, n * beam)
    prompt = synth.prompt_ids(n, P, P, SMALL["vocab"], dec.pad_id, seed=6).numpy()
    assert dec.start_beam(prompt) == P
    orc.reset()
    hyp, prob = np.zeros((n, new, beam), np.int32), np.zeros((n, beam), np.float16)
    tok = np.repeat(prompt[:, 0], beam)
    distinct_parents = 0
    for t in range(max_len - 1):
        dec.enqueue_logits()
        got = dec.logits.cpu().numpy()
        exp, _ = orc.logits(tok, t)
        np.testing.assert_allclose(got.astype(np.float32), exp.astype(np.float32), rtol=2e-2, atol=2e-2, err_msg=f"position {t}")
        if t + 1 < P:
            dec.enqueue_next()
            tok = np.repeat(prompt[:, t + 1], beam)
            continue
        g = t + 1 - P
        dec.enqueue_beam()
        e_next, e_gid, hyp, prob = O.beam_search_step(got.reshape(n, beam, -1), hyp, prob, g, beam)
        e_parent = (np.arange(n)[:, None] * beam + (np.zeros((n, beam), np.int64) if g == 0 else e_gid // beam)).reshape(-1)
        assert np.array_equal(dec.beam_next.cpu().numpy(), e_next), f"generated position {g}: next ids"
        assert np.array_equal(dec.beam_best.cpu().numpy(), e_gid), f"generated position {g}: global best ids"
        assert np.array_equal(dec.parent.cpu().numpy(), e_parent), f"generated position {g}: parents"
        assert np.array_equal(dec.hyp.cpu().numpy(), hyp) and np.array_equal(dec.prob.cpu().numpy().view(np.uint16), prob.view(np.uint16))
        assert np.array_equal(dec.ids[:, t + 1].cpu().numpy(), e_next.reshape(-1)) and int(dec.step_t.item()) == t + 1
        for layer in orc.kv:
            layer[0].cache = O.kv_reorder_dense(layer[0].cache, e_parent)
        distinct_parents += int(g > 0 and not np.array_equal(e_parent, np.arange(n * beam)))
        tok = e_next.reshape(-1)
    assert distinct_parents > 0, "the case never reordered the cache"
    assert dec.error_flag.item() == 0
    # the whole loop through run_beam gives the same containers
    out = dec.run_beam(prompt)
    assert np.array_equal(out["hyp"], hyp) and np.array_equal(out["prob"].view(np.uint16), prob.view(np.uint16))
