"""GPU parity of the Llama-2 decode loop against the numpy restatement of the reference model
(oracle/llama_np.py): fp16 logits within rtol 2e-2 / atol 2e-2, greedy token stream identical
(a divergence is tolerated only at a step where the oracle's own top-2 logits are closer than the
logit tolerance, i.e. a numerical tie)."""
import numpy as np
import pytest
import torch

from oracle import llama_np
from oracle import ops_np as O

pytestmark = pytest.mark.gpu

TINY = dict(n_layer=2, d_model=256, n_head=2, ffn=512, vocab=1000)


def _setup(cuda, batch, max_len, int4_group, seed=0, persistent=None, use_gemm=None):
    from poptransformer_b200 import llama, synth
    sd = synth.llama_state_dict(**TINY, seed=seed, device="cpu", int4_group=int4_group)
    cfg = llama.LlamaConfig(**TINY, max_len=max_len, int4_group=int4_group)
    dec = llama.LlamaDecoder(cfg, sd, batch, device=cuda, persistent=persistent, use_gemm=use_gemm)
    ocfg = llama_np.LlamaConfig(**TINY, max_len=max_len, group=int4_group)
    orc = llama_np.LlamaOracle(ocfg, {k: v.numpy() for k, v in sd.items()}, batch)
    return dec, orc


@pytest.mark.parametrize("batch,int4_group,persistent", [(1, 128, True), (2, 128, True), (1, 128, False), (2, 0, False), (1, 256, False),
                                                        (16, 128, False), (16, 128, "gemm"), (40, 128, "gemm")])
def test_logits_teacher_forced(cuda, batch, int4_group, persistent):
    """persistent=True: the whole-step kernel; False: the per-op kernels; "gemm": the per-op path with the transformer linears on the
    tcgen05 GEMM (the path of more than 16 rows, forced at 16; at 40 rows it is the only path and the fp16 LM head runs in blocks of
    32 rows).  All against the oracle."""
    from poptransformer_b200 import synth
    max_len = 72 if persistent is True else 40          # more than one KV page for the persistent kernel
    gemm = persistent == "gemm"
    persistent = False if gemm else persistent
    dec, orc = _setup(cuda, batch, max_len, int4_group, persistent=persistent, use_gemm=True if gemm else None)
    assert dec.use_gemm == gemm
    assert dec.persistent == persistent
    ids = synth.prompt_ids(batch, max_len, max_len, TINY["vocab"], dec.pad_id, seed=1)     # all prompt: every step is forced
    dec.reset(ids)
    orc.reset()
    for step in range(max_len):
        dec.step()
        got = dec.logits.cpu().numpy().astype(np.float32)
        exp, _ = orc.logits(ids[:, step].numpy(), step)
        np.testing.assert_allclose(got, exp.astype(np.float32), rtol=2e-2, atol=2e-2, err_msg=f"step {step}")
    assert dec.error_flag.item() == 0
    # KV cache contents in the reference layout: layer 0 is bit-exact (its inputs are bit-identical);
    # deeper layers inherit fp32-accumulation-order noise, so compare within the logit tolerance
    dec.step_t.fill_(max_len - 1)
    dense = dec.caches[0].export(dec.step_t, max_len).cpu().numpy()
    ref = orc.kv[0][0].cache
    assert dense.shape == ref.shape
    np.testing.assert_allclose(dense.astype(np.float32), ref.astype(np.float32), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("use_graph,persistent", [(False, False), (True, False), (False, True), (True, True)])
def test_greedy_stream(cuda, use_graph, persistent):
    from poptransformer_b200 import synth
    batch, max_len, prompt = 2, 48, 8
    dec, orc = _setup(cuda, batch, max_len, 128, seed=3, persistent=persistent)
    ids = synth.prompt_ids(batch, prompt, max_len, TINY["vocab"], dec.pad_id, seed=2)
    if use_graph:
        dec.capture()
    out = dec.run(ids, max_loop=max_len)
    got = out["Loop:0"]
    assert int(out["Loop:1"][0]) == max_len
    exp, logits = orc.generate(ids.numpy(), max_len, dec.pad_id, return_logits=True)
    assert np.array_equal(got[:, :prompt], ids[:, :prompt].numpy())
    for b in range(batch):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            t = int(diff[0])                     # token at position t was produced by the logits of step t-1
            top2 = np.sort(logits[t - 1][b].astype(np.float32))[-2:]
            assert top2[1] - top2[0] <= 2e-2, f"row {b}: streams diverge at {t} without a numerical tie (margin {top2[1]-top2[0]})"
    # the common case: identical streams
    assert (got == exp).mean() > 0.9


def test_run_twice_is_deterministic(cuda):
    from poptransformer_b200 import synth
    dec, _ = _setup(cuda, 1, 32, 128, seed=5)
    ids = synth.prompt_ids(1, 4, 32, TINY["vocab"], dec.pad_id, seed=4)
    dec.capture()
    a = dec.run(ids)["Loop:0"].copy()
    b = dec.run(ids)["Loop:0"].copy()
    assert np.array_equal(a, b)


@pytest.mark.parametrize("persistent", [True, False])
def test_early_stop_ends_where_the_reference_loop_ends(cuda, persistent):
    """early_stop (models/base_model.py:348-352): keep_going is evaluated on the stop mask as it was before an iteration's own
    update, so the loop body runs once more after the iteration that produced the last eos id.  With the eos id first
    generated for position p the final state is step = p + 1, position p + 1 written, everything after it still padding."""
    from poptransformer_b200 import llama, synth
    batch, max_len, prompt = 1, 48, 6
    sd = synth.llama_state_dict(**TINY, seed=7, device="cpu", int4_group=128)
    cfg = llama.LlamaConfig(**TINY, max_len=max_len, int4_group=128)
    ids = synth.prompt_ids(batch, prompt, max_len, TINY["vocab"], TINY["vocab"] - 1, seed=8)
    free = llama.LlamaDecoder(cfg, sd, batch, device=cuda, persistent=persistent)
    full = free.run(ids, max_loop=max_len)["Loop:0"]
    p = prompt + 9
    eos = int(full[0, p])
    first = int(np.nonzero(full[0, prompt:] == eos)[0][0]) + prompt      # the id may occur earlier in the stream
    dec = llama.LlamaDecoder(cfg, sd, batch, device=cuda, persistent=persistent, eos_id=eos, early_stop=True)
    out = dec.run(ids, max_loop=max_len, poll_every=4)
    got = out["Loop:0"]
    assert int(out["Loop:1"][0]) == first + 1
    assert np.array_equal(got[0, :first + 2], full[0, :first + 2])
    assert (got[0, first + 2:] == dec.pad_id).all()
    assert int(dec.stop_mask.item()) == 1 and int(dec.done_flag.item()) == 1
    # without early_stop the same eos id only sets the stop mask: the loop runs to the end, like the reference's
    plain = llama.LlamaDecoder(cfg, sd, batch, device=cuda, persistent=persistent, eos_id=eos)
    out = plain.run(ids, max_loop=max_len)
    assert int(out["Loop:1"][0]) == max_len and np.array_equal(out["Loop:0"], full) and int(plain.stop_mask.item()) == 1


def test_bounded_wait_runs_out_and_is_reported(cuda):
    """A tensor-parallel step whose second rank never shows up: rank 0 of a tp_size = 2 configuration is launched alone, with
    a local buffer standing in for the absent rank's exchange buffer, so nothing ever writes rank 1's arrival counter.  The
    kernel's wait for it must run out (short limit), set the error flag to the staging wait's code, and return; the host call
    must raise; and the device must stay usable."""
    from poptransformer_b200 import _lib, llama, ops, synth
    batch, max_len = 1, 32
    sd = synth.llama_state_dict(**TINY, seed=9, device="cpu", int4_group=128)
    cfg = llama.LlamaConfig(**TINY, max_len=max_len, int4_group=128)
    nbytes = _lib.lib().pt_llama_tp_buffer_bytes(batch, TINY["d_model"], 2)
    bufs = [torch.zeros((nbytes + 3) // 4, dtype=torch.int32, device=cuda) for _ in range(2)]
    dec = llama.LlamaDecoder(cfg, sd, batch, device=cuda, tp_rank=0, tp_size=2, tp_buffers=bufs, persistent=True, wait_limit=4096)
    assert dec.persistent
    ids = synth.prompt_ids(batch, 4, max_len, TINY["vocab"], dec.pad_id, seed=1)
    with pytest.raises(ops.PtError, match="error flag 10"):
        dec.run(ids, max_loop=1)
    assert int(dec.error_flag.item()) == 10
    assert int(dec.step_t.item()) == 0                    # the failed iteration did not advance the loop
    # the context is intact: an ordinary decoder still runs, and the default limit is back in force for it
    ok = llama.LlamaDecoder(cfg, sd, batch, device=cuda, persistent=True)
    assert int(ok.run(ids, max_loop=8)["Loop:1"][0]) == 8


def test_step_past_the_container_is_refused_on_the_device(cuda):
    """A launch with step >= max_len has no position left (id container, RoPE tables, page table): both paths set error flag 12
    instead of reading past their tables, and change nothing."""
    from poptransformer_b200 import ops, synth
    for persistent in (True, False):
        dec, _ = _setup(cuda, 1, 24, 128, persistent=persistent)
        ids = synth.prompt_ids(1, 4, 24, TINY["vocab"], dec.pad_id, seed=1)
        dec.run(ids, max_loop=24)
        with pytest.raises(ops.PtError):
            dec.run(ids, max_loop=25)
        dec.step_t.fill_(24)
        before = dec.ids.clone()
        dec.step()
        torch.cuda.synchronize()
        assert int(dec.error_flag.item()) == 12
        assert torch.equal(dec.ids, before)


@pytest.mark.parametrize("persistent", [True, False])
def test_multi_stream_continuous_decode(cuda, persistent):
    """Three streams over one set of weights serve five requests in turn (stream s % 3 at its own step s // 3, as KVCachePipeline's
    caches are selected): every request's id container equals what the same decoder produces for it alone."""
    from poptransformer_b200 import loop, synth
    dec, _ = _setup(cuda, 2, 72 if persistent else 40, 128, persistent=persistent)
    max_len, vocab = dec.cfg.max_len, dec.cfg.vocab
    reqs = [synth.prompt_ids(2, 3 + 2 * i, max_len, vocab, dec.pad_id, seed=20 + i) for i in range(5)]
    alone = [dec.run(r, max_loop=24)["Loop:0"].copy() for r in reqs]
    ms = loop.MultiStreamLoop(dec, 3)
    assert ms.streams[1].layers is dec.layers and ms.streams[1].caches[0].pool.data_ptr() != dec.caches[0].pool.data_ptr()
    outs = ms.run(reqs, max_loop=24)
    for i, (o, a) in enumerate(zip(outs, alone)):
        assert np.array_equal(o["Loop:0"], a), f"request {i}"
        assert int(o["Loop:1"][0]) == 24
