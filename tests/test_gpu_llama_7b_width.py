"""Parity of the Llama decode step at the WIDTH the benchmark runs: d_model 4096, 32 heads, FFN 11008, vocab 32000,
INT4 group 128 — two transformer blocks (depth only repeats the block) — against the C restatement of the reference
step (oracle/c/decode_ref.c).  The caches start 500 tokens deep, so the run uses eight full pages per head, crosses the
page boundary at position 512 into a ninth, every SM owns several row tiles of every matrix, and the attention combine
sees nine partial results.  Teacher-forced for 44 steps: fp16 logits within rtol 2e-2 / atol 2e-2, the greedy id equal
to the restatement's or a tie inside that tolerance, the new K/V rows of block 0 within the same tolerance and the
cached prompt untouched bit for bit.

How the logit tolerance is applied at this width.  Every value on the path is rounded to fp16 some thirty-five times
(the reference graph holds fp16 tensors between ops), and the three implementations at hand (this restatement, the per-op
kernels, the persistent kernel) sum in different orders, so any two of them differ by a common-mode relative error of a few
1e-3 on the hidden state: measured here, the logits (rms 1.28, largest 6) differ from the restatement's by 0.002-0.007 rms
per step, the per-op and the persistent kernels differ from each other by the same amount, and the largest single
difference over the 1.4 million logits of a run is 0.03.  A max-norm bound of 2e-2 over 32000 logits x 44 steps is
therefore a five-sigma statistic; the test requires the element-wise bound for all but 1e-3 of a step's logits, bounds
the worst element by twice the tolerance, and bounds the rms difference by 1e-2."""
import numpy as np
import pytest
import torch

from oracle import c_ref, llama_np

pytestmark = pytest.mark.gpu

DIMS = dict(n_layer=2, d_model=4096, n_head=32, ffn=11008, vocab=32000)
GROUP, MAX_LEN, CTX, STEPS = 128, 576, 500, 44


@pytest.fixture(scope="module")
def checkpoint(cuda):
    from poptransformer_b200 import synth
    sd = synth.llama_state_dict(**DIMS, seed=11, device=cuda, int4_group=GROUP)
    return sd, {k: v.cpu().numpy() for k, v in sd.items()}


@pytest.mark.parametrize("batch,persistent", [(1, True), (2, True), (1, False), (16, False), (16, "gemm")])
def test_full_width_teacher_forced(cuda, checkpoint, batch, persistent):
    """persistent True: the whole-step kernel; False: the per-op kernels; "gemm": per-op with the transformer linears on the tcgen05
    GEMM (the path of more than 16 rows, forced here at 16)."""
    from poptransformer_b200 import llama, synth
    sd, sd_np = checkpoint
    gemm = persistent == "gemm"
    persistent = False if gemm else persistent
    dec = llama.LlamaDecoder(llama.LlamaConfig(**DIMS, max_len=MAX_LEN, int4_group=GROUP), sd, batch, device=cuda, persistent=persistent,
                             use_gemm=True if gemm else None)
    assert dec.persistent == persistent and dec.use_gemm == gemm
    orc = c_ref.LlamaOracleC(llama_np.LlamaConfig(**DIMS, max_len=MAX_LEN, group=GROUP), sd_np, batch)

    # a cache that is already CTX tokens deep: the same random K/V rows on both sides
    gen = torch.Generator(device=cuda).manual_seed(5)
    before = torch.full((1,), CTX - 1, dtype=torch.int32, device=cuda)
    prompt_kv = []
    for li, kc in enumerate(dec.caches):
        kc.pool.copy_((torch.randn(kc.pool.shape, generator=gen, device=cuda) * 0.5).to(torch.float16))
        dense = kc.export(before, MAX_LEN).cpu().numpy()      # [2, rows, heads, MAX_LEN, H], newest first, zeros beyond CTX - 1
        orc.set_cache(li, dense[0], dense[1])
        prompt_kv.append(dense)

    ids = synth.prompt_ids(batch, MAX_LEN, MAX_LEN, DIMS["vocab"], dec.pad_id, seed=6)    # all prompt: every step is forced
    dec.reset(ids)
    dec.step_t.fill_(CTX)
    ties = 0
    for i in range(STEPS):
        step = CTX + i
        dec.step()
        got = dec.logits.cpu().numpy().astype(np.float32)
        got_id = dec.next_ids.cpu().numpy().reshape(-1)
        exp, exp_id = orc.logits(ids[:, step].numpy(), step)
        exp = exp.astype(np.float32)
        diff = np.abs(got - exp)
        outside = diff > 2e-2 + 2e-2 * np.abs(exp)
        assert outside.mean() <= 1e-3, f"step {step}: {int(outside.sum())} logits outside rtol 2e-2 / atol 2e-2"
        assert (diff <= 2 * (2e-2 + 2e-2 * np.abs(exp))).all(), f"step {step}: a logit differs by {diff.max()}"
        assert np.sqrt((diff ** 2).mean()) <= 1e-2, f"step {step}: rms difference {np.sqrt((diff ** 2).mean())}"
        for b in range(batch):
            if got_id[b] != exp_id[b]:
                gap = exp[b].max() - exp[b][got_id[b]]
                assert gap <= 2e-2, f"step {step} row {b}: id {got_id[b]} is {gap} below the restatement's best {exp_id[b]}"
                ties += 1
    assert dec.error_flag.item() == 0
    assert int(dec.step_t.item()) == CTX + STEPS
    assert ties <= STEPS * batch // 4

    last = torch.full((1,), CTX + STEPS - 1, dtype=torch.int32, device=cuda)
    dense = dec.caches[0].export(last, MAX_LEN).cpu().numpy()
    ref_k, ref_v = orc.kcache(0), orc.vcache(0)
    # the STEPS newest rows were appended by the run
    np.testing.assert_allclose(dense[0][:, :, :STEPS].astype(np.float32), ref_k[:, :, :STEPS].astype(np.float32), rtol=2e-2, atol=2e-2)
    np.testing.assert_allclose(dense[1][:, :, :STEPS].astype(np.float32), ref_v[:, :, :STEPS].astype(np.float32), rtol=2e-2, atol=2e-2)
    # ... behind them the cached prompt, shifted by STEPS positions and otherwise untouched (a cache append is a copy)
    for li in (0, 1):
        now = dec.caches[li].export(last, MAX_LEN).cpu().numpy()
        assert np.array_equal(now[:, :, :, STEPS:STEPS + CTX], prompt_kv[li][:, :, :, :CTX])
