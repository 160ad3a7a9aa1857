"""GPU parity of the ChatGLM2 decode loop (multi-query attention, interleaved RoPE, fp16 softmax, fused RMSNorm prologues,
fp16 and FP8-E4M3 linears) against the numpy restatement of the reference model (oracle/chatglm2_np.py).
Tolerances: rtol / atol 2e-2 on fp16 logits; with FP8 linears bit-exact where the arithmetic coincides and the 5e-2 band
applied statistically elsewhere (see the comment in the test)."""
import numpy as np
import pytest

from oracle import chatglm2_np

pytestmark = pytest.mark.gpu

SMALL = dict(n_layer=2, d_model=512, n_head=4, n_group=2, ffn=768, vocab=1000)    # head size 128, 2 KV groups like ChatGLM2-6B


def _setup(cuda, batch, max_len, precision, seed=0):
    from poptransformer_b200 import chatglm2, synth
    sd = synth.chatglm2_state_dict(**SMALL, seed=seed, device="cpu", precision=precision)
    dec = chatglm2.ChatGLM2Decoder(chatglm2.ChatGLM2Config(**SMALL, max_len=max_len, precision=precision), sd, batch, device=cuda)
    np_sd = {k: (v.numpy() if hasattr(v, "numpy") else v) for k, v in sd.items()}
    orc = chatglm2_np.ChatGLM2Oracle(chatglm2_np.ChatGLM2Config(**SMALL, max_len=max_len, precision=precision), np_sd, batch)
    return dec, orc


@pytest.mark.parametrize("batch,precision,tol", [(1, "fp16", 2e-2), (8, "fp16", 2e-2), (2, "fp8", 5e-2), (8, "fp8", 5e-2)])
def test_chatglm2_logits_teacher_forced(cuda, batch, precision, tol):
    """fp8 at 8 rows takes the tcgen05 GEMM path (RMSNorm / SwiGLU / casts as their own kernels), at 2 rows the skinny-matmul kernels."""
    from poptransformer_b200 import synth
    max_len = 70
    dec, orc = _setup(cuda, batch, max_len, precision)
    assert dec.use_gemm == (precision == "fp8" and batch >= 8)
    ids = synth.prompt_ids(batch, max_len, max_len, SMALL["vocab"], dec.pad_id, seed=1)
    dec.reset(ids)
    orc.reset()
    for step in range(max_len):
        dec.step()
        if step % 5 == 0 or step == max_len - 1:
            got = dec.logits.cpu().numpy().astype(np.float32)
        exp, _ = orc.logits(ids[:, step].numpy(), step)
        if step % 5 == 0 or step == max_len - 1:
            exp = exp.astype(np.float32)
            if precision == "fp8":
                # E4M3 casts amplify differences: a relative difference delta between two implementations' fp16 activations moves
                # a share delta / 6 % of them to the neighbouring E4M3 code (6-12 % of their value), so the next linear's outputs
                # differ by about sqrt(delta / 0.06) * 0.09 -- larger than delta below a few per cent.  Measured on B200: when the
                # arithmetic coincides the logits are bit-identical (test_chatglm2_fp8_bit_exact_where_the_arithmetic_coincides);
                # one fp16 ulp in one head's attention output (the reference rounds each probability to fp16, the kernel
                # normalises in fp32) becomes 2 % rms in the same block's MLP activations and the difference settles at 3-5 % of
                # the logits' rms from then on.  So the 5e-2 band holds for all but about 1 % of the logits: require 98 % inside
                # it, bound the worst by four times the band and the rms difference by 8 % of the logits' rms.
                err = np.abs(got - exp)
                assert np.mean(err <= tol + tol * np.abs(exp)) >= 0.98 and err.max() <= 4 * tol, f"step {step}: max {err.max()}"
                assert np.sqrt((err ** 2).mean()) <= 0.08 * np.sqrt((exp ** 2).mean()), f"step {step}: rms difference {np.sqrt((err ** 2).mean())}"
            else:
                np.testing.assert_allclose(got, exp, rtol=tol, atol=tol, err_msg=f"step {step}")
    assert dec.error_flag.item() == 0


def test_chatglm2_fp8_bit_exact_where_the_arithmetic_coincides(cuda):
    """First step of a fresh sequence (attention over one token) with a configuration in which the reference's fp16
    probability exp(s) * fp16(1 / exp(s)) is exactly 1 for every head: every cast, FP8 product sum, bias, SwiGLU and residual of
    two blocks and the head must then reproduce the restatement bit for bit, with per-tensor activation scales that differ from
    tensor to tensor.  Any change of a rounding point in the FP8 path fails this."""
    from poptransformer_b200 import synth
    dec, orc = _setup(cuda, 2, 8, "fp8")
    scales = {float(v) for k, v in orc.sd.items() if k.endswith("_act_scale")}
    assert len(scales) >= 5, "the synthetic checkpoint carries per-tensor activation scales"
    ids = synth.prompt_ids(2, 8, 8, SMALL["vocab"], dec.pad_id, seed=1)
    dec.reset(ids)
    orc.reset()
    dec.step()
    exp, _ = orc.logits(ids[:, 0].numpy(), 0)
    np.testing.assert_array_equal(dec.logits.cpu().numpy(), np.asarray(exp, dtype=np.float16))


def test_chatglm2_greedy_stream(cuda):
    from poptransformer_b200 import synth
    batch, max_len, prompt = 2, 40, 6
    dec, orc = _setup(cuda, batch, max_len, "fp16", seed=2)
    ids = synth.prompt_ids(batch, prompt, max_len, SMALL["vocab"], dec.pad_id, seed=3)
    got = dec.run(ids, max_loop=max_len)["Loop:0"]
    exp, logits = orc.generate(ids.numpy(), max_len, dec.pad_id, return_logits=True)
    for b in range(batch):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            t = int(diff[0])
            top2 = np.sort(logits[t - 1][b].astype(np.float32))[-2:]
            assert top2[1] - top2[0] <= 2e-2, f"row {b}: streams diverge at {t} without a numerical tie"
    assert (got == exp).mean() > 0.9


def test_attention_writes_the_fp8_copy_of_its_output(cuda):
    """pt_kv_append_attn with out_fp8: the E4M3 bytes are exactly the cast (pt_cast_fp8) of the fp16 output it writes beside them."""
    import ctypes
    import torch
    from poptransformer_b200 import ops
    B, n_head, n_kv, H, max_len = 3, 8, 2, 128, 200
    g = torch.Generator(device="cpu").manual_seed(4)
    cache = ops.PagedKVCache(B, n_kv, H, max_len, 64, cuda)
    cache.pool.copy_((torch.randn(cache.pool.shape, generator=g) * 0.5).half().to(cuda))
    qkv = (torch.randn((B, (n_head + 2 * n_kv) * H), generator=g) * 0.7).half().to(cuda)
    step = torch.full((1,), 150, dtype=torch.int32, device=cuda)
    out = torch.empty((B, n_head * H), dtype=torch.float16, device=cuda)
    out8 = torch.zeros((B, n_head * H), dtype=torch.uint8, device=cuda)
    ws = ops.attn_workspace(B, n_head, H, cache.max_pages, cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    scale = 2.0 / 448.0
    a = ops.attn_args(qkv, step, cache, out, n_head, ops.ROPE_NONE, ops.SOFTMAX_F32, 0.088, None, None, ws, err, out_fp8=out8, out_fp8_scale=scale)
    ops.check(ops._lib.lib().pt_kv_append_attn(ctypes.byref(a), ops._stream()), "pt_kv_append_attn")
    assert int(err.item()) == 0
    assert torch.equal(out8, ops.half_to_uint8(out, scale))
