"""Golden vectors produced by the reference's own (unmodified) model code, executed through the numpy stand-in for
popart (tests/golden/make_golden.py): they pin the oracle's restatement of the Llama decode loop, and the CUDA path."""
import glob
import os

import numpy as np
import pytest

from oracle import llama_np

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURES = sorted(glob.glob(os.path.join(HERE, "golden", "llama_*.npz")))


def _load(path):
    from poptransformer_b200 import synth
    z = np.load(path)
    dims = dict(zip(("n_layer", "d_model", "n_head", "ffn", "vocab"), (int(v) for v in z["dims"])))
    group = int(z["group"])
    sd = synth.llama_state_dict(**dims, seed=int(z["seed"]), device="cpu", int4_group=group)
    return z, dims, group, sd


def test_fixtures_exist():
    assert len(FIXTURES) >= 3


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_oracle_reproduces_reference_token_stream(path):
    z, dims, group, sd = _load(path)
    max_len, batch = int(z["max_len"]), int(z["batch"])
    # group -1 = one scale per output channel: the oracle's Int4ToHalf takes scale [n] with group 0
    cfg = llama_np.LlamaConfig(**dims, max_len=max_len, group=0)
    sd_np = {k: (v.numpy().reshape(-1) if k.endswith("_scale") else v.numpy()) for k, v in sd.items()}
    orc = llama_np.LlamaOracle(cfg, sd_np, batch)
    got = orc.generate(z["input_ids"], max_len - 1, int(z["pad_id"]))
    assert int(z["step"]) == max_len - 1
    assert np.array_equal(got, z["output_ids"]), "oracle and reference model code disagree on the greedy token stream"


@pytest.mark.gpu
@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_cuda_reproduces_reference_token_stream(path, cuda):
    from poptransformer_b200 import llama
    z, dims, group, sd = _load(path)
    max_len, batch, prompt = int(z["max_len"]), int(z["batch"]), int(z["prompt"])
    dec = llama.LlamaDecoder(llama.LlamaConfig(**dims, max_len=max_len, int4_group=group), sd, batch, device=cuda, pad_id=int(z["pad_id"]))
    out = dec.run(z["input_ids"], max_loop=max_len - 1)
    got, exp = out["Loop:0"], z["output_ids"]
    assert int(out["Loop:1"][0]) == max_len - 1
    assert np.array_equal(got[:, :prompt], exp[:, :prompt])
    # fp32 accumulation order differs from numpy's, so a row may leave the reference's stream, but only at a position where
    # the oracle's two best logits (given the reference's history) are closer than the logit tolerance; and most positions agree
    cfg = llama_np.LlamaConfig(**dims, max_len=max_len, group=0)
    sd_np = {k: (v.numpy().reshape(-1) if k.endswith("_scale") else v.numpy()) for k, v in sd.items()}
    orc = llama_np.LlamaOracle(cfg, sd_np, batch)
    orc.reset()
    logits = [orc.logits(exp[:, t], t)[0].astype(np.float32) for t in range(max_len - 1)]
    for b in range(batch):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            t = int(diff[0])
            assert t >= prompt, f"row {b}: prompt position {t} changed"
            top2 = np.sort(logits[t - 1][b])[-2:]
            assert top2[1] - top2[0] <= 2e-2, f"row {b}: leaves the reference stream at {t} with margin {top2[1] - top2[0]}"
    assert (got == exp).mean() >= 0.9


# ------------------------------------------------------------------ GPT-2 / ChatGLM2 / RWKV: the reference's model classes, fp16
OTHER = sorted(p for p in glob.glob(os.path.join(HERE, "golden", "*_tiny_fp16.npz")) if not os.path.basename(p).startswith("llama_"))


def _load_other(path):
    from oracle import chatglm2_np, gpt2_np, rwkv_np
    from poptransformer_b200 import synth
    z = np.load(path)
    kind = str(z["kind"])
    dims = dict(zip((str(k) for k in z["dims_keys"]), (int(v) for v in z["dims_vals"])))
    batch, max_len, seed = int(z["batch"]), int(z["max_len"]), int(z["seed"])
    if kind == "gpt2":
        sd = synth.gpt2_state_dict(**dims, seed=seed)
        orc = gpt2_np.GPT2Oracle(gpt2_np.GPT2Config(**dims, max_len=max_len), {k: v.numpy() for k, v in sd.items()}, batch)
    elif kind == "chatglm2":
        sd = synth.chatglm2_state_dict(**dims, seed=seed)
        orc = chatglm2_np.ChatGLM2Oracle(chatglm2_np.ChatGLM2Config(**dims, max_len=max_len), {k: v.numpy() for k, v in sd.items()}, batch)
    else:
        sd = synth.rwkv_state_dict(**dims, seed=seed)
        orc = rwkv_np.RWKVOracle(rwkv_np.RWKVConfig(**dims, max_len=max_len), {k: v.numpy() for k, v in sd.items()}, batch)
    return z, kind, dims, sd, orc


def _teacher_forced_logits(orc, kind, ids, n_steps):
    """Oracle logits along the REFERENCE stream: logits[t] are the scores for position t + 1 given the reference's tokens 0..t."""
    orc.reset()
    out = []
    for t in range(n_steps):
        out.append((orc.logits(ids[:, t]) if kind == "rwkv" else orc.logits(ids[:, t], t))[0].astype(np.float32))
    return out


def _reference_tokens_are_oracle_best(exp, logits, prompt, margin):
    """At every generated position the reference's token must be the oracle's best, or within `margin` of it."""
    for t in range(prompt - 1, len(logits)):
        for b in range(exp.shape[0]):
            gap = logits[t][b].max() - logits[t][b][exp[b, t + 1]]
            assert gap <= margin, f"row {b}, position {t + 1}: the reference's token is {gap} below the oracle's best"


def _first_divergences_are_ties(got, exp, logits, margin):
    """A row may leave the reference stream only where the oracle's two best logits (given the reference history) are within
    `margin`; after that the two streams are different continuations and are not compared."""
    for b in range(got.shape[0]):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            t = int(diff[0])
            top2 = np.sort(logits[t - 1][b])[-2:]
            assert top2[1] - top2[0] <= margin, f"row {b}: diverges at {t} with margin {top2[1] - top2[0]}"


def test_other_fixtures_exist():
    assert {os.path.basename(p).split("_")[0] for p in OTHER} == {"gpt2", "chatglm2", "rwkv"}


@pytest.mark.parametrize("path", OTHER, ids=[os.path.basename(p) for p in OTHER])
def test_oracle_reproduces_reference_model_code(path):
    """GPT-2 and RWKV: identical streams.  ChatGLM2: identical up to exact ties of two fp16 logits (the reference multiplies the
    fp16 rotate_half operand by a float32 constant, chatglm2/attention.py:107, which the stand-in evaluates in float32 and the
    oracle, like the CUDA kernel, in fp16; which of two equal logits wins then depends on the last bit of that product)."""
    z, kind, dims, sd, orc = _load_other(path)
    exp = z["output_ids"]
    logits = _teacher_forced_logits(orc, kind, exp, int(z["step"]))
    _reference_tokens_are_oracle_best(exp, logits, int(z["prompt"]), 1e-3 if kind == "chatglm2" else 0.0)
    if kind != "chatglm2":
        got = orc.generate(z["input_ids"], int(z["step"]), int(z["pad_id"]))
        assert np.array_equal(got, exp), "oracle and reference model code disagree on the greedy token stream"


@pytest.mark.gpu
@pytest.mark.parametrize("path", OTHER, ids=[os.path.basename(p) for p in OTHER])
def test_cuda_reproduces_reference_model_code(path, cuda):
    from poptransformer_b200 import chatglm2, gpt2, rwkv
    z, kind, dims, sd, orc = _load_other(path)
    batch, max_len, prompt, pad = int(z["batch"]), int(z["max_len"]), int(z["prompt"]), int(z["pad_id"])
    if kind == "gpt2":
        dec = gpt2.GPT2Decoder(gpt2.GPT2Config(**dims, max_len=max_len), sd, batch, device=cuda, pad_id=pad)
    elif kind == "chatglm2":
        dec = chatglm2.ChatGLM2Decoder(chatglm2.ChatGLM2Config(**dims, max_len=max_len), sd, batch, device=cuda, pad_id=pad)
    else:
        dec = rwkv.RWKVDecoder(rwkv.RWKVConfig(**dims, max_len=max_len), sd, batch, device=cuda, pad_id=pad)
    got = dec.run(z["input_ids"], max_loop=int(z["step"]))["Loop:0"]
    exp = z["output_ids"]
    assert np.array_equal(got[:, :prompt], exp[:, :prompt])
    _first_divergences_are_ties(got, exp, _teacher_forced_logits(orc, kind, exp, int(z["step"])), 2e-2)
    assert (got == exp).mean() > 0.8
