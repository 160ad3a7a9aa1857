"""Checkpoint ingestion (poptransformer_b200/checkpoint.py) against the reference's own pre-processing: the fixture
tests/golden/checkpoint_preprocess.npz holds tiny seeded HF-layout checkpoints and what GPT2DecModel.process_hf_model_state_dict,
RWKVDecodeModel.process_hf_model_state_dict and the ChatGLM2 splits of the reference make of them
(tests/golden/make_golden.py <reference> checkpoint_preprocess).  Bit-exact: these are copies, transposes and exact scalings."""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
Z = np.load(os.path.join(HERE, "golden", "checkpoint_preprocess.npz"))


def _part(prefix):
    return {k[len(prefix):]: Z[k] for k in Z.files if k.startswith(prefix)}


def _same(got, exp):
    assert set(got) == set(exp), sorted(set(got) ^ set(exp))
    for k in exp:
        assert np.array_equal(got[k].numpy(), exp[k]), k


def test_gpt2_prescale_and_transposes():
    from poptransformer_b200 import checkpoint
    sd = {k: torch.from_numpy(v.copy()) for k, v in _part("gpt2_in/").items()}
    _same(checkpoint.gpt2_from_hf(sd, n_embd=8, n_head=2), _part("gpt2_out/"))


def test_rwkv_rescale():
    from poptransformer_b200 import checkpoint
    sd = {k: torch.from_numpy(v.copy()) for k, v in _part("rwkv_in/").items()}
    _same(checkpoint.rwkv_from_hf(sd, rescale_every=2), _part("rwkv_out/"))


def test_chatglm2_splits():
    from poptransformer_b200 import checkpoint
    sd = {k: torch.from_numpy(v.copy()) for k, v in _part("chatglm2_in/").items()}
    _same(checkpoint.chatglm2_from_hf(sd, hidden_size=8), _part("chatglm2_out/"))


def test_int4_quantiser_produces_the_reference_checkpoint_format():
    """int8 weight under the key, fp16 `<key>_scale` of shape [out] (precision_strategy.py:24-42); embeddings and the head stay fp16; the
    numpy restatement of Int4ToHalf turns the pair back into weights within half a quantisation step."""
    from oracle import ops_np as O
    from poptransformer_b200 import checkpoint, synth
    sd = synth.llama_state_dict(n_layer=1, d_model=256, n_head=2, ffn=512, vocab=100, seed=3)
    q = checkpoint.quantize_linears_int4(checkpoint.llama_from_hf(sd), group=-1)
    assert q["model.embed_tokens.weight"].dtype == torch.float16 and q["lm_head.weight"].dtype == torch.float16
    key = "model.layers.0.mlp.down_proj.weight"
    assert q[key].dtype == torch.int8 and tuple(q[key].shape) == (256, 256) and tuple(q[key + "_scale"].shape) == (256,)
    back = O.int4_to_half(q[key].numpy(), q[key + "_scale"].numpy(), axis=1).T.astype(np.float32)      # [out, in]
    step = q[key + "_scale"].numpy().astype(np.float32)[:, None]
    assert np.all(np.abs(back - sd[key].numpy().astype(np.float32)) <= 0.51 * step + 1e-6)
    g = checkpoint.quantize_linears_int4(sd, group=128)
    assert tuple(g[key + "_scale"].shape) == (256, 4)


def test_fp8_quantiser_scale_is_amax_over_448():
    from poptransformer_b200 import checkpoint, synth
    sd = synth.llama_state_dict(n_layer=1, d_model=128, n_head=1, ffn=256, vocab=50, seed=4)
    q = checkpoint.quantize_linears_fp8(sd)
    key = "model.layers.0.self_attn.q_proj.weight"
    assert q[key].dtype == torch.uint8
    assert abs(float(q[key + "_scale"]) - float(sd[key].float().abs().max()) / 448.0) < 1e-9
