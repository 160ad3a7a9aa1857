"""The GPU front end behind the reference's own graph-building API (poptransformer_b200/frontend).

The fixtures tests/golden/llama_tiny_*_graph.json are the graphs the reference's UNMODIFIED LLAMA2DecModel emits into the product's
`popart` recorder (tests/golden/make_golden.py <reference> llama_tiny_int4:graph), stored without weights.  Where the reference
checkout is present the recording is repeated and must reproduce the fixture; everywhere, the fixture must be recognised by the
lowering; on a GPU the recorded graph is run through `popart.InferenceSession` and must reproduce the id streams that the same
model code produced through the numpy interpreter (tests/golden/llama_tiny_*.npz)."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
# the reference tree: $POPTRANSFORMER_REFERENCE, else a directory named `reference` beside the repository (absent on a GPU box)
REFERENCE = os.environ.get("POPTRANSFORMER_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
CASES = ["llama_tiny_int4", "llama_tiny_fp16"]


def _frontend():
    from poptransformer_b200 import frontend
    return frontend.install()


def _fixture(case):
    popart = _frontend()
    return popart.Builder.load(os.path.join(HERE, "golden", case + "_graph.json"))


@pytest.mark.parametrize("case", CASES)
def test_fixture_graph_is_recognised(case):
    from poptransformer_b200.frontend import lower
    z = np.load(os.path.join(HERE, "golden", case + ".npz"))
    plan = lower.analyze(_fixture(case))
    n_layer, d_model, n_head, ffn, vocab = (int(v) for v in z["dims"])
    assert (plan.family, plan.n_layer, plan.d_model, plan.n_head, plan.ffn, plan.vocab) == ("llama2", n_layer, d_model, n_head, ffn, vocab)
    assert (plan.batch, plan.max_len, plan.max_loop, plan.pad_id) == (int(z["batch"]), int(z["max_len"]), int(z["max_len"]) - 1, int(z["pad_id"]))
    assert plan.int4 == (int(z["group"]) != 0) and not plan.early_stop and abs(plan.eps - 1e-5) < 1e-9


OTHER = {"gpt2_tiny_fp16": "gpt2", "chatglm2_tiny_fp16": "chatglm2", "rwkv_tiny_fp16": "rwkv"}


def _other_dims(case):
    z = np.load(os.path.join(HERE, "golden", case + ".npz"))
    return z, dict(zip((str(k) for k in z["dims_keys"]), (int(v) for v in z["dims_vals"])))


@pytest.mark.parametrize("case", list(OTHER))
def test_other_family_fixture_graph_is_recognised(case):
    from poptransformer_b200.frontend import lower
    z, dims = _other_dims(case)
    plan = lower.analyze(_fixture(case))
    assert (plan.family, plan.n_layer, plan.d_model, plan.vocab) == (OTHER[case], dims["n_layer"], dims["d_model"], dims["vocab"])
    if plan.family == "gpt2":
        assert (plan.n_head, plan.n_positions) == (dims["n_head"], dims["n_positions"])
    elif plan.family == "chatglm2":
        assert (plan.n_head, plan.n_group, plan.ffn) == (dims["n_head"], dims["n_group"], dims["ffn"])
    else:
        assert (plan.ffn, plan.rescale_every) == (dims["ffn"], dims["rescale_every"])
    assert (plan.batch, plan.max_len, plan.max_loop, plan.pad_id) == (int(z["batch"]), int(z["max_len"]), int(z["max_len"]) - 1, int(z["pad_id"]))
    assert not plan.early_stop and abs(plan.eps - 1e-5) < 1e-9
    g = _fixture(case)
    body = next(n for n in g.nodes if n.op == "onnx.loop").attrs["body"]
    act = next(n for n in body.nodes if n.op in ("gc.gelu", "gc.swish", "onnx.relu"))
    act.op = "gc.swish" if act.op == "gc.gelu" else "gc.gelu"                 # not the reference's block any more
    with pytest.raises(lower.UnsupportedGraph, match="block 0"):
        lower.analyze(g)


def test_other_graphs_are_refused():
    from poptransformer_b200.frontend import lower
    g = _fixture("llama_tiny_fp16")
    body = next(n for n in g.nodes if n.op == "onnx.loop").attrs["body"]
    swish = next(n for n in body.nodes if n.op == "gc.swish")
    swish.op = "gc.gelu"                                   # a block that is not the reference's Llama block
    with pytest.raises(lower.UnsupportedGraph, match="block 0"):
        lower.analyze(g)
    g2 = _fixture("llama_tiny_fp16")
    g2.initializers = {k.replace("model.layers", "transformer.h"): v for k, v in g2.initializers.items()}
    with pytest.raises(lower.UnsupportedGraph, match="no Llama-2, GPT-2, ChatGLM2 or RWKV decode graph"):
        lower.analyze(g2)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "poptransformer")), reason="reference checkout not present")
@pytest.mark.parametrize("case", CASES + list(OTHER))
def test_reference_model_code_records_the_fixture(case, tmp_path):
    out = str(tmp_path / "graph.json")
    subprocess.run([sys.executable, os.path.join(HERE, "golden", "make_golden.py"), REFERENCE, case + ":graph", out], check=True, capture_output=True)
    assert json.load(open(out)) == json.load(open(os.path.join(HERE, "golden", case + "_graph.json")))


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES)
def test_session_runs_the_recorded_graph_on_the_gpu(case, cuda):
    from oracle import llama_np
    from poptransformer_b200 import synth
    popart = _frontend()
    z = np.load(os.path.join(HERE, "golden", case + ".npz"))
    dims = dict(zip(("n_layer", "d_model", "n_head", "ffn", "vocab"), (int(v) for v in z["dims"])))
    group, batch, max_len, prompt = int(z["group"]), int(z["batch"]), int(z["max_len"]), int(z["prompt"])
    sd = synth.llama_state_dict(**dims, seed=int(z["seed"]), device="cpu", int4_group=group)
    g = _fixture(case)
    for key in g.initializers:        # the checkpoint in the reference's storage layout (layers/linear.py:32, precision_strategy.py:24-42)
        a = sd[key].numpy()
        if key.endswith(("_proj.weight", "lm_head.weight")) and a.dtype != np.int8:
            a = np.ascontiguousarray(a.T)
        g.initializers[key] = a.reshape(g.initializer_info[key]["shape"])
    session = popart.InferenceSession(fnModel=g.getModelProto(), dataFlow=popart.DataFlow(1, {"Loop:0": popart.AnchorReturnType("ALL"),
                                                                                           "Loop:1": popart.AnchorReturnType("ALL")}),
                                      deviceInfo=popart.DeviceManager().acquireAvailableDevice(1), userOptions=popart.SessionOptions())
    session.prepareDevice()
    session.weightsFromHost()
    anchors = session.initAnchorArrays()
    assert session.decoder.persistent == (group != 0 and batch <= 2)
    for _ in range(2):                # Session.run twice, like examples/llama2/inference.py:26-31: the caches are re-zeroed at step 0
        session.run(popart.PyStepIO({"input_ids": z["input_ids"]}, anchors))
    got, exp = anchors["Loop:0"], z["output_ids"]
    assert int(anchors["Loop:1"]) == max_len - 1
    assert np.array_equal(got[:, :prompt], exp[:, :prompt])
    cfg = llama_np.LlamaConfig(**dims, max_len=max_len, group=0)
    sd_np = {k: (v.numpy().reshape(-1) if k.endswith("_scale") else v.numpy()) for k, v in sd.items()}
    orc = llama_np.LlamaOracle(cfg, sd_np, batch)
    orc.reset()
    logits = [orc.logits(exp[:, t], t)[0].astype(np.float32) for t in range(max_len - 1)]
    for b in range(batch):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            t = int(diff[0])
            top2 = np.sort(logits[t - 1][b])[-2:]
            assert top2[1] - top2[0] <= 2e-2, f"row {b}: leaves the reference stream at {t} with margin {top2[1] - top2[0]}"


@pytest.mark.gpu
@pytest.mark.parametrize("case", list(OTHER))
def test_session_runs_the_recorded_graph_of_another_family_on_the_gpu(case, cuda):
    """The graph the reference's unmodified GPT2DecModel / ChatGLM2DecModel / RWKVDecodeModel recorded, its initializers filled with the synthetic
    checkpoint in the reference's storage layout, through InferenceSession: the id stream of the reference's own run
    (tests/golden/<case>.npz) up to numerical ties of the restatement's top two logits."""
    from oracle import chatglm2_np, gpt2_np, rwkv_np
    from poptransformer_b200 import synth
    popart = _frontend()
    z, dims = _other_dims(case)
    fam = OTHER[case]
    batch, max_len, prompt = int(z["batch"]), int(z["max_len"]), int(z["prompt"])
    sd = {"gpt2": synth.gpt2_state_dict, "chatglm2": synth.chatglm2_state_dict, "rwkv": synth.rwkv_state_dict}[fam](**dims, seed=int(z["seed"]))
    linear = (".c_attn.weight", ".c_proj.weight", ".c_fc.weight") if fam == "gpt2" else (".weight",)
    g = _fixture(case)
    for key in g.initializers:
        if fam == "gpt2" and key == "lm_head.weight":
            continue                  # unused: the head is tied to the token embedding
        a = sd[key].numpy()
        if a.ndim == 2 and key.endswith(linear) and "embeddings" not in key and "wte" not in key and "wpe" not in key:
            a = np.ascontiguousarray(a.T)            # layers/linear.py:32 stores [in, out]
        g.initializers[key] = a.reshape(g.initializer_info[key]["shape"])
    session = popart.InferenceSession(fnModel=g.getModelProto(), dataFlow=popart.DataFlow(1, {"Loop:0": popart.AnchorReturnType("ALL"),
                                                                                           "Loop:1": popart.AnchorReturnType("ALL")}),
                                      deviceInfo=popart.DeviceManager().acquireAvailableDevice(1), userOptions=popart.SessionOptions())
    session.prepareDevice()
    session.weightsFromHost()
    anchors = session.initAnchorArrays()
    assert session.plan.family == fam
    for _ in range(2):
        session.run(popart.PyStepIO({"input_ids": z["input_ids"]}, anchors))
    got, exp = anchors["Loop:0"], z["output_ids"]
    assert int(anchors["Loop:1"]) == max_len - 1
    assert np.array_equal(got[:, :prompt], exp[:, :prompt])
    sd_np = {k: v.numpy() for k, v in sd.items()}
    if fam == "gpt2":
        orc = gpt2_np.GPT2Oracle(gpt2_np.GPT2Config(**dims, max_len=max_len), sd_np, batch)
    elif fam == "chatglm2":
        orc = chatglm2_np.ChatGLM2Oracle(chatglm2_np.ChatGLM2Config(**dims, max_len=max_len), sd_np, batch)
    else:
        orc = rwkv_np.RWKVOracle(rwkv_np.RWKVConfig(**dims, max_len=max_len), sd_np, batch)
    orc.reset()
    step_logits = (lambda t: orc.logits(exp[:, t])) if fam == "rwkv" else (lambda t: orc.logits(exp[:, t], t))
    logits = [np.asarray(step_logits(t)[0]).astype(np.float32) for t in range(max_len - 1)]
    for b in range(batch):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            t = int(diff[0])
            top2 = np.sort(logits[t - 1][b])[-2:]
            assert top2[1] - top2[0] <= 2e-2, f"row {b}: leaves the reference stream at {t} with margin {top2[1] - top2[0]}"
    assert (got == exp).mean() >= 0.9
