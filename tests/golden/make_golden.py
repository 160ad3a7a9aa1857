"""Generates the golden vectors that pin the oracle to the reference's own model code.

Runs the UNMODIFIED reference graph builders (poptransformer/models/llama2, layers, ops, utils from the reference
checkout) through the numpy stand-in for `popart` in oracle/popart_cpu, on seeded synthetic checkpoints, and stores the
inputs' seeds and the resulting id containers.  Only usable where the reference tree is available (the development
container); the fixtures it writes (tests/golden/*.npz) travel with the repository.

    python tests/golden/make_golden.py /path/to/PopTransformer [case]
"""
import logging
import os
import subprocess
import sys
import tempfile
import types

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("POPTRANSFORMER_REFERENCE", "")
if not REF:
    raise SystemExit("usage: make_golden.py /path/to/PopTransformer [case]")
sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle", "popart_cpu"), REF]

CASES = {
    # name: (dims, precision, int4 group (0 = fp16), batch, max_len, prompt_len, seed)
    "llama_tiny_fp16": (dict(n_layer=2, d_model=256, n_head=2, ffn=512, vocab=1000), "fp16", 0, 2, 40, 6, 11),
    "llama_tiny_int4": (dict(n_layer=2, d_model=256, n_head=2, ffn=512, vocab=1000), "int4", -1, 1, 40, 6, 12),
    "llama_small_int4": (dict(n_layer=3, d_model=512, n_head=4, ffn=1024, vocab=2000), "int4", -1, 2, 72, 10, 13),
}
# other model families: name: (model kind, dims, batch, max_len, prompt_len, seed); fp16 weights
OTHER = {
    "gpt2_tiny_fp16": ("gpt2", dict(n_layer=2, d_model=256, n_head=4, vocab=1000, n_positions=64), 2, 40, 6, 21),
    "chatglm2_tiny_fp16": ("chatglm2", dict(n_layer=2, d_model=512, n_head=4, n_group=2, ffn=768, vocab=1000), 2, 40, 6, 22),
    "rwkv_tiny_fp16": ("rwkv", dict(n_layer=4, d_model=256, ffn=1024, vocab=1000, rescale_every=2), 2, 40, 6, 23),
}


def run_other(name):
    """GPT-2 / ChatGLM2 / RWKV: the reference's own model classes on seeded synthetic checkpoints (fp16)."""
    kind, dims, batch, max_len, prompt, seed = OTHER[name]
    import popart                                       # the numpy stand-in
    from poptransformer_b200 import synth
    tmp = tempfile.mkdtemp()
    os.makedirs(os.path.join(tmp, "examples", kind))
    from oracle import c_ref
    os.symlink(c_ref.build(), os.path.join(tmp, "custom_ops.so"))
    os.chdir(os.path.join(tmp, "examples", kind))
    from poptransformer.utils.registry import REGISTRY
    from poptransformer.utils.tensor_type import TensorType
    for k, v in dict(num_replicas=1, batch_size=batch, batch_per_step=1, model_type="shard", enable_pipeline=False, precision="fp16").items():
        REGISTRY.register(k, v)
    REGISTRY.register("tensor_type", TensorType("fp16"))
    REGISTRY.register("logger", logging.getLogger("poptransformer"))
    pad_id = dims["vocab"] - 1
    tok = types.SimpleNamespace(pad_token_id=pad_id, eos_token_id=pad_id - 1)
    if kind == "gpt2":
        from poptransformer.models.gpt2.model import GPT2DecModel as Base
        sd = synth.gpt2_state_dict(**dims, seed=seed)
        cfg = types.SimpleNamespace(vocab_size=dims["vocab"], n_embd=dims["d_model"], layer_norm_epsilon=1e-5, n_head=dims["n_head"],
                                    n_layer=dims["n_layer"], n_positions=dims["n_positions"], pad_token_id=pad_id, eos_token_id=pad_id - 1)
        n_layer = dims["n_layer"]
    elif kind == "chatglm2":
        from poptransformer.models.chatglm2.model import ChatGLM2DecModel as Base
        sd = synth.chatglm2_state_dict(**dims, seed=seed)
        cfg = types.SimpleNamespace(padded_vocab_size=dims["vocab"], hidden_size=dims["d_model"], layernorm_epsilon=1e-5,
                                    multi_query_group_num=dims["n_group"], num_attention_heads=dims["n_head"], ffn_hidden_size=dims["ffn"],
                                    num_layers=dims["n_layer"], pad_token_id=pad_id, eos_token_id=pad_id - 1)
        n_layer = dims["n_layer"]
    else:
        from poptransformer.models.rwkv.model import RWKVDecodeModel as Base
        sd = synth.rwkv_state_dict(**dims, seed=seed)
        cfg = types.SimpleNamespace(vocab_size=dims["vocab"], hidden_size=dims["d_model"], intermediate_size=dims["ffn"],
                                    attention_hidden_size=dims["d_model"], layer_norm_epsilon=1e-5, num_hidden_layers=dims["n_layer"],
                                    rescale_every=dims["rescale_every"], pad_token_id=pad_id, eos_token_id=pad_id - 1)
        n_layer = dims["n_layer"]

    class Golden(Base):
        def prepare_state_dict(self):
            self.hf_tokenizer, self.hf_config = tok, cfg
            self.state_dict = sd
            self.register_state_dict()

    model = Golden(max_length=max_len, max_loop=max_len - 1, layer_per_ipu=[n_layer], early_stop=False, topk=1, outline_blocks=None)
    model.build_graph()
    ids = synth.prompt_ids(batch, prompt, max_len, dims["vocab"], pad_id, seed=seed).numpy()
    env = popart.run_graph(model.graph, {"input_ids": ids})
    out_ids, out_step = env["Loop:0"], env["Loop:1"]
    os.chdir(ROOT)
    np.savez(os.path.join(ROOT, "tests", "golden", name + ".npz"), input_ids=ids, output_ids=np.asarray(out_ids, dtype=np.int32),
             step=np.asarray(out_step, dtype=np.int32), kind=kind, dims_keys=np.array(list(dims.keys())), dims_vals=np.array(list(dims.values())),
             batch=batch, max_len=max_len, prompt=prompt, seed=seed, pad_id=pad_id, n_nodes=len(model.graph.nodes))
    print(name, "ok: step", out_step, "ids[0, :12]", np.asarray(out_ids)[0, :12])


def run_graph_case(name, out_path):
    """Records the graph the reference's unmodified LLAMA2DecModel emits for case `name` with the PRODUCT's recorder
    (poptransformer_b200/frontend/popart.py) and stores it without weights: the fixture the GPU front-end test lowers on a machine
    that has no reference checkout.  Same checkpoint seeds as the golden id streams of the same case."""
    if name in OTHER:
        return run_graph_case_other(name, out_path)
    dims, precision, group, batch, max_len, prompt, seed = CASES[name]
    sys.path[:0] = [os.path.join(ROOT, "poptransformer_b200", "frontend")]      # popart / poprt = the front end; hydra = the test stub
    import popart
    assert "frontend" in popart.__file__
    from poptransformer_b200 import synth
    from poptransformer_b200 import build as _b
    tmp = tempfile.mkdtemp()
    os.makedirs(os.path.join(tmp, "examples", "llama2"))
    os.symlink(_b.build(), os.path.join(tmp, "custom_ops.so"))      # the reference loads '../../custom_ops.so' at import (ops/customized.py:17-18)
    os.chdir(os.path.join(tmp, "examples", "llama2"))
    from poptransformer.utils.registry import REGISTRY
    from poptransformer.utils.tensor_type import TensorType
    for k, v in dict(num_replicas=1, batch_size=batch, batch_per_step=1, model_type="shard", enable_pipeline=False, precision=precision).items():
        REGISTRY.register(k, v)
    REGISTRY.register("tensor_type", TensorType(precision))
    REGISTRY.register("logger", logging.getLogger("poptransformer"))
    from poptransformer.models.llama2.model import LLAMA2DecModel
    pad_id = dims["vocab"] - 1
    sd = synth.llama_state_dict(**dims, seed=seed, device="cpu", int4_group=group)
    if group:
        sd = {k: (v.reshape(-1) if k.endswith("_scale") else v) for k, v in sd.items()}

    class GoldenLlama(LLAMA2DecModel):
        def prepare_state_dict(self):
            self.hf_tokenizer = types.SimpleNamespace(pad_token_id=pad_id, eos_token_id=pad_id - 1)
            self.hf_config = types.SimpleNamespace(vocab_size=dims["vocab"], hidden_size=dims["d_model"], rms_norm_eps=1e-5,
                                                   num_attention_heads=dims["n_head"], intermediate_size=dims["ffn"],
                                                   num_hidden_layers=dims["n_layer"], pad_token_id=pad_id, eos_token_id=pad_id - 1)
            self.state_dict = sd
            self.register_state_dict()

    model = GoldenLlama(max_length=max_len, max_loop=max_len - 1, layer_per_ipu=[dims["n_layer"]], early_stop=False)
    model.build_graph()
    os.chdir(ROOT)
    model.graph.save(out_path)
    # the recorded initializers are the checkpoint in the reference's storage layout: the lowering must recover the synthetic one
    from poptransformer_b200.frontend import lower
    plan = lower.analyze(model.graph)
    back = lower.state_dict_from_initializers(model.graph, plan)
    assert set(back) == set(sd) and all(np.array_equal(back[k].numpy().reshape(-1), sd[k].numpy().reshape(-1)) for k in sd)
    print(name, "graph recorded:", len(model.graph.nodes), "main nodes,", plan)


def run_graph_case_other(name, out_path):
    """The same for the reference's unmodified GPT2DecModel / ChatGLM2DecModel / RWKVDecodeModel (cases `gpt2_tiny_fp16`,
    `chatglm2_tiny_fp16`, `rwkv_tiny_fp16`): the graph recorded by the product's recorder, stored without weights, and the
    lowering's view of the checkpoint compared with the synthetic one."""
    kind, dims, batch, max_len, prompt, seed = OTHER[name]
    sys.path[:0] = [os.path.join(ROOT, "poptransformer_b200", "frontend")]
    import popart
    assert "frontend" in popart.__file__
    from poptransformer_b200 import synth
    from poptransformer_b200 import build as _b
    tmp = tempfile.mkdtemp()
    os.makedirs(os.path.join(tmp, "examples", kind))
    os.symlink(_b.build(), os.path.join(tmp, "custom_ops.so"))
    os.chdir(os.path.join(tmp, "examples", kind))
    from poptransformer.utils.registry import REGISTRY
    from poptransformer.utils.tensor_type import TensorType
    for k, v in dict(num_replicas=1, batch_size=batch, batch_per_step=1, model_type="shard", enable_pipeline=False, precision="fp16").items():
        REGISTRY.register(k, v)
    REGISTRY.register("tensor_type", TensorType("fp16"))
    REGISTRY.register("logger", logging.getLogger("poptransformer"))
    pad_id = dims["vocab"] - 1
    if kind == "gpt2":
        from poptransformer.models.gpt2.model import GPT2DecModel as Base
        sd = synth.gpt2_state_dict(**dims, seed=seed)
        cfg = types.SimpleNamespace(vocab_size=dims["vocab"], n_embd=dims["d_model"], layer_norm_epsilon=1e-5, n_head=dims["n_head"],
                                    n_layer=dims["n_layer"], n_positions=dims["n_positions"], pad_token_id=pad_id, eos_token_id=pad_id - 1)
    elif kind == "chatglm2":
        from poptransformer.models.chatglm2.model import ChatGLM2DecModel as Base
        sd = synth.chatglm2_state_dict(**dims, seed=seed)
        cfg = types.SimpleNamespace(padded_vocab_size=dims["vocab"], hidden_size=dims["d_model"], layernorm_epsilon=1e-5,
                                    multi_query_group_num=dims["n_group"], num_attention_heads=dims["n_head"], ffn_hidden_size=dims["ffn"],
                                    num_layers=dims["n_layer"], pad_token_id=pad_id, eos_token_id=pad_id - 1)
    else:
        from poptransformer.models.rwkv.model import RWKVDecodeModel as Base
        sd = synth.rwkv_state_dict(**dims, seed=seed)
        cfg = types.SimpleNamespace(vocab_size=dims["vocab"], hidden_size=dims["d_model"], intermediate_size=dims["ffn"],
                                    attention_hidden_size=dims["d_model"], layer_norm_epsilon=1e-5, num_hidden_layers=dims["n_layer"],
                                    rescale_every=dims["rescale_every"], pad_token_id=pad_id, eos_token_id=pad_id - 1)

    class GoldenGPT2(Base):
        def prepare_state_dict(self):
            self.hf_tokenizer, self.hf_config = types.SimpleNamespace(pad_token_id=pad_id, eos_token_id=pad_id - 1), cfg
            self.state_dict = sd
            self.register_state_dict()

    model = GoldenGPT2(max_length=max_len, max_loop=max_len - 1, layer_per_ipu=[dims["n_layer"]], early_stop=False, topk=1, outline_blocks=None)
    model.build_graph()
    os.chdir(ROOT)
    model.graph.save(out_path)
    from poptransformer_b200.frontend import lower
    plan = lower.analyze(model.graph)
    back = lower.state_dict_from_initializers(model.graph, plan)
    assert set(back) == set(sd) and all(np.array_equal(back[k].numpy(), sd[k].numpy()) for k in sd)
    print(name, "graph recorded:", len(model.graph.nodes), "main nodes,", plan)


def run_case(name):
    """Each case runs in a fresh interpreter: the reference keeps its graph and settings in a process-global registry."""
    dims, precision, group, batch, max_len, prompt, seed = CASES[name]
    import popart                                       # the numpy stand-in
    from poptransformer_b200 import synth
    # the reference loads '../../custom_ops.so' relative to the working directory at import time (ops/customized.py:17-18)
    tmp = tempfile.mkdtemp()
    os.makedirs(os.path.join(tmp, "examples", "llama2"))
    from oracle import c_ref
    os.symlink(c_ref.build(), os.path.join(tmp, "custom_ops.so"))
    os.chdir(os.path.join(tmp, "examples", "llama2"))

    from poptransformer.utils.registry import REGISTRY
    from poptransformer.utils.tensor_type import TensorType
    for k, v in dict(num_replicas=1, batch_size=batch, batch_per_step=1, model_type="shard", enable_pipeline=False, precision=precision).items():
        REGISTRY.register(k, v)
    REGISTRY.register("tensor_type", TensorType(precision))
    REGISTRY.register("logger", logging.getLogger("poptransformer"))
    from poptransformer.models.llama2.model import LLAMA2DecModel

    pad_id = dims["vocab"] - 1
    sd = synth.llama_state_dict(**dims, seed=seed, device="cpu", int4_group=group)
    if group:   # the reference's int4 checkpoints carry one scale per output channel, shape [out]
        sd = {k: (v.reshape(-1) if k.endswith("_scale") else v) for k, v in sd.items()}

    class GoldenLlama(LLAMA2DecModel):
        def prepare_state_dict(self):
            self.hf_tokenizer = types.SimpleNamespace(pad_token_id=pad_id, eos_token_id=pad_id - 1)
            self.hf_config = types.SimpleNamespace(vocab_size=dims["vocab"], hidden_size=dims["d_model"], rms_norm_eps=1e-5,
                                                   num_attention_heads=dims["n_head"], intermediate_size=dims["ffn"],
                                                   num_hidden_layers=dims["n_layer"], pad_token_id=pad_id, eos_token_id=pad_id - 1)
            self.state_dict = sd
            self.register_state_dict()

    model = GoldenLlama(max_length=max_len, max_loop=max_len - 1, layer_per_ipu=[dims["n_layer"]], early_stop=False)
    model.build_graph()
    ids = synth.prompt_ids(batch, prompt, max_len, dims["vocab"], pad_id, seed=seed).numpy()
    env = popart.run_graph(model.graph, {"input_ids": ids})
    out_ids, out_step = env["Loop:0"], env["Loop:1"]
    os.chdir(ROOT)
    np.savez(os.path.join(ROOT, "tests", "golden", name + ".npz"), input_ids=ids, output_ids=np.asarray(out_ids, dtype=np.int32),
             step=np.asarray(out_step, dtype=np.int32), dims=np.array([dims[k] for k in ("n_layer", "d_model", "n_head", "ffn", "vocab")]),
             group=group, batch=batch, max_len=max_len, prompt=prompt, seed=seed, pad_id=pad_id, n_nodes=len(model.graph.nodes))
    print(name, "ok: step", out_step, "ids[0, :12]", np.asarray(out_ids)[0, :12])


def run_checkpoint_preprocess(name="checkpoint_preprocess"):
    """The reference's own checkpoint pre-processing on tiny seeded checkpoints: GPT2DecModel.process_hf_model_state_dict
    (models/gpt2/model.py:154-166) and RWKVDecodeModel.process_hf_model_state_dict (models/rwkv/model.py:150-155) are called
    unbound on stand-in `hf_model` objects that hold the tensors where the HF modules hold them; the ChatGLM2 splits
    (models/chatglm2/model.py:256-276) are inline in a method that downloads the model, so their few lines are replayed here
    on the same kind of tensors."""
    import popart                                       # the numpy stand-in
    import torch
    from oracle import c_ref
    tmp = tempfile.mkdtemp()
    os.makedirs(os.path.join(tmp, "examples", "ckpt"))
    os.symlink(c_ref.build(), os.path.join(tmp, "custom_ops.so"))
    os.chdir(os.path.join(tmp, "examples", "ckpt"))
    from poptransformer.utils.registry import REGISTRY
    from poptransformer.utils.tensor_type import TensorType
    for k, v in dict(num_replicas=1, batch_size=1, batch_per_step=1, model_type="shard", enable_pipeline=False, precision="fp16").items():
        REGISTRY.register(k, v)
    REGISTRY.register("tensor_type", TensorType("fp16"))
    REGISTRY.register("logger", logging.getLogger("poptransformer"))
    from poptransformer.models.gpt2.model import GPT2DecModel
    from poptransformer.models.rwkv.model import RWKVDecodeModel
    g = torch.Generator().manual_seed(41)
    rnd = lambda *shape: torch.randn(shape, generator=g)
    out = {}
    # ---- GPT-2: 2 blocks, n_embd 8, 2 heads; HF Conv1D layout [in, out]
    n_embd, n_head, n_blocks = 8, 2, 2
    blocks, hf = [], {}
    for i in range(n_blocks):
        t = {"attn.c_attn.weight": rnd(n_embd, 3 * n_embd), "attn.c_attn.bias": rnd(3 * n_embd), "attn.c_proj.weight": rnd(n_embd, n_embd),
             "mlp.c_fc.weight": rnd(n_embd, 4 * n_embd), "mlp.c_proj.weight": rnd(4 * n_embd, n_embd)}
        for k, v in t.items():
            hf[f"transformer.h.{i}.{k}"] = v.clone()
        blocks.append(types.SimpleNamespace(attn=types.SimpleNamespace(c_attn=types.SimpleNamespace(weight=t["attn.c_attn.weight"], bias=t["attn.c_attn.bias"]),
                                                                       c_proj=types.SimpleNamespace(weight=t["attn.c_proj.weight"])),
                                            mlp=types.SimpleNamespace(c_fc=types.SimpleNamespace(weight=t["mlp.c_fc.weight"]),
                                                                      c_proj=types.SimpleNamespace(weight=t["mlp.c_proj.weight"]))))
    fake = types.SimpleNamespace(hf_config=types.SimpleNamespace(n_embd=n_embd, n_head=n_head), logger=logging.getLogger("x"),
                                 hf_model=types.SimpleNamespace(transformer=types.SimpleNamespace(h=blocks)))
    GPT2DecModel.process_hf_model_state_dict(fake)
    for k, v in hf.items():
        out["gpt2_in/" + k] = v.numpy()
    for i, b in enumerate(blocks):
        out[f"gpt2_out/transformer.h.{i}.attn.c_attn.weight"] = b.attn.c_attn.weight.numpy().copy()
        out[f"gpt2_out/transformer.h.{i}.attn.c_attn.bias"] = b.attn.c_attn.bias.numpy().copy()
        out[f"gpt2_out/transformer.h.{i}.attn.c_proj.weight"] = b.attn.c_proj.weight.numpy().copy()
        out[f"gpt2_out/transformer.h.{i}.mlp.c_fc.weight"] = b.mlp.c_fc.weight.numpy().copy()
        out[f"gpt2_out/transformer.h.{i}.mlp.c_proj.weight"] = b.mlp.c_proj.weight.numpy().copy()
    # ---- RWKV: 5 blocks, rescale_every 2
    rblocks, rin = [], {}
    for i in range(5):
        a, f = rnd(6, 6), rnd(6, 12)
        rin[f"rwkv.blocks.{i}.attention.output.weight"], rin[f"rwkv.blocks.{i}.feed_forward.value.weight"] = a.clone(), f.clone()
        rblocks.append(types.SimpleNamespace(attention=types.SimpleNamespace(output=types.SimpleNamespace(weight=a)),
                                             feed_forward=types.SimpleNamespace(value=types.SimpleNamespace(weight=f))))
    fake = types.SimpleNamespace(hf_config=types.SimpleNamespace(rescale_every=2), hf_model=types.SimpleNamespace(rwkv=types.SimpleNamespace(blocks=rblocks)))
    RWKVDecodeModel.process_hf_model_state_dict(fake)
    for k, v in rin.items():
        out["rwkv_in/" + k] = v.numpy()
    for i, b in enumerate(rblocks):
        out[f"rwkv_out/rwkv.blocks.{i}.attention.output.weight"] = b.attention.output.weight.numpy().copy()
        out[f"rwkv_out/rwkv.blocks.{i}.feed_forward.value.weight"] = b.feed_forward.value.weight.numpy().copy()
    # ---- ChatGLM2: hidden 8, 2 kv groups x 2 channels -> qkv rows 8 + 8; MLP 2 x 6 rows (chatglm2/model.py:260-276 replayed)
    hidden = 8
    cin = {"transformer.encoder.layers.0.self_attention.query_key_value.weight": rnd(16, hidden),
           "transformer.encoder.layers.0.self_attention.query_key_value.bias": rnd(16),
           "transformer.encoder.layers.0.mlp.dense_h_to_4h.weight": rnd(12, hidden),
           "transformer.encoder.layers.0.mlp.dense_4h_to_h.weight": rnd(hidden, 6)}
    sd = {k: v.clone() for k, v in cin.items()}
    for k in list(sd.keys()):
        if "query_key_value" in k:
            weight_np = sd.pop(k)
            weight_1, weight_2 = np.split(weight_np, [hidden], axis=0)
            sd[k.replace("query_key_value", "query")] = weight_1
            sd[k.replace("query_key_value", "key_value")] = weight_2
        if "dense_h_to_4h" in k:
            weight_np = sd.pop(k)
            weight_1, weight_2 = weight_np.chunk(2, dim=0)
            sd[k.replace("dense_h_to_4h", "dense_h_to_4h_1")] = weight_1
            sd[k.replace("dense_h_to_4h", "dense_h_to_4h_2")] = weight_2
    for k, v in cin.items():
        out["chatglm2_in/" + k] = v.numpy()
    for k, v in sd.items():
        out["chatglm2_out/" + k] = np.asarray(v)
    os.chdir(ROOT)
    np.savez(os.path.join(ROOT, "tests", "golden", name + ".npz"), **out)
    print(name, "ok:", len(out), "arrays")


def run_tp_strategies(name="tp_strategies"):
    """The reference's load-time weight slicing (utils/param_handler/tensor_parallel_strategy.py:21-70, the sharded embedding
    weight of :38-45 and ChatGLM2's rearrange_tp_weights, models/chatglm2/model.py:29-49) on small seeded integer-valued arrays.
    Weights are in the reference's [in, out] orientation; every result has the replica axis first."""
    import popart                                       # the numpy stand-in
    import torch
    from oracle import c_ref
    tmp = tempfile.mkdtemp()                            # poptransformer/ops/customized.py:17-18 loads ../../custom_ops.so
    os.makedirs(os.path.join(tmp, "examples", "tp"))
    os.symlink(c_ref.build(), os.path.join(tmp, "custom_ops.so"))
    os.chdir(os.path.join(tmp, "examples", "tp"))
    from poptransformer.utils.registry import REGISTRY
    from poptransformer.utils.tensor_type import TensorType
    for k, v in dict(num_replicas=2, batch_size=1, batch_per_step=1, model_type="tp", enable_pipeline=False, precision="fp16").items():
        REGISTRY.register(k, v)
    REGISTRY.register("tensor_type", TensorType("fp16"))
    REGISTRY.register("logger", logging.getLogger("poptransformer"))
    from poptransformer.utils.param_handler import tensor_parallel_strategy as T
    from poptransformer.models.chatglm2.model import rearrange_tp_weights
    rng = np.random.default_rng(31)
    arr = lambda *shape: rng.integers(-99, 100, size=shape).astype(np.float32)
    out = {}
    w, b = arr(6, 10), arr(10)
    out.update(start_w=w, start_b=b, start_w_tp4=T.shard(w, 4, -1), start_b_tp4=T.shard(b, 4, -1),     # 10 outputs padded to 12
               end_w=arr(8, 6), end_b=arr(6))
    out.update(end_w_tp2=T.shard(out["end_w"], 2, 0), end_b_tp2=T.repeat(out["end_b"], 2))
    qkv_w, qkv_b = arr(4, 24), arr(24)
    out.update(qkv_w=qkv_w, qkv_b=qkv_b, qkv_w_tp2=T.shard_fused_qkv(qkv_w, 2, -1), qkv_b_tp2=T.shard_fused_qkv(qkv_b, 2, -1))
    REGISTRY.register("query_size", 16)
    REGISTRY.register("key_value_size", 4)
    mq_w, mq_b = arr(4, 16), arr(16)                    # the ChatGLM2 query weight: the key/value parts of the split are empty
    out.update(mq_w=mq_w, mq_b=mq_b, mq_w_tp2=T.shard_multi_query_qkv(mq_w, 2, -1), mq_b_tp2=T.shard_multi_query_qkv(mq_b, 2, -1))
    mqf_w = arr(4, 24)                                  # a fused q | k | v weight: 16 query, 4 key, 4 value features
    out.update(mqf_w=mqf_w, mqf_w_tp2=T.shard_multi_query_qkv(mqf_w, 2, -1))
    emb = arr(11, 4)
    out.update(emb=emb, emb_tp4=T.build_sharded_weight(emb, 4, 11, 4))
    q_hf, dense_hf = arr(16, 4), arr(4, 16)            # HF orientation: query [out = 8 heads x 2, in], dense [out, in = 8 heads x 2]
    for n in (2, 4):
        out[f"rearr_q_tp{n}"] = rearrange_tp_weights(torch.from_numpy(q_hf), 8, n, axis=0).numpy()
        out[f"rearr_dense_tp{n}"] = rearrange_tp_weights(torch.from_numpy(dense_hf), 8, n, axis=1).numpy()
    out.update(rearr_q=q_hf, rearr_dense=dense_hf)
    np.savez(os.path.join(ROOT, "tests", "golden", name + ".npz"), **out)
    print(name, "ok:", sorted(out))


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[2].endswith(":graph"):       # e.g. llama_tiny_int4:graph [output path]
        case = sys.argv[2].split(":")[0]
        run_graph_case(case, sys.argv[3] if len(sys.argv) > 3 else os.path.join(ROOT, "tests", "golden", case + "_graph.json"))
    elif len(sys.argv) > 2:
        (run_tp_strategies if sys.argv[2] == "tp_strategies" else run_checkpoint_preprocess if sys.argv[2] == "checkpoint_preprocess"
         else run_case if sys.argv[2] in CASES else run_other)(sys.argv[2])
    else:
        for case in list(CASES) + list(OTHER) + ["tp_strategies", "checkpoint_preprocess", "llama_tiny_int4:graph", "llama_tiny_fp16:graph", "gpt2_tiny_fp16:graph", "chatglm2_tiny_fp16:graph", "rwkv_tiny_fp16:graph"]:
            subprocess.run([sys.executable, os.path.abspath(__file__), REF, case], check=True)
