"""Lowering of a recorded PopTransformer decode graph to this package's decoders.

`lower(builder)` takes the main graph recorded by `frontend/popart.py` from the reference's unmodified model code,
checks that it is the decode loop this backend implements, reads the model's shapes and its checkpoint out of the graph, and
returns (plan, decoder).  The check is structural: the loop body must consist of the embedding gather, `n_layer` blocks whose
sequence of significant ops is exactly that of the reference's block (models/llama2/model.py:28-46, llama2/attention.py:64-122,
llama2/mlp.py:20-28), the final norm + LM head + top-1 (layers/lm_head.py:47-57) and the loop carry
(models/base_model.py:313-355); anything else is refused, as PopART refuses a graph it has no lowering for.
"""
import re
from types import SimpleNamespace

import numpy as np


class UnsupportedGraph(RuntimeError):
    pass


# ops that only move / reshape / retype data, or produce constants: not part of a block's skeleton
_LAYOUT_OPS = {"onnx.constant", "onnx.reshape", "onnx.transpose", "onnx.cast", "onnx.unsqueeze", "onnx.squeeze", "onnx.split", "onnx.concat",
               "custom.Remap", "custom.Int4ToHalf"}

# the significant ops of one Llama-2 block, in the order the reference emits them
_LLAMA_BLOCK = [
    "onnx.mul", "onnx.reducemean", "onnx.add", "onnx.sqrt", "onnx.reciprocal", "onnx.mul", "onnx.mul",      # RMSNorm (layers/rms_layer_norm.py:26-36)
    "onnx.matmul", "onnx.matmul", "onnx.matmul",                                                            # q, k, v
    "onnx.matmul", "onnx.sin", "onnx.cos",                                                                  # RoPE angle = step x inv_freq (attention.py:28-38)
    "onnx.mul", "onnx.mul", "onnx.mul", "onnx.add",                                                         # rotate q
    "onnx.mul", "onnx.mul", "onnx.mul", "onnx.add",                                                         # rotate k
    "custom.KVCache",
    "onnx.matmul", "onnx.mul", "onnx.add", "custom.SoftmaxV3", "onnx.matmul",                               # scores, scale, mask, softmax, P.V
    "onnx.matmul", "onnx.add",                                                                              # o_proj + residual
    "onnx.mul", "onnx.reducemean", "onnx.add", "onnx.sqrt", "onnx.reciprocal", "onnx.mul", "onnx.mul",      # RMSNorm
    "onnx.matmul", "gc.swish", "onnx.matmul", "onnx.mul", "onnx.matmul", "onnx.add",                        # SwiGLU MLP + residual
]
_LLAMA_TAIL = [
    "onnx.mul", "onnx.reducemean", "onnx.add", "onnx.sqrt", "onnx.reciprocal", "onnx.mul", "onnx.mul",      # final norm
    "onnx.matmul", "onnx.topk",                                                                             # LM head, k = 1
    "onnx.add", "gc.dynamicupdate", "gc.dynamicslice", "onnx.equal", "onnx.where", "gc.dynamicupdate",       # step_containers
    "onnx.equal", "gc.bitwiseor",                                                                           # step_loop_cond
]


def _skeleton(nodes):
    return [n.op for n in nodes if n.op not in _LAYOUT_OPS]


def _const_of(body, main, tensor_id):
    for g in (body, main):
        for n in g.nodes:
            if n.op == "onnx.constant" and n.outputs[0] == tensor_id:
                return np.asarray(n.attrs["value"])
    raise UnsupportedGraph(f"{tensor_id} is not a constant")


def _find_loop(main):
    loops = [n for n in main.nodes if n.op == "onnx.loop"]
    if len(loops) != 1:
        raise UnsupportedGraph(f"expected one Loop in the main graph, found {len(loops)}")
    loop = loops[0]
    return loop, loop.attrs["body"], int(_const_of(main, main, loop.inputs[0]))


def analyze(main):
    """Recognises the recorded graph; returns a plan (family, shapes, ids, state_dict as numpy arrays in checkpoint layout)."""
    loop, body, max_loop = _find_loop(main)
    names = list(main.initializers)
    layer_ids = sorted({int(m.group(1)) for k in names for m in [re.match(r"model\.layers\.(\d+)\.self_attn\.q_proj\.weight$", k)] if m})
    if not layer_ids or "model.embed_tokens.weight" not in main.initializers or "lm_head.weight" not in main.initializers:
        raise UnsupportedGraph("no Llama-2 decode graph found (this front end lowers LLAMA2DecModel); initializers: " + ", ".join(names[:6]))
    n_layer = len(layer_ids)
    if layer_ids != list(range(n_layer)):
        raise UnsupportedGraph("transformer blocks are not numbered 0 .. n-1")

    # ---- the loop body: gather, blocks, tail
    nodes = body.nodes
    gathers = [i for i, n in enumerate(nodes) if n.op == "onnx.gather"]
    if len(gathers) != 1 or nodes[gathers[0]].inputs[0] != "model.embed_tokens.weight":
        raise UnsupportedGraph("expected one embedding gather from model.embed_tokens.weight")
    head = [i for i, n in enumerate(nodes) if n.op == "onnx.matmul" and "lm_head.weight" in n.inputs]
    if len(head) != 1:
        raise UnsupportedGraph("expected one LM-head matmul")
    # block l spans from the first node after the previous block to its last residual add (the node before the next block's
    # RMSNorm constant, found through the q_proj matmul's position)
    def weight_matmul(key):
        for i, n in enumerate(nodes):
            if n.op == "onnx.matmul" and (key in n.inputs or any(p.op == "custom.Int4ToHalf" and p.outputs[0] in n.inputs and p.inputs[0] == key
                                                                for p in nodes[max(0, i - 2):i])):
                return i
        raise UnsupportedGraph(f"no matmul with {key}")
    down_pos = [weight_matmul(f"model.layers.{l}.mlp.down_proj.weight") for l in range(n_layer)]
    block_end = []
    for l in range(n_layer):
        j = down_pos[l] + 1
        while j < len(nodes) and nodes[j].op != "onnx.add":
            j += 1
        block_end.append(j)
    start = gathers[0] + 1
    for l in range(n_layer):
        sk = _skeleton(nodes[start:block_end[l] + 1])
        if sk != _LLAMA_BLOCK:
            diff = next((i for i, (a, b) in enumerate(zip(sk, _LLAMA_BLOCK)) if a != b), min(len(sk), len(_LLAMA_BLOCK)))
            raise UnsupportedGraph(f"block {l} is not the reference's Llama-2 block (differs at significant op {diff}: "
                                   f"{sk[diff] if diff < len(sk) else 'end'} vs {_LLAMA_BLOCK[diff] if diff < len(_LLAMA_BLOCK) else 'end'})")
        start = block_end[l] + 1
    tail = _skeleton(nodes[start:])
    if tail[len(_LLAMA_TAIL):] == ["onnx.reducesum", "onnx.less"]:      # early_stop: keep_going = sum(stop_mask) < batch (base_model.py:348-352)
        tail = tail[:len(_LLAMA_TAIL)]
    if tail != _LLAMA_TAIL:
        raise UnsupportedGraph("the graph after the last block is not final norm + LM head + top-1 + loop carry: " + " ".join(_skeleton(nodes[start:])))

    # ---- shapes and constants
    emb = main.initializers["model.embed_tokens.weight"]
    vocab, d_model = (emb.shape if emb is not None else main.initializer_info["model.embed_tokens.weight"]["shape"])
    q_mm = nodes[weight_matmul("model.layers.0.self_attn.q_proj.weight")]
    reshape = next(n for n in nodes if n.op == "onnx.reshape" and n.inputs[0] == q_mm.outputs[0])
    batch, seq, n_head, head_dim = (int(v) for v in _const_of(body, main, reshape.inputs[1]))
    if seq != 1 or n_head * head_dim != d_model:
        raise UnsupportedGraph(f"q is reshaped to [{batch}, {seq}, {n_head}, {head_dim}]: expected one new token per step and n_head * head_dim = d_model")
    kv = [n for n in nodes if n.op == "custom.KVCache"]
    if len(kv) != n_layer or any(n.attrs.get("fp8") for n in kv) or any(n.attrs["step_len"] != 1 or n.attrs["sequence_axis"] != 3 for n in kv):
        raise UnsupportedGraph("expected one fp16 KVCache op per block with step_len 1 on axis 3")
    max_len = int(kv[0].attrs["max_len"])
    sm = [n for n in nodes if n.op == "custom.SoftmaxV3"]
    if any(n.attrs.get("stable_mode") for n in sm):
        raise UnsupportedGraph("decode softmax is expected without max subtraction (stable_mode False)")
    gate = main.initializers["model.layers.0.mlp.gate_proj.weight"]
    gate_shape = gate.shape if gate is not None else main.initializer_info["model.layers.0.mlp.gate_proj.weight"]["shape"]
    int4 = any(n.op == "custom.Int4ToHalf" for n in nodes)
    ffn = int(gate_shape[0] if int4 else gate_shape[1])          # int4 weights stay [out, in / 2]; fp16 weights are stored [in, out]
    first_norm_add = next(n for n in nodes[gathers[0]:] if n.op == "onnx.add")
    eps = float(_const_of(body, main, first_norm_add.inputs[1]))
    topk = next(n for n in nodes if n.op == "onnx.topk")
    if int(_const_of(body, main, topk.inputs[1])) != 1:
        raise UnsupportedGraph("only greedy decoding (top-k 1) is lowered")
    equals = [n for n in nodes if n.op == "onnx.equal"]
    pad_id, eos_id = int(_const_of(body, main, equals[0].inputs[1])), int(_const_of(body, main, equals[1].inputs[1]))
    cond = body.outputs[0]
    early_stop = not any(n.op == "onnx.constant" and n.outputs[0] == cond for n in nodes)
    return SimpleNamespace(family="llama2", n_layer=n_layer, d_model=int(d_model), n_head=n_head, head_dim=head_dim, ffn=ffn, vocab=int(vocab), eps=eps,
                           batch=batch, max_len=max_len, max_loop=max_loop, pad_id=pad_id, eos_id=eos_id, int4=int4, early_stop=early_stop)


def state_dict_from_initializers(main, plan):
    """The checkpoint as the decoders take it (HF layout: linear weights [out, in]).  The reference stores fp16 linear weights
    transposed, [in, out] (layers/linear.py:32), int4 weights as int8 [out, in / 2] with `<key>_scale` [out]
    (precision_strategy.py:24-42), norms and the embedding as they are; the LM head goes through Linear too."""
    import torch
    sd = {}
    for key, arr in main.initializers.items():
        if arr is None:
            raise UnsupportedGraph(f"initializer {key} has no data attached")
        a = np.asarray(arr)
        is_linear = key.endswith(("_proj.weight", "lm_head.weight"))
        if is_linear and a.dtype != np.int8:
            a = np.ascontiguousarray(a.T)
        sd[key] = torch.from_numpy(np.ascontiguousarray(a))
    return sd


def lower(main, device=None, **decoder_kwargs):
    """(plan, decoder) for the recorded graph, the decoder built on `device` (default: the current CUDA device)."""
    import torch

    from poptransformer_b200 import llama
    plan = analyze(main)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    sd = state_dict_from_initializers(main, plan)
    group = 0
    if plan.int4:
        w = sd["model.layers.0.self_attn.q_proj.weight"]
        group = (w.shape[1] * 2) // max(1, sd["model.layers.0.self_attn.q_proj.weight_scale"].numel() // w.shape[0])
    cfg = llama.LlamaConfig(n_layer=plan.n_layer, d_model=plan.d_model, n_head=plan.n_head, ffn=plan.ffn, vocab=plan.vocab, eps=plan.eps,
                            max_len=plan.max_len, int4_group=group)
    dec = llama.LlamaDecoder(cfg, sd, plan.batch, device=device, pad_id=plan.pad_id, eos_id=plan.eos_id, early_stop=plan.early_stop,
                             **decoder_kwargs)
    return plan, dec
