"""Lowering of a recorded PopTransformer decode graph to this package's decoders.

`lower(builder)` takes the main graph recorded by `frontend/popart.py` from the reference's unmodified model code,
checks that it is the decode loop this backend implements, reads the model's shapes and its checkpoint out of the graph, and
returns (plan, decoder).  The check is structural: the loop body must consist of the embedding gather(s), `n_layer` blocks whose
sequence of significant ops is exactly that of the reference's block (Llama-2: models/llama2/model.py:28-46,
llama2/attention.py:64-122, llama2/mlp.py:20-28; GPT-2: models/gpt2/model.py:28-49, gpt2/attention.py:42-86, layers/mlp.py:34-41;
ChatGLM2: models/chatglm2/model.py:95-117, chatglm2/attention.py:98-302, chatglm2/mlp.py:51-59; RWKV-4: models/rwkv/model.py:189-213,
rwkv/attention.py:46-105, rwkv/ffn.py:36-59),
the final norm + LM head + top-1 (layers/lm_head.py:47-57) and the loop carry (models/base_model.py:313-355); anything else is
refused, as PopART refuses a graph it has no lowering for.
"""
import re
from types import SimpleNamespace

import numpy as np


class UnsupportedGraph(RuntimeError):
    pass


# ops that only move / reshape / retype data, or produce constants: not part of a block's skeleton
_LAYOUT_OPS = {"onnx.constant", "onnx.reshape", "onnx.transpose", "onnx.cast", "onnx.unsqueeze", "onnx.squeeze", "onnx.split", "onnx.concat",
               "onnx.expand", "custom.Remap", "custom.Int4ToHalf"}

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


# the loop carry every decode model ends with: step_containers + step_loop_cond (models/base_model.py:313-355)
_CARRY = ["onnx.add", "gc.dynamicupdate", "gc.dynamicslice", "onnx.equal", "onnx.where", "gc.dynamicupdate", "onnx.equal", "gc.bitwiseor"]

# the significant ops of one GPT-2 block (models/gpt2/model.py:28-49, gpt2/attention.py:42-86, layers/mlp.py:34-41)
_GPT2_BLOCK = [
    "custom.NormCE", "onnx.matmul", "onnx.add",                                            # ln_1, c_attn + bias
    "custom.KVCache", "onnx.matmul", "onnx.add", "custom.SoftmaxV3", "onnx.matmul",        # cache, scores, mask, softmax, P.V
    "onnx.matmul", "onnx.add", "onnx.add",                                                 # c_proj + bias, residual
    "custom.NormCE", "onnx.matmul", "onnx.add", "gc.gelu", "onnx.matmul", "onnx.add", "onnx.add",   # ln_2, MLP, residual
]
_GPT2_TAIL = ["custom.NormCE", "onnx.matmul", "onnx.topk"] + _CARRY                        # ln_f, tied head, k = 1, loop carry


_RMSNORM = ["onnx.mul", "onnx.reducemean", "onnx.add", "onnx.sqrt", "onnx.reciprocal", "onnx.mul", "onnx.mul"]   # layers/rms_layer_norm.py:26-36
# the significant ops of one ChatGLM2 block (models/chatglm2/model.py:95-117, chatglm2/attention.py:98-302, chatglm2/mlp.py:51-59)
_CHATGLM2_BLOCK = _RMSNORM + [
    "onnx.matmul", "onnx.add", "onnx.matmul", "onnx.add",                                   # query, key_value (+bias)
    "onnx.matmul", "onnx.cos", "onnx.sin",                                                  # RoPE angle = step x inv_freq
    "onnx.mul", "onnx.mul", "onnx.mul", "onnx.add",                                         # rotate the first half of q (interleaved pairs)
    "onnx.mul", "onnx.mul", "onnx.mul", "onnx.add",                                         # rotate the first half of k
    "custom.KVCache",
    "onnx.matmul", "onnx.mul", "onnx.add", "custom.SoftmaxV3", "onnx.matmul",               # scores, scale, mask, softmax, P.V
    "onnx.matmul", "onnx.add",                                                              # dense + residual
] + _RMSNORM + ["onnx.matmul", "gc.swish", "onnx.matmul", "onnx.mul", "onnx.matmul", "onnx.add"]   # SwiGLU MLP + residual
_CHATGLM2_TAIL = _RMSNORM + ["onnx.matmul", "onnx.topk"] + _CARRY


def _common_fields(main, body, nodes, max_loop):
    """What every family's plan reads the same way: cache length, greedy head, pad / eos ids, early stop."""
    kv = [n for n in nodes if n.op == "custom.KVCache"]
    if any(n.attrs.get("fp8") for n in kv) or any(n.attrs["step_len"] != 1 or n.attrs["sequence_axis"] != 3 for n in kv):
        raise UnsupportedGraph("expected fp16 KVCache ops with step_len 1 on axis 3")
    if any(n.attrs.get("stable_mode") for n in nodes if n.op == "custom.SoftmaxV3"):
        raise UnsupportedGraph("decode softmax is expected without max subtraction (stable_mode False)")
    topk = next(n for n in nodes if n.op == "onnx.topk")
    if int(_const_of(body, main, topk.inputs[1])) != 1:
        raise UnsupportedGraph("only greedy decoding (top-k 1) is lowered")
    equals = [n for n in nodes if n.op == "onnx.equal"]
    cond = body.outputs[0]
    return dict(n_kv_ops=len(kv), max_len=int(kv[0].attrs["max_len"]), max_loop=max_loop,
                pad_id=int(_const_of(body, main, equals[0].inputs[1])), eos_id=int(_const_of(body, main, equals[1].inputs[1])),
                early_stop=not any(n.op == "onnx.constant" and n.outputs[0] == cond for n in nodes))


def _check_tail(nodes, start, want, what):
    tail = _skeleton(nodes[start:])
    if tail[len(want):] == ["onnx.reducesum", "onnx.less"]:      # early_stop: keep_going = sum(stop_mask) < batch (base_model.py:348-352)
        tail = tail[:len(want)]
    if tail != want:
        raise UnsupportedGraph(f"the graph after the last block is not {what}: " + " ".join(_skeleton(nodes[start:])))


def _analyze_gpt2(main, body, max_loop):
    """GPT2DecModel (models/gpt2/model.py): token + position embedding, blocks of NormCE / fused c_attn / KVCache attention with the
    fp16 softmax / c_proj / NormCE / GELU MLP, final NormCE and the head tied to the token embedding."""
    names = list(main.initializers)
    layer_ids = sorted({int(m.group(1)) for k in names for m in [re.match(r"transformer\.h\.(\d+)\.attn\.c_attn\.weight$", k)] if m})
    n_layer = len(layer_ids)
    if layer_ids != list(range(n_layer)) or "transformer.wpe.weight" not in main.initializers:
        raise UnsupportedGraph("GPT-2 blocks are not numbered 0 .. n-1, or the position embedding is missing")
    nodes = body.nodes
    gathers = [i for i, n in enumerate(nodes) if n.op == "onnx.gather"]
    if len(gathers) != 2 or [nodes[i].inputs[0] for i in gathers] != ["transformer.wte.weight", "transformer.wpe.weight"]:
        raise UnsupportedGraph("expected the token and the position embedding gathers")
    start = next(i for i in range(gathers[1] + 1, len(nodes)) if nodes[i].op == "onnx.add") + 1     # x = wte[id] + wpe[step]

    def weight_matmul(key):
        for i, n in enumerate(nodes):
            if n.op == "onnx.matmul" and key in n.inputs:
                return i
        raise UnsupportedGraph(f"no matmul with {key}")
    for l in range(n_layer):
        j, adds = weight_matmul(f"transformer.h.{l}.mlp.c_proj.weight") + 1, 0
        while j < len(nodes):                      # the block ends with the residual add, the second add behind the last matmul
            adds += nodes[j].op == "onnx.add"
            if adds == 2:
                break
            j += 1
        sk = _skeleton(nodes[start:j + 1])
        if sk != _GPT2_BLOCK:
            diff = next((i for i, (a, b) in enumerate(zip(sk, _GPT2_BLOCK)) if a != b), min(len(sk), len(_GPT2_BLOCK)))
            raise UnsupportedGraph(f"block {l} is not the reference's GPT-2 block (differs at significant op {diff}: "
                                   f"{sk[diff] if diff < len(sk) else 'end'} vs {_GPT2_BLOCK[diff] if diff < len(_GPT2_BLOCK) else 'end'})")
        start = j + 1
    _check_tail(nodes, start, _GPT2_TAIL, "final LayerNorm + tied head + top-1 + loop carry")
    head = next(n for n in nodes[start:] if n.op == "onnx.matmul")
    tr = next((n for n in nodes if n.op == "onnx.transpose" and n.outputs[0] in head.inputs), None)
    if tr is None or tr.inputs[0] != "transformer.wte.weight":
        raise UnsupportedGraph("the head is expected to be tied to transformer.wte.weight (layers/lm_head.py:47-57)")

    def shape_of(key):
        a = main.initializers[key]
        return tuple(a.shape) if a is not None else tuple(main.initializer_info[key]["shape"])
    vocab, d_model = shape_of("transformer.wte.weight")
    n_positions = shape_of("transformer.wpe.weight")[0]
    split = next(n for n in nodes if n.op == "onnx.split")                      # q | (k, v) of block 0
    reshape = next(n for n in nodes if n.op == "onnx.reshape" and n.inputs[0] == split.outputs[0])
    batch, seq, n_head, head_dim = (int(v) for v in _const_of(body, main, reshape.inputs[1]))
    if seq != 1 or n_head * head_dim != d_model:
        raise UnsupportedGraph(f"q is reshaped to [{batch}, {seq}, {n_head}, {head_dim}]: expected one new token per step and n_head * head_dim = d_model")
    norms = [n for n in nodes if n.op == "custom.NormCE"]
    eps = {float(n.attrs["epsilon"]) for n in norms}
    if len(norms) != 2 * n_layer + 1 or len(eps) != 1:
        raise UnsupportedGraph("expected two NormCE ops per block plus the final one, with one epsilon")
    common = _common_fields(main, body, nodes, max_loop)
    if common.pop("n_kv_ops") != n_layer:
        raise UnsupportedGraph("expected one KVCache op per block")
    return SimpleNamespace(family="gpt2", n_layer=n_layer, d_model=int(d_model), n_head=n_head, head_dim=head_dim, ffn=4 * int(d_model), vocab=int(vocab),
                           n_positions=int(n_positions), eps=eps.pop(), batch=batch, int4=False, **common)


def _analyze_chatglm2(main, body, max_loop):
    """ChatGLM2DecModel (models/chatglm2/model.py): RMSNorm, query + key_value with bias, interleaved RoPE on half of each head,
    multi-query KVCache attention with the fp16 softmax, dense, RMSNorm, SwiGLU MLP; final RMSNorm and the output layer."""
    pre = "transformer.encoder.layers."
    names = list(main.initializers)
    layer_ids = sorted({int(m.group(1)) for k in names for m in [re.match(r"transformer\.encoder\.layers\.(\d+)\.self_attention\.query\.weight$", k)] if m})
    n_layer = len(layer_ids)
    if layer_ids != list(range(n_layer)) or "transformer.output_layer.weight" not in main.initializers:
        raise UnsupportedGraph("ChatGLM2 blocks are not numbered 0 .. n-1, or the output layer is missing")
    nodes = body.nodes
    gathers = [i for i, n in enumerate(nodes) if n.op == "onnx.gather"]
    if len(gathers) != 1 or nodes[gathers[0]].inputs[0] != "transformer.embedding.word_embeddings.weight":
        raise UnsupportedGraph("expected one embedding gather from transformer.embedding.word_embeddings.weight")

    def weight_matmul(key):
        for i, n in enumerate(nodes):
            if n.op == "onnx.matmul" and key in n.inputs:
                return i
        raise UnsupportedGraph(f"no matmul with {key}")
    start = gathers[0] + 1
    for l in range(n_layer):
        j = weight_matmul(f"{pre}{l}.mlp.dense_4h_to_h.weight") + 1
        while j < len(nodes) and nodes[j].op != "onnx.add":
            j += 1
        sk = _skeleton(nodes[start:j + 1])
        if sk != _CHATGLM2_BLOCK:
            diff = next((i for i, (a, b) in enumerate(zip(sk, _CHATGLM2_BLOCK)) if a != b), min(len(sk), len(_CHATGLM2_BLOCK)))
            raise UnsupportedGraph(f"block {l} is not the reference's ChatGLM2 block (differs at significant op {diff}: "
                                   f"{sk[diff] if diff < len(sk) else 'end'} vs {_CHATGLM2_BLOCK[diff] if diff < len(_CHATGLM2_BLOCK) else 'end'})")
        start = j + 1
    _check_tail(nodes, start, _CHATGLM2_TAIL, "final RMSNorm + output layer + top-1 + loop carry")

    def shape_of(key):
        a = main.initializers[key]
        return tuple(a.shape) if a is not None else tuple(main.initializer_info[key]["shape"])
    vocab, d_model = shape_of("transformer.embedding.word_embeddings.weight")
    ffn = shape_of(f"{pre}0.mlp.dense_h_to_4h_1.weight")[1]                    # fp16 linears are stored [in, out]
    q_add = nodes[weight_matmul(f"{pre}0.self_attention.query.weight") + 1]
    q_reshape = next(n for n in nodes if n.op == "onnx.reshape" and n.inputs[0] == q_add.outputs[0])
    batch, seq, n_head, head_dim = (int(v) for v in _const_of(body, main, q_reshape.inputs[1]))
    kv_width = shape_of(f"{pre}0.self_attention.key_value.weight")[1]
    n_group = kv_width // (2 * head_dim)
    if seq != 1 or n_head * head_dim != d_model or n_group * 2 * head_dim != kv_width or n_head % max(n_group, 1):
        raise UnsupportedGraph(f"q is reshaped to [{batch}, {seq}, {n_head}, {head_dim}] and key_value has {kv_width} features: expected one new "
                               "token per step, n_head * head_dim = d_model and whole key / value groups")
    first_norm_add = next(n for n in nodes[gathers[0]:] if n.op == "onnx.add")
    eps = float(_const_of(body, main, first_norm_add.inputs[1]))
    common = _common_fields(main, body, nodes, max_loop)
    if common.pop("n_kv_ops") != n_layer:
        raise UnsupportedGraph("expected one KVCache op per block")
    return SimpleNamespace(family="chatglm2", n_layer=n_layer, d_model=int(d_model), n_head=n_head, n_group=int(n_group), head_dim=head_dim, ffn=int(ffn),
                           vocab=int(vocab), eps=eps, batch=batch, int4=False, **common)


# RWKV-4 (models/rwkv/model.py:189-213, rwkv/attention.py:46-105, rwkv/ffn.py:36-59): token-shift mix, the WKV recurrence written
# out in elementary ops, receptance gates, relu^2 channel mixing; every `rescale_every` blocks the hidden state is halved
_RWKV_MIX = ["onnx.mul", "onnx.sub", "onnx.mul", "onnx.add"]                 # x * mix + (1 - mix) * previous x
_RWKV_WKV = ["onnx.add", "onnx.greater", "onnx.where", "onnx.sub", "onnx.exp", "onnx.sub", "onnx.exp", "onnx.mul", "onnx.mul", "onnx.add", "onnx.mul",
             "onnx.add", "onnx.div",                                          # output = numerator / denominator with the running maximum
             "onnx.exp", "onnx.sub", "onnx.greater", "onnx.where", "onnx.sub", "onnx.exp", "onnx.sub", "onnx.exp", "onnx.mul", "onnx.mul", "onnx.add",
             "onnx.mul", "onnx.add"]                                          # the three new states
_RWKV_ATT = ["custom.NormCE"] + 3 * _RWKV_MIX + 3 * ["onnx.matmul"] + ["onnx.sigmoid"] + _RWKV_WKV + ["onnx.mul", "onnx.matmul", "onnx.add"]
_RWKV_FFN = ["custom.NormCE"] + 2 * _RWKV_MIX + ["onnx.matmul", "onnx.relu", "onnx.mul", "onnx.matmul", "onnx.matmul", "onnx.sigmoid", "onnx.mul", "onnx.add"]
_RWKV_CARRY = ["onnx.add", "gc.dynamicslice", "onnx.equal", "onnx.where", "gc.dynamicupdate", "onnx.equal", "gc.bitwiseor"]   # no attention mask to update
_RWKV_TAIL = ["custom.NormCE", "onnx.matmul", "onnx.topk"] + _RWKV_CARRY


def _analyze_rwkv(main, body, max_loop, loop):
    """RWKVDecodeModel (models/rwkv/model.py): the recurrent states travel as loop-carried tensors, five per block."""
    names = list(main.initializers)
    layer_ids = sorted({int(m.group(1)) for k in names for m in [re.match(r"rwkv\.blocks\.(\d+)\.ln1\.weight$", k)] if m})
    n_layer = len(layer_ids)
    if layer_ids != list(range(n_layer)) or "head.weight" not in main.initializers:
        raise UnsupportedGraph("RWKV blocks are not numbered 0 .. n-1, or the head is missing")
    nodes = body.nodes
    gathers = [i for i, n in enumerate(nodes) if n.op == "onnx.gather"]
    if len(gathers) != 1 or nodes[gathers[0]].inputs[0] != "rwkv.embeddings.weight":
        raise UnsupportedGraph("expected one embedding gather from rwkv.embeddings.weight")
    head = [i for i, n in enumerate(nodes) if n.op == "onnx.matmul" and "head.weight" in n.inputs]
    if len(head) != 1:
        raise UnsupportedGraph("expected one head matmul")
    tail_start = max(i for i in range(head[0]) if nodes[i].op == "custom.NormCE")        # ln_out
    got = _skeleton(nodes[gathers[0] + 1:tail_start])
    rescale_every = None
    for cand in range(0, n_layer + 1):
        want = []
        for l in range(n_layer):
            want += (["custom.NormCE"] if l == 0 else []) + _RWKV_ATT + _RWKV_FFN + (["onnx.div"] if cand and (l + 1) % cand == 0 else [])
        if want == got:
            rescale_every = cand
            break
    if rescale_every is None:
        raise UnsupportedGraph("block 0 .. n-1 are not the reference's RWKV-4 blocks (pre_ln, time mixing with the WKV recurrence, channel mixing, "
                               "halving every rescale_every blocks)")
    halvings = [n for n in nodes[:tail_start] if n.op == "onnx.div" and any(c.op == "onnx.constant" and c.outputs[0] == n.inputs[1] for c in nodes)]
    if any(float(_const_of(body, main, n.inputs[1])) != 2.0 for n in halvings):
        raise UnsupportedGraph("the hidden state is expected to be halved (divided by 2) at the rescale points")
    _check_tail(nodes, tail_start, _RWKV_TAIL, "final LayerNorm + head + top-1 + loop carry")

    def shape_of(key):
        a = main.initializers[key]
        return tuple(a.shape) if a is not None else tuple(main.initializer_info[key]["shape"])
    vocab, d_model = shape_of("rwkv.embeddings.weight")
    ffn = shape_of("rwkv.blocks.0.feed_forward.key.weight")[1]                 # fp16 linears are stored [in, out]
    eps = {float(n.attrs["epsilon"]) for n in nodes if n.op == "custom.NormCE"}
    if len(eps) != 1:
        raise UnsupportedGraph("expected one epsilon for every NormCE")
    info = main.input_info.get("input_ids")
    if not info or len(info["shape"]) != 2:
        raise UnsupportedGraph("input_ids is expected as a typed [batch, max_length] input of the main graph")
    batch, max_len = (int(v) for v in info["shape"])
    if len(loop.inputs) != 5 + 5 * n_layer:
        raise UnsupportedGraph(f"expected five loop-carried states per block, the loop has {len(loop.inputs) - 5} state inputs")
    topk = next(n for n in nodes if n.op == "onnx.topk")
    if int(_const_of(body, main, topk.inputs[1])) != 1:
        raise UnsupportedGraph("only greedy decoding (top-k 1) is lowered")
    equals = [n for n in nodes if n.op == "onnx.equal"]
    cond = body.outputs[0]
    return SimpleNamespace(family="rwkv", n_layer=n_layer, d_model=int(d_model), ffn=int(ffn), vocab=int(vocab), rescale_every=rescale_every, eps=eps.pop(),
                           batch=batch, max_len=max_len, max_loop=max_loop, int4=False,
                           pad_id=int(_const_of(body, main, equals[0].inputs[1])), eos_id=int(_const_of(body, main, equals[1].inputs[1])),
                           early_stop=not any(n.op == "onnx.constant" and n.outputs[0] == cond for n in nodes))


def analyze(main):
    """Recognises the recorded graph; returns a plan (family, shapes, ids, state_dict as numpy arrays in checkpoint layout)."""
    loop, body, max_loop = _find_loop(main)
    names = list(main.initializers)
    if "rwkv.embeddings.weight" in main.initializers:
        return _analyze_rwkv(main, body, max_loop, loop)
    if "transformer.embedding.word_embeddings.weight" in main.initializers and any(k.endswith("self_attention.key_value.weight") for k in names):
        return _analyze_chatglm2(main, body, max_loop)
    if "transformer.wte.weight" in main.initializers and any(k.endswith("attn.c_attn.weight") for k in names):
        return _analyze_gpt2(main, body, max_loop)
    layer_ids = sorted({int(m.group(1)) for k in names for m in [re.match(r"model\.layers\.(\d+)\.self_attn\.q_proj\.weight$", k)] if m})
    if not layer_ids or "model.embed_tokens.weight" not in main.initializers or "lm_head.weight" not in main.initializers:
        raise UnsupportedGraph("no Llama-2, GPT-2, ChatGLM2 or RWKV decode graph found (this front end lowers LLAMA2DecModel, GPT2DecModel, ChatGLM2DecModel and "
                               "RWKVDecodeModel); initializers: "
                               + ", ".join(names[:6]))
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
            if plan.family == "gpt2" and key == "lm_head.weight":
                continue
            raise UnsupportedGraph(f"initializer {key} has no data attached")
        a = np.asarray(arr)
        if plan.family == "gpt2":
            if key == "lm_head.weight":           # registered by the LM head layer but unused: the head multiplies by the transposed
                continue                          # token embedding (analyze checked that), so this is not a checkpoint tensor
            is_linear = a.ndim == 2 and key.endswith((".c_attn.weight", ".c_proj.weight", ".c_fc.weight"))
        elif plan.family == "chatglm2":
            is_linear = a.ndim == 2 and "word_embeddings" not in key
        elif plan.family == "rwkv":
            is_linear = a.ndim == 2 and key.endswith(".weight") and "embeddings" not in key
        else:
            is_linear = key.endswith(("_proj.weight", "lm_head.weight"))
        if is_linear and a.dtype != np.int8:
            a = np.ascontiguousarray(a.T)
        sd[key] = torch.from_numpy(np.ascontiguousarray(a))
    return sd


def lower(main, device=None, **decoder_kwargs):
    """(plan, decoder) for the recorded graph, the decoder built on `device` (default: the current CUDA device)."""
    import torch

    from poptransformer_b200 import chatglm2, gpt2, llama, rwkv
    plan = analyze(main)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    sd = state_dict_from_initializers(main, plan)
    if plan.family == "gpt2":
        cfg = gpt2.GPT2Config(n_layer=plan.n_layer, d_model=plan.d_model, n_head=plan.n_head, vocab=plan.vocab, n_positions=plan.n_positions,
                              max_len=plan.max_len, eps=plan.eps)
        dec = gpt2.GPT2Decoder(cfg, sd, plan.batch, device=device, pad_id=plan.pad_id, eos_id=plan.eos_id, early_stop=plan.early_stop,
                               **decoder_kwargs)
        return plan, dec
    if plan.family == "rwkv":
        cfg = rwkv.RWKVConfig(n_layer=plan.n_layer, d_model=plan.d_model, ffn=plan.ffn, vocab=plan.vocab, max_len=plan.max_len,
                              rescale_every=plan.rescale_every, eps=plan.eps)
        dec = rwkv.RWKVDecoder(cfg, sd, plan.batch, device=device, pad_id=plan.pad_id, eos_id=plan.eos_id, early_stop=plan.early_stop, **decoder_kwargs)
        return plan, dec
    if plan.family == "chatglm2":
        cfg = chatglm2.ChatGLM2Config(n_layer=plan.n_layer, d_model=plan.d_model, n_head=plan.n_head, n_group=plan.n_group, ffn=plan.ffn,
                                      vocab=plan.vocab, max_len=plan.max_len, eps=plan.eps, precision="fp16")
        dec = chatglm2.ChatGLM2Decoder(cfg, sd, plan.batch, device=device, pad_id=plan.pad_id, eos_id=plan.eos_id, early_stop=plan.early_stop,
                                       **decoder_kwargs)
        return plan, dec
    group = 0
    if plan.int4:
        w = sd["model.layers.0.self_attn.q_proj.weight"]
        group = (w.shape[1] * 2) // max(1, sd["model.layers.0.self_attn.q_proj.weight_scale"].numel() // w.shape[0])
    cfg = llama.LlamaConfig(n_layer=plan.n_layer, d_model=plan.d_model, n_head=plan.n_head, ffn=plan.ffn, vocab=plan.vocab, eps=plan.eps,
                            max_len=plan.max_len, int4_group=group)
    dec = llama.LlamaDecoder(cfg, sd, plan.batch, device=device, pad_id=plan.pad_id, eos_id=plan.eos_id, early_stop=plan.early_stop,
                             **decoder_kwargs)
    return plan, dec
