"""TEST INFRASTRUCTURE ONLY (see oracle/__init__.py): numpy restatement of the reference's ChatGLM2 decode step
(poptransformer/models/chatglm2/model.py:95-117 block, :199-254 loop body; chatglm2/attention.py:77-302 multi-query attention
with the interleaved RoPE on the first half of each head; chatglm2/mlp.py:51-59 SwiGLU; layers/rms_layer_norm.py:26-36),
one token per loop iteration, fp16 rounding after every op.

precision "fp16": fp16 matmuls.  precision "fp8": every transformer linear and the output layer take E4M3 weights with one
float32 scale per tensor and E4M3 activations with a static per-site scale (ops.half_to_uint8 + ops.fp8_matmul,
poptransformer/utils/param_handler/precision_strategy.py:44-81 in the OCP-E4M3 form)."""
from dataclasses import dataclass, field

import numpy as np

from . import ops_np as O

F16 = np.float16


@dataclass
class ChatGLM2Config:
    n_layer: int
    d_model: int
    n_head: int
    n_group: int          # multi_query_group_num
    ffn: int
    vocab: int
    max_len: int
    eps: float = 1e-5
    precision: str = "fp16"
    act_scales: dict = field(default_factory=lambda: {"norm": 8.0 / 448.0, "attn": 2.0 / 448.0, "mlp": 1.0 / 448.0})


def rearrange_tp_rows(n_rows, num_heads, num_replicas):
    """Row order that `rearrange_tp_weights` gives the query weight (chatglm2/model.py:29-49): the heads of the first and of the
    second half (= the two KV groups) are cut into `num_replicas` runs each and the runs are interleaved, so that a plain
    n-way split of the rows hands every replica heads of both halves."""
    offset, head = n_rows // 2, n_rows // num_heads
    run = num_heads // num_replicas // 2
    order = []
    for i in range(0, num_heads // 2, run):
        order += [np.arange(i * head, (i + run) * head), np.arange(offset + i * head, offset + (i + run) * head)]
    return np.concatenate(order)


class ChatGLM2Oracle:
    """tp > 1 emulates the reference's TP layers rank by rank: query rearranged and split ('multi_query_qkv' on a weight that
    only holds the query, tensor_parallel_strategy.py:59-70), key_value replicated (chatglm2/attention.py:316-346), dense and
    dense_4h_to_h 'end' with an all-reduce of fp16 partial sums, dense_h_to_4h_1/2 'start' (chatglm2/mlp.py:62-72), and the
    vocab-sharded output layer with the merge of layers/lm_head.py:75-116."""

    def __init__(self, cfg, state_dict, batch, tp=1):
        self.cfg, self.batch, self.tp = cfg, batch, tp
        self.sd = state_dict
        self.sin, self.cos = O.chatglm2_rope_tables(cfg.max_len, cfg.d_model // cfg.n_head)
        self.reset()

    def reset(self):
        self.kv = [[O.KVCacheState() for _ in range(self.tp)] for _ in range(self.cfg.n_layer)]

    def _linear(self, x, key, site, bias=None, rows=None, cols=None):
        """Linear.__call__ through the precision strategy: fp16 matmul, or cast + fp8 matmul; then the bias.
        rows / cols select a rank's output / input features of the [out, in] weight."""
        w = np.asarray(self.sd[key])
        if rows is not None:
            w = w[rows]
        if cols is not None:
            w = w[:, cols]
        if self.cfg.precision == "fp8":
            a = float(self.sd[key + "_act_scale"]) if (key + "_act_scale") in self.sd else self.cfg.act_scales[site]   # per tensor, else per site
            y = O.fp8_matmul(O.cast_fp8(x, a), np.ascontiguousarray(w.T), a, float(self.sd[key + "_scale"]))
        else:
            y = O.matmul_f16(x, np.asarray(w, dtype=F16).T)
        if not bias:
            return y
        b = np.asarray(self.sd[bias], dtype=F16)
        return O.add_f16(y, b if rows is None else b[rows])

    def _all_reduce(self, parts):
        return parts[0] if self.tp == 1 else np.sum([O.f32(p) for p in parts], axis=0, dtype=np.float32).astype(F16)

    def _logits_tp(self, ids_col, step):
        c, B, tp = self.cfg, self.batch, self.tp
        hs, N, G, d = c.d_model // c.n_head, c.n_head // tp, c.n_group, c.d_model
        order = rearrange_tp_rows(d, c.n_head, tp)
        x = O.embedding(np.asarray(self.sd["transformer.embedding.word_embeddings.weight"], dtype=F16), np.asarray(ids_col).reshape(B, 1))
        mask = O.decode_mask(B, c.max_len, step)
        fl = c.ffn // tp
        for li in range(c.n_layer):
            p = f"transformer.encoder.layers.{li}."
            h = O.rms_norm(x, np.asarray(self.sd[p + "input_layernorm.weight"], dtype=F16), c.eps).reshape(B, d)
            parts = []
            for r in range(tp):
                mine = order[r * (d // tp):(r + 1) * (d // tp)]
                q = self._linear(h, p + "self_attention.query.weight", "norm", p + "self_attention.query.bias", rows=mine)
                kv = self._linear(h, p + "self_attention.key_value.weight", "norm", p + "self_attention.key_value.bias")
                q = q.reshape(B, 1, N, hs).transpose(0, 2, 1, 3)
                k = kv[:, : G * hs].reshape(B, 1, G, hs).transpose(0, 2, 1, 3)
                v = kv[:, G * hs:].reshape(B, 1, G, hs).transpose(0, 2, 1, 3)
                q = O.chatglm2_rope_apply(q, self.sin[step], self.cos[step])
                k = O.chatglm2_rope_apply(k, self.sin[step], self.cos[step])
                past = O.kv_cache(self.kv[li][r], step, np.stack([k, v]), c.max_len, 3, 1)
                K, V = np.repeat(past[0], N // G, axis=1), np.repeat(past[1], N // G, axis=1)
                a = O.attention_decode(q, K, V, mask, hs, "float16").reshape(B, d // tp)
                parts.append(self._linear(a, p + "self_attention.dense.weight", "attn", cols=mine))
            x = O.add_f16(x, self._all_reduce(parts).reshape(B, 1, d))
            h = O.rms_norm(x, np.asarray(self.sd[p + "post_attention_layernorm.weight"], dtype=F16), c.eps).reshape(B, d)
            parts = []
            for r in range(tp):
                mine = np.arange(r * fl, (r + 1) * fl)
                g = O.swish_f16(self._linear(h, p + "mlp.dense_h_to_4h_1.weight", "norm", rows=mine))
                u = self._linear(h, p + "mlp.dense_h_to_4h_2.weight", "norm", rows=mine)
                parts.append(self._linear(O.mul_f16(u, g), p + "mlp.dense_4h_to_h.weight", "mlp", cols=mine))
            x = O.add_f16(x, self._all_reduce(parts).reshape(B, 1, d))
        hf = O.rms_norm(x, np.asarray(self.sd["transformer.encoder.final_layernorm.weight"], dtype=F16), c.eps).reshape(B, d)
        per = -(-c.vocab // tp)
        out = []
        for r in range(tp):
            mine = np.arange(r * per, min((r + 1) * per, c.vocab))
            lg = self._linear(hf, "transformer.output_layer.weight", "norm", rows=mine)
            out.append(np.pad(lg, ((0, 0), (0, per - mine.size))))               # shard() zero-pads the vocab axis
        return out, hf

    def next_ids(self, logits):
        return O.topk(logits, 1)[1][:, 0] if self.tp == 1 else O.lm_head_tp_merge(logits, self.cfg.vocab)

    def logits(self, ids_col, step):
        if self.tp > 1:
            return self._logits_tp(ids_col, step)
        c, B = self.cfg, self.batch
        hs, N, G = c.d_model // c.n_head, c.n_head, c.n_group
        x = O.embedding(np.asarray(self.sd["transformer.embedding.word_embeddings.weight"], dtype=F16), np.asarray(ids_col).reshape(B, 1))
        mask = O.decode_mask(B, c.max_len, step)
        for li in range(c.n_layer):
            p = f"transformer.encoder.layers.{li}."
            h = O.rms_norm(x, np.asarray(self.sd[p + "input_layernorm.weight"], dtype=F16), c.eps).reshape(B, c.d_model)
            q = self._linear(h, p + "self_attention.query.weight", "norm", p + "self_attention.query.bias")
            kv = self._linear(h, p + "self_attention.key_value.weight", "norm", p + "self_attention.key_value.bias")
            q = q.reshape(B, 1, N, hs).transpose(0, 2, 1, 3)
            k = kv[:, : G * hs].reshape(B, 1, G, hs).transpose(0, 2, 1, 3)
            v = kv[:, G * hs:].reshape(B, 1, G, hs).transpose(0, 2, 1, 3)
            q = O.chatglm2_rope_apply(q, self.sin[step], self.cos[step])
            k = O.chatglm2_rope_apply(k, self.sin[step], self.cos[step])
            past = O.kv_cache(self.kv[li][0], step, np.stack([k, v]), c.max_len, 3, 1)           # [2,B,G,L,hs]
            K, V = np.repeat(past[0], N // G, axis=1), np.repeat(past[1], N // G, axis=1)       # chatglm2/attention.py:238-272
            a = O.attention_decode(q, K, V, mask, hs, "float16")
            a = self._linear(a.reshape(B, c.d_model), p + "self_attention.dense.weight", "attn").reshape(B, 1, c.d_model)
            x = O.add_f16(x, a)
            h = O.rms_norm(x, np.asarray(self.sd[p + "post_attention_layernorm.weight"], dtype=F16), c.eps).reshape(B, c.d_model)
            g = O.swish_f16(self._linear(h, p + "mlp.dense_h_to_4h_1.weight", "norm"))
            u = self._linear(h, p + "mlp.dense_h_to_4h_2.weight", "norm")
            m = self._linear(O.mul_f16(u, g), p + "mlp.dense_4h_to_h.weight", "mlp").reshape(B, 1, c.d_model)
            x = O.add_f16(x, m)
        hf = O.rms_norm(x, np.asarray(self.sd["transformer.encoder.final_layernorm.weight"], dtype=F16), c.eps).reshape(B, c.d_model)
        return self._linear(hf, "transformer.output_layer.weight", "norm"), hf

    def generate(self, ids, n_steps, pad_id, return_logits=False):
        self.reset()
        ids = np.array(ids, dtype=np.int32, copy=True)
        all_logits, step = [], 0
        for _ in range(n_steps):
            lg, _ = self.logits(ids[:, step], step)
            nxt = self.next_ids(lg)
            if return_logits:
                all_logits.append(lg)
            ids, step, _ = O.step_containers(ids, step, nxt, pad_id)
        return (ids, all_logits) if return_logits else ids
