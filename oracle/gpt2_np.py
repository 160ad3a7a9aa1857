"""TEST INFRASTRUCTURE ONLY (see oracle/__init__.py): numpy restatement of the reference's GPT-2 decode step
(poptransformer/models/gpt2/model.py:23-51, :86-120, :161-197; gpt2/attention.py:35-84; gpt2/embedding.py:31-36;
layers/mlp.py:34-41; layers/lm_head.py:47-57), one token per loop iteration, fp16 rounding after every op.

Tensor parallelism (model_type 'tp') is emulated rank by rank: c_attn with the 'fused_qkv' strategy (q, k and v thirds split
separately, utils/param_handler/tensor_parallel_strategy.py:47-57), c_fc 'start', both c_proj 'end' with the bias added once
after the all-reduce (layers/linear.py:42-46), heads split over the ranks (gpt2/attention.py:88-96), and the tied head on the
vocab-sharded wte with the merge of layers/lm_head.py:75-116.  The vocab-sharded wte/wpe gather summed by an all-reduce
(gpt2/embedding.py:38-46, layers/embedding.py:41-70) adds exact zeros to fp16(wte[id] + wpe[step]) and is kept as one gather.

Weights use the reference's key names AFTER `process_hf_model_state_dict` (gpt2/model.py:154-166): linear weights in
[out, in] orientation, the query third of c_attn pre-multiplied by 1/sqrt(head_size)."""
import math
from dataclasses import dataclass

import numpy as np

from . import ops_np as O

F16 = np.float16


@dataclass
class GPT2Config:
    n_layer: int
    d_model: int
    n_head: int
    vocab: int
    n_positions: int
    max_len: int
    eps: float = 1e-5


class GPT2Oracle:
    def __init__(self, cfg, state_dict, batch, tp=1):
        self.cfg, self.batch, self.tp = cfg, batch, tp
        if cfg.n_head % tp:
            raise ValueError("n_head must be divisible by the number of replicas")
        g = lambda k: np.asarray(state_dict[k], dtype=F16)
        self.wte, self.wpe = g("transformer.wte.weight"), g("transformer.wpe.weight")
        self.layers = []
        for i in range(cfg.n_layer):
            p = f"transformer.h.{i}."
            self.layers.append({k: g(p + k) for k in (
                "ln_1.weight", "ln_1.bias", "attn.c_attn.weight", "attn.c_attn.bias", "attn.c_proj.weight", "attn.c_proj.bias",
                "ln_2.weight", "ln_2.bias", "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight", "mlp.c_proj.bias")})
        self.ln_f = (g("transformer.ln_f.weight"), g("transformer.ln_f.bias"))
        self.reset()

    def reset(self):
        self.kv = [[O.KVCacheState() for _ in range(self.tp)] for _ in range(self.cfg.n_layer)]

    @staticmethod
    def _linear(x, w, b):
        """Linear.__call__ (layers/linear.py:42-46): fp16 matmul, then ops.add of the bias."""
        return O.add_f16(O.matmul_f16(x, w.T), b)

    def _linear_end(self, xs, w, b):
        """'end' strategy: per-rank fp16 partial products over a slice of the input features, all-reduce, then the bias once."""
        k = w.shape[1] // self.tp
        parts = [O.matmul_f16(xs[r], w[:, r * k:(r + 1) * k].T) for r in range(self.tp)]
        y = parts[0] if self.tp == 1 else np.sum([O.f32(p) for p in parts], axis=0, dtype=np.float32).astype(F16)
        return O.add_f16(y, b)

    def logits(self, ids_col, step):
        if self.tp > 1:
            return self._logits_tp(ids_col, step)
        c, B = self.cfg, self.batch
        nh, hs = c.n_head, c.d_model // c.n_head
        x = O.add_f16(O.embedding(self.wte, np.asarray(ids_col).reshape(B, 1)),
                      O.embedding(self.wpe, np.full((B, 1), step, dtype=np.int32)))             # gpt2/embedding.py:31-36
        mask = O.decode_mask(B, c.max_len, step)
        for li, L in enumerate(self.layers):
            t = O.norm_ce(x, L["ln_1.weight"], L["ln_1.bias"], c.eps)
            qkv = self._linear(t.reshape(B, c.d_model), L["attn.c_attn.weight"], L["attn.c_attn.bias"])
            q = qkv[:, :c.d_model].reshape(B, 1, nh, hs).transpose(0, 2, 1, 3)                    # gpt2/attention.py:38-48
            kv = qkv[:, c.d_model:].reshape(B, 1, 2, nh, hs).transpose(2, 0, 3, 1, 4)
            past = O.kv_cache(self.kv[li][0], step, kv, c.max_len, 3, 1)
            a = O.attention_decode(q, past[0], past[1], mask, hs, "float16", pre_scaled=True)
            a = self._linear(a.reshape(B, c.d_model), L["attn.c_proj.weight"], L["attn.c_proj.bias"]).reshape(B, 1, c.d_model)
            x = O.add_f16(x, a)
            t = O.norm_ce(x, L["ln_2.weight"], L["ln_2.bias"], c.eps)
            h = O.gelu_f16(self._linear(t.reshape(B, c.d_model), L["mlp.c_fc.weight"], L["mlp.c_fc.bias"]))   # layers/mlp.py:34-41
            m = self._linear(h, L["mlp.c_proj.weight"], L["mlp.c_proj.bias"]).reshape(B, 1, c.d_model)
            x = O.add_f16(x, m)
        hfin = O.norm_ce(x, self.ln_f[0], self.ln_f[1], c.eps)
        return O.matmul_f16(hfin.reshape(B, c.d_model), self.wte.T), hfin                          # tied head, layers/lm_head.py:47-57

    def _logits_tp(self, ids_col, step):
        """The same step with the reference's TP layers; returns the per-rank logits of the vocab-sharded tied head."""
        c, B, tp = self.cfg, self.batch, self.tp
        d, hs = c.d_model, c.d_model // c.n_head
        nh, dl, fl = c.n_head // tp, c.d_model // tp, 4 * c.d_model // tp
        x = O.add_f16(O.embedding(self.wte, np.asarray(ids_col).reshape(B, 1)),
                      O.embedding(self.wpe, np.full((B, 1), step, dtype=np.int32)))
        mask = O.decode_mask(B, c.max_len, step)
        for li, L in enumerate(self.layers):
            t = O.norm_ce(x, L["ln_1.weight"], L["ln_1.bias"], c.eps).reshape(B, d)
            w, b = L["attn.c_attn.weight"], L["attn.c_attn.bias"]
            outs = []
            for r in range(tp):
                sel = np.concatenate([np.arange(j * d + r * dl, j * d + (r + 1) * dl) for j in range(3)])   # 'fused_qkv'
                qkv = self._linear(t, w[sel], b[sel])
                q = qkv[:, :dl].reshape(B, 1, nh, hs).transpose(0, 2, 1, 3)
                kv = qkv[:, dl:].reshape(B, 1, 2, nh, hs).transpose(2, 0, 3, 1, 4)
                past = O.kv_cache(self.kv[li][r], step, kv, c.max_len, 3, 1)
                outs.append(O.attention_decode(q, past[0], past[1], mask, hs, "float16", pre_scaled=True).reshape(B, dl))
            x = O.add_f16(x, self._linear_end(outs, L["attn.c_proj.weight"], L["attn.c_proj.bias"]).reshape(B, 1, d))
            t = O.norm_ce(x, L["ln_2.weight"], L["ln_2.bias"], c.eps).reshape(B, d)
            hs_r = [O.gelu_f16(self._linear(t, L["mlp.c_fc.weight"][r * fl:(r + 1) * fl], L["mlp.c_fc.bias"][r * fl:(r + 1) * fl]))
                    for r in range(tp)]
            x = O.add_f16(x, self._linear_end(hs_r, L["mlp.c_proj.weight"], L["mlp.c_proj.bias"]).reshape(B, 1, d))
        hfin = O.norm_ce(x, self.ln_f[0], self.ln_f[1], c.eps)
        per = math.ceil(c.vocab / tp)
        head = np.pad(self.wte, ((0, per * tp - c.vocab), (0, 0)))
        return [O.matmul_f16(hfin.reshape(B, d), head[r * per:(r + 1) * per].T) for r in range(tp)], hfin

    def next_ids(self, logits):
        if self.tp == 1:
            return O.topk(logits, 1)[1][:, 0]
        return O.lm_head_tp_merge(logits, self.cfg.vocab)

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

    def generate_beam(self, prompt, new_tokens, beam):
        """Beam decode with the reference's `BeamSearch` op (custom_ops/beam_search_custom_op.cpp:333-478) on top of the GPT-2 step.
        The reference registers the op but none of its Python models calls it, so the composition is the one the op's interface
        implies: every hypothesis is a cache row (this oracle is built with batch = prompts x beam, row = prompt * beam + slot),
        the prompt is fed token by token to all slots, and from the last prompt token on the fp16 logits are the scores the op
        adds to the running `prob`; the op's next ids are the next input tokens and every slot continues from the cache row of
        the hypothesis it extends.  prompt int [n_prompts, P].  Returns (hyp [n, new_tokens, beam], prob [n, beam])."""
        if self.tp != 1:
            raise ValueError("beam decode is defined for one rank")
        prompt = np.asarray(prompt, dtype=np.int32)
        n, P = prompt.shape
        assert n * beam == self.batch
        self.reset()
        hyp, prob = np.zeros((n, new_tokens, beam), np.int32), np.zeros((n, beam), F16)
        tok = np.repeat(prompt[:, 0], beam)
        for t in range(P + new_tokens - 1):
            lg, _ = self.logits(tok, t)
            if t + 1 < P:
                tok = np.repeat(prompt[:, t + 1], beam)
                continue
            g = t + 1 - P
            nxt, gid, hyp, prob = O.beam_search_step(lg.reshape(n, beam, -1), hyp, prob, g, beam)
            parent = (np.arange(n)[:, None] * beam + (np.zeros((n, beam), np.int64) if g == 0 else gid // beam)).reshape(-1)
            for layer in self.kv:
                layer[0].cache = O.kv_reorder_dense(layer[0].cache, parent)
            tok = nxt.reshape(-1)
        return hyp, prob
