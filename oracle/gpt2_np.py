"""TEST INFRASTRUCTURE ONLY (see oracle/__init__.py): numpy restatement of the reference's GPT-2 decode step
(poptransformer/models/gpt2/model.py:23-51, :86-120, :161-197; gpt2/attention.py:35-84; gpt2/embedding.py:31-36;
layers/mlp.py:34-41; layers/lm_head.py:47-57), one token per loop iteration, fp16 rounding after every op.

Weights use the reference's key names AFTER `process_hf_model_state_dict` (gpt2/model.py:154-166): linear weights in
[out, in] orientation, the query third of c_attn pre-multiplied by 1/sqrt(head_size)."""
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
    def __init__(self, cfg, state_dict, batch):
        self.cfg, self.batch = cfg, batch
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
        self.kv = [O.KVCacheState() for _ in range(self.cfg.n_layer)]

    @staticmethod
    def _linear(x, w, b):
        """Linear.__call__ (layers/linear.py:42-46): fp16 matmul, then ops.add of the bias."""
        return O.add_f16(O.matmul_f16(x, w.T), b)

    def logits(self, ids_col, step):
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
            past = O.kv_cache(self.kv[li], step, kv, c.max_len, 3, 1)
            a = O.attention_decode(q, past[0], past[1], mask, hs, "float16", pre_scaled=True)
            a = self._linear(a.reshape(B, c.d_model), L["attn.c_proj.weight"], L["attn.c_proj.bias"]).reshape(B, 1, c.d_model)
            x = O.add_f16(x, a)
            t = O.norm_ce(x, L["ln_2.weight"], L["ln_2.bias"], c.eps)
            h = O.gelu_f16(self._linear(t.reshape(B, c.d_model), L["mlp.c_fc.weight"], L["mlp.c_fc.bias"]))   # layers/mlp.py:34-41
            m = self._linear(h, L["mlp.c_proj.weight"], L["mlp.c_proj.bias"]).reshape(B, 1, c.d_model)
            x = O.add_f16(x, m)
        hfin = O.norm_ce(x, self.ln_f[0], self.ln_f[1], c.eps)
        return O.matmul_f16(hfin.reshape(B, c.d_model), self.wte.T), hfin                          # tied head, layers/lm_head.py:47-57

    def generate(self, ids, n_steps, pad_id, return_logits=False):
        self.reset()
        ids = np.array(ids, dtype=np.int32, copy=True)
        all_logits, step = [], 0
        for _ in range(n_steps):
            lg, _ = self.logits(ids[:, step], step)
            nxt = O.topk(lg, 1)[1][:, 0]
            if return_logits:
                all_logits.append(lg)
            ids, step, _ = O.step_containers(ids, step, nxt, pad_id)
        return (ids, all_logits) if return_logits else ids
