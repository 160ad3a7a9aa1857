"""numpy restatement of the reference's Llama-2 per-token decode step (test oracle only).

Follows poptransformer/models/llama2/model.py:162-197 (loop body),
llama2/attention.py:64-122, llama2/mlp.py:20-28, layers/rms_layer_norm.py:26-36,
layers/lm_head.py:47-57 and models/base_model.py:313-335 op by op, with an fp16
rounding after every op exactly where the reference graph has an fp16 tensor.
Tensor parallelism (model_type 'tp') is emulated rank by rank with the slicing of
utils/param_handler/tensor_parallel_strategy.py:21-42 and a float32 sum over ranks
rounded once to fp16 for every all-reduce.
"""
import math
import numpy as np

from . import ops_np as O

F16 = np.float16


class LlamaConfig:
    def __init__(self, n_layer, d_model, n_head, ffn, vocab, eps=1e-5, max_len=128, group=0):
        self.n_layer, self.d_model, self.n_head, self.ffn = n_layer, d_model, n_head, ffn
        self.vocab, self.eps, self.max_len, self.group = vocab, eps, max_len, group
        self.head_dim = d_model // n_head


def _dense_weight(sd, key, group):
    """Linear weight in the reference's [in, out] fp16 form.  int8 checkpoints go
    through Int4ToHalf (precision_strategy.py:24-42,56-60), fp16 ones are transposed
    (layers/linear.py:32)."""
    w = sd[key]
    if w.dtype == np.int8:
        return O.int4_to_half(w, sd[key + "_scale"], axis=1, group=group)
    return np.ascontiguousarray(np.asarray(w, dtype=F16).T)


class LlamaOracle:
    def __init__(self, cfg, state_dict, batch, tp=1):
        self.cfg, self.batch, self.tp = cfg, batch, tp
        c = cfg
        self.sin, self.cos = O.llama_rope_tables(c.max_len, c.head_dim)
        self.emb = np.asarray(state_dict["model.embed_tokens.weight"], dtype=F16)
        self.layers = []
        for i in range(c.n_layer):
            p = f"model.layers.{i}."
            self.layers.append({
                "ln1": np.asarray(state_dict[p + "input_layernorm.weight"], dtype=F16),
                "ln2": np.asarray(state_dict[p + "post_attention_layernorm.weight"], dtype=F16),
                "q": _dense_weight(state_dict, p + "self_attn.q_proj.weight", c.group),
                "k": _dense_weight(state_dict, p + "self_attn.k_proj.weight", c.group),
                "v": _dense_weight(state_dict, p + "self_attn.v_proj.weight", c.group),
                "o": _dense_weight(state_dict, p + "self_attn.o_proj.weight", c.group),
                "gate": _dense_weight(state_dict, p + "mlp.gate_proj.weight", c.group),
                "up": _dense_weight(state_dict, p + "mlp.up_proj.weight", c.group),
                "down": _dense_weight(state_dict, p + "mlp.down_proj.weight", c.group),
            })
        self.norm = np.asarray(state_dict["model.norm.weight"], dtype=F16)
        self.head = _dense_weight(state_dict, "lm_head.weight", 0)     # fp16 [d, V]
        self.reset()

    def reset(self):
        self.kv = [[O.KVCacheState() for _ in range(self.tp)] for _ in range(self.cfg.n_layer)]

    # -- linears with the reference's TP strategies ('start' = split out, 'end' = split in + all-reduce)
    def _linear_start(self, x, w, r):
        n = w.shape[1] // self.tp
        return O.matmul_f16(x, w[:, r * n:(r + 1) * n])

    def _linear_end(self, xs, w):
        k = w.shape[0] // self.tp
        parts = [O.matmul_f16(xs[r], w[r * k:(r + 1) * k]) for r in range(self.tp)]
        if self.tp == 1:
            return parts[0]
        return np.sum([O.f32(p) for p in parts], axis=0, dtype=np.float32).astype(F16)

    def logits(self, ids_col, step):
        """One decode step: ids_col int [B], step int -> fp16 logits [B, V] and the
        hidden state before the LM head."""
        c, B, tp = self.cfg, self.batch, self.tp
        nh = c.n_head // tp
        x = O.embedding(self.emb, np.asarray(ids_col).reshape(B, 1))        # [B,1,d]
        mask = O.decode_mask(B, c.max_len, step)
        for li, L in enumerate(self.layers):
            h = O.rms_norm(x, L["ln1"], c.eps)
            attn_parts = []
            for r in range(tp):
                q = self._linear_start(h, L["q"], r).reshape(B, 1, nh, c.head_dim).transpose(0, 2, 1, 3)
                k = self._linear_start(h, L["k"], r).reshape(B, 1, nh, c.head_dim).transpose(0, 2, 1, 3)
                v = self._linear_start(h, L["v"], r).reshape(B, 1, nh, c.head_dim).transpose(0, 2, 1, 3)
                q = O.llama_rope_apply(q, self.sin[step], self.cos[step])
                k = O.llama_rope_apply(k, self.sin[step], self.cos[step])
                kv = np.stack([k, v], axis=0)                                # [2,B,N,1,H]
                past = O.kv_cache(self.kv[li][r], step, kv, c.max_len, 3, 1)
                attn_parts.append(O.attention_decode(q, past[0], past[1], mask, c.head_dim, "float32"))
            a = self._linear_end(attn_parts, L["o"])
            x = O.add_f16(x, a)
            h = O.rms_norm(x, L["ln2"], c.eps).reshape(B, c.d_model)
            acts = []
            for r in range(tp):
                g = O.swish_f16(self._linear_start(h, L["gate"], r))
                u = self._linear_start(h, L["up"], r)
                acts.append(O.mul_f16(u, g))
            m = self._linear_end(acts, L["down"]).reshape(B, 1, c.d_model)
            x = O.add_f16(x, m)
        hfin = O.rms_norm(x, self.norm, c.eps)
        if tp == 1:
            return O.matmul_f16(hfin.reshape(B, c.d_model), self.head), hfin
        per = math.ceil(c.vocab / tp)
        head = np.pad(self.head, ((0, 0), (0, per * tp - c.vocab)))
        return [O.matmul_f16(hfin.reshape(B, c.d_model), head[:, r * per:(r + 1) * per]) for r in range(tp)], hfin

    def next_ids(self, logits):
        if self.tp == 1:
            return O.topk(logits, 1)[1][:, 0]
        return O.lm_head_tp_merge(logits, self.cfg.vocab)

    def generate(self, ids, n_steps, pad_id, return_logits=False):
        """ids int32 [B, max_len] right-padded with pad_id.  Runs n_steps loop
        iterations from step 0 (prompt tokens are fed one per step, F6) and returns the
        updated container (and per-step logits)."""
        self.reset()
        ids = np.array(ids, dtype=np.int32, copy=True)
        all_logits = []
        step = 0
        for _ in range(n_steps):
            lg, _ = self.logits(ids[:, step], step)
            nxt = self.next_ids(lg)
            if return_logits:
                all_logits.append(lg)
            ids, step, _ = O.step_containers(ids, step, nxt, pad_id)
        return (ids, all_logits) if return_logits else ids
