"""TEST INFRASTRUCTURE ONLY (see oracle/__init__.py): numpy restatement of the reference's RWKV-4 decode step
(poptransformer/models/rwkv/model.py:44-54 block, :98-118 stack with rescale, :157-187 state initialisation;
rwkv/attention.py:59-105 time mixing and WKV; rwkv/ffn.py:40-59 channel mixing), one token per loop iteration, fp16 rounding
after every op, WKV states in float32.

Weights use the reference's key names AFTER `process_hf_model_state_dict` (rwkv/model.py:150-155): attention.output and
feed_forward.value divided by 2^(block // rescale_every)."""
from dataclasses import dataclass

import numpy as np

from . import ops_np as O

F16, F32 = np.float16, np.float32


@dataclass
class RWKVConfig:
    n_layer: int
    d_model: int
    ffn: int
    vocab: int
    max_len: int
    rescale_every: int = 6
    eps: float = 1e-5


def gate(a, w, b):
    """gate (rwkv/attention.py:59-64): fp16(fp16(a * w) + fp16(fp16(1 - w) * b))."""
    return O.add_f16(O.mul_f16(a, w), O.mul_f16((F32(1.0) - O.f32(w)).astype(F16), b))


class RWKVOracle:
    """tp > 1 follows the reference's TP layers (rwkv/attention.py:108-147, rwkv/ffn.py:62-98): key / value / receptance are
    'start' layers whose per-rank slices (with the matching slices of time_first, time_decay and of the WKV states,
    rwkv/model.py:172-184) concatenate to exactly the unsharded result, so only the two 'end' layers (attention output,
    feed-forward value: fp16 partial products per rank, summed by the all-reduce) and the vocab-sharded head with the merge of
    layers/lm_head.py:75-116 differ from tp = 1.  The feed-forward receptance is all-gathered over the channel shards
    (rwkv/ffn.py:95); the flat gather result only lines up with the value for batch 1, and is read as a channel concatenation."""

    def __init__(self, cfg, state_dict, batch, tp=1):
        self.cfg, self.batch, self.tp = cfg, batch, tp
        self.sd = state_dict
        self.reset()

    def reset(self):
        c, B = self.cfg, self.batch
        self.state = [[np.zeros((B, c.d_model), F16), np.zeros((B, c.d_model), F16), np.zeros((B, c.d_model), F32),
                       np.zeros((B, c.d_model), F32), np.full((B, c.d_model), -1e30, F32)] for _ in range(c.n_layer)]

    def _h(self, k):
        return np.asarray(self.sd[k], dtype=F16)

    def _ln(self, x, p):
        return O.norm_ce(x, self._h(p + ".weight"), self._h(p + ".bias"), self.cfg.eps)

    def _end(self, x, w):
        """'end' layer on the [out, in] weight w: fp16 partial products over each rank's input features, then the all-reduce."""
        if self.tp == 1:
            return O.matmul_f16(x, w.T)
        k = w.shape[1] // self.tp
        parts = [O.f32(O.matmul_f16(x[:, r * k:(r + 1) * k], w[:, r * k:(r + 1) * k].T)) for r in range(self.tp)]
        return np.sum(parts, axis=0, dtype=np.float32).astype(F16)

    def next_ids(self, logits):
        return O.topk(logits, 1)[1][:, 0] if self.tp == 1 else O.lm_head_tp_merge(logits, self.cfg.vocab)

    def logits(self, ids_col):
        c, B = self.cfg, self.batch
        x = O.embedding(self._h("rwkv.embeddings.weight"), np.asarray(ids_col).reshape(B, 1)).reshape(B, c.d_model)
        for i in range(c.n_layer):
            p, st = f"rwkv.blocks.{i}.", self.state[i]
            if i == 0:
                x = self._ln(x, p + "pre_ln")
            t = self._ln(x, p + "ln1")
            a = p + "attention."
            k = gate(t, self._h(a + "time_mix_key").reshape(-1), st[1])
            v = gate(t, self._h(a + "time_mix_value").reshape(-1), st[1])
            r = gate(t, self._h(a + "time_mix_receptance").reshape(-1), st[1])
            st[1] = t
            k, v = O.matmul_f16(k, self._h(a + "key.weight").T), O.matmul_f16(v, self._h(a + "value.weight").T)
            r = O.sigmoid_f16(O.matmul_f16(r, self._h(a + "receptance.weight").T))
            wkv, st[2], st[3], st[4] = O.rwkv_wkv(k, v, np.asarray(self.sd[a + "time_first"], F32), np.asarray(self.sd[a + "time_decay"], F32),
                                                  st[2], st[3], st[4])
            x = O.add_f16(x, self._end(O.mul_f16(r, wkv.astype(F16)), self._h(a + "output.weight")))
            t = self._ln(x, p + "ln2")
            f = p + "feed_forward."
            k = gate(t, self._h(f + "time_mix_key").reshape(-1), st[0])
            r = gate(t, self._h(f + "time_mix_receptance").reshape(-1), st[0])
            st[0] = t
            k = O.matmul_f16(k, self._h(f + "key.weight").T)
            k = np.maximum(k, F16(0))
            k = O.mul_f16(k, k)
            v = self._end(k, self._h(f + "value.weight"))
            r = O.sigmoid_f16(O.matmul_f16(r, self._h(f + "receptance.weight").T))
            x = O.add_f16(x, O.mul_f16(r, v))
            if c.rescale_every > 0 and (i + 1) % c.rescale_every == 0:
                x = O.mul_f16(x, F16(0.5))                                              # ops.div by 2 (exact)
        h = self._ln(x, "rwkv.ln_out")
        if self.tp == 1:
            return O.matmul_f16(h, self._h("head.weight").T), h
        per = -(-c.vocab // self.tp)
        head = np.pad(self._h("head.weight"), ((0, per * self.tp - c.vocab), (0, 0)))            # shard() zero-pads the vocab axis
        return [O.matmul_f16(h, head[r * per:(r + 1) * per].T) for r in range(self.tp)], h

    def generate(self, ids, n_steps, pad_id, return_logits=False):
        self.reset()
        ids = np.array(ids, dtype=np.int32, copy=True)
        all_logits, step = [], 0
        for _ in range(n_steps):
            lg, _ = self.logits(ids[:, step])
            nxt = self.next_ids(lg)
            if return_logits:
                all_logits.append(lg)
            ids, step, _ = O.step_containers(ids, step, nxt, pad_id)
        return (ids, all_logits) if return_logits else ids
