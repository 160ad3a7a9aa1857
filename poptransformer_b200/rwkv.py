"""RWKV-4 decode loop on the per-op kernels: host-side mirror of the reference's RWKVDecodeModel
(poptransformer/models/rwkv/model.py:121-187, :189-213) for one token per loop iteration.

Per block (rwkv/model.py:44-54): NormCE -> token-shift gates -> key / value / receptance linears -> WKV with float32
(numerator, denominator, max) states -> sigmoid(receptance) * wkv -> output linear (+residual); NormCE -> gates -> key linear ->
relu^2 -> value linear, sigmoid(receptance) gate (+residual); hidden / 2 every `rescale_every` blocks.
The state dict uses the reference's key names after `process_hf_model_state_dict` (output / value weights pre-divided)."""
import ctypes

import torch

from . import ops


class RWKVConfig:
    def __init__(self, n_layer, d_model, ffn, vocab, max_len, rescale_every=6, eps=1e-5):
        self.n_layer, self.d_model, self.ffn, self.vocab, self.max_len, self.rescale_every, self.eps = (
            n_layer, d_model, ffn, vocab, max_len, rescale_every, eps)


class RWKVDecoder:
    def __init__(self, cfg, state_dict, batch, device="cuda", pad_id=None, eos_id=-1):
        c = cfg
        self.cfg, self.batch, self.device = cfg, batch, device
        self.pad_id = c.vocab - 1 if pad_id is None else pad_id
        self.eos_id = eos_id
        dev = device
        h = lambda k: state_dict[k].to(dev).to(torch.float16).reshape(-1).contiguous()
        f = lambda k: state_dict[k].to(dev).to(torch.float32).reshape(-1).contiguous()
        lin = lambda k: ops.PackedLinear(ops.W_FP16, state_dict[k].to(dev).to(torch.float16).contiguous())
        ln = lambda p: (h(p + ".weight"), h(p + ".bias"))
        self.emb = state_dict["rwkv.embeddings.weight"].to(dev).to(torch.float16).contiguous()
        self.layers = []
        for i in range(c.n_layer):
            p = f"rwkv.blocks.{i}."
            a, m = p + "attention.", p + "feed_forward."
            self.layers.append({
                "pre_ln": ln(p + "pre_ln") if i == 0 else None, "ln1": ln(p + "ln1"), "ln2": ln(p + "ln2"),
                "a_mix": (h(a + "time_mix_key"), h(a + "time_mix_value"), h(a + "time_mix_receptance")),
                "time_first": f(a + "time_first"), "time_decay": f(a + "time_decay"),
                "a_key": lin(a + "key.weight"), "a_value": lin(a + "value.weight"), "a_recept": lin(a + "receptance.weight"),
                "a_out": lin(a + "output.weight"),
                "f_mix": (h(m + "time_mix_key"), h(m + "time_mix_receptance")),
                "f_key": lin(m + "key.weight"), "f_value": lin(m + "value.weight"), "f_recept": lin(m + "receptance.weight"),
            })
        self.ln_out = ln("rwkv.ln_out")
        self.head = lin("head.weight")
        B, d = batch, c.d_model
        f16 = dict(dtype=torch.float16, device=dev)
        self.ids = torch.full((B, c.max_len), self.pad_id, dtype=torch.int32, device=dev)
        self.step_t = torch.zeros(1, dtype=torch.int32, device=dev)
        self.stop_mask = torch.zeros(B, dtype=torch.int32, device=dev)
        self.x, self.t, self.k, self.v, self.r, self.kk, self.vv, self.rr, self.w = (torch.empty((B, d), **f16) for _ in range(9))
        self.fk, self.fk2 = torch.empty((B, c.ffn), **f16), torch.empty((B, c.ffn), **f16)
        self.logits = torch.empty((B, c.vocab), **f16)
        self.next_val = torch.empty((B, 1), **f16)
        self.next_ids = torch.empty((B, 1), dtype=torch.int32, device=dev)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=dev)
        # states (rwkv/model.py:157-187): previous normalised hidden of the feed-forward / attention paths (fp16), WKV numerator,
        # denominator (0) and running maximum (-1e30) in float32
        self.st_ffn = [torch.zeros((B, d), **f16) for _ in range(c.n_layer)]
        self.st_att = [torch.zeros((B, d), **f16) for _ in range(c.n_layer)]
        self.st_num = [torch.zeros((B, d), dtype=torch.float32, device=dev) for _ in range(c.n_layer)]
        self.st_den = [torch.zeros((B, d), dtype=torch.float32, device=dev) for _ in range(c.n_layer)]
        self.st_max = [torch.full((B, d), -1e30, dtype=torch.float32, device=dev) for _ in range(c.n_layer)]
        self.lin_ws = ops.linear_workspace(B, max(c.ffn, c.vocab, d), 16, dev)
        torch.cuda.synchronize()

    def _linear(self, x, pl, out, epilogue=ops.EPI_STORE, residual=None):
        a = ops.linear_args(x, pl, out, epilogue=epilogue, residual=residual, workspace=self.lin_ws, error_flag=self.error_flag)
        ops.check(ops._lib.lib().pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")

    def _norm(self, x, gb, out):
        ops.check(ops._lib.lib().pt_norm_ce(ops._ptr(x), ops._ptr(gb[0]), ops._ptr(gb[1]), self.batch, self.cfg.d_model, self.cfg.eps,
                                            ops._ptr(out), ops._stream()), "pt_norm_ce")

    def enqueue_step(self):
        c, L_, P, S = self.cfg, ops._lib.lib(), ops._ptr, ops._stream
        B, d = self.batch, c.d_model
        ops.embedding(self.emb, self.ids, self.step_t, out=self.x)
        for i, L in enumerate(self.layers):
            if L["pre_ln"] is not None:
                self._norm(self.x, L["pre_ln"], self.x)
            self._norm(self.x, L["ln1"], self.t)
            mk, mv, mr = L["a_mix"]
            ops.check(L_.pt_rwkv_mix(P(self.t), P(self.st_att[i]), P(mk), P(mv), P(mr), P(self.k), P(self.v), P(self.r), B, d, S()), "pt_rwkv_mix")
            self._linear(self.k, L["a_key"], self.kk)
            self._linear(self.v, L["a_value"], self.vv)
            self._linear(self.r, L["a_recept"], self.rr)
            ops.check(L_.pt_wkv(P(self.kk), P(self.vv), P(L["time_first"]), P(L["time_decay"]), P(self.st_num[i]), P(self.st_den[i]),
                                P(self.st_max[i]), B, d, P(self.w), S()), "pt_wkv")
            ops.check(L_.pt_rwkv_act(0, P(self.rr), P(self.w), P(self.w), B * d, S()), "pt_rwkv_act")
            self._linear(self.w, L["a_out"], self.x, ops.EPI_RESIDUAL, residual=self.x)
            self._norm(self.x, L["ln2"], self.t)
            fk, fr = L["f_mix"]
            ops.check(L_.pt_rwkv_mix(P(self.t), P(self.st_ffn[i]), P(fk), P(fr), None, P(self.k), P(self.r), None, B, d, S()), "pt_rwkv_mix")
            self._linear(self.k, L["f_key"], self.fk)
            ops.check(L_.pt_rwkv_act(1, P(self.fk), None, P(self.fk2), B * c.ffn, S()), "pt_rwkv_act")
            self._linear(self.fk2, L["f_value"], self.vv)
            self._linear(self.r, L["f_recept"], self.rr)
            ops.check(L_.pt_rwkv_act(0, P(self.rr), P(self.vv), P(self.w), B * d, S()), "pt_rwkv_act")
            ops.check(L_.pt_add_f16(P(self.x), P(self.w), B * d, P(self.x), S()), "pt_add_f16")
            if c.rescale_every > 0 and (i + 1) % c.rescale_every == 0:
                ops.check(L_.pt_rwkv_act(2, P(self.x), None, P(self.x), B * d, S()), "pt_rwkv_act")
        self._norm(self.x, self.ln_out, self.t)
        self._linear(self.t, self.head, self.logits)
        ops.check(L_.pt_topk(P(self.logits), B, c.vocab, 1, 0, P(self.next_val), P(self.next_ids), S()), "topk")
        ops.step_containers(self.ids, self.step_t, self.next_ids, self.pad_id, self.eos_id, self.stop_mask)

    def reset(self, input_ids):
        self.ids.copy_(torch.as_tensor(input_ids, dtype=torch.int32).to(self.device))
        self.step_t.zero_()
        self.stop_mask.zero_()
        for i in range(self.cfg.n_layer):
            self.st_ffn[i].zero_(); self.st_att[i].zero_(); self.st_num[i].zero_(); self.st_den[i].zero_(); self.st_max[i].fill_(-1e30)

    def step(self):
        self.enqueue_step()

    def run(self, input_ids, max_loop=None):
        """Session.run analogue (poptransformer/sessions.py:47-49): returns the anchors {'Loop:0': ids, 'Loop:1': step}."""
        self.reset(input_ids)
        for _ in range(self.cfg.max_len if max_loop is None else max_loop):
            self.step()
        torch.cuda.synchronize()
        if int(self.error_flag.item()) != 0:
            raise ops.PtError("a bounded device-side wait gave up")
        return {"Loop:0": self.ids.cpu().numpy(), "Loop:1": self.step_t.cpu().numpy()}
