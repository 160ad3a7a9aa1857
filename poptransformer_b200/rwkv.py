"""RWKV-4 decode loop on the per-op kernels: host-side mirror of the reference's RWKVDecodeModel
(poptransformer/models/rwkv/model.py:121-187, :189-213) for one token per loop iteration.

Per block (rwkv/model.py:44-54): NormCE -> token-shift gates -> key / value / receptance linears -> WKV with float32
(numerator, denominator, max) states -> sigmoid(receptance) * wkv -> output linear (+residual); NormCE -> gates -> key linear ->
relu^2 -> value linear, sigmoid(receptance) gate (+residual); hidden / 2 every `rescale_every` blocks.
The state dict uses the reference's key names after `process_hf_model_state_dict` (output / value weights pre-divided).

Tensor parallel (model_type 'tp', one process per GPU; rwkv/attention.py:108-147, rwkv/ffn.py:62-98): key / value / receptance
are 'start' layers, time_first / time_decay and the WKV states are sharded with the channels (rwkv/model.py:172-184), the
attention output and the feed-forward value are 'end' layers followed by an NCCL all-reduce of the fp16 partial sums, the
feed-forward receptance is all-gathered over the channel shards, and the head is vocab-sharded with the value/id merge of
layers/lm_head.py:75-116.  The embedding stays replicated (the reference's all-reduce there adds exact zeros)."""
import ctypes

import torch

from . import ops
from .loop import DecodeLoop
from .tp import rows, vocab_rows


# Programmatic dependent launch of the linear kernels; off by default: measured 2 % slower at 32 rows on B200.
PDL_DEFAULT = 0


class RWKVConfig:
    def __init__(self, n_layer, d_model, ffn, vocab, max_len, rescale_every=6, eps=1e-5):
        self.n_layer, self.d_model, self.ffn, self.vocab, self.max_len, self.rescale_every, self.eps = (
            n_layer, d_model, ffn, vocab, max_len, rescale_every, eps)


class RWKVDecoder(DecodeLoop):
    def __init__(self, cfg, state_dict, batch, device="cuda", pad_id=None, eos_id=-1, tp_rank=0, tp_size=1, group=None, pdl_linear=None, early_stop=False):
        c = cfg
        self.pdl_linear = PDL_DEFAULT if pdl_linear is None else int(pdl_linear)
        self.tp, self.rank, self.group = tp_size, tp_rank, group
        tp, r = tp_size, tp_rank
        if c.d_model % (32 * tp) or c.ffn % (32 * tp):
            raise ops.PtError(f"d_model={c.d_model} / ffn={c.ffn} must be multiples of 32 * tp")
        dl, fl = c.d_model // tp, c.ffn // tp
        self.d_loc, self.f_loc = dl, fl
        self.cfg, self.batch, self.device = cfg, batch, device
        self.pad_id = c.vocab - 1 if pad_id is None else pad_id
        self.eos_id = eos_id
        self._init_loop(device, early_stop)
        dev = device
        h = lambda k: state_dict[k].to(dev).to(torch.float16).reshape(-1).contiguous()
        f = lambda k: state_dict[k].to(dev).to(torch.float32).reshape(-1)[r * dl:(r + 1) * dl].contiguous()   # sharded with the channels
        w16 = lambda k: state_dict[k].to(dev).to(torch.float16)
        lin = lambda k: ops.PackedLinear(ops.W_FP16, w16(k).contiguous())
        start = lambda k: ops.PackedLinear(ops.W_FP16, rows(w16(k), r, tp).contiguous())
        end = lambda k, kl: ops.PackedLinear(ops.W_FP16, w16(k)[:, r * kl:(r + 1) * kl].contiguous())
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
                "a_key": start(a + "key.weight"), "a_value": start(a + "value.weight"), "a_recept": start(a + "receptance.weight"),
                "a_out": end(a + "output.weight", dl),
                "f_mix": (h(m + "time_mix_key"), h(m + "time_mix_receptance")),
                "f_key": start(m + "key.weight"), "f_value": end(m + "value.weight", fl), "f_recept": start(m + "receptance.weight"),
            })
        self.ln_out = ln("rwkv.ln_out")
        head, self.vocab_loc = vocab_rows(w16("head.weight"), r, tp) if tp > 1 else (w16("head.weight").contiguous(), c.vocab)
        self.head = ops.PackedLinear(ops.W_FP16, head)
        B, d = batch, c.d_model
        f16 = dict(dtype=torch.float16, device=dev)
        self.ids = torch.full((B, c.max_len), self.pad_id, dtype=torch.int32, device=dev)
        self.step_t = torch.zeros(1, dtype=torch.int32, device=dev)
        self.stop_mask = torch.zeros(B, dtype=torch.int32, device=dev)
        self.x, self.t, self.k, self.v, self.r, self.vv, self.rr, self.w = (torch.empty((B, d), **f16) for _ in range(8))
        self.kk, self.vl, self.rl, self.wl = (torch.empty((B, dl), **f16) for _ in range(4))     # this rank's channels
        self.fk, self.fk2 = torch.empty((B, fl), **f16), torch.empty((B, fl), **f16)
        self.logits = torch.empty((B, self.vocab_loc), **f16)
        if tp > 1:
            self.gather_r = torch.empty((tp, B, dl), **f16)
            self.gather_val = torch.empty((tp, B), **f16)
            self.gather_ids = torch.empty((tp, B), dtype=torch.int32, device=dev)
        self.next_val = torch.empty((B, 1), **f16)
        self.next_ids = torch.empty((B, 1), dtype=torch.int32, device=dev)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=dev)
        # states (rwkv/model.py:157-187): previous normalised hidden of the feed-forward / attention paths (fp16), WKV numerator,
        # denominator (0) and running maximum (-1e30) in float32
        self.st_ffn = [torch.zeros((B, d), **f16) for _ in range(c.n_layer)]
        self.st_att = [torch.zeros((B, d), **f16) for _ in range(c.n_layer)]
        self.st_num = [torch.zeros((B, dl), dtype=torch.float32, device=dev) for _ in range(c.n_layer)]
        self.st_den = [torch.zeros((B, dl), dtype=torch.float32, device=dev) for _ in range(c.n_layer)]
        self.st_max = [torch.full((B, dl), -1e30, dtype=torch.float32, device=dev) for _ in range(c.n_layer)]
        self.lin_ws = ops.linear_workspace(B, max(fl, self.vocab_loc, d), 16, dev)
        # The key / value / receptance linears of a block read different mixes of the same hidden state and are independent:
        # on one GPU they run on three streams (fork / join by events, also inside a captured CUDA graph), each with its own
        # split-k workspace, so three short waves share the SMs instead of running back to back.
        self.side = [torch.cuda.Stream(device=dev) for _ in range(2)] if tp == 1 else []
        self.side_ws = [ops.linear_workspace(B, d, 16, dev) for _ in self.side]
        torch.cuda.synchronize()

    def _linear(self, x, pl, out, epilogue=ops.EPI_STORE, residual=None, side=None):
        """side = None: on the current stream; side = i: on side stream i (between _fork and _join), with that stream's workspace."""
        ws = self.lin_ws if side is None else self.side_ws[side]
        a = ops.linear_args(x, pl, out, epilogue=epilogue, residual=residual, workspace=ws, error_flag=self.error_flag, pdl=self.pdl_linear)
        if side is None:
            ops.check(ops._lib.lib().pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")
        else:
            with torch.cuda.stream(self.side[side]):
                ops.check(ops._lib.lib().pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")

    def _fork(self):
        main = torch.cuda.current_stream()
        for s in self.side:
            s.wait_stream(main)

    def _join(self):
        main = torch.cuda.current_stream()
        for s in self.side:
            main.wait_stream(s)

    def _norm(self, x, gb, out):
        ops.check(ops._lib.lib().pt_norm_ce(ops._ptr(x), ops._ptr(gb[0]), ops._ptr(gb[1]), self.batch, self.cfg.d_model, self.cfg.eps,
                                            ops._ptr(out), ops._stream()), "pt_norm_ce")

    def _end(self, x_in, pl, out):
        """'end' layer: out <- all_reduce(fp16(x_in . W_r^T)) over the TP group (layers/linear.py:42-46)."""
        self._linear(x_in, pl, out)
        if self.tp > 1:
            torch.distributed.all_reduce(out, group=self.group)

    def enqueue_step(self):
        c, L_, P, S = self.cfg, ops._lib.lib(), ops._ptr, ops._stream
        B, d, dl, fl = self.batch, c.d_model, self.d_loc, self.f_loc
        ops.embedding(self.emb, self.ids, self.step_t, out=self.x)
        for i, L in enumerate(self.layers):
            if L["pre_ln"] is not None:
                self._norm(self.x, L["pre_ln"], self.x)
            self._norm(self.x, L["ln1"], self.t)
            mk, mv, mr = L["a_mix"]
            ops.check(L_.pt_rwkv_mix(P(self.t), P(self.st_att[i]), P(mk), P(mv), P(mr), P(self.k), P(self.v), P(self.r), B, d, S()), "pt_rwkv_mix")
            par = bool(self.side)
            if par:
                self._fork()
            self._linear(self.k, L["a_key"], self.kk)
            self._linear(self.v, L["a_value"], self.vl, side=0 if par else None)
            self._linear(self.r, L["a_recept"], self.rl, side=1 if par else None)
            if par:
                self._join()
            ops.check(L_.pt_wkv(P(self.kk), P(self.vl), P(L["time_first"]), P(L["time_decay"]), P(self.st_num[i]), P(self.st_den[i]),
                                P(self.st_max[i]), B, dl, P(self.wl), S()), "pt_wkv")
            ops.check(L_.pt_rwkv_act(0, P(self.rl), P(self.wl), P(self.wl), B * dl, S()), "pt_rwkv_act")
            if self.tp == 1:
                self._linear(self.wl, L["a_out"], self.x, ops.EPI_RESIDUAL, residual=self.x)
            else:
                self._end(self.wl, L["a_out"], self.vv)
                ops.check(L_.pt_add_f16(P(self.x), P(self.vv), B * d, P(self.x), S()), "pt_add_f16")
            self._norm(self.x, L["ln2"], self.t)
            fk, fr = L["f_mix"]
            ops.check(L_.pt_rwkv_mix(P(self.t), P(self.st_ffn[i]), P(fk), P(fr), None, P(self.k), P(self.r), None, B, d, S()), "pt_rwkv_mix")
            if par:
                self._fork()
            self._linear(self.k, L["f_key"], self.fk)
            ops.check(L_.pt_rwkv_act(1, P(self.fk), None, P(self.fk2), B * fl, S()), "pt_rwkv_act")
            self._end(self.fk2, L["f_value"], self.vv)
            if self.tp == 1:
                self._linear(self.r, L["f_recept"], self.rr, side=0 if par else None)
                if par:
                    self._join()
            else:       # rwkv/ffn.py:95: all-gather of the receptance shards, read as a concatenation over the channels
                self._linear(self.r, L["f_recept"], self.rl)
                torch.distributed.all_gather_into_tensor(self.gather_r, self.rl, group=self.group)
                self.rr.view(B, self.tp, dl).copy_(self.gather_r.permute(1, 0, 2))
            ops.check(L_.pt_rwkv_act(0, P(self.rr), P(self.vv), P(self.w), B * d, S()), "pt_rwkv_act")
            ops.check(L_.pt_add_f16(P(self.x), P(self.w), B * d, P(self.x), S()), "pt_add_f16")
            if c.rescale_every > 0 and (i + 1) % c.rescale_every == 0:
                ops.check(L_.pt_rwkv_act(2, P(self.x), None, P(self.x), B * d, S()), "pt_rwkv_act")
        self._norm(self.x, self.ln_out, self.t)
        self._linear(self.t, self.head, self.logits)
        if self.tp == 1:
            ops.check(L_.pt_topk(P(self.logits), B, c.vocab, 1, 0, P(self.next_val), P(self.next_ids), S()), "topk")
        else:
            ops.lm_head_tp_merge(self)
        ops.step_containers(self.ids, self.step_t, self.next_ids, self.pad_id, self.eos_id, self.stop_mask, done_flag=self._loop_done_flag())

    def reset(self, input_ids):
        self.ids.copy_(torch.as_tensor(input_ids, dtype=torch.int32).to(self.device))
        self.step_t.zero_()
        self.stop_mask.zero_()
        for i in range(self.cfg.n_layer):
            self.st_ffn[i].zero_(); self.st_att[i].zero_(); self.st_num[i].zero_(); self.st_den[i].zero_(); self.st_max[i].fill_(-1e30)

    def step(self):
        self.enqueue_step()

