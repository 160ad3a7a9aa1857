"""GPT-2 decode loop on the per-op kernels: host-side mirror of the reference's GPT2DecModel
(poptransformer/models/gpt2/model.py:121-230) for one token per loop iteration.

Per block (gpt2/model.py:41-50): NormCE -> c_attn (+bias) -> KV append + attention (no RoPE, query scale folded into the
weights, softmax with the exponent in fp16, gpt2/attention.py:59-77) -> c_proj (+bias, +residual) -> NormCE -> c_fc
(+bias, GELU) -> c_proj (+bias, +residual); learned position embedding added to the token embedding
(gpt2/embedding.py:31-36); final NormCE and the LM head tied to wte (gpt2/model.py:139-146).
The state dict uses the reference's key names after `process_hf_model_state_dict` ([out, in] weights, pre-scaled query)."""
import ctypes

import numpy as np
import torch

from . import ops


class GPT2Config:
    def __init__(self, n_layer, d_model, n_head, vocab, n_positions, max_len, eps=1e-5):
        self.n_layer, self.d_model, self.n_head, self.vocab, self.n_positions, self.max_len, self.eps = (
            n_layer, d_model, n_head, vocab, n_positions, max_len, eps)
        self.head_dim = d_model // n_head


class GPT2Decoder:
    def __init__(self, cfg, state_dict, batch, device="cuda", page_size=64, pad_id=None, eos_id=-1):
        c = cfg
        if c.head_dim not in (64, 128):
            raise ops.PtError(f"head size {c.head_dim} not supported by the attention kernel (64, 128)")
        if c.max_len > c.n_positions:
            raise ops.PtError(f"max_len={c.max_len} exceeds n_positions={c.n_positions}")
        self.cfg, self.batch, self.device = cfg, batch, device
        self.pad_id = c.vocab - 1 if pad_id is None else pad_id
        self.eos_id = eos_id
        dev = device
        t = lambda k: state_dict[k].to(dev).to(torch.float16).contiguous()
        self.wte, self.wpe = t("transformer.wte.weight"), t("transformer.wpe.weight")
        self.layers = []
        for i in range(c.n_layer):
            p = f"transformer.h.{i}."
            self.layers.append({
                "ln1": (t(p + "ln_1.weight"), t(p + "ln_1.bias")), "ln2": (t(p + "ln_2.weight"), t(p + "ln_2.bias")),
                "c_attn": ops.PackedLinear(ops.W_FP16, t(p + "attn.c_attn.weight")), "b_attn": t(p + "attn.c_attn.bias"),
                "c_proj": ops.PackedLinear(ops.W_FP16, t(p + "attn.c_proj.weight")), "b_proj": t(p + "attn.c_proj.bias"),
                "c_fc": ops.PackedLinear(ops.W_FP16, t(p + "mlp.c_fc.weight")), "b_fc": t(p + "mlp.c_fc.bias"),
                "m_proj": ops.PackedLinear(ops.W_FP16, t(p + "mlp.c_proj.weight")), "b_mproj": t(p + "mlp.c_proj.bias"),
            })
        self.ln_f = (t("transformer.ln_f.weight"), t("transformer.ln_f.bias"))
        self.head = ops.PackedLinear(ops.W_FP16, self.wte)                       # tied: logits = h . wte^T
        B, d = batch, c.d_model
        f16 = dict(dtype=torch.float16, device=dev)
        self.ids = torch.full((B, c.max_len), self.pad_id, dtype=torch.int32, device=dev)
        self.pos = torch.arange(c.max_len, dtype=torch.int32, device=dev).repeat(B, 1).contiguous()   # position ids = step
        self.step_t = torch.zeros(1, dtype=torch.int32, device=dev)
        self.stop_mask = torch.zeros(B, dtype=torch.int32, device=dev)
        self.x, self.tok, self.pe, self.h = (torch.empty((B, d), **f16) for _ in range(4))
        self.qkv = torch.empty((B, 3 * d), **f16)
        self.attn = torch.empty((B, d), **f16)
        self.act = torch.empty((B, 4 * d), **f16)
        self.logits = torch.empty((B, c.vocab), **f16)
        self.next_val = torch.empty((B, 1), **f16)
        self.next_ids = torch.empty((B, 1), dtype=torch.int32, device=dev)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=dev)
        page_table = None
        self.caches = []
        for _ in range(c.n_layer):
            kc = ops.PagedKVCache(B, c.n_head, c.head_dim, c.max_len, page_size, dev, page_table)
            page_table = kc.page_table
            self.caches.append(kc)
        self.attn_ws = ops.attn_workspace(B, c.n_head, c.head_dim, self.caches[0].max_pages, dev)
        self.lin_ws = ops.linear_workspace(B, max(4 * d, c.vocab), 16, dev)
        self.graph = None
        torch.cuda.synchronize()

    def _linear(self, x, pl, out, epilogue, bias, residual=None):
        a = ops.linear_args(x, pl, out, epilogue=epilogue, bias=bias, residual=residual, workspace=self.lin_ws, error_flag=self.error_flag)
        ops.check(ops._lib.lib().pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")

    def _norm(self, x, gb, out):
        ops.check(ops._lib.lib().pt_norm_ce(ops._ptr(x), ops._ptr(gb[0]), ops._ptr(gb[1]), self.batch, self.cfg.d_model, self.cfg.eps,
                                            ops._ptr(out), ops._stream()), "pt_norm_ce")

    def enqueue_step(self):
        c, L_ = self.cfg, ops._lib.lib()
        ops.embedding(self.wte, self.ids, self.step_t, out=self.tok)
        ops.embedding(self.wpe, self.pos, self.step_t, out=self.pe)
        ops.check(L_.pt_add_f16(ops._ptr(self.tok), ops._ptr(self.pe), self.tok.numel(), ops._ptr(self.x), ops._stream()), "pt_add_f16")
        for li, L in enumerate(self.layers):
            self._norm(self.x, L["ln1"], self.h)
            self._linear(self.h, L["c_attn"], self.qkv, ops.EPI_BIAS, L["b_attn"])
            a = ops.attn_args(self.qkv, self.step_t, self.caches[li], self.attn, c.n_head, ops.ROPE_NONE, ops.SOFTMAX_F16, 1.0, None, None,
                              self.attn_ws, self.error_flag)
            ops.check(L_.pt_kv_append_attn(ctypes.byref(a), ops._stream()), "pt_kv_append_attn")
            self._linear(self.attn, L["c_proj"], self.x, ops.EPI_BIAS_RESIDUAL, L["b_proj"], residual=self.x)
            self._norm(self.x, L["ln2"], self.h)
            self._linear(self.h, L["c_fc"], self.act, ops.EPI_BIAS_GELU, L["b_fc"])
            self._linear(self.act, L["m_proj"], self.x, ops.EPI_BIAS_RESIDUAL, L["b_mproj"], residual=self.x)
        self._norm(self.x, self.ln_f, self.h)
        self._linear(self.h, self.head, self.logits, ops.EPI_STORE, None)
        ops.check(L_.pt_topk(ops._ptr(self.logits), self.batch, c.vocab, 1, 0, ops._ptr(self.next_val), ops._ptr(self.next_ids), ops._stream()),
                  "topk")
        ops.step_containers(self.ids, self.step_t, self.next_ids, self.pad_id, self.eos_id, self.stop_mask)

    def capture(self):
        saved = (self.ids.clone(), self.step_t.clone())
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.enqueue_step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.ids.copy_(saved[0])
        self.step_t.copy_(saved[1])
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.enqueue_step()
        self.graph = g
        self.ids.copy_(saved[0])
        self.step_t.copy_(saved[1])
        torch.cuda.synchronize()

    def reset(self, input_ids):
        self.ids.copy_(torch.as_tensor(input_ids, dtype=torch.int32).to(self.device))
        self.step_t.zero_()
        self.stop_mask.zero_()

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
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
