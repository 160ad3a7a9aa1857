"""GPT-2 decode loop on the per-op kernels: host-side mirror of the reference's GPT2DecModel
(poptransformer/models/gpt2/model.py:121-230) for one token per loop iteration.

Per block (gpt2/model.py:41-50): NormCE -> c_attn (+bias) -> KV append + attention (no RoPE, query scale folded into the
weights, softmax with the exponent in fp16, gpt2/attention.py:59-77) -> c_proj (+bias, +residual) -> NormCE -> c_fc
(+bias, GELU) -> c_proj (+bias, +residual); learned position embedding added to the token embedding
(gpt2/embedding.py:31-36); final NormCE and the LM head tied to wte (gpt2/model.py:139-146).
The state dict uses the reference's key names after `process_hf_model_state_dict` ([out, in] weights, pre-scaled query).

Tensor parallel (model_type 'tp', one process per GPU): c_attn 'fused_qkv', c_fc 'start', both c_proj 'end' with an NCCL
all-reduce of the fp16 partial sums and the bias added once afterwards (gpt2/attention.py:88-96, layers/mlp.py:44-58,
layers/linear.py:42-46), the tied head on the vocab-sharded wte with the value/id merge of layers/lm_head.py:75-116.  The
embedding stays replicated: the reference's vocab-sharded gathers summed by an all-reduce (gpt2/embedding.py:38-46) add
exact zeros to fp16(wte[id] + wpe[step])."""
import ctypes

import numpy as np
import torch

from . import ops
from .loop import DecodeLoop
from .tp import fused_qkv_rows, rows, vocab_rows


def pdl_default(rows):
    """Programmatic dependent launch of the (linear, attention) kernels: a kernel launched this way starts its weight prefetch
    while the previous kernel of the stream drains.  Measured on B200: 5 % faster steps for GPT-2 small at one row, where every
    kernel is a single short wave; neutral or slower (waiting blocks hold shared memory) at 16 rows."""
    return (1, 1) if rows <= 2 else (0, 0)


class GPT2Config:
    def __init__(self, n_layer, d_model, n_head, vocab, n_positions, max_len, eps=1e-5):
        self.n_layer, self.d_model, self.n_head, self.vocab, self.n_positions, self.max_len, self.eps = (
            n_layer, d_model, n_head, vocab, n_positions, max_len, eps)
        self.head_dim = d_model // n_head


class GPT2Decoder(DecodeLoop):
    def __init__(self, cfg, state_dict, batch, device="cuda", page_size=64, pad_id=None, eos_id=-1, tp_rank=0, tp_size=1, group=None,
                 spare_pages=0, pdl_linear=None, pdl_attn=None, early_stop=False):
        c = cfg
        self.tp, self.rank, self.group = tp_size, tp_rank, group
        self.pdl_linear = pdl_default(batch)[0] if pdl_linear is None else int(pdl_linear)
        self.pdl_attn = pdl_default(batch)[1] if pdl_attn is None else int(pdl_attn)
        tp, r = tp_size, tp_rank
        if c.n_head % tp:
            raise ops.PtError(f"n_head={c.n_head} not divisible by tp={tp} (gpt2/attention.py:95)")
        if c.head_dim not in (64, 128):
            raise ops.PtError(f"head size {c.head_dim} not supported by the attention kernel (64, 128)")
        if c.max_len > c.n_positions:
            raise ops.PtError(f"max_len={c.max_len} exceeds n_positions={c.n_positions}")
        self.cfg, self.batch, self.device = cfg, batch, device
        self.pad_id = c.vocab - 1 if pad_id is None else pad_id
        self.eos_id = eos_id
        self._init_loop(device, early_stop)
        dev = device
        t = lambda k: state_dict[k].to(dev).to(torch.float16).contiguous()
        self.wte, self.wpe = t("transformer.wte.weight"), t("transformer.wpe.weight")
        B, d = batch, c.d_model
        self.d_loc, self.h_loc = d // tp, c.n_head // tp
        cols = lambda w, k: w[:, r * (k // tp):(r + 1) * (k // tp)].contiguous()        # 'end': rank r's input features
        end_bias = lambda b: b if tp == 1 else b.repeat(B, 1).contiguous()           # added once, after the all-reduce
        self.layers = []
        for i in range(c.n_layer):
            p = f"transformer.h.{i}."
            self.layers.append({
                "ln1": (t(p + "ln_1.weight"), t(p + "ln_1.bias")), "ln2": (t(p + "ln_2.weight"), t(p + "ln_2.bias")),
                "c_attn": ops.PackedLinear(ops.W_FP16, fused_qkv_rows(t(p + "attn.c_attn.weight"), r, tp).contiguous()),
                "b_attn": fused_qkv_rows(t(p + "attn.c_attn.bias"), r, tp).contiguous(),
                "c_proj": ops.PackedLinear(ops.W_FP16, cols(t(p + "attn.c_proj.weight"), d)), "b_proj": end_bias(t(p + "attn.c_proj.bias")),
                "c_fc": ops.PackedLinear(ops.W_FP16, rows(t(p + "mlp.c_fc.weight"), r, tp).contiguous()),
                "b_fc": rows(t(p + "mlp.c_fc.bias"), r, tp).contiguous(),
                "m_proj": ops.PackedLinear(ops.W_FP16, cols(t(p + "mlp.c_proj.weight"), 4 * d)), "b_mproj": end_bias(t(p + "mlp.c_proj.bias")),
            })
        self.ln_f = (t("transformer.ln_f.weight"), t("transformer.ln_f.bias"))
        head, self.vocab_loc = vocab_rows(self.wte, r, tp) if tp > 1 else (self.wte, c.vocab)
        self.head = ops.PackedLinear(ops.W_FP16, head)                           # tied: logits = h . wte^T
        f16 = dict(dtype=torch.float16, device=dev)
        self.ids = torch.full((B, c.max_len), self.pad_id, dtype=torch.int32, device=dev)
        self.pos = torch.arange(c.max_len, dtype=torch.int32, device=dev).repeat(B, 1).contiguous()   # position ids = step
        self.step_t = torch.zeros(1, dtype=torch.int32, device=dev)
        self.stop_mask = torch.zeros(B, dtype=torch.int32, device=dev)
        self.x, self.tok, self.pe, self.h = (torch.empty((B, d), **f16) for _ in range(4))
        self.qkv = torch.empty((B, 3 * self.d_loc), **f16)
        self.attn = torch.empty((B, self.d_loc), **f16)
        self.act = torch.empty((B, 4 * self.d_loc), **f16)
        self.part = torch.empty((B, d), **f16)                       # row-parallel partial sums (tp > 1)
        self.logits = torch.empty((B, self.vocab_loc), **f16)
        if tp > 1:
            self.gather_val = torch.empty((tp, B), **f16)
            self.gather_ids = torch.empty((tp, B), dtype=torch.int32, device=dev)
        self.next_val = torch.empty((B, 1), **f16)
        self.next_ids = torch.empty((B, 1), dtype=torch.int32, device=dev)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=dev)
        page_table = None
        self.caches = []
        for _ in range(c.n_layer):
            kc = ops.PagedKVCache(B, self.h_loc, c.head_dim, c.max_len, page_size, dev, page_table, extra_pages=spare_pages)
            page_table = kc.page_table
            self.caches.append(kc)
        self.attn_ws = ops.attn_workspace(B, self.h_loc, c.head_dim, self.caches[0].max_pages, dev)
        self.lin_ws = ops.linear_workspace(B, max(4 * d, self.vocab_loc), 16, dev)
        self.graph = None
        torch.cuda.synchronize()

    def _linear(self, x, pl, out, epilogue, bias, residual=None, norm=None):
        """norm = (gamma, beta): the LayerNorm in front of the linear (ops.layer_norm_ce, NormCE arithmetic) runs as the kernel's
        prologue instead of as a launch of its own."""
        pro = {}
        if norm is not None and self.batch <= 8:
            pro = dict(prologue=ops.PRO_NORMCE, gamma=norm[0], beta=norm[1], eps=self.cfg.eps)
        elif norm is not None:
            # every block of the linear repeats the row statistics: from 16 rows on a launch of its own is faster
            # (measured on B200, GPT-2 XL, 16 rows: 4.12 ms per step against 4.36 fused)
            self._norm(x, norm, self.h)
            x = self.h
        a = ops.linear_args(x, pl, out, epilogue=epilogue, bias=bias, residual=residual, workspace=self.lin_ws, error_flag=self.error_flag,
                            pdl=self.pdl_linear, **pro)
        ops.check(ops._lib.lib().pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")

    def _norm(self, x, gb, out):
        ops.check(ops._lib.lib().pt_norm_ce(ops._ptr(x), ops._ptr(gb[0]), ops._ptr(gb[1]), self.batch, self.cfg.d_model, self.cfg.eps,
                                            ops._ptr(out), ops._stream()), "pt_norm_ce")

    def _row_parallel(self, x_in, pl, bias):
        """x <- fp16(x + fp16(all_reduce(fp16(x_in . W_r^T)) + bias))  (Linear 'end' + the block's ops.add, gpt2/model.py:44-49)."""
        if self.tp == 1:
            self._linear(x_in, pl, self.x, ops.EPI_BIAS_RESIDUAL, bias, residual=self.x)
            return
        L_ = ops._lib.lib()
        self._linear(x_in, pl, self.part, ops.EPI_STORE, None)
        torch.distributed.all_reduce(self.part, group=self.group)
        ops.check(L_.pt_add_f16(ops._ptr(self.part), ops._ptr(bias), self.part.numel(), ops._ptr(self.part), ops._stream()), "pt_add_f16")
        ops.check(L_.pt_add_f16(ops._ptr(self.x), ops._ptr(self.part), self.x.numel(), ops._ptr(self.x), ops._stream()), "pt_add_f16")

    def enqueue_step(self):
        self.enqueue_logits()
        self.enqueue_next()

    def enqueue_logits(self):
        """Embedding, every block, final norm and the (tied) head: fills self.logits for the token at position *step."""
        c, L_ = self.cfg, ops._lib.lib()
        ops.embedding(self.wte, self.ids, self.step_t, out=self.tok)
        ops.embedding(self.wpe, self.pos, self.step_t, out=self.pe)
        ops.check(L_.pt_add_f16(ops._ptr(self.tok), ops._ptr(self.pe), self.tok.numel(), ops._ptr(self.x), ops._stream()), "pt_add_f16")
        for li, L in enumerate(self.layers):
            self._linear(self.x, L["c_attn"], self.qkv, ops.EPI_BIAS, L["b_attn"], norm=L["ln1"])
            a = ops.attn_args(self.qkv, self.step_t, self.caches[li], self.attn, self.h_loc, ops.ROPE_NONE, ops.SOFTMAX_F16, 1.0, None, None,
                              self.attn_ws, self.error_flag, pdl=self.pdl_attn)
            ops.check(L_.pt_kv_append_attn(ctypes.byref(a), ops._stream()), "pt_kv_append_attn")
            self._row_parallel(self.attn, L["c_proj"], L["b_proj"])
            self._linear(self.x, L["c_fc"], self.act, ops.EPI_BIAS_GELU, L["b_fc"], norm=L["ln2"])
            self._row_parallel(self.act, L["m_proj"], L["b_mproj"])
        self._linear(self.x, self.head, self.logits, ops.EPI_STORE, None, norm=self.ln_f)

    def enqueue_next(self):
        """Greedy head and the loop carry (layers/lm_head.py:47-57, models/base_model.py:313-335)."""
        c, L_ = self.cfg, ops._lib.lib()
        if self.tp == 1:
            ops.check(L_.pt_topk(ops._ptr(self.logits), self.batch, c.vocab, 1, 0, ops._ptr(self.next_val), ops._ptr(self.next_ids),
                                 ops._stream()), "topk")
        else:
            ops.lm_head_tp_merge(self)
        ops.step_containers(self.ids, self.step_t, self.next_ids, self.pad_id, self.eos_id, self.stop_mask, done_flag=self._loop_done_flag())

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



class GPT2BeamDecoder(GPT2Decoder):
    """Beam decode: the `BeamSearch` custom op (custom_ops/beam_search_custom_op.cpp:333-478) on top of the GPT-2 step, with the
    beam reorder of the paged KV cache.

    The reference registers the op but none of its Python models calls it, so the composition is the one the op's interface
    implies: every hypothesis is a cache row (row = prompt * beam + slot), the prompt is fed token by token to all slots, and
    from the last prompt token on the fp16 logits [prompts, beam, vocab] are the scores the op adds to the running `prob`; its
    next ids become the next input tokens and every slot continues from the cache row of the hypothesis it extends (`parent`).
    Full cache pages are shared between rows through the page table; only the page being filled is copied, into a spare page
    per row."""

    def __init__(self, cfg, state_dict, n_prompts, beam, new_tokens, device="cuda", page_size=64, pad_id=None, **kw):
        rows = n_prompts * beam
        super().__init__(cfg, state_dict, rows, device=device, page_size=page_size, pad_id=pad_id, spare_pages=rows, **kw)
        self.n_prompts, self.beam, self.new_tokens = n_prompts, beam, new_tokens
        dev = device
        kc = self.caches[0]
        self.spare = (torch.arange(rows, dtype=torch.int32, device=dev) + rows * kc.max_pages).contiguous()
        self.table_tmp = torch.empty_like(kc.page_table)
        self.table0 = kc.page_table.clone()
        self.hyp = torch.zeros((n_prompts, new_tokens, beam), dtype=torch.int32, device=dev)
        self.prob = torch.zeros((n_prompts, beam), dtype=torch.float16, device=dev)
        self.gen_step = torch.zeros(1, dtype=torch.int32, device=dev)
        self.parent = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.beam_next = torch.empty((n_prompts, beam), dtype=torch.int32, device=dev)
        self.beam_best = torch.empty((n_prompts, beam), dtype=torch.int32, device=dev)
        L = ops._lib.lib()
        self.beam_ws = torch.empty(L.pt_beam_search_workspace_bytes(n_prompts, beam, new_tokens), dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()

    def enqueue_beam(self):
        """BeamSearch on this step's logits, the loop carry, and the cache reorder for the next step."""
        c, L, P, S = self.cfg, ops._lib.lib(), ops._ptr, ops._stream
        ops.check(L.pt_beam_search(P(self.logits), P(self.hyp), P(self.prob), P(self.gen_step), self.n_prompts, self.beam, c.vocab,
                                   self.new_tokens, 0, P(self.beam_next), P(self.beam_best), P(self.parent), P(self.beam_ws),
                                   self.beam_ws.numel(), S()), "BeamSearch")
        # the chosen ids go into the (still padded) next column of every row's container; *step becomes the next position
        ops.step_containers(self.ids, self.step_t, self.beam_next.view(-1, 1), self.pad_id, -1, self.stop_mask)
        kc = self.caches[0]
        for cache in self.caches:
            ops.check(L.pt_kv_reorder_pages(P(cache.pool), P(kc.page_table), P(self.spare), P(self.parent), P(self.step_t), self.batch,
                                            cache.n_kv, cache.head_dim, cache.page_size, cache.max_pages, S()), "pt_kv_reorder_pages")
        ops.check(L.pt_kv_reorder_table(P(kc.page_table), P(self.table_tmp), P(self.spare), P(self.parent), P(self.step_t), self.batch,
                                        kc.page_size, kc.max_pages, S()), "pt_kv_reorder_table")
        self.gen_step.add_(1)

    def start_beam(self, prompt):
        """Loads prompt int [n_prompts, P] (equal lengths, no pad ids) into every slot's container and clears the cache mapping,
        the hypothesis / score containers and the step counters.  Returns P."""
        prompt = torch.as_tensor(prompt, dtype=torch.int32)
        n, P = prompt.shape
        if n != self.n_prompts or P + self.new_tokens > self.cfg.max_len:
            raise ops.PtError(f"prompt shape {tuple(prompt.shape)} does not fit {self.n_prompts} prompts / max_len {self.cfg.max_len}")
        ids = torch.full((self.batch, self.cfg.max_len), self.pad_id, dtype=torch.int32)
        ids[:, :P] = prompt.repeat_interleave(self.beam, dim=0)
        self.reset(ids)
        self.caches[0].page_table.copy_(self.table0)
        self.spare.copy_(torch.arange(self.batch, dtype=torch.int32, device=self.device) + self.batch * self.caches[0].max_pages)
        self.hyp.zero_(); self.prob.zero_(); self.gen_step.zero_()
        return P

    def run_beam(self, prompt):
        """Returns {'hyp': [n_prompts, new_tokens, beam], 'prob': [n_prompts, beam]}: the op's hypothesis and score containers
        after `new_tokens` generated positions."""
        P = self.start_beam(prompt)
        for t in range(P + self.new_tokens - 1):
            self.enqueue_logits()
            if t + 1 < P:
                self.enqueue_next()          # the container already holds the next prompt token: only *step advances
            else:
                self.enqueue_beam()
        torch.cuda.synchronize()
        if int(self.error_flag.item()) != 0:
            raise ops.PtError("a bounded device-side wait gave up")
        return {"hyp": self.hyp.cpu().numpy(), "prob": self.prob.cpu().numpy()}
