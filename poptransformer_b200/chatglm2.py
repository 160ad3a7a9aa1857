"""ChatGLM2 decode loop on the per-op kernels: host-side mirror of the reference's ChatGLM2DecodeModel
(poptransformer/models/chatglm2/model.py:95-117, :199-254) for one token per loop iteration.

Per block: RMSNorm -> query | key_value (+bias) -> interleaved RoPE on the first half of each head, multi-query KV append and
attention with the fp16 softmax (chatglm2/attention.py:98-302) -> dense (+residual) -> RMSNorm -> SwiGLU MLP (chatglm2/mlp.py:51-59)
-> dense_4h_to_h (+residual); final RMSNorm and the output layer.  The RMSNorms and (for FP8) the activation casts run as
prologues of the linears.  Weights: fp16, or E4M3 bytes with a float `<key>_scale` per tensor.

Tensor parallel (model_type 'tp', one process per GPU): the query heads of every KV group are split over the ranks and key_value
is replicated (chatglm2/attention.py:316-346 with the weight rearrangement of chatglm2/model.py:29-49), dense and dense_4h_to_h
are 'end' layers followed by an NCCL all-reduce of the fp16 partial sums, dense_h_to_4h_1/2 are 'start' layers
(chatglm2/mlp.py:62-72), the output layer is vocab-sharded with the value/id merge of layers/lm_head.py:75-116; the embedding
stays replicated (the reference's sharded gather plus all-reduce adds exact zeros)."""
import ctypes

import numpy as np
import torch

from . import ops
from .loop import DecodeLoop
from .tp import multi_query_head_index, rows, vocab_rows


# Programmatic dependent launch of the (linear, attention) kernels; off by default: measured neutral to 4 % slower at 8 rows on B200.
PDL_DEFAULT = (0, 0)


class ChatGLM2Config:
    def __init__(self, n_layer, d_model, n_head, n_group, ffn, vocab, max_len, eps=1e-5, precision="fp16", act_scales=None):
        self.n_layer, self.d_model, self.n_head, self.n_group, self.ffn, self.vocab, self.max_len, self.eps = (
            n_layer, d_model, n_head, n_group, ffn, vocab, max_len, eps)
        self.precision = precision
        self.head_dim = d_model // n_head
        self.act_scales = act_scales or {"norm": 8.0 / 448.0, "attn": 2.0 / 448.0, "mlp": 1.0 / 448.0}


def chatglm2_rope_tables(max_len, head_dim, device):
    """sin / cos [max_len, head_dim / 4] with the reference's recipe (chatglm2/attention.py:77-96): float32 inverse frequencies
    for dim = head_dim / 2, float32 angle, cast to fp16, sin / cos of the fp16 angle rounded to fp16."""
    dim = head_dim // 2
    inv_freq = np.array([1.0 / (10000 ** (i / dim)) for i in range(0, dim, 2)]).astype(np.float32)
    ang = (np.arange(max_len, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32).astype(np.float16)
    sin, cos = np.sin(ang.astype(np.float32)).astype(np.float16), np.cos(ang.astype(np.float32)).astype(np.float16)
    return torch.from_numpy(sin).to(device), torch.from_numpy(cos).to(device)


class ChatGLM2Decoder(DecodeLoop):
    def __init__(self, cfg, state_dict, batch, device="cuda", page_size=64, pad_id=None, eos_id=-1, tp_rank=0, tp_size=1, group=None,
                 pdl_linear=None, pdl_attn=None, early_stop=False, use_gemm=None):
        """use_gemm: run the FP8 linears on the tcgen05 GEMM (pt_gemm) with the RMSNorm / SwiGLU / casts as their own small kernels.
        Default: from 8 rows on one GPU (measured on B200 at 8 rows, 65024 x 4096: 45 us against 70 us for the skinny-matmul
        kernel), when every k is a multiple of 128."""
        c = cfg
        self.pdl_linear, self.pdl_attn = PDL_DEFAULT[0] if pdl_linear is None else int(pdl_linear), PDL_DEFAULT[1] if pdl_attn is None else int(pdl_attn)
        self.tp, self.rank, self.group = tp_size, tp_rank, group
        tp, r = tp_size, tp_rank
        if (c.n_head // c.n_group) % tp or c.ffn % tp:
            raise ops.PtError(f"{c.n_head // c.n_group} query heads per group / ffn={c.ffn} not divisible by tp={tp}")
        if c.head_dim not in (64, 128) or c.n_head % c.n_group:
            raise ops.PtError(f"head size {c.head_dim} / groups {c.n_group} not supported")
        self.cfg, self.batch, self.device = cfg, batch, device
        self.pad_id = c.vocab - 1 if pad_id is None else pad_id
        self.eos_id = eos_id
        self._init_loop(device, early_stop)
        dev, fp8 = device, c.precision == "fp8"
        t = lambda k: state_dict[k].to(dev)
        self.use_gemm = bool(fp8 and tp_size == 1 and c.d_model % 128 == 0 and c.ffn % 128 == 0 and
                             (batch >= 8 if use_gemm is None else use_gemm))

        def packed(keys, site, interleave=False, pick=None):
            ws = [t(k) if pick is None or pick[j] is None else pick[j](t(k)) for j, k in enumerate(keys)]
            if fp8:
                scales = {float(state_dict[k + "_scale"]) for k in keys}
                # activation scale of the tensor (the reference casts the input with the scale stored beside the weight,
                # precision_strategy.py:62-66); `<key>_act_scale` in the checkpoint, else the configuration's value for the site
                acts = {float(state_dict[k + "_act_scale"]) if (k + "_act_scale") in state_dict else float(c.act_scales[site]) for k in keys}
                if len(scales) != 1 or len(acts) != 1:
                    raise ops.PtError("fused FP8 linears need one common weight scale and one common activation scale")
                if self.use_gemm:       # rows stay [gate features | up features]: the SwiGLU is its own kernel on this path
                    pl = ops.GemmWeight(ops.W_FP8, torch.cat(ws, 0).contiguous(), w_scale=scales.pop())
                    pl.act_scale = acts.pop()
                    return pl
                pl = ops.PackedLinear(ops.W_FP8, torch.cat(ws, 0).contiguous(), w_scale=scales.pop(), interleave_gate_up=interleave)
                pl.act_scale = acts.pop()
                return pl
            return ops.PackedLinear(ops.W_FP16, torch.cat(ws, 0).to(torch.float16).contiguous(), interleave_gate_up=interleave)

        self.emb = t("transformer.embedding.word_embeddings.weight").to(torch.float16).contiguous()
        self.h_loc, self.d_loc, self.f_loc = c.n_head // tp, c.d_model // tp, c.ffn // tp
        mine = multi_query_head_index(c.n_head, c.n_group, c.head_dim, r, tp).to(dev)       # rank r's query features
        q_rows, start = (lambda w: w[mine]), (lambda w: rows(w, r, tp))
        self.layers = []
        for i in range(c.n_layer):
            p = f"transformer.encoder.layers.{i}."
            self.layers.append({
                "ln1": t(p + "input_layernorm.weight").contiguous(), "ln2": t(p + "post_attention_layernorm.weight").contiguous(),
                "qkv": packed([p + "self_attention.query.weight", p + "self_attention.key_value.weight"], "norm", pick=[q_rows, None]),
                "b_qkv": torch.cat([t(p + "self_attention.query.bias")[mine], t(p + "self_attention.key_value.bias")]).to(torch.float16).contiguous(),
                "dense": packed([p + "self_attention.dense.weight"], "attn", pick=[lambda w: w[:, mine]]),
                "gu": packed([p + "mlp.dense_h_to_4h_1.weight", p + "mlp.dense_h_to_4h_2.weight"], "norm", interleave=True, pick=[start, start]),
                "down": packed([p + "mlp.dense_4h_to_h.weight"], "mlp", pick=[lambda w: w[:, r * self.f_loc:(r + 1) * self.f_loc]]),
            })
        self.norm = t("transformer.encoder.final_layernorm.weight").contiguous()
        self.vocab_loc = -(-c.vocab // tp) if tp > 1 else c.vocab
        self.head = packed(["transformer.output_layer.weight"], "norm", pick=[(lambda w: vocab_rows(w, r, tp)[0]) if tp > 1 else None])
        self.sin, self.cos = chatglm2_rope_tables(c.max_len, c.head_dim, dev)
        self.score_scale = float(np.float16(1.0 / np.sqrt(c.head_dim)))
        B, d = batch, c.d_model
        f16 = dict(dtype=torch.float16, device=dev)
        self.ids = torch.full((B, c.max_len), self.pad_id, dtype=torch.int32, device=dev)
        self.step_t = torch.zeros(1, dtype=torch.int32, device=dev)
        self.stop_mask = torch.zeros(B, dtype=torch.int32, device=dev)
        self.x = torch.empty((B, d), **f16)
        self.qkv = torch.empty((B, (self.h_loc + 2 * c.n_group) * c.head_dim), **f16)
        self.attn = torch.empty((B, self.d_loc), **f16)
        self.act = torch.empty((B, self.f_loc), **f16)
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
            kc = ops.PagedKVCache(B, c.n_group, c.head_dim, c.max_len, page_size, dev, page_table)
            page_table = kc.page_table
            self.caches.append(kc)
        self.attn_ws = ops.attn_workspace(B, self.h_loc, c.head_dim, self.caches[0].max_pages, dev)
        self.lin_ws = ops.linear_workspace(B, max(2 * self.f_loc, self.vocab_loc, self.qkv.shape[1], d), 16, dev)
        if self.use_gemm:
            self.gemm_ws = ops.gemm_workspace(B, max(2 * self.f_loc, self.vocab_loc, self.qkv.shape[1], d), 8, dev)
            self.x8 = torch.empty((B, max(d, self.f_loc)), dtype=torch.uint8, device=dev)      # the E4M3 input of the running linear
            self.gu_out = torch.empty((B, 2 * self.f_loc), **f16)
        self.graph = None
        torch.cuda.synchronize()

    def _linear(self, x, pl, out, site, gamma=None, epilogue=ops.EPI_STORE, bias=None, residual=None):
        fp8 = pl.wfmt == ops.W_FP8
        pro = (ops.PRO_RMSNORM_CAST_FP8 if fp8 else ops.PRO_RMSNORM) if gamma is not None else (ops.PRO_CAST_FP8 if fp8 else ops.PRO_NONE)
        a = ops.linear_args(x, pl, out, prologue=pro, epilogue=epilogue, gamma=gamma, eps=self.cfg.eps,
                            act_scale=pl.act_scale if fp8 else 0.0, bias=bias, residual=residual, workspace=self.lin_ws,
                            error_flag=self.error_flag, pdl=self.pdl_linear)
        ops.check(ops._lib.lib().pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")

    def _row_parallel(self, x_in, pl, site):
        """x <- fp16(x + all_reduce(fp16(x_in . W_r^T)))  (Linear 'end' + the block's ops.add, chatglm2/model.py:113,117)."""
        if self.tp == 1:
            self._linear(x_in, pl, self.x, site, epilogue=ops.EPI_RESIDUAL, residual=self.x)
            return
        self._linear(x_in, pl, self.part, site)
        torch.distributed.all_reduce(self.part, group=self.group)
        ops.check(ops._lib.lib().pt_add_f16(ops._ptr(self.x), ops._ptr(self.part), self.x.numel(), ops._ptr(self.x), ops._stream()), "pt_add_f16")

    def _enqueue_step_gemm(self):
        """The step with every FP8 linear on the tcgen05 GEMM: RMSNorm + cast, q|kv GEMM (+bias), attention (+cast), dense GEMM
        (+residual), RMSNorm + cast, gate|up GEMM, SwiGLU + cast, 4h_to_h GEMM (+residual); final RMSNorm + cast and the output layer."""
        c, L_, B = self.cfg, ops._lib.lib(), self.batch
        d, f = c.d_model, self.f_loc
        st = ops._stream

        def norm_cast(gamma, pl):
            ops.check(L_.pt_rms_norm_fp8(ops._ptr(self.x), ops._ptr(gamma), B, d, c.eps, pl.act_scale, ops._ptr(self.x8), st()), "pt_rms_norm_fp8")
            return self.x8.view(-1)[:B * d].view(B, d)

        def gemm(x8, pl, out, **kw):
            ops.gemm(x8, pl, out=out, x_scale=pl.act_scale, workspace=self.gemm_ws, error_flag=self.error_flag, **kw)

        ops.embedding(self.emb, self.ids, self.step_t, out=self.x)
        for li, L in enumerate(self.layers):
            gemm(norm_cast(L["ln1"], L["qkv"]), L["qkv"], self.qkv, epilogue=ops.EPI_BIAS, bias=L["b_qkv"])
            a8 = self.x8.view(-1)[:B * self.d_loc].view(B, self.d_loc)      # the attention kernel writes dense's E4M3 input itself
            a = ops.attn_args(self.qkv, self.step_t, self.caches[li], self.attn, self.h_loc, ops.ROPE_CHATGLM2, ops.SOFTMAX_F16, self.score_scale,
                              self.sin, self.cos, self.attn_ws, self.error_flag, pdl=self.pdl_attn, out_fp8=a8, out_fp8_scale=L["dense"].act_scale)
            ops.check(L_.pt_kv_append_attn(ctypes.byref(a), st()), "pt_kv_append_attn")
            gemm(a8, L["dense"], self.x, epilogue=ops.EPI_RESIDUAL, residual=self.x)
            gemm(norm_cast(L["ln2"], L["gu"]), L["gu"], self.gu_out)
            h8 = self.x8.view(-1)[:B * f].view(B, f)
            ops.check(L_.pt_swiglu_fp8(ops._ptr(self.gu_out), B, f, L["down"].act_scale, ops._ptr(h8), f, st()), "pt_swiglu_fp8")
            gemm(h8, L["down"], self.x, epilogue=ops.EPI_RESIDUAL, residual=self.x)
        gemm(norm_cast(self.norm, self.head), self.head, self.logits)
        ops.check(L_.pt_topk(ops._ptr(self.logits), B, c.vocab, 1, 0, ops._ptr(self.next_val), ops._ptr(self.next_ids), st()), "topk")
        ops.step_containers(self.ids, self.step_t, self.next_ids, self.pad_id, self.eos_id, self.stop_mask, done_flag=self._loop_done_flag())

    def enqueue_step(self):
        if self.use_gemm:
            return self._enqueue_step_gemm()
        c, L_ = self.cfg, ops._lib.lib()
        ops.embedding(self.emb, self.ids, self.step_t, out=self.x)
        for li, L in enumerate(self.layers):
            self._linear(self.x, L["qkv"], self.qkv, "norm", gamma=L["ln1"], epilogue=ops.EPI_BIAS, bias=L["b_qkv"])
            a = ops.attn_args(self.qkv, self.step_t, self.caches[li], self.attn, self.h_loc, ops.ROPE_CHATGLM2, ops.SOFTMAX_F16, self.score_scale,
                              self.sin, self.cos, self.attn_ws, self.error_flag, pdl=self.pdl_attn)
            ops.check(L_.pt_kv_append_attn(ctypes.byref(a), ops._stream()), "pt_kv_append_attn")
            self._row_parallel(self.attn, L["dense"], "attn")
            self._linear(self.x, L["gu"], self.act, "norm", gamma=L["ln2"], epilogue=ops.EPI_SWIGLU)
            self._row_parallel(self.act, L["down"], "mlp")
        self._linear(self.x, self.head, self.logits, "norm", gamma=self.norm)
        if self.tp == 1:
            ops.check(L_.pt_topk(ops._ptr(self.logits), self.batch, c.vocab, 1, 0, ops._ptr(self.next_val), ops._ptr(self.next_ids),
                                 ops._stream()), "topk")
        else:
            ops.lm_head_tp_merge(self)
        ops.step_containers(self.ids, self.step_t, self.next_ids, self.pad_id, self.eos_id, self.stop_mask, done_flag=self._loop_done_flag())

    def reset(self, input_ids):
        self.ids.copy_(torch.as_tensor(input_ids, dtype=torch.int32).to(self.device))
        self.step_t.zero_()
        self.stop_mask.zero_()

    def step(self):
        self.enqueue_step()

