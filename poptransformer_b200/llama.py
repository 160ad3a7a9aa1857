"""Llama-2 per-token decode on the B200 kernels.

Host-side mirror of the reference's LLAMA2DecModel loop body
(poptransformer/models/llama2/model.py:162-197, llama2/attention.py:64-122, llama2/mlp.py:20-28,
layers/lm_head.py:47-116, models/base_model.py:313-355): one `step()` is one iteration of the
reference's on-device Loop, i.e. one token per sequence (prompt tokens are consumed one per step, like
the reference's one-stage models; `prefill()` ingests them in one pass like its two-stage models).  The step is five kernels per layer,

    [RMSNorm ->] fused QKV linear -> RoPE + KV append + attention -> o_proj (+ residual)
    [RMSNorm ->] gate|up linear with SwiGLU epilogue -> down_proj (+ residual)

captured once in a CUDA graph and replayed per token; `step`, the id container and all activations
live on the device, so nothing crosses the host boundary between tokens.

Tensor parallelism follows the reference's TP layers (llama2/attention.py:125-144, llama2/mlp.py:31-48,
utils/param_handler/tensor_parallel_strategy.py:21-109): q/k/v/gate/up are column-parallel ('start':
output features split, so heads and FFN channels are split), o/down are row-parallel ('end': input
features split) followed by an all-reduce, the LM head is vocabulary-parallel with a top-1 merge.
One process per GPU; rank r keeps slice r.
"""
import ctypes
import math
from types import SimpleNamespace

import numpy as np
import torch

from . import ops
from .loop import DecodeLoop


class LlamaConfig:
    def __init__(self, n_layer, d_model, n_head, ffn, vocab, eps=1e-5, max_len=128, int4_group=0):
        self.n_layer, self.d_model, self.n_head, self.ffn = n_layer, d_model, n_head, ffn
        self.vocab, self.eps, self.max_len, self.int4_group = vocab, eps, max_len, int4_group
        self.head_dim = d_model // n_head


def rope_tables(max_len, head_dim, device):
    """sin/cos tables with the reference's fp16 recipe (llama2/attention.py:28-38): inv_freq rounded to
    fp16, angle = fp16(fp16(step) * inv_freq), sin/cos of the fp16 angle rounded to fp16."""
    inv_freq = np.array([1.0 / (10000 ** (i / head_dim)) for i in range(0, head_dim, 2)]).astype(np.float16)
    steps = np.arange(max_len, dtype=np.int32).astype(np.float16)
    ang = (steps.astype(np.float32)[:, None] * inv_freq.astype(np.float32)[None, :]).astype(np.float16)
    sin = np.sin(ang.astype(np.float32)).astype(np.float16)
    cos = np.cos(ang.astype(np.float32)).astype(np.float16)
    return torch.from_numpy(sin).to(device), torch.from_numpy(cos).to(device)


from .tp import KSlice as _KSlice, rows as _rows, row_parallel_int4, row_parallel_fp16  # noqa: E402


class LlamaDecoder(DecodeLoop):
    def __init__(self, cfg, state_dict, batch, device="cuda", page_size=64, fuse_norm=None, pad_id=None, eos_id=-1,
                 tp_rank=0, tp_size=1, group=None, pdl=True, persistent=None, keep_logits=True, early_stop=False, tp_buffers=None,
                 wait_limit=0, use_gemm=None, prefill=False):
        """tp_buffers: for tp_size > 1, the exchange buffers of all ranks as this process sees them (a list of tp_size int32 CUDA
        tensors of pt_llama_tp_buffer_bytes each, entry tp_rank being local memory, the others peer mappings the caller set up).
        Default: the buffers are allocated as symmetric memory over `group` (torch.distributed).
        prefill: also keep the weights in the tcgen05 GEMM's tiling so that `prefill()` can ingest a prompt in one pass.
        wait_limit: trip limit of the persistent kernel's polling loops (0 = the library default, about two seconds)."""
        self.cfg, self.batch, self.device = cfg, batch, device
        self._init_loop(device, early_stop)
        self.tp, self.rank, self.group = tp_size, tp_rank, group
        self.pdl = 1 if pdl else 0
        c = cfg
        if c.n_head % tp_size:
            raise ops.PtError(f"n_head={c.n_head} not divisible by tp={tp_size} (llama2/attention.py:130)")
        self.pad_id = c.vocab - 1 if pad_id is None else pad_id
        self.eos_id = eos_id
        self.fuse_norm = (batch <= 8) if fuse_norm is None else fuse_norm
        dev = device
        tp, r = tp_size, tp_rank
        d, f = c.d_model, c.ffn
        self.d_loc, self.f_loc, self.h_loc = d // tp, f // tp, c.n_head // tp

        def t(key):
            return state_dict[key].to(dev)

        # More than 16 rows on one GPU with INT4 weights: the transformer linears run on the tcgen05 GEMM, weights tiled once (beyond
        # 32 rows it is the only path).  Measured on B200, 7B width, 8 blocks: 16 rows 1.54 ms with the skinny-matmul kernels against
        # 1.74 ms with the GEMM; 24 rows 2.44 against 2.02 ms; 32 rows 2.87 against 2.25 ms.
        first_w = state_dict["model.layers.0.self_attn.q_proj.weight"]
        grp0 = (first_w.shape[1] * 2) // max(1, state_dict["model.layers.0.self_attn.q_proj.weight_scale"].numel() // first_w.shape[0]) \
            if first_w.dtype == torch.int8 else 0
        self.use_gemm = ((batch > 16 or use_gemm is True) and use_gemm is not False and tp_size == 1 and first_w.dtype == torch.int8 and grp0 % 128 == 0 and persistent is not True
                         and c.d_model % 128 == 0 and c.ffn % 128 == 0)

        def col_parallel(keys, interleave=False):
            ws = [_rows(t(k), r, tp) for k in keys]
            if ws[0].dtype == torch.int8:
                sc = [_rows(t(k + "_scale").reshape(t(k).shape[0], -1), r, tp) for k in keys]
                grp = (ws[0].shape[1] * 2) // sc[0].shape[1]
                if self.use_gemm:
                    return ops.GemmWeight(ops.W_INT4, torch.cat(ws, 0), torch.cat(sc, 0), group=grp)
                return ops.PackedLinear(ops.W_INT4, torch.cat(ws, 0), torch.cat(sc, 0), group=grp, interleave_gate_up=interleave)
            return ops.PackedLinear(ops.W_FP16, torch.cat(ws, 0).to(torch.float16), interleave_gate_up=interleave)

        def row_parallel(key, k_total):
            w = t(key)
            if w.dtype == torch.int8 and self.use_gemm:
                sc = t(key + "_scale").reshape(w.shape[0], -1)
                return ops.GemmWeight(ops.W_INT4, w, sc, group=(w.shape[1] * 2) // sc.shape[1]), _KSlice(k_total, 0, 1, 128)
            if w.dtype == torch.int8:
                loc, loc_s, grp_loc, ks = row_parallel_int4(w, t(key + "_scale").reshape(w.shape[0], -1), k_total, r, tp)
                return ops.PackedLinear(ops.W_INT4, loc, loc_s, group=grp_loc), ks
            loc, ks = row_parallel_fp16(w, k_total, r, tp)
            return ops.PackedLinear(ops.W_FP16, loc), ks

        def gemm_weight(keys):
            ws = [t(k) for k in keys]
            sc = [t(k + "_scale").reshape(w.shape[0], -1) for k, w in zip(keys, ws)]
            return ops.GemmWeight(ops.W_INT4, torch.cat(ws, 0), torch.cat(sc, 0), group=(ws[0].shape[1] * 2) // sc[0].shape[1])

        self.emb = t("model.embed_tokens.weight").to(torch.float16).contiguous()   # replicated: one row is read per token
        self.layers = []
        for i in range(c.n_layer):
            p = f"model.layers.{i}."
            o, o_ks = row_parallel(p + "self_attn.o_proj.weight", d)
            down, down_ks = row_parallel(p + "mlp.down_proj.weight", f)
            self.layers.append({
                "ln1": t(p + "input_layernorm.weight").contiguous(),
                "ln2": t(p + "post_attention_layernorm.weight").contiguous(),
                "qkv": col_parallel([p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"]),
                "o": o, "gu": col_parallel([p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"], interleave=True), "down": down,
            })
        self.o_ks, self.down_ks = o_ks, down_ks
        # Prompt ingestion runs hundreds of rows through every linear: those go to the tcgen05 GEMM, which wants its own tiling of
        # the weights (a second copy beside the decode kernels' packing when the decode path is not the GEMM itself).
        self.pf_layers = None
        if prefill:
            if not (tp_size == 1 and first_w.dtype == torch.int8 and grp0 % 128 == 0 and c.d_model % 128 == 0 and c.ffn % 128 == 0
                    and c.head_dim == 128 and page_size == 64):
                raise ops.PtError("prefill=True needs INT4 weights (group a multiple of 128), one GPU, head_dim 128 and 64-token pages")
            if self.use_gemm:
                self.pf_layers = self.layers
            else:
                self.pf_layers = []
                for i in range(c.n_layer):
                    p = f"model.layers.{i}."
                    self.pf_layers.append({
                        "ln1": self.layers[i]["ln1"], "ln2": self.layers[i]["ln2"],
                        "qkv": gemm_weight([p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"]),
                        "o": gemm_weight([p + "self_attn.o_proj.weight"]),
                        "gu": gemm_weight([p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"]),
                        "down": gemm_weight([p + "mlp.down_proj.weight"])})
            self._pf_bufs = {}
        self.norm = t("model.norm.weight").contiguous()
        self.vocab_loc = math.ceil(c.vocab / tp)
        head = t("lm_head.weight").to(torch.float16)
        if tp > 1:
            pad = self.vocab_loc * tp - c.vocab
            if pad:
                head = torch.cat([head, torch.zeros((pad, d), dtype=torch.float16, device=dev)], 0)   # shard() zero-pads
            head = head[r * self.vocab_loc:(r + 1) * self.vocab_loc]
        self.head = ops.PackedLinear(ops.W_FP16, head.contiguous())
        self.sin, self.cos = rope_tables(c.max_len, c.head_dim, dev)
        self.score_scale = float(np.float16(1 / math.sqrt(c.head_dim)))
        self._state_opts = dict(page_size=page_size, persistent=persistent, keep_logits=keep_logits, tp_buffers=tp_buffers, wait_limit=wait_limit)
        self._weights_in_stream_order = False
        self._alloc_state()

    def new_stream(self):
        """A second decode stream over the SAME weights: its own id container, step, KV caches, activations, workspaces and (once
        `capture()` is called on it) CUDA graph.  This is what KVCachePipeline's `max_bps` caches are for in the reference
        (custom_ops/kv_cache_pipeline.cpp:392-439): several independent generations share one model and take turns."""
        import copy
        s = copy.copy(self)
        s._init_loop(self.device, self.early_stop)
        if self.pf_layers is not None:
            s._pf_bufs = {}
        s._alloc_state()
        return s

    def _alloc_state(self):
        """Everything a decode stream owns (nothing here depends on the checkpoint values)."""
        c, dev, batch = self.cfg, self.device, self.batch
        tp, r, group = self.tp, self.rank, self.group
        d, f = c.d_model, c.ffn
        page_size, persistent, keep_logits = self._state_opts["page_size"], self._state_opts["persistent"], self._state_opts["keep_logits"]
        tp_buffers, wait_limit = self._state_opts["tp_buffers"], self._state_opts["wait_limit"]
        B = batch
        f16 = dict(dtype=torch.float16, device=dev)
        self.ids = torch.full((B, c.max_len), self.pad_id, dtype=torch.int32, device=dev)
        self.step_t = torch.zeros(1, dtype=torch.int32, device=dev)
        self.stop_mask = torch.zeros(B, dtype=torch.int32, device=dev)
        self.x = torch.empty((B, d), **f16)
        self.h = torch.empty((B, d), **f16)
        self.part = torch.empty((B, d), **f16)                       # row-parallel partial sums (tp > 1)
        self.qkv = torch.empty((B, 3 * self.d_loc), **f16)
        self.attn = torch.zeros((B, self.o_ks.width), **f16)         # zero pads outside the rank's k-range stay zero
        self.act = torch.zeros((B, self.down_ks.width), **f16)
        self.logits = torch.empty((B, self.vocab_loc if tp > 1 else c.vocab), **f16)
        self.next_val = torch.empty((B, 1), **f16)
        self.next_ids = torch.empty((B, 1), dtype=torch.int32, device=dev)
        if tp > 1:
            self.gather_val = torch.empty((tp, B), **f16)
            self.gather_ids = torch.empty((tp, B), dtype=torch.int32, device=dev)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=dev)
        page_table = None
        self.caches = []
        for _ in range(c.n_layer):
            kc = ops.PagedKVCache(B, self.h_loc, c.head_dim, c.max_len, page_size, dev, page_table)
            page_table = kc.page_table
            self.caches.append(kc)
        self.attn_ws = ops.attn_workspace(B, self.h_loc, c.head_dim, self.caches[0].max_pages, dev)
        self.lin_ws = ops.linear_workspace(B, max(3 * self.d_loc, 2 * self.f_loc, d, self.logits.shape[1]), 16, dev)
        if self.use_gemm:
            self.gemm_ws = ops.gemm_workspace(B, max(3 * d, 2 * f), 8, dev)
            self.gu_out = torch.empty((B, 2 * f), **f16)
        self.graph = None
        # The persistent whole-step kernel covers INT4, batch <= 2, on one GPU or tensor-parallel over up to 8 (the all-reduces are
        # then fused into the kernel as peer stores); everything else takes the per-op kernels and NCCL.
        can_persist = (not self.use_gemm and batch <= 2 and c.head_dim == 128 and page_size == 64 and self.layers[0]["qkv"].wfmt == ops.W_INT4
                       and d % 128 == 0 and f % 128 == 0)
        if tp > 1:
            can_persist = (can_persist and tp <= 8 and self.d_loc % 128 == 0 and self.f_loc % 8 == 0 and self.o_ks.offset == 0
                           and self.o_ks.width == self.d_loc and self.down_ks.offset % 8 == 0)
        self.persistent = can_persist if persistent is None else (persistent and can_persist)
        if self.persistent:
            L = ops._lib.lib()

            def to_stream(pl):
                """Packed tiles -> the order in which each SM's consumer warps read them (the per-op kernels cannot use it)."""
                out = torch.empty_like(pl.packed_w)
                ops.check(L.pt_llama_stream_permute(pl.wfmt, ops._ptr(pl.packed_w), ops._ptr(out), pl.n_out, pl.k_in, ops._stream()),
                          "pt_llama_stream_permute")
                pl.packed_w = out

            if not self._weights_in_stream_order:     # once per set of weights; further streams share the permuted tiles
                for lay in self.layers:
                    for k in ("qkv", "o", "gu", "down"):
                        to_stream(lay[k])
                to_stream(self.head)
                self._weights_in_stream_order = True
            arr = (ops._lib.LlamaLayer * c.n_layer)()
            for i, lay in enumerate(self.layers):
                arr[i].qkv, arr[i].o = lay["qkv"].packed_w.data_ptr(), lay["o"].packed_w.data_ptr()
                arr[i].gu, arr[i].down = lay["gu"].packed_w.data_ptr(), lay["down"].packed_w.data_ptr()
                arr[i].ln1, arr[i].ln2 = lay["ln1"].data_ptr(), lay["ln2"].data_ptr()
                arr[i].pool = self.caches[i].pool.data_ptr()
            self.mk_layers = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(dev)
            self.mk_ws = torch.zeros(L.pt_llama_step_workspace_bytes(B, self.h_loc, c.head_dim, self.caches[0].max_pages), dtype=torch.uint8, device=dev)
            a = ops._lib.LlamaStepArgs()
            a.batch, a.d_model, a.n_head, a.head_dim, a.n_layer = B, d, self.h_loc, c.head_dim, c.n_layer
            a.ffn, a.vocab = self.down_ks.width, (self.vocab_loc if tp > 1 else c.vocab)
            a.max_len, a.page_size, a.max_pages, a.pad_id, a.eos_id = c.max_len, page_size, self.caches[0].max_pages, self.pad_id, self.eos_id
            a.norm_eps, a.score_scale = c.eps, self.score_scale
            a.layers, a.norm, a.head, a.emb = self.mk_layers.data_ptr(), self.norm.data_ptr(), self.head.packed_w.data_ptr(), self.emb.data_ptr()
            a.rope_sin, a.rope_cos = self.sin.data_ptr(), self.cos.data_ptr()
            a.ids, a.step_dev, a.stop_mask, a.next_ids = self.ids.data_ptr(), self.step_t.data_ptr(), self.stop_mask.data_ptr(), self.next_ids.data_ptr()
            a.page_table = self.caches[0].page_table.data_ptr()
            # the kernel's own activation scratch: 32-bit words (fp16 value + phase tag), zeroed once
            self.mk_act = [torch.zeros((B, n), dtype=torch.int32, device=dev)
                           for n in ((2 if tp > 1 else 1) * d, 3 * self.d_loc, self.d_loc, self.down_ks.width)]
            a.x, a.qkv, a.attn, a.act = (t.data_ptr() for t in self.mk_act)
            if tp > 1:
                nbytes = L.pt_llama_tp_buffer_bytes(B, d, tp)
                a.tp_size, a.tp_rank = tp, r
                a.ffn_offset, a.ffn_valid, a.vocab_offset, a.emb_rows = self.down_ks.offset, self.f_loc, r * self.vocab_loc, c.vocab
                if tp_buffers is not None:
                    if len(tp_buffers) != tp or any(b.numel() * b.element_size() < nbytes for b in tp_buffers):
                        raise ops.PtError(f"tp_buffers: need {tp} buffers of at least {nbytes} bytes")
                    self.tp_bufs = list(tp_buffers)
                    for i in range(tp):
                        a.tp_buffers[i] = self.tp_bufs[i].data_ptr()
                else:
                    # exchange buffer for the fused all-reduces: symmetric memory, every rank maps every rank's buffer; plain peer
                    # loads / stores only (no multicast object is requested)
                    import torch.distributed._symmetric_memory as symm_mem
                    grp = group if group is not None else torch.distributed.group.WORLD
                    self.tp_buf = symm_mem.empty((nbytes + 3) // 4, dtype=torch.int32, device=dev)
                    self.tp_buf.zero_()
                    self.tp_hdl = symm_mem.rendezvous(self.tp_buf, grp)
                    for i in range(tp):
                        a.tp_buffers[i] = int(self.tp_hdl.buffer_ptrs[i])
                    torch.cuda.synchronize()
                    torch.distributed.barrier(group=grp)
            a.logits = self.logits.data_ptr() if keep_logits else None
            a.workspace, a.workspace_bytes = self.mk_ws.data_ptr(), self.mk_ws.numel()
            a.error_flag = self.error_flag.data_ptr()
            a.done_flag = self.done_flag.data_ptr() if self.early_stop else None
            a.wait_limit = int(wait_limit)
            self.mk_args = a
        torch.cuda.synchronize()

    # ---- accounting -------------------------------------------------------------------------
    def weight_bytes(self):
        """Algorithmic weight bytes this rank streams per step (every linear once, norm weights)."""
        n = sum(L[k].nbytes for L in self.layers for k in ("qkv", "o", "gu", "down")) + self.head.nbytes
        return n + (2 * self.cfg.n_layer + 1) * self.cfg.d_model * 2

    def weight_bytes_total(self):
        """The same for the whole model (all ranks), counted from the logical shapes."""
        c = self.cfg
        lin = c.n_layer * (4 * c.d_model * c.d_model + 3 * c.d_model * c.ffn)
        g = self.layers[0]["qkv"].group
        per_w = (0.5 + 2.0 / g) if self.layers[0]["qkv"].wfmt == ops.W_INT4 else 2.0
        return int(lin * per_w + c.vocab * c.d_model * 2 + (2 * c.n_layer + 1) * c.d_model * 2)

    def kv_bytes_per_token_total(self):
        """KV bytes per cached token per sequence over all layers and heads (read once per step)."""
        c = self.cfg
        return 2 * c.n_layer * c.n_head * c.head_dim * 2

    # ---- one loop iteration -------------------------------------------------------------------
    def _all_reduce(self, tns):
        if self.tp > 1:
            torch.distributed.all_reduce(tns, group=self.group)

    def _norm_linear(self, x, gamma, pl, out, epilogue=ops.EPI_STORE, out_ld=0):
        if x.shape[0] > 32:
            # beyond the skinny-matmul kernels' 32 rows (the fp16 LM head of a large batch, whose transformer linears run on the
            # GEMM): normalise once, then the linear in blocks of 32 rows
            L = ops._lib.lib()
            ops.check(L.pt_rms_norm(ops._ptr(x), None, ops._ptr(gamma), x.shape[0], x.shape[1], self.cfg.eps, ops._ptr(self.h), None,
                                    ops._stream()), "pt_rms_norm")
            for r0 in range(0, x.shape[0], 32):
                ops.linear(self.h[r0:r0 + 32], pl, out[r0:r0 + 32], epilogue=epilogue, workspace=self.lin_ws, out_ld=out_ld, pdl=self.pdl)
            return
        if self.fuse_norm:
            ops.linear(x, pl, out, prologue=ops.PRO_RMSNORM, gamma=gamma, eps=self.cfg.eps, epilogue=epilogue, workspace=self.lin_ws,
                       out_ld=out_ld, pdl=self.pdl)
        else:
            L = ops._lib.lib()
            ops.check(L.pt_rms_norm(ops._ptr(x), None, ops._ptr(gamma), x.shape[0], x.shape[1], self.cfg.eps, ops._ptr(self.h), None,
                                    ops._stream()), "pt_rms_norm")
            ops.linear(self.h, pl, out, epilogue=epilogue, workspace=self.lin_ws, out_ld=out_ld, pdl=self.pdl)

    def _row_parallel(self, x_in, pl):
        """x <- fp16(x + all_reduce(fp16(x_in . W_r^T)))  (Linear 'end' + ops.add, llama2/model.py:42,45)."""
        if self.tp == 1:
            ops.linear(x_in, pl, self.x, epilogue=ops.EPI_RESIDUAL, residual=self.x, workspace=self.lin_ws, pdl=self.pdl)
        else:
            ops.linear(x_in, pl, self.part, workspace=self.lin_ws, pdl=self.pdl)
            self._all_reduce(self.part)
            L = ops._lib.lib()
            ops.check(L.pt_add_f16(ops._ptr(self.x), ops._ptr(self.part), self.x.numel(), ops._ptr(self.x), ops._stream()), "pt_add_f16")

    def enqueue_step(self):
        c = self.cfg
        L_ = ops._lib.lib()
        if self.persistent:
            ops.check(L_.pt_llama_decode_step(ctypes.byref(self.mk_args), ops._stream()), "pt_llama_decode_step")
            return
        ops.embedding(self.emb, self.ids, self.step_t, out=self.x)
        if self.use_gemm:
            self._enqueue_layers_gemm()
            self._enqueue_head()
            return
        attn_out = self.attn.data_ptr() + 2 * self.o_ks.offset      # column offset inside the zero-padded k-window
        act_out = self.act.data_ptr() + 2 * self.down_ks.offset
        for li, L in enumerate(self.layers):
            self._norm_linear(self.x, L["ln1"], L["qkv"], self.qkv)
            a = ops.attn_args(self.qkv, self.step_t, self.caches[li], self.attn, self.h_loc, ops.ROPE_LLAMA, ops.SOFTMAX_F32, self.score_scale,
                              self.sin, self.cos, self.attn_ws, self.error_flag, pdl=self.pdl)
            a.out = attn_out
            a.out_ld = self.attn.shape[1]
            ops.check(L_.pt_kv_append_attn(ctypes.byref(a), ops._stream()), "pt_kv_append_attn")
            self._row_parallel(self.attn, L["o"])
            self._norm_linear_raw(self.x, L["ln2"], L["gu"], act_out, self.act.shape[1])
            self._row_parallel(self.act, L["down"])
        self._enqueue_head()

    def _enqueue_layers_gemm(self):
        """The transformer blocks at 16 or more rows: RMSNorm kernel, tcgen05 GEMMs (residual adds in their epilogues), SwiGLU kernel."""
        c = self.cfg
        L_ = ops._lib.lib()

        def norm(gamma):
            ops.check(L_.pt_rms_norm(ops._ptr(self.x), None, ops._ptr(gamma), self.batch, c.d_model, c.eps, ops._ptr(self.h), None, ops._stream()),
                      "pt_rms_norm")

        for li, L in enumerate(self.layers):
            norm(L["ln1"])
            ops.gemm(self.h, L["qkv"], out=self.qkv, workspace=self.gemm_ws, error_flag=self.error_flag)
            a = ops.attn_args(self.qkv, self.step_t, self.caches[li], self.attn, self.h_loc, ops.ROPE_LLAMA, ops.SOFTMAX_F32, self.score_scale,
                              self.sin, self.cos, self.attn_ws, self.error_flag)
            ops.check(L_.pt_kv_append_attn(ctypes.byref(a), ops._stream()), "pt_kv_append_attn")
            ops.gemm(self.attn, L["o"], out=self.x, epilogue=ops.EPI_RESIDUAL, residual=self.x, workspace=self.gemm_ws, error_flag=self.error_flag)
            norm(L["ln2"])
            ops.gemm(self.h, L["gu"], out=self.gu_out, workspace=self.gemm_ws, error_flag=self.error_flag)
            ops.check(L_.pt_swiglu(ops._ptr(self.gu_out), self.batch, c.ffn, ops._ptr(self.act), self.act.shape[1], ops._stream()), "pt_swiglu")
            ops.gemm(self.act, L["down"], out=self.x, epilogue=ops.EPI_RESIDUAL, residual=self.x, workspace=self.gemm_ws, error_flag=self.error_flag)

    def prefill(self, n_tokens=None, chunk=1024):
        """Ingests the first `n_tokens` positions of every sequence in one pass (the work of the reference's first stage,
        models/base_model.py:358-494) instead of one loop iteration per token: their keys and values go to the caches and the step
        counter moves to `n_tokens`, so the next `step()` is loop iteration `n_tokens` of the token-by-token loop.  Default: one less
        than the shortest prompt (leading ids that are not the pad id), so that the first decode step processes the last prompt
        token every sequence has and ragged prompts keep the loop's rule (a pad position takes the generated id).  Call right
        after `reset()`.  Returns the number of positions ingested.  With `early_stop`, the loop condition is not evaluated over the
        ingested positions (a batch whose prompts all contain the eos id stops on the first decode step, not inside the prompt)."""
        if self.pf_layers is None:
            raise ops.PtError("this decoder was built without prefill=True")
        c, B = self.cfg, self.batch
        if n_tokens is None:
            lead = (self.ids != self.pad_id).to(torch.int32).cumprod(1).sum(1).min()
            n_tokens = int(lead.item()) - 1
        n = int(n_tokens)
        if n <= 0:
            return 0
        if n >= c.max_len:
            raise ops.PtError(f"prefill: n_tokens={n} leaves no decode position (max_len={c.max_len})")
        L_ = ops._lib.lib()
        d, f = c.d_model, c.ffn
        for s0 in range(0, n, chunk):
            P = min(chunk, n - s0)
            rows = B * P
            if rows not in self._pf_bufs:
                f16 = dict(dtype=torch.float16, device=self.device)
                self._pf_bufs = {rows: SimpleNamespace(x=torch.empty((rows, d), **f16), h=torch.empty((rows, d), **f16), qkv=torch.empty((rows, 3 * d), **f16),
                                                       attn=torch.empty((rows, d), **f16), gu=torch.empty((rows, 2 * f), **f16),
                                                       act=torch.empty((rows, f), **f16), ws=ops.gemm_workspace(rows, max(3 * d, 2 * f), 8, self.device))}
            w = self._pf_bufs[rows]
            ops.check(L_.pt_prefill_embed(ops._ptr(self.emb), ops._ptr(self.ids), c.max_len, B, P, s0, d, c.vocab, self.eos_id, ops._ptr(self.stop_mask),
                                          ops._ptr(w.x), ops._stream()), "pt_prefill_embed")

            def norm(gamma):
                ops.check(L_.pt_rms_norm(ops._ptr(w.x), None, ops._ptr(gamma), rows, d, c.eps, ops._ptr(w.h), None, ops._stream()), "pt_rms_norm")

            for li, L in enumerate(self.pf_layers):
                norm(L["ln1"])
                ops.gemm(w.h, L["qkv"], out=w.qkv, workspace=w.ws, error_flag=self.error_flag)
                ops.prefill_attn(w.qkv, self.caches[li], B, P, s0, c.n_head, self.score_scale, self.sin, self.cos, out=w.attn)
                ops.gemm(w.attn, L["o"], out=w.x, epilogue=ops.EPI_RESIDUAL, residual=w.x, workspace=w.ws, error_flag=self.error_flag)
                norm(L["ln2"])
                ops.gemm(w.h, L["gu"], out=w.gu, workspace=w.ws, error_flag=self.error_flag)
                ops.check(L_.pt_swiglu(ops._ptr(w.gu), rows, f, ops._ptr(w.act), f, ops._stream()), "pt_swiglu")
                ops.gemm(w.act, L["down"], out=w.x, epilogue=ops.EPI_RESIDUAL, residual=w.x, workspace=w.ws, error_flag=self.error_flag)
        self.step_t.fill_(n)
        return n

    def _enqueue_head(self):
        c = self.cfg
        L_ = ops._lib.lib()
        self._norm_linear(self.x, self.norm, self.head, self.logits)
        if self.tp == 1:
            ops.check(L_.pt_topk(ops._ptr(self.logits), self.batch, c.vocab, 1, 0, ops._ptr(self.next_val), ops._ptr(self.next_ids),
                                 ops._stream()), "topk")
        else:
            ops.lm_head_tp_merge(self)
        ops.step_containers(self.ids, self.step_t, self.next_ids, self.pad_id, self.eos_id, self.stop_mask, done_flag=self._loop_done_flag())

    def _norm_linear_raw(self, x, gamma, pl, out_ptr, out_ld):
        """gate|up linear with the SwiGLU epilogue writing at a column offset of the (zero-padded) activation buffer."""
        L_ = ops._lib.lib()
        src = x
        pro = ops.PRO_RMSNORM
        if not self.fuse_norm:
            ops.check(L_.pt_rms_norm(ops._ptr(x), None, ops._ptr(gamma), x.shape[0], x.shape[1], self.cfg.eps, ops._ptr(self.h), None,
                                     ops._stream()), "pt_rms_norm")
            src, pro = self.h, ops.PRO_NONE
        a = ops.linear_args(src, pl, self.act, prologue=pro, gamma=gamma if pro else None, eps=self.cfg.eps, epilogue=ops.EPI_SWIGLU,
                            workspace=self.lin_ws, out_ld=out_ld, pdl=self.pdl)
        a.out = out_ptr
        ops.check(L_.pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")

    def enqueue_linears_only(self):
        """Every INT4/FP16 transformer linear of one step, back to back (used to time the dominant kernel alone)."""
        if self.use_gemm:
            for L in self.layers:
                ops.gemm(self.h, L["qkv"], out=self.qkv, workspace=self.gemm_ws)
                ops.gemm(self.attn, L["o"], out=self.part, workspace=self.gemm_ws)
                ops.gemm(self.h, L["gu"], out=self.gu_out, workspace=self.gemm_ws)
                ops.gemm(self.act, L["down"], out=self.part, workspace=self.gemm_ws)
            return
        for L in self.layers:
            self._norm_linear(self.x, L["ln1"], L["qkv"], self.qkv)
            ops.linear(self.attn, L["o"], self.part, workspace=self.lin_ws)
            self._norm_linear_raw(self.x, L["ln2"], L["gu"], self.act.data_ptr(), self.act.shape[1])
            ops.linear(self.act, L["down"], self.part, workspace=self.lin_ws)

    def capture(self):
        """Captures one loop iteration in a CUDA graph (one eager iteration first so lazy initialisation is done)."""
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
        """input_ids int32 [batch, max_len] (host or device), right-padded with pad_id; step <- 0."""
        ids = torch.as_tensor(input_ids, dtype=torch.int32)
        self.ids.copy_(ids.to(self.device, non_blocking=True))
        self.step_t.zero_()
        self.stop_mask.zero_()

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.enqueue_step()
