"""Host-side mirror of the reference's custom-op surface (poptransformer/ops/customized.py)
on CUDA tensors.  Same op names and argument meanings; every function enqueues kernels of
libpt_b200.so on torch's current stream.  PyTorch is used for device memory and streams only.

Reference op            -> function here
  KVCache               -> kv_cache            (dense reference layout, bit-exact)
  KVCachePipeline       -> kv_cache_pipeline
  Int4ToHalf            -> int4_to_half
  SoftmaxV3             -> softmax_ce
  NormCE                -> layer_norm_ce
  CastToUint8...        -> half_to_uint8
  FP8MatMul...          -> fp8_matmul
  BeamSearch            -> beam_search
  Remap                 -> remap_tensor        (layout hint on IPU; identity here)
plus the fused decode stages that replace chains of reference ops: PackedLinear / linear,
rms_norm, kv_append_attn, topk, embedding, step_containers, wkv.
"""
import ctypes

import torch

from . import _lib
from ._lib import AttnArgs, GemmArgs, LinearArgs, PtError, check

W_INT4, W_FP16, W_FP8 = 0, 1, 2
PRO_NONE, PRO_RMSNORM, PRO_CAST_FP8, PRO_RMSNORM_CAST_FP8, PRO_NORMCE = 0, 1, 2, 3, 4
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL = 0, 1, 2, 3, 4, 5
ROPE_NONE, ROPE_LLAMA, ROPE_CHATGLM2 = 0, 1, 2
SOFTMAX_F32, SOFTMAX_F16 = 0, 1


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise PtError("libpt_b200 ops need CUDA tensors (there is no CPU path)")
    if not t.is_contiguous():
        raise PtError("libpt_b200 ops need contiguous tensors")
    return ctypes.c_void_p(t.data_ptr())


def launch_count():
    return int(_lib.lib().pt_launch_count())


# ------------------------------------------------------------------------------------------ Int4ToHalf
def int4_to_half(x, scale, ref=None, axis=1, remap=1, group=0):
    """ops.int4_to_half (customized.py:115-124).  x int8 [n, m]; scale fp16 [n] (axis 1) / [m]
    (axis 0) or [n, 2m/group].  `ref` and `remap` only steer the IPU layout and are ignored."""
    n, m = x.shape
    out = torch.empty((2 * m, n) if axis == 1 else (2 * n, m), dtype=torch.float16, device=x.device)
    check(_lib.lib().pt_int4_to_half(_ptr(x), _ptr(scale), n, m, axis, group, _ptr(out), _stream()), "Int4ToHalf")
    return out


# ------------------------------------------------------------------------------------------ linear
class PackedLinear:
    """A weight matrix in the streaming kernel's tile order (built once at load time).

    w: [n_out, k] with k contiguous — INT4: int8 [n_out, k/2] in the reference checkpoint format
    (precision_strategy.py:24-42) with fp16 scales [n_out] or [n_out, k/group]; FP16: fp16 [n_out, k]
    (the HF [out, in] layout, i.e. before the reference's load-time transpose, layers/linear.py:32);
    FP8: uint8 E4M3 [n_out, k] with a per-tensor scale."""

    def __init__(self, wfmt, w, scale=None, group=0, interleave_gate_up=False, w_scale=1.0):
        L = _lib.lib()
        self.wfmt = wfmt
        self.n_out = w.shape[0]
        self.k_in = w.shape[1] * 2 if wfmt == W_INT4 else w.shape[1]
        self.w_scale = float(w_scale)
        self.interleaved = bool(interleave_gate_up)
        if wfmt == W_INT4:
            self.group = int(group) if group else self.k_in
            scale = scale.reshape(self.n_out, self.k_in // self.group).contiguous()
        else:
            self.group = 0
        nbytes = L.pt_linear_packed_bytes(wfmt, self.n_out, self.k_in)
        self.packed_w = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
        check(L.pt_linear_repack(wfmt, _ptr(w.contiguous()), _ptr(scale) if scale is not None else None, self.n_out, self.k_in,
                                 self.group, 1 if interleave_gate_up else 0, _ptr(self.packed_w), _stream()), "pt_linear_repack")

    @property
    def nbytes(self):
        """Algorithmic bytes one launch streams from HBM: weights plus one fp16 scale per row and group.  (The
        packed tiles repeat a scale for every 128-k chunk of its group, so the buffer itself can be larger.)"""
        sb = self.n_out * (self.k_in // self.group) * 2 if self.wfmt == W_INT4 else 0
        wb = self.n_out * self.k_in // 2 if self.wfmt == W_INT4 else self.n_out * self.k_in * (2 if self.wfmt == W_FP16 else 1)
        return wb + sb


def linear_workspace(batch, n_out_max, max_ksplit=16, device="cuda"):
    """Zero-initialised split-k workspace shared by all linears of a stream (counters must start at 0;
    every launch leaves them at 0)."""
    n = _lib.lib().pt_linear_workspace_bytes(batch, n_out_max, max_ksplit)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def linear_args(x, pl, out, prologue=PRO_NONE, epilogue=EPI_STORE, gamma=None, eps=0.0, act_scale=0.0, bias=None,
                residual=None, workspace=None, ksplit=0, out_ld=0, pdl=0, error_flag=None, beta=None):
    a = LinearArgs()
    a.wfmt, a.batch, a.n_out, a.k_in, a.group = pl.wfmt, x.shape[0], pl.n_out, pl.k_in, pl.group
    a.prologue, a.epilogue, a.ksplit = prologue, epilogue, ksplit
    a.x, a.packed_w = _ptr(x), _ptr(pl.packed_w)
    a.norm_gamma, a.norm_eps, a.act_scale, a.w_scale = _ptr(gamma), eps, act_scale, pl.w_scale
    a.bias, a.residual, a.out, a.out_ld, a.pdl = _ptr(bias), _ptr(residual), _ptr(out), out_ld, pdl
    a.error_flag, a.norm_beta = _ptr(error_flag), _ptr(beta)
    a.workspace = _ptr(workspace)
    a.workspace_bytes = workspace.numel() if workspace is not None else 0
    return a


def linear(x, pl, out=None, **kw):
    """y = epilogue(prologue(x) @ W^T).  x fp16 [batch <= 32, k]."""
    if x.shape[1] != pl.k_in:
        raise PtError(f"linear: x has k={x.shape[1]}, weight has k={pl.k_in}")
    n = pl.n_out // 2 if kw.get("epilogue", EPI_STORE) == EPI_SWIGLU else pl.n_out
    if out is None:
        out = torch.empty((x.shape[0], n), dtype=torch.float16, device=x.device)
    a = linear_args(x, pl, out, **kw)
    check(_lib.lib().pt_linear(ctypes.byref(a), _stream()), "pt_linear")
    return out


# ------------------------------------------------------------------------------------------ tensor-core GEMMs (16+ rows)
class GemmWeight:
    """A weight matrix tiled once for pt_gemm (pt_gemm_repack): FP8 bytes [n_out, k], or INT4 rows in the reference's int8
    [n_out, k/2] format plus fp16 scales [n_out, k/group]."""

    def __init__(self, wfmt, w, scale=None, group=0, w_scale=1.0):
        L = _lib.lib()
        self.wfmt, self.n_out, self.w_scale = wfmt, w.shape[0], float(w_scale)
        if wfmt == W_INT4:
            self.k_in = w.shape[1] * 2
            self.group = int(group) if group else self.k_in
            self.scales = scale.reshape(self.n_out, self.k_in // self.group).to(torch.float16).contiguous()
        elif wfmt == W_FP8:
            self.k_in, self.group, self.scales = w.shape[1], 0, None
        else:
            raise PtError("GemmWeight: INT4 or FP8")
        self.w = torch.empty(L.pt_gemm_packed_bytes(wfmt, self.n_out, self.k_in), dtype=torch.uint8, device=w.device)
        check(L.pt_gemm_repack(wfmt, _ptr(w.contiguous()), self.n_out, self.k_in, _ptr(self.w), _stream()), "pt_gemm_repack")

    @property
    def nbytes(self):
        """Algorithmic bytes one launch streams from HBM."""
        wb = self.n_out * self.k_in // 2 if self.wfmt == W_INT4 else self.n_out * self.k_in
        return wb + (self.scales.numel() * 2 if self.scales is not None else 0)


def gemm_workspace(m, n_out_max, max_ksplit=8, device="cuda"):
    return torch.zeros(_lib.lib().pt_gemm_workspace_bytes(m, n_out_max, max_ksplit), dtype=torch.uint8, device=device)


def gemm(x, gw, out=None, x_scale=1.0, epilogue=EPI_STORE, residual=None, workspace=None, ksplit=0, error_flag=None, bias=None):
    """y = x @ W^T on the tcgen05 GEMM.  INT4: x fp16 [m, k]; FP8: x E4M3 bytes [m, k] quantised with `x_scale`."""
    m = x.shape[0]
    if x.shape[1] != gw.k_in:
        raise PtError(f"gemm: x has k={x.shape[1]}, weight has k={gw.k_in}")
    if out is None:
        out = torch.empty((m, gw.n_out), dtype=torch.float16, device=x.device)
    a = GemmArgs()
    a.wfmt, a.m, a.n_out, a.k_in, a.group, a.epilogue, a.ksplit = gw.wfmt, m, gw.n_out, gw.k_in, gw.group, epilogue, ksplit
    a.w_tiled = 1
    a.x, a.w, a.scales = _ptr(x), _ptr(gw.w), _ptr(gw.scales)
    a.x_scale, a.w_scale = float(x_scale), gw.w_scale
    a.residual, a.out, a.out_ld = _ptr(residual), _ptr(out), 0
    a.workspace, a.workspace_bytes = _ptr(workspace), (workspace.numel() if workspace is not None else 0)
    a.error_flag, a.bias = _ptr(error_flag), _ptr(bias)
    check(_lib.lib().pt_gemm(ctypes.byref(a), _stream()), "pt_gemm")
    return out


# ------------------------------------------------------------------------------------------ norms / softmax
def layer_norm_ce(x, gamma, beta, eps, batch_size=None, sequence_length=None, input_size=None):
    """ops.layer_norm_ce (customized.py:69-102): LayerNorm over the last dim with the NormCE arithmetic."""
    dim = x.shape[-1]
    rows = x.numel() // dim
    out = torch.empty_like(x)
    check(_lib.lib().pt_norm_ce(_ptr(x), _ptr(gamma), _ptr(beta), rows, dim, float(eps), _ptr(out), _stream()), "NormCE")
    return out


def rms_norm(x, gamma, eps, residual=None):
    """RMSLayerNorm (layers/rms_layer_norm.py:26-36); with `residual` returns (norm(x + residual), x + residual)."""
    dim = x.shape[-1]
    rows = x.numel() // dim
    out = torch.empty_like(x)
    s = torch.empty_like(x) if residual is not None else None
    check(_lib.lib().pt_rms_norm(_ptr(x), _ptr(residual), _ptr(gamma), rows, dim, float(eps), _ptr(out), _ptr(s), _stream()), "pt_rms_norm")
    return (out, s) if residual is not None else out


def softmax_ce(x, dim=-1, stable_mode=True):
    """ops.softmax_ce (customized.py:57-65) over the last axis; fp16 or fp32 input."""
    if dim not in (-1, x.dim() - 1):
        raise PtError("SoftmaxV3: only the last axis is supported (the reference flattens to [rows, last])")
    n = x.shape[-1]
    out = torch.empty_like(x)
    dt = {torch.float16: 0, torch.float32: 1}.get(x.dtype)
    if dt is None:
        raise PtError("SoftmaxV3: dtype must be fp16 or fp32")
    check(_lib.lib().pt_softmax(_ptr(x), x.numel() // n, n, 1 if stable_mode else 0, dt, _ptr(out), _stream()), "SoftmaxV3")
    return out


# ------------------------------------------------------------------------------------------ KV cache (reference layout)
class KVCacheOp:
    """One `KVCache` call site: owns the persistent cache like the reference op instance
    (custom_ops/kv_cache.cpp:108-116), re-zeroed when step == 0."""

    def __init__(self, max_len, sequence_axis, step_len=1, fp8=False, fp8_scale=1.0):
        """fp8=True is the op's `fp8` attribute (customized.py:32; kv_cache.cpp:100-104, :183-185): the cache is kept as 8-bit floats
        (E4M3 bytes of updater / fp8_scale) and returned cast back to fp16."""
        self.max_len, self.axis, self.step_len = max_len, sequence_axis, step_len
        self.fp8, self.fp8_scale = bool(fp8), float(fp8_scale)
        self.cache = self.scratch = None

    def __call__(self, step, updater):
        shape = list(updater.shape)
        if shape[self.axis] != self.step_len:
            raise PtError(f"KVCache: updater has {shape[self.axis]} positions on axis {self.axis}, step_len is {self.step_len}")
        outer = 1
        for d in shape[: self.axis]:
            outer *= d
        inner = 1
        for d in shape[self.axis + 1:]:
            inner *= d
        shape[self.axis] = self.max_len
        if self.fp8:
            if self.cache is None:
                self.cache = torch.zeros(shape, dtype=torch.uint8, device=updater.device)
            out = torch.empty(shape, dtype=torch.float16, device=updater.device)
            check(_lib.lib().pt_kv_cache_fp8(_ptr(step), _ptr(updater), _ptr(self.cache), _ptr(out), self.fp8_scale, outer, self.max_len,
                                             self.step_len, inner, _stream()), "KVCache")
            return out
        if self.cache is None:
            self.cache = torch.zeros(shape, dtype=updater.dtype, device=updater.device)
            self.scratch = torch.empty_like(self.cache)
        check(_lib.lib().pt_kv_cache(_ptr(step), _ptr(updater), _ptr(self.cache), _ptr(self.scratch), outer, self.max_len,
                                     self.step_len, inner, _stream()), "KVCache")
        return self.cache


def kv_cache(state, step, updater):
    """ops.kv_cache (customized.py:21-35) with the op instance's state made explicit."""
    return state(step, updater)


class KVCachePipelineOp:
    """One `KVCachePipeline` call site (custom_ops/kv_cache_pipeline.cpp:374-451): `max_bps` caches, cache step % max_bps receives the
    shifted insert and is returned.  transpose=1 is the op's second storage layout (kv_cache_pipeline.hpp:107-113, vertex
    GetBpsKvCacheLastDim, kv_cache_codelet.cpp:170-212): the caches are kept as [..., H, max_len] and shifted along their LAST
    dimension; the op returns the tensor transposed back (kv_cache_pipeline.cpp:441-446), so callers see the same values."""

    def __init__(self, max_len, max_bps, sequence_axis, step_len=1, transpose=0, fp8=False, fp8_scale=1.0):
        """fp8=True: the caches hold E4M3 bytes of updater / fp8_scale and the op returns fp16 (kv_cache_pipeline.cpp:386-388, :437-439)."""
        self.max_len, self.max_bps, self.axis, self.step_len, self.transpose = max_len, max_bps, sequence_axis, step_len, int(transpose)
        self.fp8, self.fp8_scale = bool(fp8), float(fp8_scale)
        self.caches = None

    def __call__(self, step, updater):
        shape = list(updater.shape)
        if self.axis != len(shape) - 2:
            raise PtError("KVCachePipeline: sequence_axis must be rank - 2 (kv_cache_pipeline.hpp:83-88)")
        if shape[self.axis] != self.step_len:
            raise PtError(f"KVCachePipeline: updater has {shape[self.axis]} positions on axis {self.axis}, step_len is {self.step_len}")
        if self.transpose:
            upd = updater.transpose(-1, -2).contiguous()           # [..., H, step_len]: the sequence is the last dimension
            outer, inner = upd.numel() // self.step_len, 1
            store = list(upd.shape[:-1]) + [self.max_len]
        else:
            upd = updater
            outer = 1
            for d in shape[: self.axis]:
                outer *= d
            inner = shape[-1]
            store = shape[: self.axis] + [self.max_len, shape[-1]]
        if self.caches is None:
            self.caches = torch.zeros([self.max_bps] + store, dtype=torch.uint8 if self.fp8 else updater.dtype, device=updater.device)
        out = torch.empty(store, dtype=updater.dtype, device=updater.device)
        if self.fp8:
            check(_lib.lib().pt_kv_cache_pipeline_fp8(_ptr(step), _ptr(upd), _ptr(self.caches), _ptr(out), self.fp8_scale, self.max_bps, outer,
                                                      self.max_len, self.step_len, inner, _stream()), "KVCachePipeline")
        else:
            check(_lib.lib().pt_kv_cache_pipeline(_ptr(step), _ptr(upd), _ptr(self.caches), _ptr(out), self.max_bps, outer, self.max_len,
                                                  self.step_len, inner, _stream()), "KVCachePipeline")
        return out.transpose(-1, -2).contiguous() if self.transpose else out


def kv_cache_pipeline(state, step, updater):
    return state(step, updater)


# ------------------------------------------------------------------------------------------ paged cache + attention
class PagedKVCache:
    """Page pool of one layer plus the (shared) page table.  pool[page][2][n_kv][page_size][head_dim]."""

    def __init__(self, rows, n_kv, head_dim, max_len, page_size=64, device="cuda", page_table=None, extra_pages=0):
        self.rows, self.n_kv, self.head_dim, self.page_size = rows, n_kv, head_dim, page_size
        self.max_len = max_len
        self.max_pages = (max_len + page_size - 1) // page_size
        n_pages = rows * self.max_pages + extra_pages
        self.pool = torch.zeros((n_pages, 2, n_kv, page_size, head_dim), dtype=torch.float16, device=device)
        if page_table is None:
            page_table = torch.arange(rows * self.max_pages, dtype=torch.int32, device=device).reshape(rows, self.max_pages)
        self.page_table = page_table

    def export(self, step, max_len):
        """Reference-layout view [2, rows, n_kv, max_len, head_dim], newest first, zeros beyond step."""
        out = torch.empty((2, self.rows, self.n_kv, max_len, self.head_dim), dtype=torch.float16, device=self.pool.device)
        check(_lib.lib().pt_kv_export(_ptr(self.pool), _ptr(self.page_table), _ptr(step), self.rows, self.n_kv, self.head_dim,
                                      self.page_size, self.max_pages, max_len, _ptr(out), _stream()), "pt_kv_export")
        return out


def attn_workspace(batch, n_head, head_dim, max_pages, device="cuda"):
    n = _lib.lib().pt_attn_workspace_bytes(batch, n_head, head_dim, max_pages)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def attn_args(qkv, step, cache, out, n_head, rope_mode, softmax_mode, score_scale, rope_sin, rope_cos, workspace, error_flag, pdl=0,
              out_fp8=None, out_fp8_scale=0.0):
    a = AttnArgs()
    a.batch, a.n_head, a.n_kv, a.head_dim = qkv.shape[0], n_head, cache.n_kv, cache.head_dim
    a.page_size, a.max_pages, a.rope_mode, a.softmax_mode = cache.page_size, cache.max_pages, rope_mode, softmax_mode
    a.score_scale = score_scale
    a.step_dev, a.qkv, a.rope_sin, a.rope_cos = _ptr(step), _ptr(qkv), _ptr(rope_sin), _ptr(rope_cos)
    a.pool, a.page_table, a.out, a.out_ld = _ptr(cache.pool), _ptr(cache.page_table), _ptr(out), 0
    a.workspace, a.workspace_bytes = _ptr(workspace), workspace.numel()
    a.error_flag = _ptr(error_flag)
    a.pdl = pdl
    a.max_len = cache.max_len
    a.out_fp8, a.out_fp8_scale = _ptr(out_fp8), float(out_fp8_scale)
    return a


def kv_append_attn(qkv, step, cache, n_head, rope_mode=ROPE_NONE, softmax_mode=SOFTMAX_F32, score_scale=1.0, rope_sin=None,
                   rope_cos=None, workspace=None, error_flag=None, out=None):
    """RoPE + KV append + decode attention for one new token per row.  qkv fp16 [rows, (n_head + 2 n_kv) * H]."""
    if out is None:
        out = torch.empty((qkv.shape[0], n_head * cache.head_dim), dtype=torch.float16, device=qkv.device)
    if workspace is None:
        workspace = attn_workspace(qkv.shape[0], n_head, cache.head_dim, cache.max_pages, qkv.device)
    a = attn_args(qkv, step, cache, out, n_head, rope_mode, softmax_mode, score_scale, rope_sin, rope_cos, workspace, error_flag)
    check(_lib.lib().pt_kv_append_attn(ctypes.byref(a), _stream()), "pt_kv_append_attn")
    return out


def prefill_attn(qkv, cache, batch, n_tokens, start, n_head, score_scale, rope_sin, rope_cos, out=None):
    """Causal attention over a whole prompt chunk (the reference's sequence_length != 1 attention, llama2/attention.py:64-114):
    qkv fp16 [batch * n_tokens, 3 * n_head * H], row b * n_tokens + t = position start + t of sequence b.  Rotates q in place,
    appends rotated k and v to the paged cache and returns softmax(q K^T * scale + causal mask) V, [batch * n_tokens, n_head * H]."""
    if qkv.shape != (batch * n_tokens, 3 * n_head * cache.head_dim) or cache.n_kv != n_head:
        raise PtError(f"prefill_attn: qkv {tuple(qkv.shape)} does not match batch={batch} n_tokens={n_tokens} n_head={n_head} (no grouped KV heads)")
    if out is None:
        out = torch.empty((batch * n_tokens, n_head * cache.head_dim), dtype=torch.float16, device=qkv.device)
    a = _lib.PrefillAttnArgs()
    a.batch, a.n_tokens, a.start, a.n_head, a.head_dim = batch, n_tokens, start, n_head, cache.head_dim
    a.page_size, a.max_pages, a.max_len, a.score_scale = cache.page_size, cache.max_pages, cache.max_len, score_scale
    a.qkv, a.rope_sin, a.rope_cos, a.pool, a.page_table, a.out = _ptr(qkv), _ptr(rope_sin), _ptr(rope_cos), _ptr(cache.pool), _ptr(cache.page_table), _ptr(out)
    check(_lib.lib().pt_prefill_attn(ctypes.byref(a), _stream()), "pt_prefill_attn")
    return out


# ------------------------------------------------------------------------------------------ top-k / beam search
def topk(x, k, axis=-1):
    """ops.topk (popart.py:135-137) on the last axis: (values, int32 indices), ties -> lowest index."""
    if axis not in (-1, x.dim() - 1):
        raise PtError("topk: only the last axis is supported")
    dim = x.shape[-1]
    rows = x.numel() // dim
    dt = {torch.float16: 0, torch.float32: 1}[x.dtype]
    vals = torch.empty(x.shape[:-1] + (k,), dtype=x.dtype, device=x.device)
    ids = torch.empty(x.shape[:-1] + (k,), dtype=torch.int32, device=x.device)
    check(_lib.lib().pt_topk(_ptr(x), rows, dim, k, dt, _ptr(vals), _ptr(ids), _stream()), "topk")
    return vals, ids


def beam_search(logits, hyp_container, prob_container, step, beam_size, parent=None, workspace=None):
    """`BeamSearch` custom op (beam_search_custom_op.cpp:333-478).  logits [B, beam, V]; hyp int32
    [B, max_len, beam] and prob [B, beam] are updated in place.  Returns (next_id, global_best_id, hyp, prob)."""
    b, beam, vocab = logits.shape
    if beam != beam_size:
        raise PtError("BeamSearch: logits.shape[1] must equal beam_size")
    max_len = hyp_container.shape[1]
    dt = {torch.float16: 0, torch.float32: 1}[logits.dtype]
    L = _lib.lib()
    if workspace is None:
        workspace = torch.empty(L.pt_beam_search_workspace_bytes(b, beam, max_len), dtype=torch.uint8, device=logits.device)
    next_id = torch.empty((b, beam), dtype=torch.int32, device=logits.device)
    gbest = torch.empty((b, beam), dtype=torch.int32, device=logits.device)
    check(L.pt_beam_search(_ptr(logits), _ptr(hyp_container), _ptr(prob_container), _ptr(step), b, beam, vocab, max_len, dt,
                           _ptr(next_id), _ptr(gbest), _ptr(parent), _ptr(workspace), workspace.numel(), _stream()), "BeamSearch")
    return next_id, gbest, hyp_container, prob_container


# ------------------------------------------------------------------------------------------ FP8
def _require_e4m3(op, fp8_format):
    """The reference's formats are Graphcore's F143 / F152 (exponent bias and range differ from OCP E4M3, the arithmetic is
    closed): bytes in those formats would decode to other values here, so they are refused instead of silently misread."""
    if fp8_format in ("F143", "F152"):
        raise PtError(f"{op}: Graphcore {fp8_format} bytes are not OCP E4M3 and are not supported; re-quantise the fp16/fp32 tensor "
                      "with poptransformer_b200.quant.quantize_fp8 (E4M3, per-tensor scale amax/448)")
    if fp8_format != "E4M3":
        raise PtError(f"{op}: unsupported format {fp8_format}")


def half_to_uint8(x, fp8_scale, fp8_format="E4M3"):
    """ops.half_to_uint8 (customized.py:127-135) with OCP E4M3 and a float per-tensor scale."""
    _require_e4m3("CastToUint8", fp8_format)
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    check(_lib.lib().pt_cast_fp8(_ptr(x), float(fp8_scale), x.numel(), _ptr(out), _stream()), "CastToUint8")
    return out


def fp8_matmul(input_l, input_r, fp8_scale_lhs, fp8_scale_rhs, fp8_format_lhs="E4M3", fp8_format_rhs="E4M3"):
    """ops.fp8_matmul (customized.py:137-148): input_l e4m3 [m, k], input_r e4m3 [n, k] (k contiguous) -> fp16 [m, n]."""
    _require_e4m3("FP8MatMul", fp8_format_lhs)
    _require_e4m3("FP8MatMul", fp8_format_rhs)
    m, k = input_l.shape
    n = input_r.shape[0]
    out = torch.empty((m, n), dtype=torch.float16, device=input_l.device)
    check(_lib.lib().pt_fp8_matmul(_ptr(input_l), _ptr(input_r), float(fp8_scale_lhs), float(fp8_scale_rhs), m, n, k, _ptr(out), _stream()),
          "FP8MatMul")
    return out


# ------------------------------------------------------------------------------------------ misc
def wkv(k, v, time_first, time_decay, num, den, max_state):
    out = torch.empty_like(k)
    b, c = k.shape
    check(_lib.lib().pt_wkv(_ptr(k), _ptr(v), _ptr(time_first), _ptr(time_decay), _ptr(num), _ptr(den), _ptr(max_state), b, c, _ptr(out),
                            _stream()), "pt_wkv")
    return out


def embedding(table, ids, step=None, out=None):
    """ids int32 [batch, stride]; gathers table[ids[b, *step]] (step None -> column 0)."""
    batch, stride = ids.shape
    vocab, dim = table.shape
    if out is None:
        out = torch.empty((batch, dim), dtype=table.dtype, device=table.device)
    check(_lib.lib().pt_embedding(_ptr(table), _ptr(ids), stride, _ptr(step), batch, dim, vocab, _ptr(out), _stream()), "pt_embedding")
    return out


def step_containers(ids, step, next_ids, pad_id, eos_id=-1, stop_mask=None, done_flag=None):
    """step_containers + step_loop_cond (models/base_model.py:313-355).  With `done_flag` (device int32, zeroed per generation)
    the reference's early stop applies: the flag is set by the iteration that found every sequence already stopped, and the
    calls after it change nothing."""
    batch, max_len = ids.shape
    if done_flag is None:
        check(_lib.lib().pt_step_containers(_ptr(ids), batch, max_len, _ptr(step), _ptr(next_ids), int(pad_id), int(eos_id), _ptr(stop_mask),
                                            _stream()), "pt_step_containers")
    else:
        check(_lib.lib().pt_step_containers_early_stop(_ptr(ids), batch, max_len, _ptr(step), _ptr(next_ids), int(pad_id), int(eos_id),
                                                       _ptr(stop_mask), _ptr(done_flag), _stream()), "pt_step_containers_early_stop")


def lm_head_tp_merge(dec):
    """TPLMHead.__call__ after the matmul (layers/lm_head.py:86-115) for a decoder holding its vocab shard's logits: exact-zero
    logits -> -10000, local top-1, + rank * vocab_per_rank, all-gather of (value, id) over the TP group, arg-max over ranks.
    Uses the decoder's logits, next_val, next_ids, gather_val, gather_ids, vocab_loc, rank, tp and group."""
    L = _lib.lib()
    check(L.pt_lm_head_local_topk(_ptr(dec.logits), dec.batch, dec.vocab_loc, dec.rank * dec.vocab_loc, _ptr(dec.next_val),
                                  _ptr(dec.next_ids), _stream()), "pt_lm_head_local_topk")
    torch.distributed.all_gather_into_tensor(dec.gather_val, dec.next_val.view(1, -1), group=dec.group)
    torch.distributed.all_gather_into_tensor(dec.gather_ids, dec.next_ids.view(1, -1), group=dec.group)
    check(L.pt_lm_head_tp_pick(_ptr(dec.gather_val), _ptr(dec.gather_ids), dec.tp, dec.batch, _ptr(dec.next_ids), _stream()),
          "pt_lm_head_tp_pick")


def random_sample(logits, k, generator=None):
    """ops.random_sample (popart.py:25-29): top-k of the logits on their last axis, then one of the k candidates picked by the arg-max
    of k standard-normal draws (one draw vector shared by all rows, shape [1, k] as in the reference).  The draws come from torch's
    generator (the reference's come from PopART's RNG: the choice is not reproducible across the two, the candidate set is)."""
    vals, ids = topk(logits, k)
    noise = torch.randn((1, k), generator=generator, device=logits.device, dtype=torch.float32)
    pick = torch.argmax(noise, dim=1)                               # [1]
    return ids[..., pick.item()].unsqueeze(-1).contiguous()


def add(a, b):
    out = torch.empty_like(a)
    check(_lib.lib().pt_add_f16(_ptr(a), _ptr(b), a.numel(), _ptr(out), _stream()), "pt_add_f16")
    return out


def remap_tensor(x, fwd_after_matmul=0, name="remap"):
    """ops.remap_tensor (customized.py:38-54): an IPU tile-layout hint with no numeric effect."""
    return x
