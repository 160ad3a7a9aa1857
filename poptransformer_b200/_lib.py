"""ctypes binding of libpt_b200.so (the C-ABI declared in include/pt_b200.h).

There is no CPU fallback: if the library cannot be loaded every op raises.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("PT_B200_LIB", os.path.join(HERE, "libpt_b200.so"))

c_void_p, c_int, c_float, c_size_t, c_int64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_int64


class PtError(RuntimeError):
    """Raised when a libpt_b200 entry point reports an error (the reference raises
    popart::error / poplar_error at graph-build time for the same violations)."""


class LinearArgs(ctypes.Structure):
    _fields_ = [
        ("wfmt", c_int), ("batch", c_int), ("n_out", c_int), ("k_in", c_int), ("group", c_int),
        ("prologue", c_int), ("epilogue", c_int), ("ksplit", c_int),
        ("x", c_void_p), ("packed_w", c_void_p), ("norm_gamma", c_void_p),
        ("norm_eps", c_float), ("act_scale", c_float), ("w_scale", c_float),
        ("bias", c_void_p), ("residual", c_void_p), ("out", c_void_p), ("out_ld", c_int), ("pdl", c_int),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("error_flag", c_void_p), ("norm_beta", c_void_p),
    ]


class AttnArgs(ctypes.Structure):
    _fields_ = [
        ("batch", c_int), ("n_head", c_int), ("n_kv", c_int), ("head_dim", c_int),
        ("page_size", c_int), ("max_pages", c_int), ("rope_mode", c_int), ("softmax_mode", c_int),
        ("score_scale", c_float),
        ("step_dev", c_void_p), ("qkv", c_void_p), ("rope_sin", c_void_p), ("rope_cos", c_void_p),
        ("pool", c_void_p), ("page_table", c_void_p), ("out", c_void_p), ("out_ld", c_int),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("error_flag", c_void_p), ("pdl", c_int), ("max_len", c_int),
        ("out_fp8", c_void_p), ("out_fp8_scale", c_float),
    ]


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("wfmt", c_int), ("m", c_int), ("n_out", c_int), ("k_in", c_int), ("group", c_int), ("epilogue", c_int), ("ksplit", c_int),
        ("w_tiled", c_int), ("x", c_void_p), ("w", c_void_p), ("scales", c_void_p), ("x_scale", c_float), ("w_scale", c_float),
        ("residual", c_void_p), ("out", c_void_p), ("out_ld", c_int), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("error_flag", c_void_p), ("bias", c_void_p),
    ]


class PrefillAttnArgs(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("batch", "n_tokens", "start", "n_head", "head_dim", "page_size", "max_pages", "max_len")] + \
               [("score_scale", c_float), ("qkv", c_void_p), ("rope_sin", c_void_p), ("rope_cos", c_void_p), ("pool", c_void_p),
                ("page_table", c_void_p), ("out", c_void_p)]


class LlamaLayer(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("qkv", "o", "gu", "down", "ln1", "ln2", "pool")]


class LlamaStepArgs(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("batch", "d_model", "n_head", "head_dim", "ffn", "vocab", "n_layer", "max_len", "page_size",
                                     "max_pages", "pad_id", "eos_id")] + [("norm_eps", c_float), ("score_scale", c_float)] + \
               [(n, c_void_p) for n in ("layers", "norm", "head", "emb", "rope_sin", "rope_cos", "ids", "step_dev", "stop_mask", "next_ids",
                                        "page_table", "x", "qkv", "attn", "act", "logits", "workspace")] + \
               [("workspace_bytes", c_size_t), ("error_flag", c_void_p), ("trace", c_void_p), ("debug", c_int)] + \
               [(n, c_int) for n in ("tp_size", "tp_rank", "ffn_offset", "ffn_valid", "vocab_offset", "emb_rows")] + [("tp_buffers", c_void_p * 8)] + \
               [("done_flag", c_void_p), ("wait_limit", c_int)]


# name -> (restype, argtypes); mirrors include/pt_b200.h one to one
SIGNATURES = {
    "pt_last_error": (ctypes.c_char_p, []),
    "pt_version": (c_int, []),
    "pt_launch_count": (ctypes.c_uint64, []),
    "pt_int4_to_half": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "pt_linear_packed_bytes": (c_size_t, [c_int, c_int, c_int]),
    "pt_linear_repack": (c_int, [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "pt_linear_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "pt_linear": (c_int, [ctypes.POINTER(LinearArgs), c_void_p]),
    "pt_linear_static_scratch": (c_int, [ctypes.POINTER(LinearArgs), c_void_p]),
    "pt_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "pt_gemm": (c_int, [ctypes.POINTER(GemmArgs), c_void_p]),
    "pt_gemm_packed_bytes": (c_size_t, [c_int, c_int, c_int]),
    "pt_gemm_repack": (c_int, [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "pt_norm_ce": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p]),
    "pt_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "pt_softmax": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "pt_kv_cache": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_void_p]),
    "pt_kv_cache_pipeline": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_void_p]),
    "pt_kv_cache_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int, c_int, c_int64, c_void_p]),
    "pt_kv_cache_pipeline_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int64, c_int, c_int, c_int64, c_void_p]),
    "pt_attn_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "pt_kv_append_attn": (c_int, [ctypes.POINTER(AttnArgs), c_void_p]),
    "pt_prefill_attn": (c_int, [ctypes.POINTER(PrefillAttnArgs), c_void_p]),
    "pt_prefill_embed": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "pt_kv_export": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "pt_kv_reorder_pages": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "pt_kv_reorder_table": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "pt_llama_stream_permute": (c_int, [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "pt_llama_step_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "pt_llama_tp_buffer_bytes": (c_size_t, [c_int, c_int, c_int]),
    "pt_llama_decode_step": (c_int, [ctypes.POINTER(LlamaStepArgs), c_void_p]),
    "pt_topk": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "pt_lm_head_local_topk": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "pt_lm_head_tp_pick": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "pt_beam_search_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "pt_beam_search": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_size_t, c_void_p]),
    "pt_cast_fp8": (c_int, [c_void_p, c_float, c_int64, c_void_p, c_void_p]),
    "pt_fp8_matmul": (c_int, [c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int, c_void_p, c_void_p]),
    "pt_rwkv_mix": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "pt_rwkv_act": (c_int, [c_int, c_void_p, c_void_p, c_void_p, ctypes.c_int64, c_void_p]),
    "pt_wkv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "pt_embedding": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "pt_step_containers": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "pt_step_containers_early_stop": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "pt_swiglu": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p]),
    "pt_rms_norm_fp8": (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p, c_void_p]),
    "pt_swiglu_fp8": (c_int, [c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p]),
    "pt_add_f16": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
}

_lib = None


def lib():
    """Loads libpt_b200.so (building it with nvcc if it is missing and nvcc is present)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build as _build
        _build.build()
    try:
        handle = ctypes.CDLL(LIB_PATH)
    except OSError as e:  # no fallback on purpose
        raise PtError(f"libpt_b200.so could not be loaded from {LIB_PATH}: {e}") from e
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype, fn.argtypes = res, args
    _lib = handle
    return _lib


def check(code, what=""):
    if code != 0:
        msg = lib().pt_last_error().decode(errors="replace")
        raise PtError(f"{what or 'libpt_b200'} failed ({code}): {msg}")
