"""Checkpoint ingestion: HF `state_dict`s -> the key naming and pre-processing the reference applies before its layers look
weights up, plus the offline quantisers.  Everything here is load-time host work (torch tensors on the CPU); the decoders pack
the result for the kernels.

  GPT-2     models/gpt2/model.py:154-166: HF GPT-2 stores Conv1D weights [in, out]; the query third of c_attn (weight and bias)
            is multiplied by 1 / sqrt(head_size) so that attention needs no score scale, and c_attn / c_proj / c_fc / mlp.c_proj
            are transposed to [out, in].
  ChatGLM2  models/chatglm2/model.py:256-276: query_key_value is split into `query` (hidden_size rows) and `key_value`,
            dense_h_to_4h into dense_h_to_4h_1 / _2 (the two halves).
  RWKV-4    models/rwkv/model.py:150-155: attention.output.weight and feed_forward.value.weight of block b are divided by
            2 ** (b // rescale_every).
  Llama-2   keys are used as HF stores them (llama2/model.py:114-132 via layers/linear.py:28-40).
  INT4      a checkpoint tensor that is already int8 takes the int4 path, its scale under `<key>_scale`
            (utils/param_handler/precision_strategy.py:24-42); `quantize_linears_int4` produces that format (or the group-128
            extension) from fp16 weights.
"""
import re

import torch

from .quant import quantize_fp8, quantize_int4


def load_state_dict(path):
    """A checkpoint file as a flat {key: CPU tensor} dict: .safetensors (if the safetensors package is present), torch .bin / .pt / .pth."""
    if path.endswith(".safetensors"):
        try:
            from safetensors.torch import load_file
        except ImportError as e:
            raise RuntimeError("reading .safetensors needs the safetensors package") from e
        return load_file(path)
    sd = torch.load(path, map_location="cpu", weights_only=True)
    return sd.get("state_dict", sd) if isinstance(sd, dict) else sd


def gpt2_from_hf(sd, n_embd, n_head):
    """GPT2LMHeadModel state_dict -> the reference's pre-processed one (gpt2/model.py:154-166).  Returns a new dict."""
    scale = float(1 / (n_embd // n_head) ** 0.5)
    out = {}
    for k, v in sd.items():
        v = v.clone()
        if re.search(r"\.attn\.c_attn\.weight$", k):
            v[:, :n_embd] = v[:, :n_embd] * scale
            v = v.transpose(0, 1).contiguous()
        elif re.search(r"\.attn\.c_attn\.bias$", k):
            v[:n_embd] = v[:n_embd] * scale
        elif re.search(r"\.(attn\.c_proj|mlp\.c_fc|mlp\.c_proj)\.weight$", k):
            v = v.transpose(0, 1).contiguous()
        out[k] = v
    return out


def chatglm2_from_hf(sd, hidden_size):
    """ChatGLM2 state_dict -> the reference's (chatglm2/model.py:256-276): fused tensors split, other keys unchanged."""
    out = {}
    for k, v in sd.items():
        if "query_key_value" in k:
            out[k.replace("query_key_value", "query")] = v[:hidden_size].clone()
            out[k.replace("query_key_value", "key_value")] = v[hidden_size:].clone()
        elif "dense_h_to_4h" in k:
            a, b = v.chunk(2, dim=0)
            out[k.replace("dense_h_to_4h", "dense_h_to_4h_1")] = a.clone()
            out[k.replace("dense_h_to_4h", "dense_h_to_4h_2")] = b.clone()
        else:
            out[k] = v
    return out


def rwkv_from_hf(sd, rescale_every):
    """RwkvForCausalLM state_dict -> the reference's (rwkv/model.py:150-155)."""
    out = {}
    for k, v in sd.items():
        m = re.match(r"rwkv\.blocks\.(\d+)\.(attention\.output|feed_forward\.value)\.weight$", k)
        if m and rescale_every > 0:
            v = v / (2 ** (int(m.group(1)) // rescale_every))
        out[k] = v
    return out


def llama_from_hf(sd):
    return dict(sd)


_LINEAR = re.compile(r"(_proj|query|key_value|dense|dense_h_to_4h_[12]|dense_4h_to_h|c_attn|c_proj|c_fc|key|value|receptance|output)\.weight$")


def quantize_linears_int4(sd, group=128, match=_LINEAR, skip=("embed", "lm_head", "wte", "wpe", "word_embeddings", "output_layer", "head.")):
    """fp16 / fp32 linear weights [out, in] -> int8 packed nibbles under the same key + fp16 `<key>_scale` ([out] when group is -1:
    one scale per output channel, the reference's format; [out, in / group] otherwise).  Embeddings and LM heads stay as they are
    (precision_strategy.py:25: only int8 tensors take the int4 path)."""
    out = {}
    for k, v in sd.items():
        if v.ndim == 2 and match.search(k) and not any(s in k for s in skip) and v.dtype in (torch.float16, torch.float32, torch.bfloat16):
            g = v.shape[1] if group < 0 else group
            q, s = quantize_int4(v, g)
            out[k], out[k + "_scale"] = q, (s.reshape(-1) if group < 0 else s)
        else:
            out[k] = v
    return out


def quantize_linears_fp8(sd, match=_LINEAR, skip=("embed", "wte", "wpe", "word_embeddings"), act_amax=None):
    """Linear weights -> E4M3 bytes + a float32 per-tensor scale amax / 448 under `<key>_scale`.  act_amax: optional
    {weight key: largest input magnitude seen in calibration}; stored as the tensor's activation scale `<key>_act_scale`
    = amax / 448 (linears that share their input must be given the same value)."""
    out = {}
    for k, v in sd.items():
        if v.ndim == 2 and match.search(k) and not any(s in k for s in skip) and v.dtype in (torch.float16, torch.float32, torch.bfloat16):
            q, s = quantize_fp8(v)
            out[k], out[k + "_scale"] = q, torch.tensor(s, dtype=torch.float32)
            if act_amax and k in act_amax:
                out[k + "_act_scale"] = torch.tensor(float(act_amax[k]) / 448.0, dtype=torch.float32)
        else:
            out[k] = v
    return out
