"""Weight-only quantisers for the synthetic benchmark weights (torch, CPU or CUDA tensors).

INT4: symmetric signed nibbles, two per byte with the EVEN k index in the high nibble (the
layout the reference's Int4ToHalf expects, custom_ops/int4_to_half_custom_op.cpp:139-147),
one fp16 scale per output row and per group of `group` inputs; group == in_features is the
reference's one-scale-per-output-channel checkpoint format
(poptransformer/utils/param_handler/precision_strategy.py:24-42).
FP8: OCP E4M3 with one float32 scale per tensor, scale = amax / 448.
"""
import torch


def quantize_int4(w, group):
    """w [out, in] float -> (int8 [out, in/2], fp16 scale [out, in/group])."""
    w = w.float()
    n, k = w.shape
    if k % group or k % 2:
        raise ValueError(f"in_features={k} must be even and a multiple of group={group}")
    wg = w.reshape(n, k // group, group)
    s = (wg.abs().amax(dim=2) / 7.0).to(torch.float16)
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = torch.clamp(torch.round(wg / s.float().unsqueeze(-1)), -8, 7).to(torch.int32).reshape(n, k)
    packed = (((q[:, 0::2] & 0xF) << 4) | (q[:, 1::2] & 0xF)).to(torch.uint8).view(torch.int8)
    return packed.contiguous(), s.contiguous()


def quantize_fp8(w):
    """w float -> (uint8 E4M3 bits, float scale); saturating round-to-nearest-even."""
    amax = float(w.float().abs().max())
    scale = amax / 448.0 if amax > 0 else 1.0
    q = torch.clamp(w.float() / scale, -448.0, 448.0).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).contiguous(), scale
