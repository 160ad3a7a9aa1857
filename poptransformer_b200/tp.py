"""Tensor-parallel weight slicing (host side, works on CPU or CUDA tensors).

Mirrors the reference's TP strategies (poptransformer/utils/param_handler/tensor_parallel_strategy.py:21-109 and the int4
scale handling of precision_strategy.py:34-40) for weights kept in the HF [out, in] orientation:
  'start' (column parallel: q/k/v/gate/up, LM head) -> split the OUTPUT features: rows().
  'end'   (row parallel: o_proj/down_proj)          -> split the INPUT features: row_parallel_*(), followed by an all-reduce.
"""
import torch


def rows(t, r, n):
    """'start' strategy: rank r's block of output features (rows of the [out, in] matrix)."""
    per = t.shape[0] // n
    if per * n != t.shape[0]:
        raise ValueError(f"out_features={t.shape[0]} not divisible by tp={n}")
    return t[r * per:(r + 1) * per]


class KSlice:
    """'end' strategy: rank r's range [k0, k1) of input features, widened to [a0, a1) on multiples of `align`.
    Weights outside [k0, k1) are zero and the producer of the activations writes at column `offset` of a zero-initialised
    buffer of `width` columns, so group scales that are defined on global k positions stay valid for every rank."""

    def __init__(self, k_total, r, n, align):
        per = k_total // n
        if per * n != k_total:
            raise ValueError(f"in_features={k_total} not divisible by tp={n}")
        self.k0, self.k1 = r * per, (r + 1) * per
        self.a0 = (self.k0 // align) * align
        self.a1 = -(-self.k1 // align) * align
        self.offset, self.width = self.k0 - self.a0, self.a1 - self.a0


def row_parallel_int4(w, scale, k_total, r, n):
    """w int8 [out, k_total/2] (two nibbles per byte), scale fp16 [out, k_total/group] -> (local w, local scale, local group, KSlice)."""
    grp = k_total // scale.shape[1]
    ks = KSlice(k_total, r, n, max(grp, 128) if grp < k_total else 128)
    if grp == k_total:                      # one scale per output row: any 128-aligned window works
        loc_s, grp_loc = scale, ks.width
    else:
        loc_s, grp_loc = scale[:, ks.a0 // grp: ks.a1 // grp], grp
    loc = w[:, ks.a0 // 2: ks.a1 // 2].clone()
    loc[:, : ks.offset // 2] = 0            # nibble pairs outside the rank's range contribute exactly 0
    loc[:, (ks.k1 - ks.a0) // 2:] = 0
    return loc.contiguous(), loc_s.contiguous(), grp_loc, ks


def row_parallel_fp16(w, k_total, r, n):
    ks = KSlice(k_total, r, n, 32)
    loc = torch.zeros((w.shape[0], ks.width), dtype=torch.float16, device=w.device)
    loc[:, ks.offset: ks.offset + (ks.k1 - ks.k0)] = w[:, ks.k0: ks.k1]
    return loc, ks
