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


def fused_qkv_rows(t, r, n, parts=3):
    """'fused_qkv' strategy (tensor_parallel_strategy.py:47-57): the q, k and v thirds of the output features are split
    separately and rank r's pieces are concatenated, so every rank keeps whole heads of all three."""
    return torch.cat([rows(p, r, n) for p in torch.chunk(t, parts, dim=0)], 0)


def multi_query_head_index(n_head, n_group, head_dim, r, n):
    """Feature indices of rank r's query heads for multi-query attention with replicated KV groups: the heads of every KV
    group are split n ways and rank r takes its share of EACH group, group by group, so that local head j still belongs to
    local group j // (n_head / n / n_group).  This is the order the reference produces with `rearrange_tp_weights` (two
    groups, chatglm2/model.py:29-49) followed by the 'multi_query_qkv' split of the query (tensor_parallel_strategy.py:59-70)."""
    per_group = n_head // n_group
    if per_group % n:
        raise ValueError(f"{per_group} query heads per KV group not divisible by tp={n}")
    share = per_group // n
    heads = torch.cat([torch.arange(g * per_group + r * share, g * per_group + (r + 1) * share) for g in range(n_group)])
    return (heads[:, None] * head_dim + torch.arange(head_dim)[None, :]).reshape(-1)


def vocab_rows(w, r, n):
    """Vocab-parallel head ('start' on the vocab axis with shard()'s zero padding, tensor_parallel_strategy.py:21-30):
    returns rank r's rows and the number of rows per rank."""
    per = -(-w.shape[0] // n)
    pad = per * n - w.shape[0]
    if pad:
        w = torch.cat([w, torch.zeros((pad,) + tuple(w.shape[1:]), dtype=w.dtype, device=w.device)], 0)
    return w[r * per:(r + 1) * per].contiguous(), per


def cols(t, r, n):
    """'end' strategy for a weight in [out, in] orientation: rank r's block of input features.  The bias of an 'end' layer is
    kept whole on every rank and added once, after the all-reduce (tensor_parallel_strategy.py:85-90, layers/linear.py:42-46)."""
    per = t.shape[1] // n
    if per * n != t.shape[1]:
        raise ValueError(f"in_features={t.shape[1]} not divisible by tp={n}")
    return t[:, r * per:(r + 1) * per]


def multi_query_qkv_rows(t, r, n, q_size, kv_size):
    """'multi_query_qkv' strategy (tensor_parallel_strategy.py:59-70) on a fused q | k | v weight: the query, key and value
    feature ranges are each split n ways and rank r's pieces concatenated.  (ChatGLM2 applies it to a weight that holds only the
    query, chatglm2/attention.py:318-329, where it is a plain n-way split of the rearranged heads.)"""
    q, k, v = t[:q_size], t[q_size:q_size + kv_size], t[q_size + kv_size:]
    return torch.cat([rows(p, r, n) for p in (q, k, v) if p.shape[0]], 0)
