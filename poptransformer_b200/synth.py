"""Seeded synthetic checkpoints with the benchmark configurations' shapes and value distributions
(no tokenizer or pretrained weights are available offline).  Keys follow the HF / reference naming
that the reference layers look up (e.g. llama2/model.py:114-132 via layers/linear.py:28-40);
INT4 linears are stored as int8 `<key>` + fp16 `<key>_scale` like the reference's int4 checkpoints."""
import torch

from .quant import quantize_fp8, quantize_int4


def _normal(shape, gen, device, std=0.02):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(torch.float16)


def llama_state_dict(n_layer, d_model, n_head, ffn, vocab, seed=0, device="cpu", int4_group=0):
    """Llama-2 architecture, weights ~ N(0, 0.02) fp16, RMSNorm weights 1 + N(0, 0.02).
    int4_group > 0 quantises every transformer linear (not the embedding / LM head) with that scale group along the input
    features; int4_group = -1 uses one scale per output channel (group = in_features), the reference's checkpoint format."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    sd = {}

    def lin(key, out_f, in_f):
        w = _normal((out_f, in_f), gen, device)
        if int4_group:
            sd[key], sd[key + "_scale"] = quantize_int4(w, in_f if int4_group < 0 else int4_group)
        else:
            sd[key] = w

    sd["model.embed_tokens.weight"] = _normal((vocab, d_model), gen, device)
    for i in range(n_layer):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = (1.0 + _normal((d_model,), gen, device).float()).to(torch.float16)
        sd[p + "post_attention_layernorm.weight"] = (1.0 + _normal((d_model,), gen, device).float()).to(torch.float16)
        for nm in ("q_proj", "k_proj", "v_proj", "o_proj"):
            lin(p + f"self_attn.{nm}.weight", d_model, d_model)
        lin(p + "mlp.gate_proj.weight", ffn, d_model)
        lin(p + "mlp.up_proj.weight", ffn, d_model)
        lin(p + "mlp.down_proj.weight", d_model, ffn)
    sd["model.norm.weight"] = (1.0 + _normal((d_model,), gen, device).float()).to(torch.float16)
    sd["lm_head.weight"] = _normal((vocab, d_model), gen, device)
    return sd


def gpt2_state_dict(n_layer, d_model, n_head, vocab, n_positions, seed=0, device="cpu"):
    """GPT-2 architecture with the reference's key names after its checkpoint pre-processing (gpt2/model.py:154-166): linear
    weights [out, in], the query third of c_attn (weight and bias) multiplied by 1/sqrt(head_size).  fp16, N(0, 0.02);
    LayerNorm weights 1 + N(0, 0.02), biases N(0, 0.02)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    sd = {"transformer.wte.weight": _normal((vocab, d_model), gen, device), "transformer.wpe.weight": _normal((n_positions, d_model), gen, device)}
    scale = float(1.0 / (d_model // n_head) ** 0.5)

    def ln(key):
        sd[key + ".weight"] = (1.0 + _normal((d_model,), gen, device).float()).to(torch.float16)
        sd[key + ".bias"] = _normal((d_model,), gen, device)

    for i in range(n_layer):
        p = f"transformer.h.{i}."
        ln(p + "ln_1")
        w, b = _normal((3 * d_model, d_model), gen, device).float(), _normal((3 * d_model,), gen, device).float()
        w[:d_model] *= scale
        b[:d_model] *= scale
        sd[p + "attn.c_attn.weight"], sd[p + "attn.c_attn.bias"] = w.to(torch.float16), b.to(torch.float16)
        sd[p + "attn.c_proj.weight"], sd[p + "attn.c_proj.bias"] = _normal((d_model, d_model), gen, device), _normal((d_model,), gen, device)
        ln(p + "ln_2")
        sd[p + "mlp.c_fc.weight"], sd[p + "mlp.c_fc.bias"] = _normal((4 * d_model, d_model), gen, device), _normal((4 * d_model,), gen, device)
        sd[p + "mlp.c_proj.weight"], sd[p + "mlp.c_proj.bias"] = _normal((d_model, 4 * d_model), gen, device), _normal((d_model,), gen, device)
    ln("transformer.ln_f")
    return sd


def chatglm2_state_dict(n_layer, d_model, n_head, n_group, ffn, vocab, seed=0, device="cpu", precision="fp16"):
    """ChatGLM2 architecture with the reference's key names after its checkpoint pre-processing (chatglm2/model.py:256-289:
    query / key_value and the two halves of dense_h_to_4h split).  precision "fp8" stores every transformer linear and the output
    layer as E4M3 bytes plus a float `<key>_scale` and a per-tensor activation scale `<key>_act_scale`; linears that the decoder fuses (query | key_value, the two MLP halves) are
    quantised with one common scale."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    hs = d_model // n_head
    sd = {"transformer.embedding.word_embeddings.weight": _normal((vocab, d_model), gen, device)}

    n_lin = [0]

    def lin(group, act_range):
        ws = {k: _normal(shape, gen, device) for k, shape in group}
        if precision == "fp8":
            amax = max(float(w.float().abs().max()) for w in ws.values())
            scale = amax / 448.0
            # per-tensor activation scale `<key>_act_scale`: the largest input magnitude the linear is calibrated for / 448, a
            # different value for every tensor (the same for linears that share their input)
            act = act_range * (1.0, 1.25, 0.8)[n_lin[0] % 3] / 448.0
            n_lin[0] += 1
            for k, w in ws.items():
                sd[k] = torch.clamp(w.float() / scale, -448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
                sd[k + "_scale"] = scale
                sd[k + "_act_scale"] = act
        else:
            sd.update(ws)

    for i in range(n_layer):
        p = f"transformer.encoder.layers.{i}."
        sd[p + "input_layernorm.weight"] = (1.0 + _normal((d_model,), gen, device).float()).to(torch.float16)
        sd[p + "post_attention_layernorm.weight"] = (1.0 + _normal((d_model,), gen, device).float()).to(torch.float16)
        lin([(p + "self_attention.query.weight", (d_model, d_model)), (p + "self_attention.key_value.weight", (2 * n_group * hs, d_model))], 8.0)
        sd[p + "self_attention.query.bias"] = _normal((d_model,), gen, device)
        sd[p + "self_attention.key_value.bias"] = _normal((2 * n_group * hs,), gen, device)
        lin([(p + "self_attention.dense.weight", (d_model, d_model))], 2.0)
        lin([(p + "mlp.dense_h_to_4h_1.weight", (ffn, d_model)), (p + "mlp.dense_h_to_4h_2.weight", (ffn, d_model))], 8.0)
        lin([(p + "mlp.dense_4h_to_h.weight", (d_model, ffn))], 1.0)
    sd["transformer.encoder.final_layernorm.weight"] = (1.0 + _normal((d_model,), gen, device).float()).to(torch.float16)
    lin([("transformer.output_layer.weight", (vocab, d_model))], 8.0)
    return sd


def rwkv_state_dict(n_layer, d_model, ffn, vocab, rescale_every=6, seed=0, device="cpu"):
    """RWKV-4 architecture with the reference's key names after its checkpoint pre-processing (rwkv/model.py:150-155: attention.output
    and feed_forward.value weights divided by 2^(block // rescale_every)).  fp16 weights N(0, 0.02) (key / receptance / value of
    the mixers N(0, 0.05) so that the WKV states move), time_decay ~ U(-5, -1), time_first ~ U(-1, 1), time_mix_* ~ U(0, 1)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    uni = lambda lo, hi: (torch.rand((d_model,), generator=gen, device=device) * (hi - lo) + lo)
    sd = {"rwkv.embeddings.weight": _normal((vocab, d_model), gen, device, std=1.0)}

    def ln(key):
        sd[key + ".weight"] = (1.0 + _normal((d_model,), gen, device).float()).to(torch.float16)
        sd[key + ".bias"] = _normal((d_model,), gen, device)

    for i in range(n_layer):
        p = f"rwkv.blocks.{i}."
        if i == 0:
            ln(p + "pre_ln")
        ln(p + "ln1")
        ln(p + "ln2")
        div = float(2 ** (i // rescale_every)) if rescale_every > 0 else 1.0
        a, m = p + "attention.", p + "feed_forward."
        sd[a + "time_decay"], sd[a + "time_first"] = uni(-5.0, -1.0).float(), uni(-1.0, 1.0).float()
        for nm in ("time_mix_key", "time_mix_value", "time_mix_receptance"):
            sd[a + nm] = uni(0.0, 1.0).to(torch.float16).reshape(1, 1, d_model)
        for nm in ("key", "value", "receptance"):
            sd[a + nm + ".weight"] = _normal((d_model, d_model), gen, device, std=0.05)
        sd[a + "output.weight"] = (_normal((d_model, d_model), gen, device, std=0.05).float() / div).to(torch.float16)
        for nm in ("time_mix_key", "time_mix_receptance"):
            sd[m + nm] = uni(0.0, 1.0).to(torch.float16).reshape(1, 1, d_model)
        sd[m + "key.weight"] = _normal((ffn, d_model), gen, device, std=0.05)
        sd[m + "receptance.weight"] = _normal((d_model, d_model), gen, device, std=0.05)
        sd[m + "value.weight"] = (_normal((d_model, ffn), gen, device, std=0.05).float() / div).to(torch.float16)
    ln("rwkv.ln_out")
    sd["head.weight"] = _normal((vocab, d_model), gen, device)
    return sd


def prompt_ids(batch, prompt_len, max_len, vocab, pad_id, seed=0):
    """Uniform-random prompt ids excluding pad_id, right-padded to max_len with pad_id (int32, CPU)."""
    gen = torch.Generator().manual_seed(seed)
    ids = torch.full((batch, max_len), pad_id, dtype=torch.int32)
    p = torch.randint(0, vocab - 1, (batch, prompt_len), generator=gen, dtype=torch.int32)
    p = torch.where(p >= pad_id, p + 1, p)
    ids[:, :prompt_len] = p
    return ids
