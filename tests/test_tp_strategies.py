"""The host-side tensor-parallel weight slicing against the reference's own load-time functions
(poptransformer/utils/param_handler/tensor_parallel_strategy.py:21-70, models/chatglm2/model.py:29-49), whose outputs on small
seeded arrays are stored in tests/golden/tp_strategies.npz by tests/golden/make_golden.py.  The reference keeps weights as
[in, out] with the replica axis first; this package keeps [out, in] and slices per rank, hence the transposes."""
import os

import numpy as np
import pytest
import torch

from oracle import chatglm2_np
from poptransformer_b200 import tp

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tp_strategies.npz"))
T = lambda a: torch.from_numpy(np.ascontiguousarray(a))


def test_start_splits_output_features_with_zero_padding():
    w, b = G["start_w"], G["start_b"]                  # [in 6, out 10]; 10 outputs over 4 ranks -> padded to 12
    for r in range(4):
        loc, per = tp.vocab_rows(T(w.T), r, 4)
        assert per == 3 and np.array_equal(loc.numpy().T, G["start_w_tp4"][r])
        assert np.array_equal(tp.vocab_rows(T(b), r, 4)[0].numpy(), G["start_b_tp4"][r])
    with pytest.raises(ValueError):
        tp.rows(T(w.T), 0, 4)                          # without padding the split must be even


def test_end_splits_input_features_and_repeats_the_bias():
    w = G["end_w"]                                     # [in 8, out 6]
    for r in range(2):
        assert np.array_equal(tp.cols(T(w.T), r, 2).numpy().T, G["end_w_tp2"][r])
        assert np.array_equal(G["end_b_tp2"][r], G["end_b"])
        ks = tp.KSlice(8, r, 2, 1)
        assert (ks.k0, ks.k1) == (4 * r, 4 * r + 4)


def test_fused_qkv_keeps_whole_thirds_per_rank():
    for r in range(2):
        assert np.array_equal(tp.fused_qkv_rows(T(G["qkv_w"].T), r, 2).numpy().T, G["qkv_w_tp2"][r])
        assert np.array_equal(tp.fused_qkv_rows(T(G["qkv_b"]), r, 2).numpy(), G["qkv_b_tp2"][r])


def test_multi_query_qkv():
    for r in range(2):
        assert np.array_equal(tp.multi_query_qkv_rows(T(G["mq_w"].T), r, 2, 16, 4).numpy().T, G["mq_w_tp2"][r])
        assert np.array_equal(tp.multi_query_qkv_rows(T(G["mq_b"]), r, 2, 16, 4).numpy(), G["mq_b_tp2"][r])
        assert np.array_equal(tp.multi_query_qkv_rows(T(G["mqf_w"].T), r, 2, 16, 4).numpy().T, G["mqf_w_tp2"][r])


@pytest.mark.parametrize("n", [2, 4])
def test_chatglm2_head_rearrangement(n):
    """rearrange_tp_weights followed by the n-way split of the query (and of the dense layer's input features) hands rank r
    the features multi_query_head_index(…, r, n) names; the oracle's restatement of the row order agrees."""
    q, dense = G["rearr_q"], G["rearr_dense"]          # HF orientation: [out = 8 heads x 2, in] and [out, in = 8 heads x 2]
    order = chatglm2_np.rearrange_tp_rows(16, 8, n)
    assert np.array_equal(q[order], G[f"rearr_q_tp{n}"])
    assert np.array_equal(dense[:, order], G[f"rearr_dense_tp{n}"])
    for r in range(n):
        idx = tp.multi_query_head_index(8, 2, 2, r, n).numpy()
        assert np.array_equal(q[idx], tp.rows(T(G[f"rearr_q_tp{n}"]), r, n).numpy())
        assert np.array_equal(dense[:, idx], tp.cols(T(G[f"rearr_dense_tp{n}"]), r, n).numpy())


def test_sharded_embedding_plus_all_reduce_equals_one_gather():
    """TPEmbedding (layers/embedding.py:41-70): every rank gathers from its vocab shard, ids outside the shard read the appended
    zero row, and the all-reduce sums the ranks.  The sum has one non-zero term, so the replicated table this package keeps gives
    the same fp16 values."""
    emb, sharded = G["emb"], G["emb_tp4"]              # [11, 4] -> [4, 3 + 1, 4]
    per = sharded.shape[1] - 1
    for r in range(4):
        assert np.array_equal(sharded[r, :per][: max(0, min(per, 11 - r * per))], emb[r * per:(r + 1) * per])
        assert not sharded[r, per].any()
    for tok in range(11):
        total = np.zeros(4, np.float32)
        for r in range(4):
            idx = tok - r * per
            total += sharded[r, per if (idx < 0 or idx > per) else idx]
        assert np.array_equal(total, emb[tok])


@pytest.mark.parametrize("kind", ["gpt2", "chatglm2", "chatglm2_fp8", "rwkv"])
@pytest.mark.parametrize("world", [2, 4])
def test_oracle_tp_emulation_agrees_with_one_rank(kind, world):
    """The rank-by-rank emulation differs from the unsharded model only by the fp16 rounding of the 'end' layers' partial sums:
    over a few teacher-forced steps the concatenated vocab shards stay within 4e-3 (fp16) / 5e-2 (FP8, where a changed last bit
    can move an activation to the next E4M3 value) of the one-rank logits,
    the padded vocab tail is exactly zero, and the value/id merge picks the arg-max of the concatenation."""
    from oracle import chatglm2_np, gpt2_np, ops_np, rwkv_np
    from poptransformer_b200 import synth
    batch, max_len, vocab = 2, 16, 301
    if kind == "gpt2":
        dims = dict(n_layer=2, d_model=128, n_head=4, vocab=vocab, n_positions=32)
        sd = {k: v.numpy() for k, v in synth.gpt2_state_dict(**dims, seed=3).items()}
        make = lambda n: gpt2_np.GPT2Oracle(gpt2_np.GPT2Config(**dims, max_len=max_len), sd, batch, tp=n)
    elif kind.startswith("chatglm2"):
        prec = "fp8" if kind.endswith("fp8") else "fp16"
        dims = dict(n_layer=2, d_model=256, n_head=8, n_group=2, ffn=384, vocab=vocab)
        sd = {k: (v.numpy() if hasattr(v, "numpy") else v) for k, v in synth.chatglm2_state_dict(**dims, seed=3, precision=prec).items()}
        make = lambda n: chatglm2_np.ChatGLM2Oracle(chatglm2_np.ChatGLM2Config(**dims, max_len=max_len, precision=prec), sd, batch, tp=n)
    else:
        dims = dict(n_layer=2, d_model=128, ffn=512, vocab=vocab)
        sd = {k: v.numpy() for k, v in synth.rwkv_state_dict(**dims, seed=3).items()}
        make = lambda n: rwkv_np.RWKVOracle(rwkv_np.RWKVConfig(**dims, max_len=max_len), sd, batch, tp=n)
    one, many = make(1), make(world)
    ids = synth.prompt_ids(batch, 6, max_len, vocab, vocab - 1, seed=5).numpy()
    per = -(-vocab // world)
    tol = 5e-2 if kind.endswith("fp8") else 4e-3
    for t in range(5):
        args = (ids[:, t],) if kind == "rwkv" else (ids[:, t], t)
        a, shards = one.logits(*args)[0], many.logits(*args)[0]
        assert len(shards) == world and all(s.shape == (batch, per) for s in shards)
        cat = np.concatenate(shards, axis=1)
        assert not cat[:, vocab:].any()
        if kind.endswith("fp8"):   # E4M3 casts amplify a changed last bit to a few per cent: the band holds for all but a few logits
            err = np.abs(cat[:, :vocab].astype(np.float32) - a.astype(np.float32))
            assert np.mean(err <= tol + tol * np.abs(a.astype(np.float32))) >= 0.98 and err.max() <= 4 * tol
        else:
            np.testing.assert_allclose(cat[:, :vocab].astype(np.float32), a.astype(np.float32), atol=tol, rtol=tol)
        masked = np.where(cat == 0, np.float16(-10000), cat)
        assert np.array_equal(many.next_ids(shards), np.argmax(masked.astype(np.float32), axis=1))
