"""Tensor-parallel host logic on CPU ranks (gloo, world_size 2 and 4): slicing with the reference's 'start' / 'end'
strategies, all-reduce of row-parallel partial sums, and the vocabulary-parallel LM-head merge, against the single-rank oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ops_np as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from poptransformer_b200 import quant, tp
    g = torch.Generator().manual_seed(0)
    d, f, vocab, group = 256, 2816, 1000, 128          # f / 4 = 704 = 5.5 scale groups, like 11008 / 8 = 10.75
    x = torch.randn((2, d), generator=g).half()
    w_up = torch.randn((f, d), generator=g) * 0.05
    w_down = torch.randn((d, f), generator=g) * 0.05
    head = (torch.randn((vocab, d), generator=g) * 0.05).half()
    up_q, up_s = quant.quantize_int4(w_up, group)
    down_q, down_s = quant.quantize_int4(w_down, group)

    # single-rank oracle
    up_full = O.int4_to_half(up_q.numpy(), up_s.numpy(), axis=1, group=group)          # [d, f]
    act_full = O.matmul_f16(x.numpy(), up_full)                                          # [2, f]
    down_full = O.int4_to_half(down_q.numpy(), down_s.numpy(), axis=1, group=group)     # [f, d]
    y_full = np.matmul(act_full.astype(np.float32), down_full.astype(np.float32))

    # this rank: column-parallel up projection, row-parallel down projection over a group-aligned window
    up_loc, ups_loc = tp.rows(up_q, rank, world), tp.rows(up_s, rank, world)
    act_loc = O.matmul_f16(x.numpy(), O.int4_to_half(up_loc.numpy(), ups_loc.numpy(), axis=1, group=group))    # [2, f/world]
    assert np.array_equal(act_loc, act_full[:, rank * (f // world):(rank + 1) * (f // world)])
    dq, ds, grp_loc, ks = tp.row_parallel_int4(down_q, down_s, f, rank, world)
    assert ks.width % 128 == 0 and 0 <= ks.offset < 128 and grp_loc == group
    window = np.zeros((2, ks.width), np.float16)
    window[:, ks.offset: ks.offset + act_loc.shape[1]] = act_loc
    part = np.matmul(window.astype(np.float32), O.int4_to_half(dq.numpy(), ds.numpy(), axis=1, group=grp_loc).astype(np.float32))
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    np.testing.assert_allclose(t.numpy(), y_full, rtol=1e-4, atol=1e-4 * np.abs(y_full).max())

    # vocabulary-parallel LM head: local top-1 (+ offset), all-gather, first maximum wins
    per = -(-vocab // world)
    head_pad = torch.cat([head, torch.zeros((per * world - vocab, d), dtype=torch.float16)], 0)
    logits_loc = O.matmul_f16(x.numpy(), head_pad[rank * per:(rank + 1) * per].numpy().T)
    lg = np.where(logits_loc == 0, np.float16(-10000.0), logits_loc)
    v, i = O.topk(lg, 1)
    pair = torch.tensor(np.stack([v[:, 0].astype(np.float32), (i[:, 0] + rank * per).astype(np.float32)], 1))
    gathered = [torch.zeros_like(pair) for _ in range(world)]
    dist.all_gather(gathered, pair)
    vals = np.stack([gt[:, 0].numpy() for gt in gathered], 1)
    ids = np.stack([gt[:, 1].numpy() for gt in gathered], 1).astype(np.int32)
    merged = ids[np.arange(2), np.argmax(vals, axis=1)]
    full_logits = [O.matmul_f16(x.numpy(), head_pad[r * per:(r + 1) * per].numpy().T) for r in range(world)]
    assert np.array_equal(merged, O.lm_head_tp_merge(full_logits, vocab))
    assert np.array_equal(merged, O.topk(O.matmul_f16(x.numpy(), head.numpy().T), 1)[1][:, 0])
    open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tp_slicing_allreduce_and_head_merge(world, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_kslice_windows_cover_llama_7b_shards():
    from poptransformer_b200 import tp
    for world in (1, 2, 4, 8):
        covered = np.zeros(11008, int)
        for r in range(world):
            ks = tp.KSlice(11008, r, world, 128)
            assert ks.a0 % 128 == 0 and ks.a1 % 128 == 0 and ks.a0 <= ks.k0 < ks.k1 <= ks.a1 <= 11008 + 127
            covered[ks.k0:ks.k1] += 1
        assert (covered == 1).all()
