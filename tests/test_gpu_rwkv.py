"""GPU parity of the RWKV-4 decode loop (NormCE, token-shift gates, WKV states, receptance gates, relu^2 channel mixing, rescale)
against the numpy restatement of the reference model (oracle/rwkv_np.py)."""
import numpy as np
import pytest

from oracle import rwkv_np

pytestmark = pytest.mark.gpu

SMALL = dict(n_layer=4, d_model=256, ffn=1024, vocab=1000, rescale_every=2)


def _setup(cuda, batch, max_len, seed=0):
    from poptransformer_b200 import rwkv, synth
    sd = synth.rwkv_state_dict(**SMALL, seed=seed, device="cpu")
    dec = rwkv.RWKVDecoder(rwkv.RWKVConfig(**SMALL, max_len=max_len), sd, batch, device=cuda)
    orc = rwkv_np.RWKVOracle(rwkv_np.RWKVConfig(**SMALL, max_len=max_len), {k: v.numpy() for k, v in sd.items()}, batch)
    return dec, orc


@pytest.mark.parametrize("batch", [1, 4])
def test_rwkv_logits_and_states_teacher_forced(cuda, batch):
    from poptransformer_b200 import synth
    max_len = 48
    dec, orc = _setup(cuda, batch, max_len)
    ids = synth.prompt_ids(batch, max_len, max_len, SMALL["vocab"], dec.pad_id, seed=1)
    dec.reset(ids)
    orc.reset()
    for step in range(max_len):
        dec.step()
        exp, _ = orc.logits(ids[:, step].numpy())
        np.testing.assert_allclose(dec.logits.cpu().numpy().astype(np.float32), exp.astype(np.float32), rtol=2e-2, atol=2e-2, err_msg=f"step {step}")
    for i in (0, SMALL["n_layer"] - 1):   # WKV states after 48 tokens
        np.testing.assert_allclose(dec.st_max[i].cpu().numpy(), orc.state[i][4], rtol=2e-2, atol=2e-2)
        np.testing.assert_allclose(dec.st_den[i].cpu().numpy(), orc.state[i][3], rtol=3e-2, atol=2e-2)
    assert dec.error_flag.item() == 0


def test_rwkv_greedy_stream(cuda):
    from poptransformer_b200 import synth
    batch, max_len, prompt = 2, 40, 6
    dec, orc = _setup(cuda, batch, max_len, seed=2)
    ids = synth.prompt_ids(batch, prompt, max_len, SMALL["vocab"], dec.pad_id, seed=3)
    got = dec.run(ids, max_loop=max_len)["Loop:0"]
    exp, logits = orc.generate(ids.numpy(), max_len, dec.pad_id, return_logits=True)
    for b in range(batch):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            t = int(diff[0])
            top2 = np.sort(logits[t - 1][b].astype(np.float32))[-2:]
            assert top2[1] - top2[0] <= 2e-2, f"row {b}: streams diverge at {t} without a numerical tie"
    assert (got == exp).mean() > 0.9
