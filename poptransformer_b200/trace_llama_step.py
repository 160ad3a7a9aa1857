"""Where a step of the persistent Llama kernel spends its time: reads the in-kernel stamps of a diagnostics build.

The persistent kernel (csrc/decode_llama.cu) can stamp its phase boundaries with the global timer and, when the library is
built with -DPT_MK_TRACE_WAITS, also accumulates SM-cycle counts inside the staging and multiplication code.  Build a second
library with that flag and point this script at it; the production library is not touched:

    PT_NVCC_EXTRA=-DPT_MK_TRACE_WAITS PT_B200_LIB=/tmp/libpt_trace.so python -m poptransformer_b200.build
    PT_B200_LIB=/tmp/libpt_trace.so python -m poptransformer_b200.trace_llama_step [--layers 8] [--no-math]

Prints, per transformer block and averaged over the SMs (also the slowest / fastest SM): the time of each staging, linear phase
and of the attention phase, the split of a staging (wait for the producers / loads / RMSNorm / quantise) and of a linear phase
(set-up / multiplication loop / reduction + epilogue / publish), and per matrix how many cycles an iteration of the loop waits
for its stage against how many it loads and multiplies.  --no-math consumes the weight tiles without multiplying them, which
shows the pace of the weight stream alone.  The diagnostics build runs about a quarter slower than the production build."""
import argparse

import numpy as np
import torch

from . import llama, synth

TRS = 64   # trace slots per (SM, block) of the diagnostics build


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--no-math", action="store_true")
    args = ap.parse_args()
    nl = args.layers
    dev = torch.device("cuda", 0)
    dims = dict(n_layer=nl, d_model=4096, n_head=32, ffn=11008, vocab=32000)
    cfg = llama.LlamaConfig(**dims, max_len=args.ctx + 256, int4_group=128)
    sd = synth.llama_state_dict(**dims, seed=0, device=dev, int4_group=128)
    dec = llama.LlamaDecoder(cfg, sd, 1, device=dev, keep_logits=False)
    if not dec.persistent:
        raise SystemExit("the persistent kernel does not cover this configuration")
    del sd
    ids = synth.prompt_ids(1, args.ctx, cfg.max_len, cfg.vocab, dec.pad_id, seed=0)
    gen = torch.Generator(device=dev).manual_seed(1)
    for kc in dec.caches:
        kc.pool.copy_((torch.randn(kc.pool.shape, generator=gen, device=dev) * 0.5).to(torch.float16))
    nsm = torch.cuda.get_device_properties(0).multi_processor_count
    tr = torch.zeros((nsm, nl, TRS), dtype=torch.int64, device=dev)
    dec.reset(ids)
    dec.step_t.fill_(args.ctx - 1)
    for _ in range(4):
        dec.step()
    torch.cuda.synchronize()
    dec.mk_args.trace = tr.data_ptr()
    dec.mk_args.debug = 1 if args.no_math else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        dec.step()
    e1.record()
    torch.cuda.synchronize()
    print("ms per step (diagnostics build, %d blocks): %.4f, error flag %d" % (nl, e0.elapsed_time(e1) / args.steps, dec.error_flag.item()))
    t = tr.cpu().numpy().astype(np.float64)       # stamps belong to the last step; the cycle counters add up over all steps
    if t[:, 1:, 48:].sum() == 0:
        print("(no cycle counters: this library was built without -DPT_MK_TRACE_WAITS; only the stamps are shown)")
    L = slice(1, nl)                               # block 0 starts behind the embedding: left out

    def d(a, b):
        x = t[:, L, b] - t[:, L, a]
        return x.mean() / 1e3, x.max(axis=0).mean() / 1e3, x.min(axis=0).mean() / 1e3

    for name, a, b in [("staging q|k|v", 0, 1), ("q|k|v", 1, 2), ("attention", 3, 4), ("staging o", 4, 5), ("o_proj", 5, 6), ("staging gate|up", 7, 8),
                       ("gate|up", 8, 9), ("staging down", 9, 10), ("down_proj", 10, 11), ("block", 0, 12)]:
        print("%-16s mean %6.2f us   slowest SM %6.2f   fastest SM %6.2f" % ((name,) + d(a, b)))
    print("attention (us): q poll + RoPE %.2f, wait for K/V %.2f, scores %.2f, softmax %.2f, P.V %.2f, publish %.2f; all units %.2f" % (
        d(3, 13)[0], d(13, 15)[0], d(15, 16)[0], d(16, 17)[0], d(17, 18)[0], d(18, 19)[0], d(13, 14)[0]))
    norm = nsm * (nl - 1) * args.steps
    clk = torch.cuda.get_device_properties(0).clock_rate / 1e3      # cycles per microsecond at the maximum SM clock
    for i, w in enumerate(("q|k|v", "o_proj", "gate|up", "down_proj")):
        a = t[:, L, 32 + 4 * i: 36 + 4 * i].sum(axis=(0, 1))
        n = max(a[3], 1)
        print("%-10s loop iteration (two tiles per warp): waits %.0f cycles for its stage, loads + multiplies %.0f cycles; %.1f iterations per block"
              % (w, a[0] / n, a[2] / n, a[3] / norm))
    sq = t[:, L, 48:53].sum(axis=(0, 1)) / norm / clk
    print("the four stagings of a block (us): wait for producers %.2f, loads %.2f, RMSNorm %.2f, quantise %.2f, barrier %.2f" % tuple(sq))
    pq = t[:, L, 56:61].sum(axis=(0, 1)) / norm / clk
    print("the four linear phases of a block (us): set-up %.2f, loop %.2f, barrier %.2f, reduction + epilogue %.2f, publish %.2f" % tuple(pq))
    print("weight-stream wait of warp 0 per block %.2f us; producer blocked on a full ring per block %.2f us" % (
        t[:, L, 23].mean() / 1e3, t[:, L, 27].mean() / 1e3))


if __name__ == "__main__":
    main()
