"""Host side of the reference's decode loop, shared by the decoders.

The reference builds one PopART Loop around the model graph (poptransformer/ops/popart.py:170-178,
models/base_model.py:271-290) and `Session.run` executes it once per generation
(poptransformer/sessions.py:47-49), returning the anchors `Loop:0` (the id container) and `Loop:1`
(the step).  Here the loop body is one `step()` of a decoder (CUDA-graph replay or kernel launches) and
the loop itself is this host `for`: nothing but the launches crosses the host boundary per token.

`early_stop` (HFDecBaseModel.early_stop, models/base_model.py:348-352): the reference's loop condition is
"some sequence had not produced its eos id before this iteration".  The device keeps that condition in
`done_flag`: the loop-carry kernel sets it, and once set every later step leaves ids, step and stop mask
untouched, so the host only needs to look at the flag every `poll_every` steps and still returns exactly the
state at which the reference's loop ends.
"""
import torch

from ._lib import PtError


class DecodeLoop:
    early_stop = False
    done_flag = None

    def _init_loop(self, device, early_stop=False):
        self.early_stop = bool(early_stop)
        self.done_flag = torch.zeros(1, dtype=torch.int32, device=device)

    def _loop_done_flag(self):
        """The device flag handed to the loop-carry kernel (None when the loop always runs max_loop iterations)."""
        return self.done_flag if self.early_stop else None

    def run(self, input_ids, max_loop=None, poll_every=16, prefill=False):
        """Session.run equivalent (poptransformer/sessions.py:47-49): feeds the id container, runs at most `max_loop` loop
        iterations on the device and returns the reference's anchors {'Loop:0': ids, 'Loop:1': step}.  `prefill=True` (decoders that
        have `prefill()`): the iterations that only consume prompt tokens are replaced by one pass over the prompt."""
        max_len = self.cfg.max_len
        n = max_len if max_loop is None else int(max_loop)
        if n < 0 or n > max_len:
            raise PtError(f"max_loop={n} outside 0..max_length={max_len}")
        self.reset(input_ids)
        if self.done_flag is not None:
            self.done_flag.zero_()
        first = min(n, self.prefill()) if prefill else 0     # loop iterations the one-pass prompt ingestion stands for
        for i in range(first, n):
            self.step()
            if self.early_stop and (i + 1) % poll_every == 0 and int(self.done_flag.item()):
                break
        out = {"Loop:0": self.ids.cpu().numpy(), "Loop:1": self.step_t.cpu().numpy()}
        err = int(self.error_flag.item())
        if err != 0:
            raise PtError(f"device-side error flag {err} during decode (a bounded wait gave up, or the step left the id container)")
        return out


class MultiStreamLoop:
    """`max_bps` decode streams over ONE set of weights, served in turn (continuous decode).

    Global iteration s runs one loop iteration of stream s % max_bps, which is that stream's own step s // max_bps: the
    (bpsIdx, stepTrue) pair the reference's GetStepBps vertex derives from the loop counter (custom_ops/kv_cache_codelet.cpp:18-36)
    and by which KVCachePipeline picks one of its `max_bps` caches (custom_ops/kv_cache_pipeline.cpp:392-439).  Each stream owns
    its id container, step, stop mask, KV caches and CUDA graph (`decoder.new_stream()`); the weights exist once.  A stream whose
    generation has ended (its `max_loop` iterations are done, or with `early_stop` every sequence has produced its eos id) takes
    the next waiting request while the other streams keep going, so the device never idles behind the longest generation."""

    def __init__(self, decoder, max_bps, capture=True):
        if max_bps < 1:
            raise PtError(f"max_bps={max_bps}")
        if not hasattr(decoder, "new_stream"):
            raise PtError(f"{type(decoder).__name__} has no new_stream(): its weights cannot be shared between streams")
        self.streams = [decoder] + [decoder.new_stream() for _ in range(max_bps - 1)]
        if capture:
            for s in self.streams:
                if s.graph is None:
                    s.capture()
        self.max_bps = max_bps

    def run(self, requests, max_loop=None, poll_every=16):
        """requests: a list of id containers ([batch, max_len] int32 each).  Returns one {'Loop:0', 'Loop:1'} per request, each
        identical to what `decoder.run(request, max_loop)` returns on its own."""
        first = self.streams[0]
        max_len = first.cfg.max_len
        n = max_len if max_loop is None else int(max_loop)
        if n < 0 or n > max_len:
            raise PtError(f"max_loop={n} outside 0..max_length={max_len}")
        results = [None] * len(requests)
        waiting = list(range(len(requests)))
        serving = [None] * self.max_bps         # request index each stream is working on
        done_steps = [0] * self.max_bps         # stepTrue of each stream

        def start(k):
            serving[k] = waiting.pop(0) if waiting else None
            if serving[k] is not None:
                st = self.streams[k]
                st.reset(requests[serving[k]])
                if st.done_flag is not None:
                    st.done_flag.zero_()
                done_steps[k] = 0

        def finish(k):
            st = self.streams[k]
            results[serving[k]] = {"Loop:0": st.ids.cpu().numpy().copy(), "Loop:1": st.step_t.cpu().numpy().copy()}   # the stream's buffers are reused
            err = int(st.error_flag.item())
            if err != 0:
                raise PtError(f"device-side error flag {err} on stream {k}")

        for k in range(self.max_bps):
            start(k)
        s = 0
        while any(r is not None for r in serving):
            k = s % self.max_bps               # bpsIdx
            s += 1
            if serving[k] is None:
                continue
            st = self.streams[k]
            ended = done_steps[k] >= n
            if not ended:
                st.step()
                done_steps[k] += 1
                ended = done_steps[k] >= n or (st.early_stop and done_steps[k] % poll_every == 0 and int(st.done_flag.item()))
            if ended:
                finish(k)
                start(k)
        return results
