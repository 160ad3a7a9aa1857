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
