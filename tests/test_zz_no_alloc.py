"""pt_linear_static_scratch: the linear layer for hosts that cannot allocate device memory where they call it (a plugin
inside a process that owns the memory pool, a no-allocation callback).  Its split-k scratch is a fixed array inside the
library, so the tests check through the C-ABI: results equal pt_linear's on two calls in a row (the array is shared and
keeps the previous call's contents) for every weight format, with and without a k-split, and when the output width
changes between calls; neither torch's allocator nor the device's free memory moves during the calls; and a shape whose
scratch would not fit is refused with a message instead of being run."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _packed(ops, cuda, g, wfmt, n, k):
    if wfmt == ops.W_INT4:
        w = torch.randint(-128, 128, (n, k // 2), generator=g, dtype=torch.int8).to(cuda)
        s = (torch.rand((n, k // 128), generator=g) * 0.004 + 0.004).half().to(cuda)
        return ops.PackedLinear(ops.W_INT4, w, s, group=128)
    if wfmt == ops.W_FP16:
        return ops.PackedLinear(ops.W_FP16, (torch.randn((n, k), generator=g) * 0.02).half().to(cuda))
    w = torch.randint(0, 120, (n, k), generator=g, dtype=torch.int32).to(torch.uint8).to(cuda)   # positive E4M3 codes below 448
    return ops.PackedLinear(ops.W_FP8, w, w_scale=0.01)


@pytest.mark.parametrize("fmt,ksplit", [("int4", 0), ("fp16", 0), ("fp8", 0), ("int4", 1), ("fp16", 5)])
def test_static_scratch_matches_workspace_variant_twice(cuda, fmt, ksplit):
    from poptransformer_b200 import _lib, ops
    L = _lib.lib()
    wfmt = {"int4": ops.W_INT4, "fp16": ops.W_FP16, "fp8": ops.W_FP8}[fmt]
    g = torch.Generator(device="cpu").manual_seed(0)
    k, batch = 4096, 2
    widths = (4096, 12288)                             # the output width changes between the two calls
    pls = [_packed(ops, cuda, g, wfmt, n, k) for n in widths]
    ws = ops.linear_workspace(batch, max(widths), 32, cuda)
    xs = [torch.randn((batch, k), generator=g).half().to(cuda) for _ in range(2)]
    outs = [(torch.empty((batch, n), dtype=torch.float16, device=cuda), torch.empty((batch, n), dtype=torch.float16, device=cuda)) for n in widths]
    # the address of the built-in array is looked up by the first call on a device: make that call before measuring
    warm = ops.linear_args(xs[0], pls[0], outs[0][1], ksplit=ksplit)
    _lib.check(L.pt_linear_static_scratch(ctypes.byref(warm), ops._stream()), "pt_linear_static_scratch")
    torch.cuda.synchronize()
    for call, (x, pl, (out_ref, out_new)) in enumerate(zip(xs, pls, outs)):     # two calls in a row on the same stream
        a = ops.linear_args(x, pl, out_ref, workspace=ws, ksplit=ksplit)
        _lib.check(L.pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")
        b = ops.linear_args(x, pl, out_new, ksplit=ksplit)    # no workspace from the caller
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        _lib.check(L.pt_linear_static_scratch(ctypes.byref(b), ops._stream()), "pt_linear_static_scratch")
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before, "the device's free memory changed during the call"
        ref, new = out_ref.float().cpu().numpy(), out_new.float().cpu().numpy()
        assert np.isfinite(new).all()
        # same kernel, same split, same summation order
        assert np.array_equal(new, ref), f"call {call}"


def test_static_scratch_rejects_oversized_shapes(cuda):
    from poptransformer_b200 import _lib, ops
    L = _lib.lib()
    n, k, batch = 65536, 4096, 32                      # 16 splits x 32 rows x 65536 outputs x 4 B > 4 MiB
    pl = ops.PackedLinear(ops.W_FP16, torch.zeros((n, k), dtype=torch.float16, device=cuda))
    x = torch.zeros((batch, k), dtype=torch.float16, device=cuda)
    out = torch.zeros((batch, n), dtype=torch.float16, device=cuda)
    a = ops.linear_args(x, pl, out, ksplit=16)
    rc = L.pt_linear_static_scratch(ctypes.byref(a), ops._stream())
    assert rc == -1
    msg = L.pt_last_error().decode()
    assert "built-in scratch" in msg and "pt_linear" in msg
    torch.cuda.synchronize()
    assert torch.count_nonzero(out).item() == 0        # nothing ran
