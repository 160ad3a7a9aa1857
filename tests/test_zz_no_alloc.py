"""pt_linear_static_scratch: the linear layer for hosts that cannot allocate device memory where they call it (a plugin
inside a process that owns the memory pool, a no-allocation callback).  Its split-k scratch is a fixed array inside the
library, so the test checks three things through the C-ABI: results equal pt_linear's on two calls in a row (the array
is shared and keeps the previous call's contents), no torch allocation happens during the calls, and a shape whose
scratch would not fit is refused with a message instead of being run."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_variant_twice(cuda):
    from poptransformer_b200 import _lib, ops
    L = _lib.lib()
    g = torch.Generator(device="cpu").manual_seed(0)
    n, k, batch = 4096, 4096, 2
    w = torch.randint(-128, 128, (n, k // 2), generator=g, dtype=torch.int8).to(cuda)
    s = (torch.rand((n, k // 128), generator=g) * 0.004 + 0.004).half().to(cuda)
    pl = ops.PackedLinear(ops.W_INT4, w, s, group=128)
    ws = ops.linear_workspace(batch, n, 32, cuda)
    out_ref = torch.empty((batch, n), dtype=torch.float16, device=cuda)
    out_new = torch.empty_like(out_ref)
    xs = [torch.randn((batch, k), generator=g).half().to(cuda) for _ in range(2)]
    torch.cuda.synchronize()
    for call, x in enumerate(xs):                      # two calls in a row on the same stream
        a = ops.linear_args(x, pl, out_ref, workspace=ws)
        _lib.check(L.pt_linear(ctypes.byref(a), ops._stream()), "pt_linear")
        b = ops.linear_args(x, pl, out_new)            # no workspace from the caller
        before = torch.cuda.memory_allocated()
        _lib.check(L.pt_linear_static_scratch(ctypes.byref(b), ops._stream()), "pt_linear_static_scratch")
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        ref, new = out_ref.float().cpu().numpy(), out_new.float().cpu().numpy()
        assert np.isfinite(new).all()
        np.testing.assert_allclose(new, ref, rtol=2e-3, atol=2e-3 * np.abs(ref).max(), err_msg=f"call {call}")


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
