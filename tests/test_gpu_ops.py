"""GPU parity: every C-ABI op against the numpy oracle on the same seeded inputs.
Bit-exact for integer / copy / fp16-elementwise work; stated tolerances for accumulations."""
import numpy as np
import pytest
import torch

from oracle import ops_np as O

pytestmark = pytest.mark.gpu


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def rng(seed):
    return np.random.default_rng(seed)


# ------------------------------------------------------------------ Int4ToHalf (bit-exact)
@pytest.mark.parametrize("n,m", [(16, 64), (48, 96), (33, 17), (4096, 128)])
def test_int4_to_half_axis1_per_channel(cuda, n, m):
    from poptransformer_b200 import ops
    r = rng(1)
    w = r.integers(-128, 128, size=(n, m), dtype=np.int8)
    s = (r.random(n) * 0.01 + 1e-3).astype(np.float16)
    got = ops.int4_to_half(dev(w, cuda), dev(s, cuda), axis=1).cpu().numpy()
    exp = O.int4_to_half(w, s, axis=1)
    assert got.shape == exp.shape and np.array_equal(got.view(np.uint16), exp.view(np.uint16))


def test_int4_to_half_all_bytes_lut(cuda):
    """All 256 byte values: equals the reference's 256x2 LUT (int4_to_half_custom_op.cpp:139-166)."""
    from poptransformer_b200 import ops
    w = np.arange(256, dtype=np.uint8).view(np.int8).reshape(1, 256)
    s = np.ones(1, dtype=np.float16)
    got = ops.int4_to_half(dev(w, cuda), dev(s, cuda), axis=1).cpu().numpy().reshape(256, 2)
    for b in range(256):
        sb = b - 256 if b >= 128 else b
        hi = sb >> 4
        lo = ((b << 4) & 0xFF)
        lo = (lo - 256 if lo >= 128 else lo) >> 4
        assert got[b, 0] == hi and got[b, 1] == lo


def test_int4_to_half_group_and_axis0(cuda):
    from poptransformer_b200 import ops
    r = rng(2)
    w = r.integers(-128, 128, size=(24, 128), dtype=np.int8)
    sg = (r.random((24, 2)) * 0.01 + 1e-3).astype(np.float16)
    got = ops.int4_to_half(dev(w, cuda), dev(sg, cuda), axis=1, group=128).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), O.int4_to_half(w, sg, axis=1, group=128).view(np.uint16))
    s0 = (r.random(128) * 0.01 + 1e-3).astype(np.float16)
    got0 = ops.int4_to_half(dev(w, cuda), dev(s0, cuda), axis=0).cpu().numpy()
    assert np.array_equal(got0.view(np.uint16), O.int4_to_half(w, s0, axis=0).view(np.uint16))


# ------------------------------------------------------------------ linear (fp32-accumulation tolerance)
def _lin_ref(x, wt):
    return (x.astype(np.float32) @ wt.astype(np.float32))


@pytest.mark.parametrize("batch,n,k,group", [(1, 64, 256, 128), (1, 4096, 4096, 128), (3, 48, 512, 512), (8, 256, 1024, 128),
                                             (16, 128, 2048, 128), (1, 4096, 11008, 128), (32, 64, 512, 256)])
def test_linear_int4(cuda, batch, n, k, group):
    from poptransformer_b200 import ops
    r = rng(3)
    w = (r.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scale = O.quantize_int4(w, group)
    x = (r.standard_normal((batch, k))).astype(np.float16)
    wt = O.int4_to_half(packed, scale, axis=1, group=group)          # [k, n] fp16, the reference's dequantised weight
    exp = _lin_ref(x, wt)
    pl = ops.PackedLinear(ops.W_INT4, dev(packed, cuda), dev(scale, cuda), group=group)
    ws = ops.linear_workspace(batch, n, 16, cuda)
    for ksplit in (0, 1, 3):
        got = ops.linear(dev(x, cuda), pl, workspace=ws, ksplit=ksplit).cpu().numpy().astype(np.float32)
        # exact fp16 products, fp32 accumulation in a different order than numpy: tiny relative error + fp16 output rounding
        np.testing.assert_allclose(got, exp.astype(np.float16).astype(np.float32), rtol=2e-3, atol=2e-3 * np.abs(exp).max())
    assert torch.count_nonzero(ws[:8192]).item() == 0, "split-k counters must return to zero"


def test_linear_shared_workspace_across_widths(cuda):
    """One split-k workspace serves linears of different widths, as the decoders use it: a narrow linear (its partial sums start
    right behind the counter region) followed by wide ones whose row groups need more counters than a 256-byte region held,
    twice in a row.  Shapes: o_proj-like 4096 x 4096, then 16384 and 22016 (Llama-7B gate|up) and 27392 (ChatGLM2-6B gate|up)
    output rows.  Every output row must be written (none stale) and match the oracle's dequantised-weight matmul."""
    from poptransformer_b200 import ops
    r = rng(31)
    k, batch = 4096, 4
    x = r.standard_normal((batch, k)).astype(np.float16)
    widths = (4096, 16384, 22016, 27392)
    ws = ops.linear_workspace(batch, max(widths), 16, cuda)
    layers = []
    for n in widths:
        packed = r.integers(-128, 128, size=(n, k // 2), dtype=np.int8)
        scale = (r.random((n, k // 128), dtype=np.float32) * 0.004 + 0.004).astype(np.float16)
        wt = O.int4_to_half(packed, scale, axis=1, group=128)
        layers.append((ops.PackedLinear(ops.W_INT4, dev(packed, cuda), dev(scale, cuda), group=128), _lin_ref(x, wt)))
    xd = dev(x, cuda)
    for rep in range(2):
        for (pl, exp), n in zip(layers, widths):
            out = torch.full((batch, n), float("nan"), dtype=torch.float16, device=cuda)
            ops.linear(xd, pl, out, workspace=ws, ksplit=4)
            got = out.cpu().numpy().astype(np.float32)
            assert np.isfinite(got).all(), f"rep {rep} n_out {n}: rows left unwritten"
            np.testing.assert_allclose(got, exp.astype(np.float16).astype(np.float32), rtol=2e-3, atol=2e-3 * np.abs(exp).max(),
                                       err_msg=f"rep {rep} n_out {n}")
    assert torch.count_nonzero(ws[:8192]).item() == 0


@pytest.mark.parametrize("batch,n,k", [(1, 32000, 512), (4, 50257, 768), (2, 100, 1600), (16, 300, 64)])
def test_linear_fp16(cuda, batch, n, k):
    from poptransformer_b200 import ops
    r = rng(4)
    w = (r.standard_normal((n, k)) * 0.02).astype(np.float16)
    x = r.standard_normal((batch, k)).astype(np.float16)
    exp = _lin_ref(x, w.T)
    pl = ops.PackedLinear(ops.W_FP16, dev(w, cuda))
    ws = ops.linear_workspace(batch, n, 16, cuda)
    got = ops.linear(dev(x, cuda), pl, workspace=ws).cpu().numpy().astype(np.float32)
    np.testing.assert_allclose(got, exp.astype(np.float16).astype(np.float32), rtol=2e-3, atol=2e-3 * np.abs(exp).max())


def test_linear_fp8(cuda):
    from poptransformer_b200 import ops
    r = rng(5)
    n, k, batch = 96, 512, 8
    w = (r.standard_normal((n, k)) * 0.02).astype(np.float32)
    ws_ = float(np.abs(w).max() / 448.0)
    wb = O.e4m3_encode(w / ws_)
    x = r.standard_normal((batch, k)).astype(np.float16)
    xs_ = float(np.abs(x.astype(np.float32)).max() / 448.0)
    xb = O.cast_fp8(x, xs_)
    exp = O.fp8_matmul(xb, np.ascontiguousarray(wb.T), xs_, ws_).astype(np.float32)
    pl = ops.PackedLinear(ops.W_FP8, dev(wb, cuda), w_scale=ws_)
    ws = ops.linear_workspace(batch, n, 16, cuda)
    got = ops.linear(dev(x, cuda), pl, prologue=ops.PRO_CAST_FP8, act_scale=xs_, workspace=ws).cpu().numpy().astype(np.float32)
    np.testing.assert_allclose(got, exp, rtol=2e-3, atol=2e-3 * np.abs(exp).max())
    # the standalone ops: cast is bit-exact, matmul within accumulation tolerance
    cast = ops.half_to_uint8(dev(x, cuda), xs_).cpu().numpy()
    assert np.array_equal(cast, xb)
    mm = ops.fp8_matmul(dev(xb, cuda), dev(wb, cuda), xs_, ws_).cpu().numpy().astype(np.float32)
    np.testing.assert_allclose(mm, exp, rtol=2e-3, atol=2e-3 * np.abs(exp).max())


def test_linear_epilogues_and_prologue(cuda):
    from poptransformer_b200 import ops
    r = rng(6)
    batch, d, f = 2, 256, 384
    x = r.standard_normal((batch, d)).astype(np.float16)
    gamma = (1 + 0.1 * r.standard_normal(d)).astype(np.float16)
    wg = (r.standard_normal((f, d)) * 0.05).astype(np.float16)
    wu = (r.standard_normal((f, d)) * 0.05).astype(np.float16)
    wd = (r.standard_normal((d, f)) * 0.05).astype(np.float16)
    bias = (r.standard_normal(d) * 0.1).astype(np.float16)
    ws = ops.linear_workspace(batch, 2 * f, 16, cuda)
    # RMSNorm prologue + SwiGLU epilogue
    h = O.rms_norm(x, gamma, 1e-5)
    g = O.swish_f16(O.matmul_f16(h, wg.T))
    u = O.matmul_f16(h, wu.T)
    exp_act = O.mul_f16(u, g).astype(np.float32)
    pl = ops.PackedLinear(ops.W_FP16, dev(np.concatenate([wg, wu]), cuda), interleave_gate_up=True)
    act = ops.linear(dev(x, cuda), pl, prologue=ops.PRO_RMSNORM, gamma=dev(gamma, cuda), eps=1e-5, epilogue=ops.EPI_SWIGLU, workspace=ws)
    np.testing.assert_allclose(act.cpu().numpy().astype(np.float32), exp_act, rtol=1e-2, atol=2e-3)
    # residual (in place) and bias epilogues
    a16 = exp_act.astype(np.float16)
    pld = ops.PackedLinear(ops.W_FP16, dev(wd, cuda))
    y = O.matmul_f16(a16, wd.T)
    xres = dev(x, cuda).clone()
    ops.linear(dev(a16, cuda), pld, xres, epilogue=ops.EPI_RESIDUAL, residual=xres, workspace=ws)
    np.testing.assert_allclose(xres.cpu().numpy().astype(np.float32), O.add_f16(x, y).astype(np.float32), rtol=1e-2, atol=4e-3)
    yb = ops.linear(dev(a16, cuda), pld, epilogue=ops.EPI_BIAS, bias=dev(bias, cuda), workspace=ws)
    np.testing.assert_allclose(yb.cpu().numpy().astype(np.float32), O.add_f16(y, bias).astype(np.float32), rtol=1e-2, atol=4e-3)
    yg = ops.linear(dev(a16, cuda), pld, epilogue=ops.EPI_BIAS_GELU, bias=dev(bias, cuda), workspace=ws)
    np.testing.assert_allclose(yg.cpu().numpy().astype(np.float32), O.gelu_f16(O.add_f16(y, bias)).astype(np.float32), rtol=1e-2, atol=4e-3)


def test_linear_rejects_bad_shapes(cuda):
    from poptransformer_b200 import ops
    w = torch.zeros((16, 100), dtype=torch.float16, device=cuda)
    with pytest.raises(ops.PtError):
        ops.PackedLinear(ops.W_FP16, w)          # k not a multiple of 32
    pl = ops.PackedLinear(ops.W_FP16, torch.zeros((16, 64), dtype=torch.float16, device=cuda))
    with pytest.raises(ops.PtError):
        ops.linear(torch.zeros((33, 64), dtype=torch.float16, device=cuda), pl)   # batch > 32
    with pytest.raises(ops.PtError):
        ops.linear(torch.zeros((1, 32), dtype=torch.float16, device=cuda), pl)    # k mismatch


# ------------------------------------------------------------------ norms / softmax
@pytest.mark.parametrize("rows,dim", [(1, 768), (1, 1600), (2, 768), (16, 1600), (32, 2048)])
def test_norm_ce(cuda, rows, dim):
    from poptransformer_b200 import ops
    r = rng(7)
    x = r.standard_normal((rows, dim)).astype(np.float16)
    g = (1 + 0.1 * r.standard_normal(dim)).astype(np.float16)
    b = (0.1 * r.standard_normal(dim)).astype(np.float16)
    got = ops.layer_norm_ce(dev(x, cuda), dev(g, cuda), dev(b, cuda), 1e-5).cpu().numpy()
    exp = O.norm_ce(x, g, b, 1e-5)
    # The fp32 statistics are summed in a different order than numpy's.  The fp16 chain after them is identical, so a row
    # differs only when the fp16 rounding of its mean or inverse std-dev flips by one ulp, which moves the elements of that
    # row by at most a few fp16 ulps of the output.
    diff = np.abs(got.astype(np.float32) - exp.astype(np.float32))
    assert diff.max() <= 4e-3
    # with the kernel's own rounded statistics recovered from its output, the fp16 chain must be reproducible exactly:
    # re-run the oracle's chain with (m, r) perturbed by at most one ulp and require one combination to match bit for bit
    xf = x.astype(np.float32)
    for row in range(rows):
        n = dim
        if rows == 1:
            mean = xf[row].sum(dtype=np.float32) / np.float32(n)
            var = (xf[row] * xf[row]).sum(dtype=np.float32) / np.float32(n) - mean * mean + np.float32(1e-5)
            m0 = np.float16(mean)
        else:
            m0 = np.float16(xf[row].sum(dtype=np.float32) / np.float32(n))
            var = max((xf[row] * xf[row]).sum(dtype=np.float32) / np.float32(n) - np.float32(m0) ** 2, np.float32(0)) + np.float32(1e-5)
        r0 = np.float16(np.float32(1.0) / np.sqrt(np.float32(var)))
        found = False
        for dm in (0, 1, -1):
            for dr in (0, 1, -1):
                m = np.array(int(m0.view(np.uint16)) + dm, dtype=np.uint16).view(np.float16)[()] if dm else m0
                r = np.array(int(r0.view(np.uint16)) + dr, dtype=np.uint16).view(np.float16)[()] if dr else r0
                t = (xf[row] - np.float32(m)).astype(np.float16)
                t = (t.astype(np.float32) * np.float32(r)).astype(np.float16)
                t = (t.astype(np.float32) * g.astype(np.float32)).astype(np.float16)
                t = (t.astype(np.float32) + b.astype(np.float32)).astype(np.float16)
                found |= np.array_equal(t.view(np.uint16), got[row].view(np.uint16))
        assert found, f"row {row}: fp16 chain not reproducible from statistics within one ulp"


def test_norm_ce_rejects_like_reference(cuda):
    from poptransformer_b200 import ops
    for dim in (770, 8192):
        x = torch.zeros((2, dim), dtype=torch.float16, device=cuda)
        with pytest.raises(ops.PtError):
            ops.layer_norm_ce(x, x[0].clone(), x[0].clone(), 1e-5)


@pytest.mark.parametrize("rows,dim", [(1, 4096), (16, 4096), (3, 100)])
def test_rms_norm(cuda, rows, dim):
    from poptransformer_b200 import ops
    r = rng(8)
    x = r.standard_normal((rows, dim)).astype(np.float16)
    res = r.standard_normal((rows, dim)).astype(np.float16)
    g = (1 + 0.1 * r.standard_normal(dim)).astype(np.float16)
    got = ops.rms_norm(dev(x, cuda), dev(g, cuda), 1e-5).cpu().numpy()
    exp = O.rms_norm(x, g, 1e-5)
    assert (got.view(np.uint16) == exp.view(np.uint16)).mean() > 0.99
    assert np.abs(got.astype(np.float32) - exp.astype(np.float32)).max() <= 4e-3
    got2, s = ops.rms_norm(dev(x, cuda), dev(g, cuda), 1e-5, residual=dev(res, cuda))
    assert np.array_equal(s.cpu().numpy().view(np.uint16), O.add_f16(x, res).view(np.uint16))
    exp2 = O.rms_norm(O.add_f16(x, res), g, 1e-5)
    assert np.abs(got2.cpu().numpy().astype(np.float32) - exp2.astype(np.float32)).max() <= 8e-3


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("stable", [False, True])
def test_softmax_v3(cuda, dtype, stable):
    from poptransformer_b200 import ops
    r = rng(9)
    x = (r.standard_normal((24, 768)) * 2).astype(dtype)
    got = ops.softmax_ce(dev(x, cuda), -1, stable_mode=stable).cpu().numpy()
    exp = O.softmax_v3(x, stable)
    tol = 2e-3 if dtype == np.float16 else 1e-6
    np.testing.assert_allclose(got.astype(np.float32), exp.astype(np.float32), rtol=tol, atol=tol * 1e-2)


@pytest.mark.parametrize("rows,dim", [(1, 768), (16, 1600), (4, 2048)])
def test_linear_normce_prologue(cuda, rows, dim):
    """LayerNorm (NormCE arithmetic, one-row and many-row forms) as the prologue of the linear kernel against the op followed by
    the plain linear: the normalised activations differ at most in the last fp16 bit of a few elements (statistics summed in
    another order), so the outputs agree to the linear-layer tolerance."""
    from poptransformer_b200 import ops
    r = rng(30 + rows)
    n = 1024
    x = (r.standard_normal((rows, dim)) * 1.5 + 0.3).astype(np.float16)
    g = (1 + 0.1 * r.standard_normal(dim)).astype(np.float16)
    bt = (0.1 * r.standard_normal(dim)).astype(np.float16)
    w = (r.standard_normal((n, dim)) * 0.02).astype(np.float16)
    bias = r.standard_normal(n).astype(np.float16)
    pl = ops.PackedLinear(ops.W_FP16, dev(w, cuda))
    ws = ops.linear_workspace(rows, n, 16, cuda)
    got = ops.linear(dev(x, cuda), pl, prologue=ops.PRO_NORMCE, gamma=dev(g, cuda), beta=dev(bt, cuda), eps=1e-5, epilogue=ops.EPI_BIAS,
                     bias=dev(bias, cuda), workspace=ws).cpu().numpy().astype(np.float32)
    h = O.norm_ce(x, g, bt, 1e-5)
    exp = O.add_f16(O.matmul_f16(h, np.ascontiguousarray(w.T)), bias[None, :]).astype(np.float32)
    np.testing.assert_allclose(got, exp, rtol=4e-3, atol=4e-3 * np.abs(exp).max())
    with pytest.raises(ops.PtError, match="norm_beta"):
        ops.linear(dev(x, cuda), pl, prologue=ops.PRO_NORMCE, gamma=dev(g, cuda), eps=1e-5, workspace=ws)


def test_fp8_activation_kernels(cuda):
    """pt_rms_norm_fp8 and pt_swiglu_fp8 (the activation side of the FP8 linears that run on the GEMM) against the restatements:
    the casts are exact, so bytes only differ where the fp16 value in front of the cast differs by its last bit (the RMSNorm
    statistic is summed in another order)."""
    import ctypes
    from poptransformer_b200 import _lib, ops
    L = _lib.lib()
    r = rng(21)
    rows, d, f, scale = 8, 4096, 13696, 8.0 / 448.0
    x = r.standard_normal((rows, d)).astype(np.float16)
    g = (1 + 0.1 * r.standard_normal(d)).astype(np.float16)
    out = torch.empty((rows, d), dtype=torch.uint8, device=cuda)
    xd, gd = dev(x, cuda), dev(g, cuda)
    _lib.check(L.pt_rms_norm_fp8(ops._ptr(xd), ops._ptr(gd), rows, d, 1e-5, scale, ops._ptr(out), ops._stream()), "pt_rms_norm_fp8")
    exp = O.cast_fp8(O.rms_norm(x, g, 1e-5), scale)
    got = out.cpu().numpy()
    assert (got == exp).mean() > 0.99
    assert np.abs(O.e4m3_decode(got) - O.e4m3_decode(exp)).max() <= 0.13 * np.abs(O.e4m3_decode(exp)).max()      # one E4M3 step at most
    gu = r.standard_normal((rows, 2 * f)).astype(np.float16)
    out2 = torch.empty((rows, f), dtype=torch.uint8, device=cuda)
    gud = dev(gu, cuda)
    _lib.check(L.pt_swiglu_fp8(ops._ptr(gud), rows, f, 1.0 / 448.0, ops._ptr(out2), f, ops._stream()), "pt_swiglu_fp8")
    act = O.mul_f16(gu[:, f:], O.swish_f16(gu[:, :f]))
    exp2 = O.cast_fp8(act, 1.0 / 448.0)
    assert (out2.cpu().numpy() == exp2).mean() > 0.999        # expf differs from numpy's by an ulp now and then


# ------------------------------------------------------------------ KV cache (bit-exact)
def test_kv_cache_dense(cuda):
    from poptransformer_b200 import ops
    r = rng(10)
    B, N, L, H = 2, 3, 8, 16
    st_o = O.KVCacheState()
    op = ops.KVCacheOp(max_len=L, sequence_axis=3)
    step_t = torch.zeros(1, dtype=torch.int32, device=cuda)
    for rep in range(2):                      # second pass checks the re-zero at step 0
        for step in range(L + 2 if rep == 0 else 3):
            kv = r.standard_normal((2, B, N, 1, H)).astype(np.float16)
            step_t.fill_(step)
            got = ops.kv_cache(op, step_t, dev(kv, cuda)).cpu().numpy()
            exp = O.kv_cache(st_o, step, kv, L, 3, 1)
            assert np.array_equal(got.view(np.uint16), exp.view(np.uint16)), f"step {step}"


def test_kv_cache_pipeline(cuda):
    from poptransformer_b200 import ops
    r = rng(11)
    B, N, L, H, bps = 2, 2, 6, 8, 3
    st_o = O.KVCachePipelineState()
    op = ops.KVCachePipelineOp(max_len=L, max_bps=bps, sequence_axis=2)
    step_t = torch.zeros(1, dtype=torch.int32, device=cuda)
    for step in list(range(10)) + [0, 1, 2]:
        kv = r.standard_normal((B, N, 1, H)).astype(np.float16)
        step_t.fill_(step)
        got = ops.kv_cache_pipeline(op, step_t, dev(kv, cuda)).cpu().numpy()
        exp = O.kv_cache_pipeline(st_o, step, kv, L, bps, 2, 1)
        assert np.array_equal(got.view(np.uint16), exp.view(np.uint16)), f"step {step}"


@pytest.mark.parametrize("scale", [1.0, 0.03125, 0.013])
def test_kv_cache_fp8_storage(cuda, scale):
    """The `fp8` attribute of KVCache and KVCachePipeline: bytes in the cache, fp16 out; bit-exact against the restatement, through
    the zeroing at step 0, more steps than the cache holds, and values beyond the E4M3 range (saturating cast)."""
    from poptransformer_b200 import ops
    r = rng(12)
    B, N, L, H, bps = 2, 3, 7, 16, 3
    st_o, st_p = O.KVCacheState(), O.KVCachePipelineState()
    op = ops.KVCacheOp(max_len=L, sequence_axis=3, fp8=True, fp8_scale=scale)
    pipe = ops.KVCachePipelineOp(max_len=L, max_bps=bps, sequence_axis=2, fp8=True, fp8_scale=scale)
    step_t = torch.zeros(1, dtype=torch.int32, device=cuda)
    for step in list(range(L + 3)) + [0, 1, 2]:
        kv = (r.standard_normal((2, B, N, 1, H)) * (600.0 * scale if step == 2 else 3.0 * scale)).astype(np.float16)
        step_t.fill_(step)
        got = ops.kv_cache(op, step_t, dev(kv, cuda)).cpu().numpy()
        exp = O.kv_cache(st_o, step, kv, L, 3, 1, fp8=True, fp8_scale=scale)
        assert got.dtype == np.float16 and np.array_equal(got.view(np.uint16), exp.view(np.uint16)), f"KVCache step {step}"
        assert np.array_equal(op.cache.cpu().numpy(), st_o.cache), f"KVCache bytes, step {step}"
        got = ops.kv_cache_pipeline(pipe, step_t, dev(kv[0], cuda)).cpu().numpy()
        exp = O.kv_cache_pipeline(st_p, step, kv[0], L, bps, 2, 1, fp8=True, fp8_scale=scale)
        assert np.array_equal(got.view(np.uint16), exp.view(np.uint16)), f"KVCachePipeline step {step}"
        assert np.array_equal(pipe.caches.cpu().numpy(), np.stack(st_p.caches)), f"KVCachePipeline bytes, step {step}"


def test_kv_cache_pipeline_last_dim_layout(cuda):
    """transpose=1: the caches are stored [..., H, L] and shifted along the last dimension (GetBpsKvCacheLastDim); the op hands the
    result back transposed, so the values equal the plain layout's."""
    from poptransformer_b200 import ops
    r = rng(12)
    B, N, L, H, bps = 2, 3, 9, 8, 2
    st_o = O.KVCachePipelineState()
    op = ops.KVCachePipelineOp(max_len=L, max_bps=bps, sequence_axis=2, transpose=1)
    step_t = torch.zeros(1, dtype=torch.int32, device=cuda)
    for step in list(range(12)) + [0, 1]:
        kv = r.standard_normal((B, N, 1, H)).astype(np.float16)
        step_t.fill_(step)
        got = ops.kv_cache_pipeline(op, step_t, dev(kv, cuda)).cpu().numpy()
        exp = O.kv_cache_pipeline(st_o, step, kv, L, bps, 2, 1)
        assert np.array_equal(got.view(np.uint16), exp.view(np.uint16)), f"step {step}"
    assert tuple(op.caches.shape) == (bps, B, N, H, L)
    # the stored layout really is the shifted last dimension: newest token in column 0 of the cache that took the last insert
    assert np.array_equal(op.caches[1 % bps].cpu().numpy()[..., 0].view(np.uint16), kv[:, :, 0, :].view(np.uint16))


def test_random_sample_picks_one_of_the_top_k(cuda):
    from poptransformer_b200 import ops
    r = rng(13)
    x = r.standard_normal((3, 1, 500)).astype(np.float16)
    g = torch.Generator(device=cuda).manual_seed(0)
    seen = set()
    for _ in range(8):
        ids = ops.random_sample(dev(x, cuda), 4, generator=g).cpu().numpy()
        assert ids.shape == (3, 1, 1)
        top4 = O.topk(x, 4)[1]
        for b in range(3):
            assert ids[b, 0, 0] in top4[b, 0]
        seen.add(int(np.nonzero(top4[0, 0] == ids[0, 0, 0])[0][0]))
    assert len(seen) > 1            # the pick varies with the draws


# ------------------------------------------------------------------ fused RoPE + paged append + attention
@pytest.mark.parametrize("B,N,G,H,L,page,mode", [(1, 4, 4, 128, 40, 16, "llama"), (2, 8, 8, 128, 150, 64, "llama"),
                                                (2, 4, 4, 64, 70, 32, "gpt2"), (2, 8, 2, 128, 70, 64, "none_gqa"),
                                                (2, 8, 2, 128, 70, 64, "chatglm2"),
                                                # 8 and 16 q heads per kv group: the group's heads are shared out over 2 and 4 blocks
                                                (2, 16, 2, 128, 70, 64, "chatglm2"), (1, 32, 2, 128, 150, 64, "chatglm2"),
                                                (2, 16, 2, 64, 40, 16, "none_gqa")])
def test_kv_append_attn(cuda, B, N, G, H, L, page, mode):
    from poptransformer_b200 import ops
    from poptransformer_b200.llama import rope_tables
    r = rng(12)
    sin_o, cos_o = O.llama_rope_tables(L, H)
    sin_t, cos_t = rope_tables(L, H, cuda)
    assert np.array_equal(sin_t.cpu().numpy().view(np.uint16), sin_o.view(np.uint16))
    sin_c, cos_c = O.chatglm2_rope_tables(L, H)
    cache = ops.PagedKVCache(B, G, H, L, page, cuda)
    # scramble the page table to prove the indirection is honoured
    perm = torch.randperm(B * cache.max_pages, generator=torch.Generator().manual_seed(0)).to(torch.int32)
    cache.page_table.copy_(perm.reshape(B, cache.max_pages).to(cuda))
    st_o = O.KVCacheState()
    step_t = torch.zeros(1, dtype=torch.int32, device=cuda)
    ws = ops.attn_workspace(B, N, H, cache.max_pages, cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    scale = float(np.float16(1 / np.sqrt(H)))
    for step in range(L):
        qkv = (r.standard_normal((B, (N + 2 * G) * H)) * 0.5).astype(np.float16)
        q = qkv[:, : N * H].reshape(B, N, 1, H)
        k = qkv[:, N * H:(N + G) * H].reshape(B, G, 1, H)
        v = qkv[:, (N + G) * H:].reshape(B, G, 1, H)
        if mode == "llama":
            q = O.llama_rope_apply(q, sin_o[step], cos_o[step])
            k = O.llama_rope_apply(k, sin_o[step], cos_o[step])
        if mode == "chatglm2":       # multi-query groups, interleaved pairs on the first half of each head, fp16 softmax
            q = O.chatglm2_rope_apply(q, sin_c[step], cos_c[step])
            k = O.chatglm2_rope_apply(k, sin_c[step], cos_c[step])
        past = O.kv_cache(st_o, step, np.stack([k, v]), L, 3, 1)          # [2,B,G,L,H]
        step_t.fill_(step)
        kw = dict(rope_mode=ops.ROPE_LLAMA, softmax_mode=ops.SOFTMAX_F32, score_scale=scale, rope_sin=sin_t, rope_cos=cos_t) if mode == "llama" \
            else dict(rope_mode=ops.ROPE_CHATGLM2, softmax_mode=ops.SOFTMAX_F16, score_scale=scale, rope_sin=dev(sin_c, cuda),
                      rope_cos=dev(cos_c, cuda)) if mode == "chatglm2" else dict(rope_mode=ops.ROPE_NONE, softmax_mode=ops.SOFTMAX_F16 if mode == "gpt2" else ops.SOFTMAX_F32,
                      score_scale=1.0 if mode == "gpt2" else scale)
        got = ops.kv_append_attn(dev(qkv, cuda), step_t, cache, N, workspace=ws, error_flag=err, **kw).cpu().numpy()
        if step % 7 == 0 or step == L - 1:
            rep = N // G
            K = np.repeat(past[0], rep, axis=1)
            V = np.repeat(past[1], rep, axis=1)
            exp = O.attention_decode(q, K, V, O.decode_mask(B, L, step), H, "float16" if mode in ("gpt2", "chatglm2") else "float32",
                                     pre_scaled=(mode == "gpt2")).reshape(B, N * H)
            np.testing.assert_allclose(got.astype(np.float32), exp.astype(np.float32), rtol=2e-2, atol=2e-3, err_msg=f"step {step}")
            # cache contents, exported to the reference layout, are bit-exact
            dense = cache.export(step_t, L).cpu().numpy()
            assert np.array_equal(dense.view(np.uint16), past.view(np.uint16)), f"cache mismatch at step {step}"
    assert err.item() == 0
    assert torch.count_nonzero(ws[: B * N * 4]).item() == 0


# ------------------------------------------------------------------ top-k / beam search (bit-exact indices)
@pytest.mark.parametrize("rows,dim,k,dtype", [(1, 32000, 1, np.float16), (4, 50257, 4, np.float16), (3, 1000, 8, np.float32)])
def test_topk(cuda, rows, dim, k, dtype):
    from poptransformer_b200 import ops
    r = rng(13)
    x = r.standard_normal((rows, dim)).astype(dtype)
    x[:, 5] = x[:, 77] = x.max() + 1           # forced tie: lowest index must win
    v, i = ops.topk(dev(x, cuda), k)
    ev, ei = O.topk(x, k)
    assert np.array_equal(i.cpu().numpy(), ei)
    assert np.array_equal(v.cpu().numpy(), ev)


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_beam_search(cuda, dtype):
    from poptransformer_b200 import ops
    r = rng(14)
    B, beam, V, max_len = 3, 4, 5000, 12
    hyp = np.zeros((B, max_len, beam), dtype=np.int32)
    prob = np.zeros((B, beam), dtype=dtype)
    hyp_t, prob_t = dev(hyp, cuda), dev(prob, cuda)
    step_t = torch.zeros(1, dtype=torch.int32, device=cuda)
    parent = torch.zeros(B * beam, dtype=torch.int32, device=cuda)
    for step in range(max_len):
        logits = np.log(r.random((B, beam, V)) + 1e-6).astype(dtype)
        if step == 0:
            logits[:] = logits[:, :1]                    # identical beams at the first step
        step_t.fill_(step)
        nid, gid, hyp_t, prob_t = ops.beam_search(dev(logits, cuda), hyp_t, prob_t, step_t, beam, parent=parent)
        e_nid, e_gid, hyp, prob = O.beam_search_step(logits, hyp, prob, step, beam)
        assert np.array_equal(nid.cpu().numpy(), e_nid), f"step {step}"
        assert np.array_equal(gid.cpu().numpy(), e_gid), f"step {step}"
        assert np.array_equal(hyp_t.cpu().numpy(), hyp), f"step {step}"
        assert np.array_equal(prob_t.cpu().numpy(), prob), f"step {step}"
        if step > 0:
            exp_parent = (np.arange(B)[:, None] * beam + e_gid // beam).reshape(-1)
            assert np.array_equal(parent.cpu().numpy(), exp_parent)


# ------------------------------------------------------------------ RWKV WKV, embedding, loop carry
def test_wkv(cuda):
    from poptransformer_b200 import ops
    r = rng(15)
    B, C = 4, 512
    tf = r.uniform(-1, 1, C).astype(np.float32)
    td = r.uniform(-5, -1, C).astype(np.float32)
    num = np.zeros((B, C), np.float32); den = np.zeros((B, C), np.float32); mx = np.full((B, C), -1e30, np.float32)
    num_t, den_t, mx_t = dev(num, cuda), dev(den, cuda), dev(mx, cuda)
    for _ in range(5):
        k = r.standard_normal((B, C)).astype(np.float16)
        v = r.standard_normal((B, C)).astype(np.float16)
        out = ops.wkv(dev(k, cuda), dev(v, cuda), dev(tf, cuda), dev(td, cuda), num_t, den_t, mx_t).cpu().numpy()
        e_out, num, den, mx = O.rwkv_wkv(k, v, tf, td, num, den, mx)
        np.testing.assert_allclose(out.astype(np.float32), e_out.astype(np.float16).astype(np.float32), rtol=2e-3, atol=1e-4)
        np.testing.assert_allclose(num_t.cpu().numpy(), num, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(mx_t.cpu().numpy(), mx, rtol=1e-5, atol=1e-6)


def test_embedding_and_step_containers(cuda):
    from poptransformer_b200 import ops
    r = rng(16)
    B, L, V, d, pad = 3, 10, 50, 64, 49
    table = r.standard_normal((V, d)).astype(np.float16)
    ids = np.full((B, L), pad, dtype=np.int32)
    ids[:, :4] = r.integers(0, pad, size=(B, 4))
    ids_t = dev(ids, cuda)
    step_t = torch.zeros(1, dtype=torch.int32, device=cuda)
    step = 0
    for it in range(L):
        e = ops.embedding(dev(table, cuda), ids_t, step_t).cpu().numpy()
        assert np.array_equal(e, O.embedding(table, ids[:, step]))
        nxt = r.integers(0, pad, size=(B, 1)).astype(np.int32)
        ops.step_containers(ids_t, step_t, dev(nxt, cuda), pad)
        ids, step, _ = O.step_containers(ids, step, nxt, pad)
        assert np.array_equal(ids_t.cpu().numpy(), ids) and step_t.item() == step


# ------------------------------------------------------------------ beam reorder of the paged cache, TP head ops
def test_kv_reorder_pages_and_table(cuda):
    """Row r continues from row parent[r]: full pages are shared through the page table, the page being filled is copied
    into the row's spare page.  Checked through the reference-layout export, twice in a row (spare pages swap roles)."""
    from poptransformer_b200 import _lib, ops
    L = _lib.lib()
    rows, n_kv, hd, page, max_len, step = 4, 2, 128, 64, 200, 150
    kc = ops.PagedKVCache(rows, n_kv, hd, max_len, page, cuda, extra_pages=rows)
    g = torch.Generator(device=cuda).manual_seed(3)
    kc.pool.copy_(torch.randn(kc.pool.shape, generator=g, device=cuda).to(torch.float16))
    spare = (torch.arange(rows, dtype=torch.int32, device=cuda) + rows * kc.max_pages).contiguous()
    tmp = torch.empty_like(kc.page_table)
    step_t = torch.tensor([step], dtype=torch.int32, device=cuda)
    dense = kc.export(step_t, max_len).cpu().numpy()
    for parent in ([2, 2, 0, 1], [3, 0, 0, 2]):
        par = torch.tensor(parent, dtype=torch.int32, device=cuda)
        ops.check(L.pt_kv_reorder_pages(ops._ptr(kc.pool), ops._ptr(kc.page_table), ops._ptr(spare), ops._ptr(par), ops._ptr(step_t), rows, n_kv, hd,
                                        page, kc.max_pages, ops._stream()), "pt_kv_reorder_pages")
        ops.check(L.pt_kv_reorder_table(ops._ptr(kc.page_table), ops._ptr(tmp), ops._ptr(spare), ops._ptr(par), ops._ptr(step_t), rows, page,
                                        kc.max_pages, ops._stream()), "pt_kv_reorder_table")
        got = kc.export(step_t, max_len).cpu().numpy()
        dense = O.kv_reorder_dense(dense, parent)
        assert np.array_equal(got.view(np.uint16), dense.view(np.uint16))
        # every row owns its current page exclusively (appending to one row must not touch another)
        cur = kc.page_table[:, step // page].cpu().numpy()
        assert len(set(cur.tolist())) == rows and not set(cur.tolist()) & set(spare.cpu().numpy().tolist())


def test_lm_head_tp_ops(cuda):
    from poptransformer_b200 import _lib, ops
    L = _lib.lib()
    r = rng(21)
    tp, rows, vocab = 4, 3, 1001
    per = -(-vocab // tp)
    full = r.standard_normal((rows, per * tp)).astype(np.float16)
    full[:, vocab:] = 0                       # zero-padded shard rows
    full[1, 5] = 0                            # an exact zero inside the vocabulary is read as -10000 too
    shards = [full[:, k * per:(k + 1) * per].copy() for k in range(tp)]
    vals = torch.empty((tp, rows), dtype=torch.float16, device=cuda)
    ids = torch.empty((tp, rows), dtype=torch.int32, device=cuda)
    for k in range(tp):
        ops.check(L.pt_lm_head_local_topk(ops._ptr(dev(shards[k], cuda)), rows, per, k * per, ops._ptr(vals[k]), ops._ptr(ids[k]), ops._stream()),
                  "pt_lm_head_local_topk")
    nxt = torch.empty(rows, dtype=torch.int32, device=cuda)
    ops.check(L.pt_lm_head_tp_pick(ops._ptr(vals), ops._ptr(ids), tp, rows, ops._ptr(nxt), ops._stream()), "pt_lm_head_tp_pick")
    assert np.array_equal(nxt.cpu().numpy(), O.lm_head_tp_merge(shards, vocab))
