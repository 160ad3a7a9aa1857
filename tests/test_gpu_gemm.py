"""GPU parity of the tensor-core GEMMs (pt_gemm) against the numpy restatements of the reference ops: FP8MatMul
(oracle.ops_np.fp8_matmul, custom_ops/matmul_fp8.cpp:885-1091 in its E4M3 form) and Int4ToHalf followed by the fp16 matmul
(oracle.ops_np.int4_to_half, precision_strategy.py:56-60).  Products are exact in fp32 on both sides, so the only difference
is the fp32 summation order: 2e-3 relative to the largest output, the bar of the other linear-layer tests."""
import numpy as np
import pytest
import torch

from oracle import ops_np as O

pytestmark = pytest.mark.gpu


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _check(got, exp):
    exp16 = exp.astype(np.float16).astype(np.float32)
    np.testing.assert_allclose(got, exp16, rtol=2e-3, atol=2e-3 * np.abs(exp).max())


# (n_out, k_in, m): ChatGLM2-6B dense at every row count; h_to_4h x 2, 4h_to_h and the head at one or two each (the numpy
# reference of the wide ones takes seconds per case)
FP8_CASES = [(4096, 4096, 8), (4096, 4096, 16), (4096, 4096, 32), (4096, 4096, 128), (27392, 4096, 16), (27392, 4096, 128),
             (4096, 13696, 8), (4096, 13696, 32), (65024, 4096, 8), (65024, 4096, 32)]


@pytest.mark.parametrize("n,k,m", FP8_CASES)
def test_gemm_fp8(cuda, n, k, m):
    from poptransformer_b200 import ops
    r = np.random.default_rng(n + k + m)
    w = (r.standard_normal((n, k), dtype=np.float32) * 0.02)
    ws_ = float(np.abs(w).max() / 448.0)
    wb = O.e4m3_encode(w / ws_)
    x = r.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    xs_ = float(np.abs(x.astype(np.float32)).max() / 448.0)
    xb = O.cast_fp8(x, xs_)
    exp = O.fp8_matmul(xb, np.ascontiguousarray(wb.T), xs_, ws_).astype(np.float32)
    gw = ops.GemmWeight(ops.W_FP8, dev(wb, cuda), w_scale=ws_)
    ws = ops.gemm_workspace(m, n, 8, cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    for ksplit in (0, 1):
        got = ops.gemm(dev(xb, cuda), gw, x_scale=xs_, workspace=ws, ksplit=ksplit, error_flag=err).cpu().numpy().astype(np.float32)
        assert int(err.item()) == 0
        _check(got, exp)
    # the reference op's entry point routes here
    mm = ops.fp8_matmul(dev(xb, cuda), dev(wb, cuda), xs_, ws_).cpu().numpy().astype(np.float32)
    _check(mm, exp)


@pytest.mark.parametrize("n,k,group,m", [(4096, 4096, 128, 16), (4096, 4096, 128, 32), (4096, 4096, 128, 128), (22016, 4096, 128, 16),
                                         (22016, 4096, 128, 128), (4096, 11008, 128, 16), (4096, 11008, 128, 32), (1000, 512, 256, 16),
                                         (1000, 512, 256, 128)])
def test_gemm_int4(cuda, n, k, group, m):
    from poptransformer_b200 import ops
    r = np.random.default_rng(n + k + m)
    packed = r.integers(-128, 128, size=(n, k // 2), dtype=np.int8)
    scale = (r.random((n, k // group), dtype=np.float32) * 0.004 + 0.004).astype(np.float16)
    x = r.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    wt = O.int4_to_half(packed, scale, axis=1, group=group)               # [k, n] fp16: the reference's dequantised weight
    exp = x.astype(np.float32) @ wt.astype(np.float32)
    gw = ops.GemmWeight(ops.W_INT4, dev(packed, cuda), dev(scale, cuda), group=group)
    ws = ops.gemm_workspace(m, n, 8, cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    for ksplit in (0, 1, 3):
        got = ops.gemm(dev(x, cuda), gw, workspace=ws, ksplit=ksplit, error_flag=err).cpu().numpy().astype(np.float32)
        assert int(err.item()) == 0
        _check(got, exp)


def test_gemm_widths_share_one_workspace(cuda):
    """GEMMs of different widths take their k-slice counters from one workspace, as the layers of a decoder do: a narrow one (32
    weight tiles, eight k-slices), then a wide one (96 tiles, three k-slices), twice over.  The narrow GEMM's partial sums must not
    land where the wide one counts its arrivals."""
    from poptransformer_b200 import ops
    r = np.random.default_rng(77)
    m, k = 16, 4096
    x = r.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    cases = []
    for n in (4096, 12288):
        packed = r.integers(-128, 128, size=(n, k // 2), dtype=np.int8)
        scale = (r.random((n, k // 128), dtype=np.float32) * 0.004 + 0.004).astype(np.float16)
        exp = x.astype(np.float32) @ O.int4_to_half(packed, scale, axis=1, group=128).astype(np.float32)
        cases.append((ops.GemmWeight(ops.W_INT4, dev(packed, cuda), dev(scale, cuda), group=128), exp))
    ws = ops.gemm_workspace(m, 12288, 8, cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    for _ in range(2):
        for gw, exp in cases:
            got = ops.gemm(dev(x, cuda), gw, workspace=ws, error_flag=err).cpu().numpy().astype(np.float32)
            assert int(err.item()) == 0
            _check(got, exp)


def test_gemm_more_rows_than_one_tile_and_residual(cuda):
    """300 activation rows (two row tiles of the kernel, the second ragged), a width that is no multiple of 128, residual epilogue."""
    from poptransformer_b200 import ops
    r = np.random.default_rng(5)
    m, n, k = 300, 1000, 1024
    packed = r.integers(-128, 128, size=(n, k // 2), dtype=np.int8)
    scale = (r.random((n, k // 128), dtype=np.float32) * 0.004 + 0.004).astype(np.float16)
    x = r.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    res = r.standard_normal((m, n), dtype=np.float32).astype(np.float16)
    wt = O.int4_to_half(packed, scale, axis=1, group=128)
    acc = (x.astype(np.float32) @ wt.astype(np.float32)).astype(np.float16)
    exp = (res.astype(np.float32) + acc.astype(np.float32)).astype(np.float16).astype(np.float32)
    gw = ops.GemmWeight(ops.W_INT4, dev(packed, cuda), dev(scale, cuda), group=128)
    got = ops.gemm(dev(x, cuda), gw, epilogue=ops.EPI_RESIDUAL, residual=dev(res, cuda), workspace=ops.gemm_workspace(m, n, 8, cuda)).cpu().numpy()
    np.testing.assert_allclose(got.astype(np.float32), exp, rtol=4e-3, atol=4e-3 * np.abs(exp).max())


def test_gemm_bias_epilogue(cuda):
    """y = fp16(fp16(acc * scales) + bias) (layers/linear.py:42-46), with and without k-slices."""
    from poptransformer_b200 import ops
    r = np.random.default_rng(9)
    m, n, k = 8, 4608, 4096
    w = r.standard_normal((n, k), dtype=np.float32) * 0.02
    ws_ = float(np.abs(w).max() / 448.0)
    wb = O.e4m3_encode(w / ws_)
    x = r.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    xs_ = float(np.abs(x.astype(np.float32)).max() / 448.0)
    xb = O.cast_fp8(x, xs_)
    bias = r.standard_normal(n).astype(np.float16)
    acc = O.fp8_matmul(xb, np.ascontiguousarray(wb.T), xs_, ws_)
    exp = O.add_f16(acc, bias[None, :]).astype(np.float32)
    gw = ops.GemmWeight(ops.W_FP8, dev(wb, cuda), w_scale=ws_)
    ws = ops.gemm_workspace(m, n, 8, cuda)
    for ksplit in (0, 1):
        got = ops.gemm(dev(xb, cuda), gw, x_scale=xs_, workspace=ws, ksplit=ksplit, epilogue=ops.EPI_BIAS, bias=dev(bias, cuda)).cpu().numpy()
        np.testing.assert_allclose(got.astype(np.float32), exp, rtol=2e-3, atol=2e-3 * np.abs(exp).max())


def test_gemm_rejects_bad_shapes(cuda):
    from poptransformer_b200 import ops
    gw = ops.GemmWeight(ops.W_FP8, torch.zeros((64, 256), dtype=torch.uint8, device=cuda))
    gw.k_in = 192
    with pytest.raises(ops.PtError, match="multiple of 128"):
        ops.gemm(torch.zeros((16, 192), dtype=torch.uint8, device=cuda), gw)
