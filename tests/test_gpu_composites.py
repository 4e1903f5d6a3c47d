"""Hadamard rotation, the two-layout quantize and microscaling attention."""

import pytest
import torch

import cases as C
from golden_io import bits_equal, describe_mismatch, golden_cases
from oracle import tables as OT

pytestmark = pytest.mark.gpu

_CASES = golden_cases(OT.quantization_map)


def _impl():
    from cuda_impl import CudaImpl

    return CudaImpl


def _close_in_bf16(got, want, max_fraction=2e-3):
    """Equal except for single-ulp differences (fp32 summation order) on a small fraction."""
    assert got.shape == want.shape and got.dtype == want.dtype
    g, w = got.float(), want.float()
    diff = (g - w).abs()
    ulp = torch.maximum(g.abs(), w.abs()) * 2.0 ** -7 + 1e-30
    assert bool((diff <= ulp).all()), float((diff / ulp).max())
    assert float((diff > 0).float().mean()) <= max_fraction


@pytest.mark.parametrize("name", ["hadamard_last", "hadamard_rows"])
def test_hadamard(name):
    op, args, kwargs, expected = _CASES[name]
    got = C.run_case(_impl(), op, args, kwargs)
    _close_in_bf16(got[0], expected[0])


def test_quantize_mx_transpose():
    op, args, kwargs, expected = _CASES["mx_transpose_nvfp4"]
    got = C.run_case(_impl(), op, args, kwargs)
    # the untransposed layout involves no rotation: bit-exact
    assert bits_equal(got[0], expected[0]), describe_mismatch(got[0], expected[0])
    assert bits_equal(got[1], expected[1]), describe_mismatch(got[1], expected[1])
    # the rotated transpose can differ where an fp32 sum lands on a rounding boundary
    assert got[2].shape == expected[2].shape and got[3].shape == expected[3].shape
    assert float((got[2].float() != expected[2].float()).float().mean()) < 0.05
    assert float((got[3].float() != expected[3].float()).float().mean()) < 0.02


def test_sdpa_mx():
    import voyager_b200

    op, args, kwargs, expected = _CASES["sdpa_mx_int8"]
    got = C.run_case(_impl(), op, args, kwargs)
    voyager_b200.ops.gemm_status()
    g, w = got[0].float(), expected[0].float()
    assert g.shape == w.shape
    assert float((g - w).abs().max() / w.abs().max()) <= 2e-2


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_conv2d_mx_reads_its_operands_back_and_convolves(layout):
    """``conv2d_mx`` = ``dequantize_mx`` of both operands (bit-exact kernels) + the convolution, in either layout."""
    import torch.nn.functional as F

    import voyager_b200 as vb

    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 32, 9, 9, generator=g).bfloat16().cuda()
    w = (torch.randn(16, 32, 3, 3, generator=g) * 0.1).bfloat16().cuda()
    bias = torch.randn(16, generator=g).bfloat16().cuda()
    table = vb.get_quantization_map("int8").cuda()
    Q = torch.ops.quantized_ops
    xs, ws = (x.permute(0, 2, 3, 1).contiguous(), w.permute(2, 3, 1, 0).contiguous()) if layout == "nhwc" else (x, w)
    axis_x, axis_w = (-1, -2) if layout == "nhwc" else (1, 1)            # blocks along the input channels
    sx, cx = Q.quantize_mx(xs, table, [axis_x], 16, 127.0, True)
    sw, cw = Q.quantize_mx(ws, table, [axis_w], 16, 127.0, True)
    got = Q.conv2d_mx(cx, cw, bias, [1, 1], [1, 1], [1, 1], 1, input_scale=sx, weight_scale=sw, block_size=16,
                      layout=layout, out_dtype=torch.float32)
    dx, dw = Q.dequantize_mx(cx, sx, 16), Q.dequantize_mx(cw, sw, 16)
    if layout == "nhwc":
        dx, dw = dx.permute(0, 3, 1, 2), dw.permute(3, 2, 0, 1)
    want = F.conv2d(dx.float(), dw.float(), bias.float(), 1, 1)
    if layout == "nhwc":
        want = want.permute(0, 2, 3, 1)
    assert got.shape == want.shape and got.dtype == torch.float32
    assert float((got - want).abs().max()) <= 1e-3 * float(want.abs().max())
