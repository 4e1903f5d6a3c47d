"""The tensor-core GEMM and the microscaling linear / matmul built on it.

Codes and scales feeding the GEMM must be bit-exact; the product is compared
with the reference's dequantize-then-fp32-matmul within 1e-2 of the largest
output (the stated tolerance for accumulation-order differences), and with an
fp64 product of the same bf16 operands within 2e-5 when the output is fp32.
"""

import pytest
import torch

import cases as C
from golden_io import bits_equal, describe_mismatch, golden_cases
from oracle import gemm as OG
from oracle import quantizers as OQ
from oracle import tables as OT

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2
_CASES = {k: v for k, v in golden_cases(OT.quantization_map).items()
          if v[0] in ("linear_mx_chain", "matmul_mx_chain")}


def _impl():
    from cuda_impl import CudaImpl

    return CudaImpl


def _status():
    import voyager_b200

    voyager_b200.ops.gemm_status()


def rel_err(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("name", sorted(_CASES))
def test_mx_gemm_golden(name):
    op, args, kwargs, expected = _CASES[name]
    got = C.run_case(_impl(), op, args, kwargs)
    _status()
    for i in range(4):
        assert bits_equal(got[i], expected[i]), f"{name} output {i}: " + describe_mismatch(got[i], expected[i])
    assert got[4].shape == expected[4].shape and got[4].dtype == expected[4].dtype
    assert rel_err(got[4], expected[4]) <= REL_TOL, rel_err(got[4], expected[4])


@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (16, 256, 64), (100, 264, 72), (128, 256, 4096), (300, 1000, 520),
                                   (257, 513, 136), (2048, 512, 256)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_shapes(m, n, k, out_dtype):
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = torch.randn(n, k, generator=g).bfloat16()
    bias = torch.randn(n, generator=g).bfloat16()
    want = (a.double() @ b.double().T + bias.double())
    got = _impl().linear(a, b, bias, out_dtype=out_dtype)
    _status()
    assert got.dtype == out_dtype and got.shape == (m, n)
    tol = 2e-5 if out_dtype == torch.float32 else 4e-3
    assert rel_err(got, want) <= tol, rel_err(got, want)


def test_gemm_batched_and_alpha():
    g = torch.Generator().manual_seed(3)
    a = torch.randn(3, 2, 70, 96, generator=g).bfloat16()
    b = torch.randn(3, 2, 96, 40, generator=g).bfloat16()  # [K, N]: matmul layout
    got = _impl().matmul(a, b, out_dtype=torch.float32)
    _status()
    want = a.double() @ b.double()
    assert got.shape == (3, 2, 70, 40)
    assert rel_err(got, want) <= 2e-5
    # kx output and f16 operands
    a16, b16 = a[0, 0].half(), b[0, 0].half()
    got = _impl().matmul(a16, b16, layout="xc,ck->kx")
    _status()
    assert got.shape == (40, 70) and got.dtype == torch.float16
    assert rel_err(got, (a16.double() @ b16.double()).T) <= 2e-3


def test_linear_mx_config1_shape():
    """MXINT8 linear at the benchmark shape against the oracle's fp32 product."""
    x = C.randn(0, 2048, 4096, outliers=0.001)
    w = C.randn(1, 4096, 4096, std=0.02)
    table = OT.quantization_map("int8")
    impl = _impl()
    sx, cx = impl.quantize_mx(x, table, [-1], 16, 127.0, True)
    sw, cw = impl.quantize_mx(w, table, [-1], 16, 127.0, True)
    y = impl.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=16)
    _status()
    want = OG.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=16)
    assert y.dtype == torch.bfloat16 and y.shape == (2048, 4096)
    assert rel_err(y, want) <= REL_TOL, rel_err(y, want)
    y32 = impl.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=16, out_dtype=torch.float32)
    a = OQ.decode_and_scale(cx, sx, None, 16).double()
    b = OQ.decode_and_scale(cw, sw, None, 16).double()
    assert rel_err(y32, a @ b.T) <= 2e-5
