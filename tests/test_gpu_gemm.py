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


# ---------------------------------------------------------------------------
# Block scales applied inside the GEMM's main loop (vq_gemm_mx): the same operands, tiles and
# summation order as dequantize-then-GEMM, so the two must agree bit for bit.
# ---------------------------------------------------------------------------
def _mx_problem(batch, m, n, k, bs, seed, scaled=("a", "b"), batched_weight=False):
    import voyager_b200

    g = torch.Generator().manual_seed(seed)
    table = voyager_b200.get_quantization_map("int8").cuda()
    a = torch.randn(*batch, m, k, generator=g).bfloat16().cuda()
    b = (torch.randn(*(batch if batched_weight else ()), n, k, generator=g) * 0.05).bfloat16().cuda()
    q = torch.ops.quantized_ops.quantize_mx
    sa, ca = q(a, table, [-1], bs, 127.0, True) if "a" in scaled else (None, a)
    sb, cb = q(b, table, [-1], bs, 127.0, True) if "b" in scaled else (None, b)
    return ca, sa, cb, sb


@pytest.mark.parametrize("batch,m,n,k,bs", [
    ((), 300, 200, 264, 8), ((), 129, 8, 64, 32), ((), 2048, 4096, 4096, 32), ((), 1000, 520, 200, 32),
    ((), 512, 384, 1024, 16), ((), 640, 256, 512, 64), ((), 257, 136, 768, 128), ((), 384, 640, 1024, 256),
    ((3,), 200, 264, 128, 32), ((2, 2), 160, 96, 320, 16),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_mx_gemm_in_mainloop_equals_dequantize_then_gemm(batch, m, n, k, bs, out_dtype, monkeypatch):
    import voyager_b200
    from voyager_b200 import ops

    monkeypatch.setattr(ops, "MX_IN_MAINLOOP", "always")
    ca, sa, cb, sb = _mx_problem(batch, m, n, k, bs, seed=m + n + k + bs)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    alpha = torch.tensor(0.75, device="cuda")
    got = torch.ops.quantized_ops.linear_mx(ca, cb, bias, input_scale=sa, weight_scale=sb, block_size=bs,
                                            alpha=alpha, out_dtype=out_dtype)
    da = ops._decode_and_scale(ca, sa, None, bs)
    db = ops._decode_and_scale(cb, sb, None, bs)
    want = ops.gemm_tn(da, db, out_dtype=out_dtype, alpha=alpha, bias=bias)
    _status()
    assert got.shape == want.shape and got.dtype == want.dtype
    assert torch.equal(got, want), describe_mismatch(got.cpu(), want.cpu())
    ref = 0.75 * (da.double() @ db.double().mT) + bias.double()
    assert rel_err(got, ref) <= (2e-5 if out_dtype == torch.float32 else REL_TOL)


@pytest.mark.parametrize("scaled", [("a",), ("b",)])
def test_mx_gemm_in_mainloop_one_scaled_operand(scaled, monkeypatch):
    from voyager_b200 import ops

    monkeypatch.setattr(ops, "MX_IN_MAINLOOP", "always")
    ca, sa, cb, sb = _mx_problem((), 384, 320, 512, 32, seed=5, scaled=scaled)
    got = torch.ops.quantized_ops.linear_mx(ca, cb, None, input_scale=sa, weight_scale=sb, block_size=32)
    want = ops.gemm_tn(ops._read_operand(ca, sa, None, 32), ops._read_operand(cb, sb, None, 32))
    _status()
    assert torch.equal(got, want)


def test_mx_gemm_in_mainloop_batched_weight(monkeypatch):
    from voyager_b200 import ops

    monkeypatch.setattr(ops, "MX_IN_MAINLOOP", "always")
    ca, sa, cb, sb = _mx_problem((4,), 256, 192, 128, 32, seed=9, batched_weight=True)
    got = ops._mx_gemm_in_mainloop(ops.LINEAR_LAYOUT, ca, cb, None, sa, sb, 32, None, ops.LINEAR_LAYOUT, torch.bfloat16)
    assert got is not None
    want = ops.gemm_tn(ops._decode_and_scale(ca, sa, None, 32), ops._decode_and_scale(cb, sb, None, 32))
    _status()
    assert torch.equal(got, want)


@pytest.mark.parametrize("m", [1, 16, 100, 128])
def test_mx_gemm_in_mainloop_few_rows(m, monkeypatch):
    """At most 128 rows: the second CTA of each pair multiplies zero padding; the result is the same."""
    from voyager_b200 import ops

    monkeypatch.setattr(ops, "MX_IN_MAINLOOP", "always")
    ca, sa, cb, sb = _mx_problem((), m, 520, 1024, 32, seed=m)
    got = torch.ops.quantized_ops.linear_mx(ca, cb, None, input_scale=sa, weight_scale=sb, block_size=32,
                                            out_dtype=torch.float32)
    da, db = ops._decode_and_scale(ca, sa, None, 32), ops._decode_and_scale(cb, sb, None, 32)
    _status()
    assert rel_err(got, da.double() @ db.double().T) <= 2e-5


def test_mx_gemm_in_mainloop_is_the_path_a_weight_bound_linear_mx_takes(monkeypatch):
    """A K-contiguous block-scaled bfloat16 linear whose read-back would cost more than the transform warps do
    launches no read-back kernel; a compute-bound one keeps the read-back."""
    from voyager_b200 import ops

    calls = []
    real = ops._decode_and_scale
    monkeypatch.setattr(ops, "_decode_and_scale", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    ca, sa, cb, sb = _mx_problem((), 256, 4096, 1024, 32, seed=2)
    torch.ops.quantized_ops.linear_mx(ca, cb, None, input_scale=sa, weight_scale=sb, block_size=32)
    assert not calls
    ca, sa, cb, sb = _mx_problem((), 4096, 4096, 1024, 32, seed=3)
    torch.ops.quantized_ops.linear_mx(ca, cb, None, input_scale=sa, weight_scale=sb, block_size=32)
    assert len(calls) == 2
    assert not ops._in_mainloop_pays(2048, 4096, 4096, 1, True, True, True)
    assert ops._in_mainloop_pays(16, 4096, 4096, 1, True, True, True)
