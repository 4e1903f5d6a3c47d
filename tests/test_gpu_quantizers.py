"""Bit-exact parity of the CUDA quantizers with the reference (golden
fixtures) and with the CPU oracle, through the registered operators."""

import pytest
import torch

import cases as C
from golden_io import bits_equal, describe_mismatch, golden_cases, golden_tables
from oracle import quantizers as OQ
from oracle import tables as OT

pytestmark = pytest.mark.gpu

QUANTIZER_OPS = {"vmap", "quantize", "dequantize", "calculate_mx_qparam", "quantize_mx", "dequantize_mx",
                 "quantize_affine", "calculate_global_scale"}
_CASES = {k: v for k, v in golden_cases(OT.quantization_map).items() if v[0] in QUANTIZER_OPS}


def _impl():
    from cuda_impl import CudaImpl

    return CudaImpl


@pytest.mark.parametrize("name", sorted(_CASES))
def test_golden_case(name):
    op, args, kwargs, expected = _CASES[name]
    got = C.run_case(_impl(), op, args, kwargs)
    assert len(got) == len(expected)
    for i, (g, w) in enumerate(zip(got, expected)):
        assert bits_equal(g, w), f"{name} output {i}: " + describe_mismatch(g, w)


@pytest.mark.parametrize("name", sorted(golden_tables()))
def test_vmap_exhaustive(name):
    """Every bfloat16 input through every format: the kernel's rounding (an
    arithmetic form where the table is recognised) equals the reference table."""
    table = golden_tables()[name]
    got = _impl().vmap(OT.all_bf16(), table)
    assert bits_equal(got, table), describe_mismatch(got, table)


@pytest.mark.parametrize("name", ["int8", "fp8_e4m3", "fp4_e2m1", "lut4_to_int6", "posit8_1", "uint2"])
def test_vmap_exhaustive_f32_f16(name):
    table = golden_tables()[name]
    x32 = OT.all_bf16().float()
    x32 = torch.cat([x32, x32 * 1.001, x32 * 0.999])  # values between bf16 points round first
    got = _impl().vmap(x32, table)
    want = OQ.vmap(x32, table)
    assert bits_equal(got, want), describe_mismatch(got, want)
    x16 = OT.all_bf16().to(torch.float16)
    got = _impl().vmap(x16, table)
    want = OQ.vmap(x16, table)
    assert bits_equal(got, want), describe_mismatch(got, want)


@pytest.mark.parametrize("spec", [
    ("int8", 16, 127.0, True, None),
    ("int8", 32, 127.0, True, None),
    ("fp8_e4m3", 32, 448.0, True, None),
    ("fp4_e2m1", 16, 6.0, False, "fp8_e4m3"),
    ("lut4_to_int6", 64, 31.0, False, "fp8_e5m3"),
    ("int6", 64, 31.0, False, "fp8_e5m3"),
    ("posit8_1", 16, 4096.0, True, None),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quantize_mx_every_magnitude(spec, dtype):
    """Blocks whose amax sweeps every positive bfloat16 value (subnormals,
    infinities and NaN included) with mixed-sign contents."""
    name, bs, qmax, pot, scale_name = spec
    amax = OT.all_bf16()[: 0x8000].float()
    g = torch.Generator().manual_seed(5)
    body = (torch.rand(amax.numel(), bs, generator=g) * 2 - 1) * amax[:, None]
    body[:, 0] = amax
    x = body.to(dtype)
    table = OT.quantization_map(name)
    stable = None if scale_name is None else OT.quantization_map(scale_name)
    want = OQ.quantize_mx(x, table, [-1], bs, qmax, pot, stable)
    got = _impl().quantize_mx(x, table, [-1], bs, qmax, pot, stable)
    for i, (gg, ww) in enumerate(zip(got, want)):
        assert bits_equal(gg, ww), f"output {i}: " + describe_mismatch(gg, ww)


def test_quantize_mx_config1_shape():
    """MXINT8 at the benchmark's activation shape against the oracle."""
    x = C.randn(0, 2048, 4096, outliers=0.001)
    table = OT.quantization_map("int8")
    want = OQ.quantize_mx(x, table, [-1], 16, 127.0, True)
    got = _impl().quantize_mx(x, table, [-1], 16, 127.0, True)
    for gg, ww in zip(got, want):
        assert bits_equal(gg, ww), describe_mismatch(gg, ww)


def test_quantize_per_tensor_exhaustive():
    """Every bfloat16 input divided by awkward per-tensor scales."""
    x = OT.all_bf16()
    table = OT.quantization_map("fp8_e4m3")
    for s in (0.0123, 1.0, 3.3e-5, 7.7e3):
        scale = torch.tensor(s, dtype=torch.bfloat16)
        want = OQ.quantize(x, scale, qmap=table)
        got = _impl().quantize(x, scale, None, None, None, table)
        assert bits_equal(got, want), describe_mismatch(got, want)
        s32 = torch.tensor(s, dtype=torch.float32)
        want = OQ.quantize(x, s32, qmap=table)
        got = _impl().quantize(x, s32, None, None, None, table)
        assert bits_equal(got, want), describe_mismatch(got, want)


def test_empty_inputs():
    table = OT.quantization_map("int8")
    impl = _impl()
    assert impl.vmap(torch.empty(0, dtype=torch.bfloat16), table).shape == (0,)
    s, c = impl.quantize_mx(torch.empty(0, 32, dtype=torch.bfloat16), table, [-1], 16, 127.0, True)
    assert s.shape == (0, 2) and c.shape == (0, 32)


def test_cpu_tensors_have_no_kernel():
    import voyager_b200  # noqa: F401

    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.quantized_ops.vmap(torch.zeros(4, dtype=torch.bfloat16), OT.quantization_map("int8"))
