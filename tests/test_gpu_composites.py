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
