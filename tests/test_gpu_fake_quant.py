"""The fake-quant operators (``torch.ops.quantization.*``) against the reference's own CPU
outputs (golden fixtures), bit for bit, and their straight-through gradients."""

import pytest
import torch

import cases as C
from golden_io import bits_equal, describe_mismatch, golden_cases
from oracle import tables as OT

pytestmark = pytest.mark.gpu

FAKE_QUANT_OPS = {"fake_quant", "group_wise_affine_fake_quant", "mx_fake_quant", "hadamard_amax", "amax_observer"}
_CASES = {k: v for k, v in golden_cases(OT.quantization_map).items() if v[0] in FAKE_QUANT_OPS}


def _impl():
    from cuda_impl import CudaImpl

    return CudaImpl


@pytest.mark.parametrize("name", sorted(_CASES))
def test_golden_case(name):
    op, args, kwargs, expected = _CASES[name]
    got = C.run_case(_impl(), op, args, kwargs)
    assert len(got) == len(expected)
    for i, (g, w) in enumerate(zip(got, expected)):
        assert g.shape == w.shape and g.dtype == w.dtype, f"{name} output {i}: {g.shape} {g.dtype}"
        assert bits_equal(g, w), f"{name} output {i}: " + describe_mismatch(g, w)


def test_straight_through_gradients():
    import voyager_b200  # noqa: F401

    FQ = torch.ops.quantization
    table = OT.quantization_map("int8").cuda()
    x = torch.randn(6, 40, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = FQ.mx_fake_quant(x, table, [-1], 16, 127.0, True, None, None, None, None, None)
    g = torch.randn_like(y)
    y.backward(g)
    assert torch.equal(x.grad, g)
    # a rotation pads the axis to whole runs of 16; the gradient drops the padding
    x2 = torch.randn(3, 8, 40, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    h = voyager_b200.ops.hadamard_matrix("cuda")
    y2 = FQ.mx_fake_quant(x2, table, [-1], 16, 127.0, True, None, None, None, h, -1)
    assert y2.shape == (3, 8, 48)
    g2 = torch.randn_like(y2)
    y2.backward(g2)
    assert torch.equal(x2.grad, g2[..., :40])
    x3 = torch.randn(4, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out, scale, zp = FQ.group_wise_affine_fake_quant(x3, [-1], 32, 0.0, 15.0, None)
    assert not scale.requires_grad and not zp.requires_grad
    out.sum().backward()
    assert torch.equal(x3.grad, torch.ones_like(x3))
