"""The outlier side stream (filter_outlier, quantize_mx_outlier, slice_csr_tensor, spmm_csr and the
outlier arguments of linear_mx) against the reference's CPU outputs: CSR structure and quantizer
outputs bit for bit, products within the GEMM tolerance."""

import pytest
import torch

import cases as C
from golden_io import bits_equal, describe_mismatch, golden_cases
from oracle import tables as OT

pytestmark = pytest.mark.gpu

OPS = {"filter_outlier", "quantize_mx_outlier", "slice_csr_chain", "spmm_chain", "linear_mx_outlier_chain"}
_CASES = {k: v for k, v in golden_cases(OT.quantization_map).items() if v[0] in OPS}


def _impl():
    from cuda_impl import CudaImpl

    return CudaImpl


@pytest.mark.parametrize("name", sorted(_CASES))
def test_golden_case(name):
    op, args, kwargs, expected = _CASES[name]
    got = C.run_case(_impl(), op, args, kwargs)
    assert len(got) == len(expected)
    for i, (g, w) in enumerate(zip(got, expected)):
        assert g.shape == w.shape and g.dtype == w.dtype, f"{name} output {i}: {g.shape} {g.dtype} vs {w.shape} {w.dtype}"
        product = (op == "spmm_chain") or (op == "linear_mx_outlier_chain" and i == len(expected) - 1)
        if product:
            err = (g.double() - w.double()).abs().max() / w.double().abs().max().clamp_min(1e-30)
            assert float(err) <= 1e-2, f"{name} output {i}: relative error {float(err):.3e}"
        else:
            assert bits_equal(g, w), f"{name} output {i}: " + describe_mismatch(g, w)


def test_filter_outlier_is_graph_capturable():
    import voyager_b200  # noqa: F401

    Q = torch.ops.quantized_ops
    x = torch.randn(2, 32, 64, device="cuda", dtype=torch.bfloat16) * 3
    want = Q.filter_outlier(x, 6.0, 0.1)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got = Q.filter_outlier(x, 6.0, 0.1)
    graph.replay()
    torch.cuda.synchronize()
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    # nothing lost: inlier + scattered outliers give the input back
    data, indices, indptr, inlier = [t.cpu() for t in got]
    rebuilt = inlier.clone()
    for b in range(2):
        for r in range(32):
            for e in range(int(indptr[b, r]), int(indptr[b, r + 1])):
                rebuilt[b, r, int(indices[b, e])] = data[b, e]
    assert torch.equal(rebuilt, x.cpu())
