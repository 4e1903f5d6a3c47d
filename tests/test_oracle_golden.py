"""The CPU oracle against the reference's own outputs (committed fixtures)."""

import pytest
import torch

import cases as C
from golden_io import bits_equal, describe_mismatch, golden_cases, golden_tables
from oracle import fake_quant as fq_oracle
from oracle import observers as obs_oracle
from oracle import outliers as out_oracle
from oracle import gemm, gptq, quantizers, tables


class OracleImpl:
    vmap = staticmethod(quantizers.vmap)
    quantize = staticmethod(quantizers.quantize)
    dequantize = staticmethod(quantizers.dequantize)
    calculate_mx_qparam = staticmethod(quantizers.calculate_mx_qparam)
    quantize_mx = staticmethod(quantizers.quantize_mx)
    dequantize_mx = staticmethod(quantizers.dequantize_mx)
    quantize_affine = staticmethod(quantizers.quantize_affine)
    calculate_global_scale = staticmethod(quantizers.calculate_global_scale)
    hadamard_rotate = staticmethod(quantizers.hadamard_rotate)
    hadamard_matrix = staticmethod(quantizers.hadamard_matrix)
    quantize_mx_transpose = staticmethod(quantizers.quantize_mx_transpose)
    linear_mx = staticmethod(gemm.linear_mx)
    matmul_mx = staticmethod(gemm.matmul_mx)
    sdpa_mx = staticmethod(gemm.sdpa_mx)
    dense_linear = staticmethod(torch.nn.functional.linear)
    compensate_weight = staticmethod(gptq.compensate_weight)
    fake_quant = staticmethod(fq_oracle.fake_quant)
    group_wise_affine_fake_quant = staticmethod(fq_oracle.group_wise_affine_fake_quant)
    mx_fake_quant = staticmethod(fq_oracle.mx_fake_quant)
    hadamard_amax = staticmethod(fq_oracle.hadamard_amax)
    amax_observer = staticmethod(obs_oracle.amax_observer)
    filter_outlier = staticmethod(out_oracle.filter_outlier)
    quantize_mx_outlier = staticmethod(out_oracle.quantize_mx_outlier)
    slice_csr_tensor = staticmethod(out_oracle.slice_csr_tensor)
    spmm_csr = staticmethod(out_oracle.spmm_csr)


@pytest.mark.parametrize("name", sorted(golden_tables()))
def test_table_matches_reference(name):
    want = golden_tables()[name]
    got = tables.quantization_map(name)
    assert bits_equal(got, want), describe_mismatch(got, want)


_CASES = golden_cases(tables.quantization_map)


@pytest.mark.parametrize("name", sorted(_CASES))
def test_oracle_case(name):
    op, args, kwargs, expected = _CASES[name]
    got = C.run_case(OracleImpl, op, args, kwargs)
    assert len(got) == len(expected)
    for i, (g, w) in enumerate(zip(got, expected)):
        assert bits_equal(g, w), f"{name} output {i}: " + describe_mismatch(g, w)
