"""Seeded parity cases shared by the fixture generator and the tests.

``build_cases(table)`` returns ``[(name, op, args, kwargs), ...]`` where
``table(dtype_name)`` supplies the 65 536-entry lookup table for a dtype
(the reference's own when generating fixtures, the oracle's or the product's
when checking).  All inputs come from a CPU ``torch.Generator`` and are also
stored in the fixture file, so the GPU box never depends on RNG agreement.

The shapes are small versions of the benchmark configurations (MXINT8 linear,
FP8 per-tensor layer, NF4 / KIVI decode, NVFP4 prefill, GPTQ) plus the edge
cases the reference handles explicitly: partial blocks, axes shorter than a
block, blocks along the second-to-last axis, two-axis blocks, all-zero and
subnormal blocks, infinities and NaNs, float32 inputs.
"""

import math

import numpy as np
import torch

BF16 = torch.bfloat16


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def randn(seed, *shape, std=1.0, dtype=BF16, outliers=0.0):
    g = _gen(seed)
    x = torch.randn(*shape, generator=g) * std
    if outliers:
        mask = torch.rand(*shape, generator=g) < outliers
        x = torch.where(mask, x * 20, x)
    return x.to(dtype)


def edge_blocks(dtype=BF16):
    """Rows of 16 that hit the power-of-two scale's corner cases."""
    rows = [
        torch.zeros(16),
        torch.full((16,), 2.0 ** -120),
        torch.full((16,), 2.0 ** -126),
        torch.full((16,), 2.0 ** -127),
        torch.full((16,), 2.0 ** -130),
        torch.full((16,), 2.0 ** -133),
        torch.linspace(-3, 3, 16),
        torch.tensor([float("inf")] + [1.0] * 15),
        torch.tensor([float("-inf")] + [0.5] * 15),
        torch.tensor([float("nan")] + [2.0] * 15),
        torch.tensor([3.0e38, -3.0e38] + [1.0] * 14),
        torch.tensor([127.0, 127.5, 128.0, 63.5, -63.5, 0.5, 1.5, 2.5, -2.5, -0.0, 0.0, 1e-3, 7.0, 96.0, -96.0, 100.0]),
    ]
    return torch.stack(rows).to(dtype)


def build_cases(table):
    cases = []

    def add(name, op, *args, **kwargs):
        cases.append((name, op, list(args), dict(kwargs)))

    int8, int6, int4 = table("int8"), table("int6"), table("int4")
    e4m3, e5m2, e5m3, e8m0 = table("fp8_e4m3"), table("fp8_e5m2"), table("fp8_e5m3"), table("fp8_e8m0")
    e2m1, posit8 = table("fp4_e2m1"), table("posit8_1")
    nf4 = table("lut4_to_int6")
    uint2, uint4 = table("uint2"), table("uint4")
    nf4_levels = torch.unique(nf4)
    nf4_index = torch.searchsorted(nf4_levels, nf4).to(torch.int64)
    nf4_mid = (nf4_levels[:-1] + nf4_levels[1:]) / 2

    # ---- vmap ---------------------------------------------------------
    add("vmap_int8_bf16", "vmap", randn(1, 33, 70, std=40.0), int8)
    add("vmap_e4m3_f32", "vmap", randn(2, 5, 129, std=100.0, dtype=torch.float32), e4m3)
    add("vmap_index_table", "vmap", randn(3, 257, std=10.0), nf4_index)
    add("vmap_e2m1_f16", "vmap", randn(4, 19, 64, std=2.0, dtype=torch.float16), e2m1)

    # ---- quantize_mx, power-of-two scales -----------------------------
    x_c1 = randn(10, 64, 256, outliers=0.001)
    add("mx_int8_pot_c1", "quantize_mx", x_c1, int8, [-1], 16, 127.0, True)
    add("mx_int8_pot_weight", "quantize_mx", randn(11, 48, 128, std=0.02), int8, [-1], 16, 127.0, True)
    add("mx_int8_pot_edges", "quantize_mx", edge_blocks(), int8, [-1], 16, 127.0, True)
    add("mx_int8_pot_edges_f32", "quantize_mx", edge_blocks(torch.float32), int8, [-1], 16, 127.0, True)
    add("mx_int8_pot_partial", "quantize_mx", randn(12, 3, 40), int8, [-1], 16, 127.0, True)
    add("mx_int8_pot_short", "quantize_mx", randn(13, 3, 8), int8, [-1], 16, 127.0, True)
    add("mx_int8_pot_axis2", "quantize_mx", randn(14, 2, 48, 40), int8, [-2], 16, 127.0, True)
    add("mx_int8_pot_axis2_partial", "quantize_mx", randn(15, 2, 37, 24), int8, [-2], 16, 127.0, True)
    add("mx_int6_pot_2axis", "quantize_mx", randn(16, 1, 2, 128, 128), int6, [-2, -1], 64, 31.0, True)
    add("mx_int6_2axis_e5m3", "quantize_mx", randn(17, 1, 2, 128, 192), int6, [-2, -1], 64, 31.0, False, e5m3)
    add("mx_e4m3_pot_bs32", "quantize_mx", randn(18, 32, 128, std=3.0), e4m3, [-1], 32, 448.0, True)
    add("mx_e2m1_pot_bs32", "quantize_mx", randn(19, 32, 128, std=3.0), e2m1, [-1], 32, 6.0, True)
    add("mx_posit8_pot", "quantize_mx", randn(20, 16, 64, std=5.0), posit8, [-1], 16, 4096.0, True)
    add("mx_int8_pot_f32", "quantize_mx", randn(21, 16, 64, dtype=torch.float32), int8, [-1], 16, 127.0, True)
    add("mx_int8_pot_f16", "quantize_mx", randn(22, 16, 64, dtype=torch.float16), int8, [-1], 16, 127.0, True)
    add("mx_int8_pot_3d", "quantize_mx", randn(23, 2, 5, 96), int8, [-1], 16, 127.0, True)

    # ---- quantize_mx, table scales ------------------------------------
    x_nf = randn(30, 32, 256, outliers=0.002)
    add("mx_nf4_e5m3_values", "quantize_mx", x_nf, nf4, [-1], 64, 31.0, False, e5m3)
    add("mx_nf4_e5m3_index", "quantize_mx", x_nf, nf4_index, [-1], 64, 31.0, False, e5m3, nf4_mid)
    add("mx_nf4_e5m3_codebook", "quantize_mx", x_nf, nf4_levels, [-1], 64, 31.0, False, e5m3, nf4_mid)
    add("mx_nf4_e5m3_weight", "quantize_mx", randn(31, 24, 192, std=0.02), nf4, [-1], 64, 31.0, False, e5m3)
    add("mx_e4m3_e8m0_table", "quantize_mx", randn(32, 16, 128), e4m3, [-1], 32, 448.0, False, e8m0)
    add("mx_int4_noscalemap", "quantize_mx", randn(33, 16, 128), int4, [-1], 32, 7.0, False, None)
    add("mx_nf4_e5m3_edges", "quantize_mx", edge_blocks(), nf4, [-1], 16, 31.0, False, e5m3)
    x_nv = randn(34, 32, 128, outliers=0.002)
    t_nv = (x_nv.abs().amax() / (6.0 * 448.0)).clamp_min(torch.finfo(torch.float32).tiny)
    add("mx_nvfp4_global", "quantize_mx", x_nv, e2m1, [-1], 16, 6.0, False, e4m3, None, None, t_nv)
    w_nv = randn(35, 48, 64, std=0.02)
    t_w = (w_nv.abs().amax() / (6.0 * 448.0)).clamp_min(torch.finfo(torch.float32).tiny)
    add("mx_nvfp4_global_weight", "quantize_mx", w_nv, e2m1, [-1], 16, 6.0, False, e4m3, None, None, t_w)
    add("mx_nvfp4_global_f32", "quantize_mx", x_nv.float(), e2m1, [-1], 16, 6.0, False, e4m3, None, None, t_nv.float())
    add("mx_nvfp4_2axis", "quantize_mx", w_nv, e2m1, [-2, -1], 16, 6.0, False, e4m3, None, None, t_w)
    add("mx_nvfp4_zero", "quantize_mx", torch.zeros(4, 32, dtype=BF16), e2m1, [-1], 16, 6.0, False, e4m3, None, None,
        torch.tensor(torch.finfo(torch.float32).tiny, dtype=BF16))

    # ---- stochastic rounding -------------------------------------------
    seed = torch.tensor(123456789012345, dtype=torch.int64)
    add("mx_nvfp4_sr", "quantize_mx", x_nv, e2m1, [-1], 16, 6.0, False, e4m3, None, seed, t_nv)
    add("mx_int8_sr", "quantize_mx", randn(36, 7, 48), int8, [-1], 16, 127.0, True, None, None, seed)
    add("quantize_sr_per_tensor", "quantize", randn(37, 5, 33, std=3.0), torch.tensor(0.05, dtype=BF16), None, None,
        None, e4m3, None, seed)

    # ---- calculate_mx_qparam -------------------------------------------
    add("qparam_pot", "calculate_mx_qparam", x_c1, [-1], 16, 127.0, True)
    add("qparam_e5m3", "calculate_mx_qparam", x_nf, [-1], 64, 31.0, False, e5m3)
    add("qparam_global", "calculate_mx_qparam", x_nv, [-1], 16, 6.0, False, e4m3, t_nv)

    # ---- quantize / dequantize ------------------------------------------
    x_pt = randn(40, 2, 64, 96, std=1.5, outliers=0.001)
    s_pt = (x_pt.abs().amax() / 448.0)
    add("quantize_per_tensor_e4m3", "quantize", x_pt, s_pt, None, None, None, e4m3)
    add("quantize_per_tensor_1elem", "quantize", x_pt, s_pt.reshape(1), None, None, None, e4m3)
    add("quantize_per_tensor_e5m2", "quantize", x_pt, s_pt, None, None, None, e5m2)
    add("quantize_per_tensor_int8_f32", "quantize", x_pt.float(), (x_pt.float().abs().amax() / 127.0), None, None,
        None, int8)
    w_pc = randn(41, 48, 64, std=0.02)
    s_pc = w_pc.abs().amax(1, keepdim=True) / 448.0
    add("quantize_per_channel_e4m3", "quantize", w_pc, s_pc, None, None, None, e4m3)
    add("quantize_per_channel_last", "quantize", w_pc, (w_pc.abs().amax(0) / 127.0), None, None, None, int8)
    add("quantize_no_qmap", "quantize", x_pt, s_pt)
    add("quantize_block_scale", "quantize", x_c1, (x_c1.reshape(64, 16, 16).abs().amax(-1) / 127.0).clamp_min(1e-3),
        None, [-1], 16, int8)
    zp = torch.full((64, 16), 3.0, dtype=BF16)
    add("quantize_block_zp", "quantize", x_c1, torch.full((64, 16), 0.25, dtype=BF16), zp, [-1], 16, uint4)
    add("quantize_codebook", "quantize", x_nf, torch.tensor(0.1, dtype=BF16), None, None, None, nf4_levels)
    add("quantize_codebook_bounds", "quantize", x_nf, torch.tensor(0.1, dtype=BF16), None, None, None, nf4_levels,
        nf4_mid)
    heads = torch.stack([nf4_levels.float() * f for f in (1.0, 0.5, 2.0, 1.5)]).reshape(1, 4, 1, 1, 16)
    x_h = randn(42, 2, 4, 6, 32, std=10.0)
    add("quantize_codebook_per_head", "quantize", x_h, torch.tensor(1.0, dtype=BF16), None, None, None, heads)

    y_pt = randn(43, 2, 32, 80, std=200.0)
    add("dequantize_per_tensor_outmap", "dequantize", y_pt, torch.tensor(0.00037, dtype=BF16), None, None, None, None,
        table(None))
    add("dequantize_per_tensor_plain", "dequantize", y_pt, torch.tensor(0.00037, dtype=BF16))
    add("dequantize_per_channel", "dequantize", y_pt, randn(44, 80, std=0.01).abs() + 0.001)
    add("dequantize_input_map", "dequantize", y_pt, torch.tensor(0.5, dtype=BF16), None, None, None, e4m3, None)
    add("dequantize_f32", "dequantize", y_pt.float(), torch.tensor(0.00037))

    # ---- KIVI: group-wise affine ------------------------------------------
    k_cache = randn(50, 1, 2, 128, 64)
    v_cache = randn(51, 1, 2, 128, 64)
    add("affine_k_uint2_e4m3", "quantize_affine", k_cache, uint2, [-2], 64, 0.0, 3.0, e4m3)
    add("affine_v_uint2_e4m3", "quantize_affine", v_cache, uint2, [-1], 64, 0.0, 3.0, e4m3)
    add("affine_k_uint2_e5m3", "quantize_affine", k_cache, uint2, [-2], 64, 0.0, 3.0, e5m3)
    add("affine_v_uint2_e5m3", "quantize_affine", v_cache, uint2, [-1], 64, 0.0, 3.0, e5m3)
    add("affine_uint4_noscalemap", "quantize_affine", randn(52, 8, 256, std=0.02), uint4, [-1], 128, 0.0, 15.0, None)
    add("affine_partial", "quantize_affine", randn(53, 3, 40) + 2.0, uint4, [-1], 16, 0.0, 15.0, None)
    add("affine_const_block", "quantize_affine", torch.full((2, 32), 0.75, dtype=BF16), uint2, [-1], 16, 0.0, 3.0, e4m3)
    add("affine_f32", "quantize_affine", randn(54, 4, 64, dtype=torch.float32), uint4, [-1], 32, 0.0, 15.0, None)

    # dequantize with zero point + blocks + re-encode (KIVI fused read)
    codes = torch.randint(0, 4, (1, 2, 128, 64), generator=_gen(55)).to(BF16)
    sc = (randn(56, 1, 2, 2, 64).abs() * 0.3 + 0.05)
    zpk = torch.randint(0, 4, (1, 2, 2, 64), generator=_gen(57)).to(BF16)
    add("dequantize_kivi_k", "dequantize", codes, sc, zpk, [-2], 64)
    add("dequantize_kivi_k_reencode", "dequantize", codes, sc, zpk, [-2], 64, None, e4m3)
    scv = (randn(58, 1, 2, 128, 1).abs() * 0.3 + 0.05)
    zpv = torch.randint(0, 4, (1, 2, 128, 1), generator=_gen(59)).to(BF16)
    add("dequantize_kivi_v", "dequantize", codes, scv, zpv, [-1], 64)

    # ---- dequantize_mx -------------------------------------------------------
    idx = torch.randint(0, 16, (8, 128), generator=_gen(60)).to(BF16)
    sc_mx = (randn(61, 8, 2).abs() + 0.01)
    add("dequantize_mx_code", "dequantize_mx", idx, sc_mx, 64, nf4_levels)
    add("dequantize_mx_code_global", "dequantize_mx", idx, sc_mx, 64, nf4_levels, torch.tensor(0.0123, dtype=BF16))
    add("dequantize_mx_plain", "dequantize_mx", randn(62, 8, 128, std=30).round(), sc_mx, 64)

    # ---- GEMMs -----------------------------------------------------------------
    xa, wa = randn(70, 32, 128, outliers=0.001), randn(71, 48, 128, std=0.02)
    add("linear_mx_int8", "linear_mx_chain", xa, wa, None, spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True))
    add("linear_mx_int8_bias", "linear_mx_chain", xa, wa, randn(72, 48, std=0.1),
        spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True))
    add("linear_mx_int8_batched", "linear_mx_chain", randn(73, 2, 9, 64), randn(74, 24, 64, std=0.02), None,
        spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True))
    add("linear_mx_nf4", "linear_mx_chain", xa, wa, None,
        spec=dict(qmap=nf4_index, bs=64, qmax=31.0, pot=False, scale_qmap=e5m3, bounds=nf4_mid, code=nf4_levels))
    add("linear_mx_nvfp4", "linear_mx_chain", xa, wa, randn(75, 48, std=0.1),
        spec=dict(qmap=e2m1, bs=16, qmax=6.0, pot=False, scale_qmap=e4m3, global_scale=(6.0, 448.0)))
    add("linear_mx_int8_kx", "linear_mx_chain", xa, wa, None,
        spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True, layout="xc,kc->kx"))
    add("linear_mx_int8_f32out", "linear_mx_chain", xa, wa, None,
        spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True, out_dtype=torch.float32))
    add("matmul_mx_int8", "matmul_mx_chain", randn(76, 2, 3, 16, 64), randn(77, 2, 3, 64, 24),
        spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True))
    add("matmul_mx_nf4", "matmul_mx_chain", randn(78, 2, 16, 128), randn(79, 2, 128, 32),
        spec=dict(qmap=nf4_index, bs=64, qmax=31.0, pot=False, scale_qmap=e5m3, bounds=nf4_mid, code=nf4_levels))

    # ---- per-tensor FP8 linear (quantize -> aten.linear -> dequantize) ---------
    add("fp8_linear_chain", "fp8_linear_chain", randn(80, 24, 96, std=1.2, outliers=0.002), randn(81, 40, 96, std=0.02),
        spec=dict(qmap=e4m3, qmax=448.0, out_map=table(None)))

    # ---- global scale ------------------------------------------------------------
    add("global_scale_bf16", "calculate_global_scale", x_nv, 6.0, 448.0)
    add("global_scale_zero", "calculate_global_scale", torch.zeros(4, 4, dtype=BF16), 6.0, 448.0)
    add("global_scale_f32", "calculate_global_scale", x_nv.float(), 6.0, 448.0)

    # ---- Hadamard / transpose ---------------------------------------------------
    add("hadamard_last", "hadamard_rotate", randn(85, 3, 8, 40), -1, "hadamard")
    add("hadamard_rows", "hadamard_rotate", randn(86, 3, 24, 8), -2, "hadamard")
    add("mx_transpose_nvfp4", "quantize_mx_transpose", randn(87, 32, 48), e2m1, 16, 6.0, False, e4m3, None, None,
        torch.tensor(0.002, dtype=BF16), None, torch.tensor(0.002, dtype=BF16), "hadamard")

    # ---- attention ------------------------------------------------------------------
    add("sdpa_mx_int8", "sdpa_mx_chain", randn(88, 1, 4, 16, 32), randn(89, 1, 2, 32, 32), randn(90, 1, 2, 32, 32),
        spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True))

    # ---- GPTQ --------------------------------------------------------------------------
    def hess(seed, tokens, k, rank):
        g = _gen(seed)
        x = 0.7 * torch.randn(tokens, k, generator=g) + 0.3 * (
            torch.randn(tokens, rank, generator=g) @ torch.randn(rank, k, generator=g)) / math.sqrt(rank)
        return x.T @ x, tokens

    h1, t1 = hess(95, 512, 128, 8)
    w1 = randn(96, 32, 128, std=0.02, dtype=torch.float32)
    add("gptq_nf4_e5m3", "gptq", w1, h1, t1,
        spec=dict(qmap=nf4, scale_qmap=e5m3, qmax=31.0, bs=64, damping=0.01, act_order=False, shrink=False))
    add("gptq_nf4_e5m3_shrink", "gptq", w1, h1, t1,
        spec=dict(qmap=nf4, scale_qmap=e5m3, qmax=31.0, bs=64, damping=0.01, act_order=False, shrink=True))
    add("gptq_nf4_e5m3_actorder", "gptq", w1, h1, t1,
        spec=dict(qmap=nf4, scale_qmap=e5m3, qmax=31.0, bs=64, damping=0.01, act_order=True, shrink=False))
    add("gptq_int4_bs32", "gptq", w1, h1, t1,
        spec=dict(qmap=int4, scale_qmap=e5m3, qmax=7.0, bs=32, damping=0.01, act_order=False, shrink=False))
    h2, t2 = hess(97, 96, 160, 4)  # rank-deficient -> damping escalation; partial last block
    add("gptq_partial_block", "gptq", randn(98, 16, 160, std=0.02, dtype=torch.float32), h2, t2,
        spec=dict(qmap=nf4, scale_qmap=e5m3, qmax=31.0, bs=64, damping=0.01, act_order=False, shrink=False))

    # ---- fake-quant ops (quantization/ops.py) --------------------------------------------
    xf = randn(120, 6, 48, 64, std=1.5, outliers=0.002)
    add("fq_tensor_e4m3", "fake_quant", xf, e4m3, torch.tensor(0.011, dtype=BF16))
    add("fq_tensor_f32_scale", "fake_quant", xf, int8, torch.tensor(0.0437, dtype=torch.float32))
    add("fq_channel_int8", "fake_quant", randn(121, 40, 96, std=0.02),
        int8, (randn(122, 40, 1, std=1.0).abs() * 4e-4 + 1e-4))
    add("fq_f32_input", "fake_quant", randn(123, 5, 77, dtype=torch.float32), int6, torch.tensor(0.09))
    add("gwa_uint4_bs32", "group_wise_affine_fake_quant", randn(124, 3, 16, 128), [-1], 32, 0.0, 15.0, None)
    add("gwa_uint2_rows_e5m3", "group_wise_affine_fake_quant", randn(125, 1, 2, 128, 64), [-2], 64, 0.0, 3.0, e5m3)
    add("gwa_partial_block", "group_wise_affine_fake_quant", randn(126, 5, 40), [-1], 16, 0.0, 255.0, None)
    add("gwa_edges", "group_wise_affine_fake_quant", edge_blocks(), [-1], 16, 0.0, 15.0, e5m3)
    add("mxfq_int8_pot", "mx_fake_quant", xf, int8, [-1], 16, 127.0, True, None, None, None, None, None)
    add("mxfq_e2m1_e4m3_global", "mx_fake_quant", xf, e2m1, [-1], 16, 6.0, False, e4m3, None,
        torch.tensor(0.0021, dtype=BF16), None, None)
    add("mxfq_nf4_e5m3_rows", "mx_fake_quant", randn(127, 2, 128, 48), nf4, [-2], 64, 31.0, False, e5m3, None, None,
        None, None)
    add("mxfq_hadamard", "mx_fake_quant", randn(128, 3, 8, 40), e2m1, [-1], 16, 6.0, False, e4m3, None,
        torch.tensor(0.002, dtype=BF16), "hadamard", -1)
    add("mxfq_edges", "mx_fake_quant", edge_blocks(), int8, [-1], 16, 127.0, True, None, None, None, None, None)
    add("mxfq_stochastic", "mx_fake_quant", randn(129, 4, 64, std=3.0), torch.arange(-7.0, 8.0).to(BF16), [-1], 16, 7.0,
        True, None, torch.tensor(1234, dtype=torch.int64), None, None, None)
    add("hadamard_amax_last", "hadamard_amax", randn(130, 3, 8, 40), -1, "hadamard")
    add("hadamard_amax_rows", "hadamard_amax", randn(131, 3, 24, 8), -2, "hadamard")

    # ---- delayed-scaling observer (fake_quantize.py:406-437): a sequence of inputs through one module ----
    seq = torch.stack([randn(140 + i, 6, 32, std=0.5 * (i + 1)) for i in range(5)])
    add("observer_tensor_e4m3", "amax_observer", seq, "fp8_e4m3", 448.0, 3, None, False)
    add("observer_tensor_int8_pow2", "amax_observer", seq, "int8", 127.0, 2, None, True)
    add("observer_channel_e4m3", "amax_observer", seq, "fp8_e4m3", 448.0, 4, 0, False)
    zeros_first = seq.clone()
    zeros_first[0] = 0
    zeros_first[2, 0, 0] = float("inf")
    add("observer_zero_and_inf", "amax_observer", zeros_first, "fp8_e4m3", 448.0, 2, None, False)

    # ---- outlier side stream (ops/quantized.py:1286-1644) ------------------------------------
    xo = randn(150, 2, 24, 64, outliers=0.02)
    add("outlier_filter", "filter_outlier", xo, 6.0, 0.05)
    add("outlier_filter_overflow", "filter_outlier", xo, 2.0, 0.02)          # more outliers than capacity
    add("outlier_filter_f32_2d", "filter_outlier", randn(151, 16, 40, dtype=torch.float32, outliers=0.03), 5.0, 0.1)
    add("outlier_quantize_mx", "quantize_mx_outlier", xo, int8, [-1], 16, 127.0, True, None, None, 6.0, 0.05, 3)
    add("outlier_slice_rows", "slice_csr_chain", xo[0], 6.0, 0.05, 0, 5, 17, 1.0)
    add("outlier_slice_cols", "slice_csr_chain", xo[0], 6.0, 0.05, 1, 16, 48, 0.5)
    add("outlier_spmm_kc", "spmm_chain", xo, randn(152, 40, 64, std=0.05), "kc", spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True))
    add("outlier_spmm_ck", "spmm_chain", xo[0], randn(153, 64, 40, std=0.05), "ck", spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True))
    add("outlier_linear_mx", "linear_mx_outlier_chain", randn(154, 48, 128, outliers=0.01), randn(155, 72, 128, std=0.02),
        spec=dict(qmap=int8, bs=16, qmax=127.0, pot=True, threshold=6.0, max_pct=0.03))
    return cases


# ----------------------------------------------------------------------------
# running a case against an implementation of the ops
# ----------------------------------------------------------------------------
def run_case(impl, op, args, kwargs):
    """Run one case.  ``impl`` exposes the reference's op names as attributes
    (``vmap``, ``quantize``, ``quantize_mx``, ``linear_mx`` ...).  Returns a
    tuple of tensors."""
    spec = kwargs.get("spec")
    args = [impl.hadamard_matrix() if isinstance(a, str) and a == "hadamard" else a for a in args]

    def qmx(x, axes=(-1,)):
        gs = None
        if "global_scale" in spec:
            gs = impl.calculate_global_scale(x, *spec["global_scale"])
        s, c = impl.quantize_mx(x, spec["qmap"], list(axes), spec["bs"], spec["qmax"], spec["pot"],
                                spec.get("scale_qmap"), spec.get("bounds"), None, gs)
        return s, c, gs

    if op == "linear_mx_chain":
        x, w, bias = args
        sx, cx, gx = qmx(x)
        sw, cw, gw = qmx(w)
        alpha = None if gx is None else gx * gw
        extra = {k: spec[k] for k in ("layout", "out_dtype") if k in spec}
        y = impl.linear_mx(cx, cw, bias, input_scale=sx, weight_scale=sw, block_size=spec["bs"],
                           input_code=spec.get("code"), weight_code=spec.get("code"), alpha=alpha, **extra)
        return sx, cx, sw, cw, y
    if op == "matmul_mx_chain":
        a, b = args
        sa, ca, _ = qmx(a, (-1,))
        sb, cb, _ = qmx(b, (-2,))
        y = impl.matmul_mx(ca, cb, input_scale=sa, weight_scale=sb, block_size=spec["bs"],
                           input_code=spec.get("code"), weight_code=spec.get("code"))
        return sa, ca, sb, cb, y
    if op == "sdpa_mx_chain":
        q, k, v = args
        sq, cq, _ = qmx(q, (-1,))
        sk, ck, _ = qmx(k, (-1,))
        sv, cv, _ = qmx(v, (-2,))
        y = impl.sdpa_mx(cq, ck, cv, None, 0.0, True, enable_gqa=True, query_scale=sq, key_scale=sk,
                         value_scale=sv, block_size=spec["bs"], probs_qmap=spec["qmap"],
                         probs_quant_max=spec["qmax"], force_scale_power_of_two=spec["pot"])
        return (y,)
    if op == "fp8_linear_chain":
        x, w = args
        sa = x.abs().amax() / spec["qmax"]
        sw = w.abs().amax() / spec["qmax"]
        cx = impl.quantize(x, sa, None, None, None, spec["qmap"])
        cw = impl.quantize(w, sw, None, None, None, spec["qmap"])
        y = impl.dense_linear(cx, cw)
        out = impl.dequantize(y, sa * sw, None, None, None, None, spec["out_map"])
        return cx, cw, y, out
    if op == "slice_csr_chain":
        x, threshold, max_pct, dim, start, end, size_factor = args
        data, indices, indptr, _ = impl.filter_outlier(x, threshold, max_pct)
        return tuple(impl.slice_csr_tensor(data, indices, indptr, dim, start, end, size_factor))
    if op == "spmm_chain":
        x, w, weight_layout = args
        data, indices, indptr, _ = impl.filter_outlier(x, 6.0, 0.05)
        sw, cw, _ = qmx(w, (-1,) if weight_layout == "kc" else (-2,))
        return (impl.spmm_csr(data, indices, indptr, cw, sw, None, spec["bs"], weight_layout, out_dtype=torch.float32),)
    if op == "linear_mx_outlier_chain":
        x, w = args
        data, indices, indptr, sx, cx = impl.quantize_mx_outlier(x, spec["qmap"], [-1], spec["bs"], spec["qmax"],
                                                                  spec["pot"], None, None, spec["threshold"],
                                                                  spec["max_pct"])
        sw, cw, _ = qmx(w)
        y = impl.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=spec["bs"], A_data=data,
                           A_indices=indices, A_indptr=indptr)
        return data, indices, indptr, sx, cx, y
    if op == "gptq":
        w, h, tokens = args
        return (impl.compensate_weight(w, h.clone(), tokens, spec["qmap"], spec["scale_qmap"], spec["qmax"],
                                       spec["bs"], spec["damping"], spec["act_order"], True, spec["shrink"]),)
    out = getattr(impl, op)(*args)
    return tuple(out) if isinstance(out, (tuple, list)) else (out,)


# ----------------------------------------------------------------------------
# (de)serialisation: tensors as numpy arrays, bfloat16 as its uint16 bits
# ----------------------------------------------------------------------------
def to_numpy(t):
    if t.dtype == BF16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16), "bf16"
    if t.dtype == torch.float16:
        return t.contiguous().numpy(), "f16"
    return t.contiguous().numpy(), str(t.dtype).replace("torch.", "")


def from_numpy(a, tag):
    if tag == "bf16":
        return torch.from_numpy(a.view(np.int16).copy()).view(BF16)
    return torch.from_numpy(a.copy())
