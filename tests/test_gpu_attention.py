"""The fused FP8 attention kernel against the sequence of kernels it replaces:
``fp8_gemm`` (Q K^T), ``softmax_quantize_fp8``, ``fp8_gemm`` (P V) and the cast of the context."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _vb():
    import voyager_b200 as vb
    return vb


def _operands(T, kv, groups, seed):
    g = torch.Generator().manual_seed(seed)
    d = 128
    q = torch.randn(kv, groups * T, d, generator=g).to(torch.float8_e4m3fn).view(torch.uint8).cuda()
    k = torch.randn(kv, T, d, generator=g).to(torch.float8_e4m3fn).view(torch.uint8).cuda()
    vt = torch.randn(kv, d, T, generator=g).to(torch.float8_e4m3fn).view(torch.uint8).cuda()
    return q, k, vt


def _separate(vb, q, k, vt, alpha_qk, score_scale, p_scale, alpha_pv, T):
    scores = vb.fp8.fp8_gemm(q, k, alpha_qk, causal=("scores", T))
    p8 = vb.fp8.softmax_quantize_fp8(scores, score_scale, p_scale, causal_period=T)
    return vb.fp8.fp8_gemm(p8, vt, alpha_pv, causal=("probabilities", T))


@pytest.mark.parametrize("T,kv,groups", [(128, 1, 1), (256, 2, 2), (384, 1, 3), (1024, 2, 4), (2048, 2, 2)])
def test_attention_matches_separate_kernels(T, kv, groups):
    vb = _vb()
    q, k, vt = _operands(T, kv, groups, T + kv + groups)
    alpha_qk = torch.tensor(0.37, dtype=torch.float32).cuda()
    alpha_pv = torch.tensor(1.0 / 448.0 * 0.9, dtype=torch.float32).cuda()
    p_scale = torch.tensor(1.0 / 448.0, dtype=torch.bfloat16).cuda()
    score_scale = 1.0 / math.sqrt(128)
    want = _separate(vb, q, k, vt, alpha_qk, score_scale, p_scale, alpha_pv, T).float()
    got = vb.fp8.attention_fp8(q, k, vt, alpha_qk, score_scale, p_scale, alpha_pv).float()
    assert vb.fp8.attention_status() == 0
    vb.ops.gemm_status()
    # a probability code differs by one step only at a rounding boundary: the contexts agree to
    # bfloat16 resolution almost everywhere
    err = (got - want).abs()
    assert float(err.max()) <= 1e-2 * float(want.abs().max())
    assert float((err > 0).float().mean()) < 0.05


@pytest.mark.parametrize("T,kv,groups", [(256, 2, 2), (1024, 2, 4)])
def test_attention_fp8_output_is_the_cast_of_the_context(T, kv, groups):
    vb = _vb()
    q, k, vt = _operands(T, kv, groups, 7 * T)
    alpha_qk = torch.tensor(0.2, dtype=torch.float32).cuda()
    alpha_pv = torch.tensor(1.0 / 448.0, dtype=torch.float32).cuda()
    p_scale = torch.tensor(1.0 / 448.0, dtype=torch.bfloat16).cuda()
    score_scale = 1.0 / math.sqrt(128)
    ctx = vb.fp8.attention_fp8(q, k, vt, alpha_qk, score_scale, p_scale, alpha_pv)
    ctx_scale = (ctx.float().abs().amax() / 448.0).to(torch.bfloat16)
    want = vb.fp8.transpose_heads_quantize_fp8(ctx.view(kv * groups, T, 128), ctx_scale)
    got = vb.fp8.attention_fp8(q, k, vt, alpha_qk, score_scale, p_scale, alpha_pv, ctx_scale)
    assert vb.fp8.attention_status() == 0
    assert torch.equal(got.view(want.shape), want.view(torch.uint8) if want.dtype != torch.uint8 else want)


def test_attention_is_deterministic_and_rejects_other_shapes():
    vb = _vb()
    q, k, vt = _operands(512, 2, 2, 3)
    a = torch.tensor(0.3, dtype=torch.float32).cuda()
    s = torch.tensor(1.0 / 448.0, dtype=torch.bfloat16).cuda()
    one = vb.fp8.attention_fp8(q, k, vt, a, 0.088, s, a)
    two = vb.fp8.attention_fp8(q, k, vt, a, 0.088, s, a)
    assert torch.equal(one, two)
    with pytest.raises(Exception):
        vb.fp8.attention_fp8(q[:, :, :64].contiguous(), k[:, :, :64].contiguous(), vt[:, :64].contiguous(), a, 0.088, s, a)


def test_attention_matches_a_torch_restatement():
    """Every step of the operator sequence written with torch ops on the dequantized codes."""
    vb = _vb()
    T, kv, groups, d = 256, 2, 2, 128
    q, k, vt = _operands(T, kv, groups, 11)
    alpha_qk, alpha_pv, sp, scale = 0.37, 0.9 / 448.0, 1.0 / 448.0, 1.0 / math.sqrt(d)
    f8 = lambda t: t.view(torch.float8_e4m3fn).float()
    scores = (torch.matmul(f8(q), f8(k).transpose(1, 2)) * alpha_qk).bfloat16()            # [kv, groups*T, T]
    s = (scores.float() * scale).bfloat16()
    pos = torch.arange(groups * T, device="cuda") % T
    s = s.float().masked_fill(torch.arange(T, device="cuda")[None, :] > pos[:, None], float("-inf"))
    p = torch.softmax(s, -1).bfloat16()
    p8 = (p.float() / torch.tensor(sp, dtype=torch.bfloat16).float()).bfloat16().to(torch.float8_e4m3fn)
    want = (torch.matmul(p8.float(), f8(vt).transpose(1, 2)) * alpha_pv).bfloat16().float()
    dev = lambda v, dt: torch.tensor(v, dtype=dt).cuda()
    got = vb.fp8.attention_fp8(q, k, vt, dev(alpha_qk, torch.float32), scale, dev(sp, torch.bfloat16),
                               dev(alpha_pv, torch.float32)).float()
    assert vb.fp8.attention_status() == 0
    assert float((got - want).abs().max()) <= 1e-2 * float(want.abs().max())
