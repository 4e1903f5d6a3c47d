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


# ---------------------------------------------------------------------------
# bfloat16 operands: the eager attention of a graph whose attention matmuls are not quantized
# ---------------------------------------------------------------------------
def _eager_bf16_attention(q, k, v, round_scores=True):
    """matmul -> scale + mask -> softmax -> matmul on bfloat16 tensors (float32 accumulation, every node's
    output rounded to bfloat16), computed per KV group in float64-free plain torch."""
    T, heads, d = q.shape
    kv = k.shape[1]
    groups = heads // kv
    mask = torch.full((T, T), float("-inf"), device=q.device).triu(1)
    qg = q.reshape(T, kv, groups, d).permute(1, 2, 0, 3).float()
    scores = torch.matmul(qg, k.permute(1, 2, 0)[:, None].float())
    if round_scores:
        scores = scores.bfloat16().float()
    s = (scores * (1.0 / d ** 0.5) + mask).bfloat16().float()
    p = torch.softmax(s, -1).bfloat16().float()
    ctx = torch.matmul(p, v.transpose(0, 1)[:, None].float()).bfloat16()
    return ctx.permute(2, 0, 1, 3).reshape(T, heads * d)


@pytest.mark.parametrize("T,kv,groups", [(128, 1, 1), (256, 2, 2), (384, 1, 4), (1024, 2, 4), (2048, 8, 4)])
@pytest.mark.parametrize("round_acc", [True, False])
def test_attention_bf16_matches_the_eager_graph(T, kv, groups, round_acc):
    from voyager_b200 import fp8 as F8

    g = torch.Generator().manual_seed(T + kv + groups)
    q = (torch.randn(T, kv * groups, 128, generator=g) * 1.5).bfloat16().cuda()
    k = (torch.randn(T, kv, 128, generator=g) * 1.5).bfloat16().cuda()
    v = torch.randn(T, kv, 128, generator=g).bfloat16().cuda()
    got = F8.attention_bf16(q, k, v, round_acc=round_acc)
    assert F8.attention_status() == 0
    want = _eager_bf16_attention(q, k, v, round_scores=round_acc)
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    diff = (got.float() - want.float()).abs()
    # probabilities that sit on a bfloat16 rounding boundary may flip by one step (ex2.approx against expf, the
    # row sum in another order); the context then differs by at most a few of its own rounding steps
    assert float(diff.max()) <= 2e-2 * float(want.float().abs().max()), float(diff.max())
    assert float(diff.pow(2).mean().sqrt()) <= 2e-3 * float(want.float().pow(2).mean().sqrt())
    assert float((got != want).float().mean()) <= 0.25
    again = F8.attention_bf16(q, k, v, round_acc=round_acc)
    assert torch.equal(got, again)


def test_attention_bf16_first_rows_are_exact():
    """Row 0 attends to key 0 only: p = 1 and the context is v[0], bit for bit."""
    from voyager_b200 import fp8 as F8

    g = torch.Generator().manual_seed(3)
    q = torch.randn(256, 4, 128, generator=g).bfloat16().cuda()
    k = torch.randn(256, 2, 128, generator=g).bfloat16().cuda()
    v = torch.randn(256, 2, 128, generator=g).bfloat16().cuda()
    got = F8.attention_bf16(q, k, v).reshape(256, 4, 128)
    assert F8.attention_status() == 0
    for h in range(4):
        assert torch.equal(got[0, h], v[0, h // 2])


def test_attention_bf16_rejects_other_shapes():
    from voyager_b200 import fp8 as F8

    q = torch.zeros(100, 2, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        F8.attention_bf16(q, q, q)
    q = torch.zeros(128, 2, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        F8.attention_bf16(q, q, q)


def test_rope_heads_bf16_equals_the_elementwise_graph():
    """One kernel against x * cos + rotate_half(x) * sin on bfloat16 tensors, bit for bit, from a strided slice of a
    merged projection, written head-major."""
    from voyager_b200 import fp8 as F8
    from voyager_b200.workloads import apply_rope

    g = torch.Generator().manual_seed(6)
    T, heads, kv, d = 256, 8, 2, 128
    qkv = torch.randn(T, (heads + 2 * kv) * d, generator=g).bfloat16().cuda()
    cos = torch.randn(T, d, generator=g).bfloat16().cuda()
    sin = torch.randn(T, d, generator=g).bfloat16().cuda()
    for lo, n in ((0, heads), (heads * d, kv)):
        x = qkv[:, lo:lo + n * d].unflatten(1, (n, d))
        got = F8.rope_heads_bf16(x, cos, sin)
        want = apply_rope(x, cos, sin).permute(1, 0, 2)
        assert got.shape == (n, T, d) and torch.equal(got, want)


def test_attention_bf16_heads_is_attention_bf16_on_prepared_operands():
    from voyager_b200 import fp8 as F8

    g = torch.Generator().manual_seed(8)
    T = 384
    q = torch.randn(T, 8, 128, generator=g).bfloat16().cuda()
    k = torch.randn(T, 2, 128, generator=g).bfloat16().cuda()
    v = torch.randn(T, 2, 128, generator=g).bfloat16().cuda()
    a = F8.attention_bf16(q, k, v)
    b = F8.attention_bf16_heads(q.permute(1, 0, 2).contiguous(), k.permute(1, 0, 2).contiguous(),
                                v.permute(1, 2, 0).contiguous())
    assert F8.attention_status() == 0
    assert torch.equal(a, b)
