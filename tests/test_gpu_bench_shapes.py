"""Parity at the shapes the benchmark runs (Llama-3.1-8B layer, 2048 tokens), against the
CPU oracle and against torch restatements of the operator sequence -- never against the
package's own kernels."""

import math

import pytest
import torch

from oracle import layers as OL

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn


def _vb():
    import voyager_b200

    return voyager_b200


def rel_err(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def test_fp8_decoder_layer_llama8b_2048_tokens_matches_converted_graph():
    """The benchmark's c2 step itself: LLAMA_8B, T=2048, merged QKV, fused attention (32 heads),
    SwiGLU-epilogue GEMM 2048x28672x4096, residual epilogues -- against the converted-graph
    semantics computed by the CPU oracle on the same seeded input."""
    vb = _vb()
    W = vb.workloads
    shape, T = W.LLAMA_8B, 2048
    params = W.make_layer_params(7, shape)
    x = W.make_hidden_states(100, T, shape)
    scales = W.calibrate_fp8_scales(x, params, shape)
    want = OL.fp8_decoder_layer(x, params, scales, shape, W.rope_tables(T, shape, "cpu"), W.causal_mask(T, "cpu"))
    layer = W.Fp8DecoderLayer({k: v.cuda() for k, v in params.items()}, {k: v.cuda() for k, v in scales.items()}, shape)
    assert layer.fuse_attention and layer.LAUNCHES == 10
    got = layer(x.cuda()).cpu()
    vb.ops.gemm_status()
    assert vb.fp8.attention_status() == 0
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    # The graph rounds each GEMM to bfloat16 before its scale; the FP8 GEMM rounds once after it.
    assert rel_err(got, want) <= 2e-2, rel_err(got, want)
    rms = float((got.double() - want.double()).pow(2).mean().sqrt() / want.double().pow(2).mean().sqrt())
    assert rms <= 1e-2, rms


def attention_restatement(q, k, vt, alpha_qk, score_scale, p_scale, alpha_pv, T, groups):
    """Every step of the operator sequence (Q K^T GEMM rounded to bfloat16, scale, causal mask, float32
    softmax rounded to bfloat16, e4m3 cast of the probabilities, P V GEMM rounded to bfloat16) written
    with torch ops on the decoded FP8 bytes, one KV head at a time."""
    f8 = lambda t: t.view(E4M3).float()
    out = []
    pos = torch.arange(groups * T, device=q.device) % T
    masked = torch.arange(T, device=q.device)[None, :] > pos[:, None]
    sp = torch.tensor(p_scale, dtype=torch.bfloat16, device=q.device).float()
    for h in range(q.shape[0]):
        scores = (torch.matmul(f8(q[h]), f8(k[h]).t()) * alpha_qk).bfloat16()
        s = (scores.float() * score_scale).bfloat16().float().masked_fill(masked, float("-inf"))
        p = torch.softmax(s, -1).bfloat16()
        p8 = (p.float() / sp).bfloat16().to(E4M3)
        out.append((torch.matmul(p8.float(), f8(vt[h]).t()) * alpha_pv).bfloat16())
    return torch.stack(out)


def test_attention_fp8_at_the_benchmark_shape_matches_a_torch_restatement():
    """8 KV heads x 4 query heads each x 2048 tokens x 128: the launch the c2 layer makes."""
    vb = _vb()
    T, kv, groups, d = 2048, 8, 4, 128
    g = torch.Generator().manual_seed(5)
    q = torch.randn(kv, groups * T, d, generator=g).to(E4M3).view(torch.uint8).cuda()
    k = torch.randn(kv, T, d, generator=g).to(E4M3).view(torch.uint8).cuda()
    vt = torch.randn(kv, d, T, generator=g).to(E4M3).view(torch.uint8).cuda()
    alpha_qk, alpha_pv, sp, scale = 0.37, 0.9 / 448.0, 1.0 / 448.0, 1.0 / math.sqrt(d)
    want = attention_restatement(q, k, vt, alpha_qk, scale, sp, alpha_pv, T, groups).float()
    dev = lambda v, dt: torch.tensor(v, dtype=dt).cuda()
    got = vb.fp8.attention_fp8(q, k, vt, dev(alpha_qk, torch.float32), scale, dev(sp, torch.bfloat16),
                               dev(alpha_pv, torch.float32)).float()
    assert vb.fp8.attention_status() == 0
    err = (got - want).abs()
    assert float(err.max()) <= 1e-2 * float(want.abs().max()), float(err.max())
    # a probability code moves by one FP8 step only where a value sits on a rounding boundary
    assert float((err > 0).float().mean()) < 0.05


def test_gated_fp8_gemm_2048x28672x4096_matches_fp64():
    """The merged gate/up projection with the SwiGLU + cast epilogue (the roofline kernel of c2)
    against a float64 product of the decoded bytes followed by the graph's rounding steps."""
    vb = _vb()
    FP8 = vb.fp8
    T, K, I = 2048, 4096, 14336
    g = torch.Generator().manual_seed(9)
    a = torch.randn(T, K, generator=g).to(E4M3).cuda()
    wg = (torch.randn(I, K, generator=g) * 0.5).to(E4M3).cuda()
    wu = (torch.randn(I, K, generator=g) * 0.5).to(E4M3).cuda()
    alpha_g = (torch.rand(I, generator=g) * 0.02 + 0.01).cuda()     # one float32 factor per output column
    alpha_u = (torch.rand(I, generator=g) * 0.02 + 0.01).cuda()
    w = FP8.interleave_gate_up(wg.view(torch.uint8), wu.view(torch.uint8))
    cols = FP8.interleave_gate_up(alpha_g, alpha_u)
    gate_ref = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
    up_ref = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
    a64 = a.double()
    for lo in range(0, I, 2048):                                      # float64 in slices: bounded memory
        hi = min(I, lo + 2048)
        gate_ref[:, lo:hi] = (a64 @ wg[lo:hi].double().t() * alpha_g[lo:hi].double()).to(torch.bfloat16)
        up_ref[:, lo:hi] = (a64 @ wu[lo:hi].double().t() * alpha_u[lo:hi].double()).to(torch.bfloat16)
    act = torch.nn.functional.silu(gate_ref) * up_ref                 # bf16(bf16(silu(g)) * u)
    s_act = (act.float().abs().amax() / 448.0).to(torch.bfloat16)
    want = (act / s_act).float().clamp(-448, 448).to(E4M3).float()    # e4m3(bf16(a / s))
    got = FP8.fp8_gemm(a.view(torch.uint8), w, alpha_cols=cols, gated_scale=s_act)
    vb.ops.gemm_status()
    assert got.shape == (T, I) and got.dtype == torch.uint8
    got = got.view(E4M3).float()
    diff = (got - want).abs()
    # the float32 accumulation order differs from float64: a value on a bfloat16 rounding boundary may
    # move, and with it the code by one FP8 step
    step = torch.maximum(want.abs(), got.abs()) * 0.126 + 2.0 ** -9
    assert bool((diff <= step).all()), float(diff.max())
    assert float((diff > 0).float().mean()) < 1e-2, float((diff > 0).float().mean())


def test_merged_qkv_and_residual_gemms_at_the_benchmark_shape_match_fp64():
    """[2048,4096] x [6144,4096]^T with per-column scales, and [2048,14336] x [4096,14336]^T with
    the residual added after the rounding."""
    vb = _vb()
    FP8 = vb.fp8
    g = torch.Generator().manual_seed(10)
    a = torch.randn(2048, 4096, generator=g).to(E4M3).cuda()
    w = (torch.randn(6144, 4096, generator=g) * 0.5).to(E4M3).cuda()
    cols = (torch.rand(6144, generator=g) * 0.02 + 0.01).cuda()
    want = (a.double() @ w.double().t()) * cols.double()
    got = FP8.fp8_gemm(a.view(torch.uint8), w.view(torch.uint8), alpha_cols=cols, out_dtype=torch.float32)
    vb.ops.gemm_status()
    assert rel_err(got, want) <= 2e-5, rel_err(got, want)
    a = torch.randn(2048, 14336, generator=g).to(E4M3).cuda()
    w = (torch.randn(4096, 14336, generator=g) * 0.5).to(E4M3).cuda()
    res = torch.randn(2048, 4096, generator=g).bfloat16().cuda()
    alpha = torch.tensor(0.003, dtype=torch.bfloat16).cuda()
    y = ((a.double() @ w.double().t()) * alpha.double()).to(torch.bfloat16)
    want = (res + y).float()
    got = FP8.fp8_gemm(a.view(torch.uint8), w.view(torch.uint8), alpha, residual=res).float()
    vb.ops.gemm_status()
    diff = (got - want).abs()
    assert float(diff.max()) <= 2.0 ** -7 * float(want.abs().max())      # one bfloat16 step of the largest value
    assert float((diff > 0).float().mean()) < 1e-2
