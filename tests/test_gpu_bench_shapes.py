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


def _stats(got, want):
    """(largest difference over the largest magnitude, rms difference over rms, fraction of differing elements)."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    d = (got - want).abs()
    return (float(d.max() / want.abs().max()), float(d.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()),
            float((d > 0).float().mean()))


def test_fp8_decoder_layer_llama8b_2048_tokens_matches_converted_graph():
    """The benchmark's c2 step itself: LLAMA_8B, T=2048, merged QKV, fused attention (32 heads),
    SwiGLU-epilogue GEMM 2048x28672x4096, residual epilogues -- against the converted-graph
    semantics computed by the CPU oracle on the same seeded input.

    Two statements.  (1) Kernel by kernel, each fed the *oracle's* tensor for its input, the
    outputs are the oracle's up to float32 summation order: codes differ on at most 0.1 % of
    elements.  (2) End to end the difference is what that noise becomes after the layer's five
    FP8 re-quantizations (a code that flips moves a value by up to 1/8): about 1 % rms."""
    vb = _vb()
    W, FP8 = vb.workloads, vb.fp8
    shape, T = W.LLAMA_8B, 2048
    params = W.make_layer_params(7, shape)
    x = W.make_hidden_states(100, T, shape)
    scales = W.calibrate_fp8_scales(x, params, shape)
    rec = {}
    want = OL.fp8_decoder_layer(x, params, scales, shape, W.rope_tables(T, shape, "cpu"), W.causal_mask(T, "cpu"),
                                record=rec.__setitem__)
    s = {k: v.cuda() for k, v in scales.items()}
    layer = W.Fp8DecoderLayer({k: v.cuda() for k, v in params.items()}, s, shape)
    assert layer.fuse_attention and layer.LAUNCHES == 8 and layer.ra
    got = layer(x.cuda())
    vb.ops.gemm_status()
    assert vb.fp8.attention_status() == 0
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    worst, rms, _ = _stats(got, want)
    assert worst <= 6e-2 and rms <= 2e-2, (worst, rms)

    # ---- kernel by kernel on the oracle's own intermediates
    sh, d = shape, shape.head_dim
    codes = lambda t: t.float().to(E4M3).view(torch.uint8).cuda()          # bfloat16-valued codes -> FP8 bytes
    values = lambda b: b.view(E4M3).float()
    xd = x.cuda()
    (cos, sin), _ = layer._tables(T, xd.device)
    h8 = FP8.rmsnorm_quantize_fp8(xd, layer.ln1, sh.eps, s["h"])
    assert _stats(values(h8), rec["h8"])[2] <= 1e-4
    qkv = FP8.fp8_gemm(codes(rec["h8"]), layer.w8_qkv, alpha_cols=layer.alpha_qkv, round_acc=True)
    nq, nkv = sh.heads * d, sh.kv_heads * d
    for name, lo, hi, heads in (("q_lin", 0, nq, sh.heads), ("k_lin", nq, nq + nkv, sh.kv_heads),
                                ("v_lin", nq + nkv, nq + 2 * nkv, sh.kv_heads)):
        worst, rms, frac = _stats(qkv[:, lo:hi].reshape(T, heads, d), rec[name])
        assert frac <= 1e-3 and worst <= 1e-2, (name, worst, rms, frac)
    q8 = FP8.rope_quantize_fp8(rec["q_lin"].cuda(), cos, sin, s["q"])
    k8 = FP8.rope_quantize_fp8(rec["k_lin"].cuda(), cos, sin, s["k"])
    vt8 = FP8.transpose_quantize_fp8(rec["v_lin"].cuda(), s["v"])
    for name, got8 in (("q8", q8), ("k8", k8), ("v8", vt8)):
        assert _stats(values(got8), rec[name])[2] <= 1e-3, name
    ctx8 = FP8.attention_fp8(codes(rec["q8"]).view(sh.kv_heads, sh.groups * T, d), codes(rec["k8"]), codes(rec["v8"]),
                             layer.alpha_qk, 1.0 / math.sqrt(d), s["p"], layer.alpha_pv, s["ctx"], round_acc=True)
    assert vb.fp8.attention_status() == 0
    worst, rms, frac = _stats(values(ctx8), rec["ctx8"])
    assert frac <= 5e-3 and rms <= 5e-3, ("ctx8", worst, rms, frac)
    x1 = FP8.fp8_gemm(codes(rec["ctx8"]), layer.w8["o"], layer.alpha["o"], residual=xd, round_acc=True)
    worst, rms, frac = _stats(x1, rec["x1"])
    assert frac <= 1e-2 and rms <= 1e-3 and worst <= 1e-2, ("x1", worst, rms, frac)
    h28 = FP8.rmsnorm_quantize_fp8(rec["x1"].cuda(), layer.ln2, sh.eps, s["h2"])
    assert _stats(values(h28), rec["h28"])[2] <= 1e-4
    act8 = FP8.fp8_gemm(codes(rec["h28"]), layer.w8_swiglu, alpha_cols=layer.alpha_swiglu, gated_scale=s["act"],
                        round_acc=True)
    worst, rms, frac = _stats(values(act8), rec["act8"])
    assert frac <= 1e-3 and rms <= 2e-3, ("act8", worst, rms, frac)
    out = FP8.fp8_gemm(codes(rec["act8"]), layer.w8["down"], layer.alpha["down"], residual=rec["x1"].cuda(),
                       round_acc=True)
    worst, rms, frac = _stats(out, want)
    assert frac <= 1e-2 and rms <= 1e-3 and worst <= 1e-2, ("out", worst, rms, frac)
    vb.ops.gemm_status()


def attention_restatement(q, k, vt, alpha_qk, score_scale, p_scale, alpha_pv, T, groups, round_acc=False):
    """Every step of the operator sequence (Q K^T GEMM rounded to bfloat16, scale, causal mask, float32
    softmax rounded to bfloat16, e4m3 cast of the probabilities, P V GEMM rounded to bfloat16) written
    with torch ops on the decoded FP8 bytes, one KV head at a time.  ``round_acc``: each product is
    rounded to bfloat16 before its scale is applied (matmul, then dequantize)."""
    f8 = lambda t: t.view(E4M3).float()
    first = (lambda t: t.bfloat16().float()) if round_acc else (lambda t: t)
    out = []
    pos = torch.arange(groups * T, device=q.device) % T
    masked = torch.arange(T, device=q.device)[None, :] > pos[:, None]
    sp = torch.tensor(p_scale, dtype=torch.bfloat16, device=q.device).float()
    for h in range(q.shape[0]):
        scores = (first(torch.matmul(f8(q[h]), f8(k[h]).t())) * alpha_qk).bfloat16()
        s = (scores.float() * score_scale).bfloat16().float().masked_fill(masked, float("-inf"))
        p = torch.softmax(s, -1).bfloat16()
        p8 = (p.float() / sp).bfloat16().to(E4M3)
        out.append((first(torch.matmul(p8.float(), f8(vt[h]).t())) * alpha_pv).bfloat16())
    return torch.stack(out)


@pytest.mark.parametrize("round_acc", [False, True])
def test_attention_fp8_at_the_benchmark_shape_matches_a_torch_restatement(round_acc):
    """8 KV heads x 4 query heads each x 2048 tokens x 128: the launch the c2 layer makes."""
    vb = _vb()
    T, kv, groups, d = 2048, 8, 4, 128
    g = torch.Generator().manual_seed(5)
    q = torch.randn(kv, groups * T, d, generator=g).to(E4M3).view(torch.uint8).cuda()
    k = torch.randn(kv, T, d, generator=g).to(E4M3).view(torch.uint8).cuda()
    vt = torch.randn(kv, d, T, generator=g).to(E4M3).view(torch.uint8).cuda()
    alpha_qk, alpha_pv, sp, scale = 0.37, 0.9 / 448.0, 1.0 / 448.0, 1.0 / math.sqrt(d)
    want = attention_restatement(q, k, vt, alpha_qk, scale, sp, alpha_pv, T, groups, round_acc).float()
    dev = lambda v, dt: torch.tensor(v, dtype=dt).cuda()
    got = vb.fp8.attention_fp8(q, k, vt, dev(alpha_qk, torch.float32), scale, dev(sp, torch.bfloat16),
                               dev(alpha_pv, torch.float32), round_acc=round_acc).float()
    assert vb.fp8.attention_status() == 0
    err = (got - want).abs()
    assert float(err.max()) <= 1e-2 * float(want.abs().max()), float(err.max())
    # a probability code moves by one FP8 step only where a value sits on a rounding boundary
    assert float((err > 0).float().mean()) < 0.05


@pytest.mark.parametrize("round_acc", [False, True])
def test_gated_fp8_gemm_2048x28672x4096_matches_fp64(round_acc):
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
    first = (lambda t: t.to(torch.bfloat16).double()) if round_acc else (lambda t: t)
    for lo in range(0, I, 2048):                                      # float64 in slices: bounded memory
        hi = min(I, lo + 2048)
        gate_ref[:, lo:hi] = (first(a64 @ wg[lo:hi].double().t()) * alpha_g[lo:hi].double()).to(torch.bfloat16)
        up_ref[:, lo:hi] = (first(a64 @ wu[lo:hi].double().t()) * alpha_u[lo:hi].double()).to(torch.bfloat16)
    act = torch.nn.functional.silu(gate_ref) * up_ref                 # bf16(bf16(silu(g)) * u)
    s_act = (act.float().abs().amax() / 448.0).to(torch.bfloat16)
    want = (act / s_act).float().clamp(-448, 448).to(E4M3).float()    # e4m3(bf16(a / s))
    got = FP8.fp8_gemm(a.view(torch.uint8), w, alpha_cols=cols, gated_scale=s_act, round_acc=round_acc)
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
