"""Real-FP8 path: the cast's bytes encode exactly the codes the table quantizer
yields, the FP8 GEMM matches an fp64 product of the decoded bytes, and the FP8
decoder layer tracks the converted-graph semantics (oracle) within the
per-tensor-FP8 tolerance."""

import pytest
import torch

from oracle import layers as OL
from oracle import quantizers as OQ
from oracle import tables as OT

pytestmark = pytest.mark.gpu


def _vb():
    import voyager_b200

    return voyager_b200


def rel_err(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("dtype,torch_dtype", [("fp8_e4m3", torch.float8_e4m3fn), ("fp8_e5m2", torch.float8_e5m2)])
def test_fp8_cast_bytes_are_the_table_codes(dtype, torch_dtype):
    vb = _vb()
    table = OT.quantization_map(dtype)
    x = torch.cat([OT.all_bf16(), OT.all_bf16().flip(0)])  # every bf16 value, twice
    x = torch.where(torch.isnan(x), torch.zeros_like(x), x)
    for s in (1.0, 0.0123, 3.3e-5, 7.7e3):
        for sdt in (torch.bfloat16, torch.float32):
            scale = torch.tensor(s, dtype=sdt)
            want = OQ.quantize(x, scale, qmap=table)
            got = vb.fp8.quantize_fp8(x.cuda(), scale.cuda(), dtype).cpu()
            decoded = got.view(torch_dtype).float()
            assert torch.equal(decoded, want.float()), (dtype, s, sdt)
            # -0 never appears from a -0 input; tiny negatives keep their sign, as in the table
            assert torch.equal(torch.signbit(decoded), torch.signbit(want.float()))


def test_fp8_cast_per_row_scales():
    vb = _vb()
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(48, 64, generator=g) * 0.02).bfloat16()
    s = (w.abs().amax(1, keepdim=True) / 448.0)
    want = OQ.quantize(w, s, qmap=OT.quantization_map("fp8_e4m3"))
    got = vb.fp8.quantize_fp8(w.cuda(), s.cuda()).cpu().view(torch.float8_e4m3fn).float()
    assert torch.equal(got, want.float())


@pytest.mark.parametrize("m,n,k,batch", [(64, 48, 128, 1), (300, 520, 272, 1), (256, 128, 2048, 3), (130, 2048, 128, 2)])
def test_fp8_gemm(m, n, k, batch):
    vb = _vb()
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(batch, m, k, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(batch, n, k, generator=g).to(torch.float8_e4m3fn)
    alpha = torch.tensor(0.37, dtype=torch.bfloat16)
    want = torch.matmul(a.double(), b.double().transpose(-1, -2)) * float(alpha)
    got = vb.fp8.fp8_gemm(a.view(torch.uint8).cuda(), b.view(torch.uint8).cuda(), alpha.cuda(),
                          out_dtype=torch.float32).cpu()
    vb.ops.gemm_status()
    assert got.shape == (batch, m, n)
    assert rel_err(got, want) <= 2e-5, rel_err(got, want)


def test_fp8_decoder_layer_matches_converted_graph():
    vb = _vb()
    W = vb.workloads
    shape = W.TINY
    T = 64
    params = W.make_layer_params(0, shape)
    x = W.make_hidden_states(1, T, shape)
    scales = W.calibrate_fp8_scales(x, params, shape)
    want = OL.fp8_decoder_layer(x, params, scales, shape, W.rope_tables(T, shape, "cpu"), W.causal_mask(T, "cpu"))
    layer = W.Fp8DecoderLayer({k: v.cuda() for k, v in params.items()}, {k: v.cuda() for k, v in scales.items()}, shape)
    got = layer(x.cuda()).cpu()
    vb.ops.gemm_status()
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    # The graph rounds each GEMM to bfloat16 before its scale; the FP8 GEMM rounds once after it.
    assert rel_err(got, want) <= 2e-2, rel_err(got, want)
    ref = W.bf16_layer_forward(x, params, shape)
    assert rel_err(got, ref) <= 0.15


def test_fp8_decoder_layer_with_fused_attention_matches_converted_graph():
    """head_dim 128 and T a multiple of 128: the attention runs in the fused kernel."""
    vb = _vb()
    W = vb.workloads
    shape = W.LlamaShape(hidden=512, heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=1024)
    T = 256
    params = W.make_layer_params(0, shape)
    x = W.make_hidden_states(1, T, shape)
    scales = W.calibrate_fp8_scales(x, params, shape)
    want = OL.fp8_decoder_layer(x, params, scales, shape, W.rope_tables(T, shape, "cpu"), W.causal_mask(T, "cpu"))
    layer = W.Fp8DecoderLayer({k: v.cuda() for k, v in params.items()}, {k: v.cuda() for k, v in scales.items()}, shape)
    assert layer.fuse_attention and layer.LAUNCHES == 8
    got = layer(x.cuda()).cpu()
    vb.ops.gemm_status()
    assert vb.fp8.attention_status() == 0
    assert rel_err(got, want) <= 2e-2, rel_err(got, want)
    layer.fuse_attention = False
    separate = layer(x.cuda()).cpu()
    assert rel_err(got, separate) <= 1e-2


@pytest.mark.parametrize("rows,cols,period", [(8, 64, 0), (96, 256, 32), (64, 2048, 64), (10, 520, 0), (12, 4096, 0)])
def test_softmax_quantize_fused_matches_unfused(rows, cols, period):
    """The fused pass against the unfused bf16 op sequence on the CPU oracle."""
    vb = _vb()
    g = torch.Generator().manual_seed(rows + cols)
    scores = (torch.randn(rows, cols, generator=g) * 6).bfloat16()
    scale = 0.125
    sp = torch.tensor(1.0 / 448.0, dtype=torch.bfloat16)
    mask = None
    if period:
        t = torch.arange(rows) % period
        mask = torch.where(torch.arange(cols)[None, :] > t[:, None], float("-inf"), 0.0).bfloat16()
    s = scores * scale
    if mask is not None:
        s = s + mask
    p = torch.softmax(s.float(), -1).bfloat16()
    want = OQ.quantize(p, sp, qmap=OT.quantization_map("fp8_e4m3")).float()
    got = vb.fp8.softmax_quantize_fp8(scores.cuda(), scale, sp.cuda(), causal_period=period).cpu()
    got = got.view(torch.float8_e4m3fn).float()
    # expf may differ from the CPU's in the last bit: allow a single FP8 step on a tiny fraction of entries
    diff = (got - want).abs()
    step = torch.maximum(want.abs(), got.abs()) * 0.126 + 2.0 ** -9
    assert bool((diff <= step).all()), float(diff.max())
    assert float((diff > 0).float().mean()) < 2e-3
    if mask is not None:
        got2 = vb.fp8.softmax_quantize_fp8(scores.cuda(), scale, sp.cuda(), mask=mask.cuda()).cpu()
        assert torch.equal(got2.view(torch.float8_e4m3fn).float(), got)
