"""NVFP4: the fused cast and the packer reproduce quantize_mx's codes and scales bit for bit,
and the native block-scaled GEMM matches linear_mx on the same operands."""

import numpy as np
import pytest
import torch

import cases as C
from oracle import gemm as OG
from oracle import quantizers as OQ
from oracle import tables as OT

pytestmark = pytest.mark.gpu

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _vb():
    import voyager_b200

    return voyager_b200


def unpack(packed, rows, k):
    """Decode packed codes / scale tiles back to float tensors [rows, K] and [rows, K/16]."""
    codes = packed.codes.cpu().reshape(rows, k // 2)
    lo, hi = codes & 0xF, codes >> 4
    nib = torch.stack([lo, hi], -1).reshape(rows, k).long()
    val = E2M1_VALUES[nib & 7] * torch.where(nib & 8 != 0, -1.0, 1.0)
    sbytes = packed.scales.cpu().reshape(-1)
    r = torch.arange(rows)[:, None]
    kb = torch.arange(k // 16)[None, :]
    off = ((r // 128) * (k // 64) + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    scale = sbytes[off].view(torch.float8_e4m3fn).float()
    return val, scale


def reference_quantize(x):
    e2m1, e4m3 = OT.quantization_map("fp4_e2m1"), OT.quantization_map("fp8_e4m3")
    t = OQ.calculate_global_scale(x, 6.0, 448.0)
    scale, codes = OQ.quantize_mx(x, e2m1, [-1], 16, 6.0, False, e4m3, None, None, t)
    return t, scale, codes


@pytest.mark.parametrize("rows,k,seed", [(128, 256, 1), (200, 64, 2), (64, 1024, 3), (300, 320, 4)])
def test_fused_cast_matches_quantize_mx(rows, k, seed):
    vb = _vb()
    x = C.randn(seed, rows, k, outliers=0.002)
    x[0, :16] = 0  # an all-zero block
    t, scale, codes = reference_quantize(x)
    packed = vb.nvfp4.cast_nvfp4(x.cuda(), t.cuda())
    val, sc = unpack(packed, rows, k)
    assert torch.equal(sc, scale.float())
    assert torch.equal(val, codes.float())
    repacked = vb.nvfp4.pack_nvfp4(codes.cuda(), scale.cuda())
    val2, sc2 = unpack(repacked, rows, k)
    assert torch.equal(sc2, scale.float()) and torch.equal(val2, codes.float())


def test_packer_rejects_unrepresentable_values():
    vb = _vb()
    codes = torch.full((128, 64), 2.5, dtype=torch.bfloat16, device="cuda")
    scale = torch.ones(128, 4, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        vb.nvfp4.pack_nvfp4(codes, scale)


@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (64, 48, 64), (300, 264, 320), (256, 512, 4096), (2048, 1024, 1024),
                                   (129, 72, 64), (520, 1000, 448), (1024, 4096, 2048)])
def test_native_gemm_matches_linear_mx(m, n, k):
    vb = _vb()
    x = C.randn(10 + m, m, k, outliers=0.002)
    w = C.randn(20 + n, n, k, std=0.02)
    tx, sx, cx = reference_quantize(x)
    tw, sw, cw = reference_quantize(w)
    alpha = tx * tw
    bias = C.randn(5, n, std=0.1)
    want = OG.linear_mx(cx, cw, bias, input_scale=sx, weight_scale=sw, block_size=16, alpha=alpha)
    a = vb.nvfp4.cast_nvfp4(x.cuda(), tx.cuda())
    b = vb.nvfp4.cast_nvfp4(w.cuda(), tw.cuda())
    got = vb.nvfp4.nvfp4_gemm(a, b, alpha.cuda(), bias.cuda()).cpu()
    vb.ops.gemm_status()
    assert got.shape == want.shape and got.dtype == want.dtype
    err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
    assert err <= 1e-2, err
    got32 = vb.nvfp4.nvfp4_gemm(a, b, None, None, out_dtype=torch.float32).cpu()
    da = (cx.double() * OQ.expand_blocks(sx, cx, 16).double())
    db = (cw.double() * OQ.expand_blocks(sw, cw, 16).double())
    ref = da @ db.T
    err32 = float((got32.double() - ref).abs().max() / ref.abs().max())
    assert err32 <= 1e-4, err32


@pytest.mark.parametrize("shape,axis", [((3, 40, 128), -1), ((128, 256), 0), ((200, 64), -1)])
def test_reference_signatures(shape, axis):
    """quantize_nvfp4 / unpack_nvfp4 / nvfp4_linear / emulate_nvfp4_linear as the reference spells them."""
    vb = _vb()
    x = C.randn(sum(shape), *shape, outliers=0.002)
    codes, scales, t = vb.nvfp4.quantize_nvfp4(x.cuda(), axis)
    moved = x.movedim(axis, -1)
    t_want, scale_want, codes_want = reference_quantize(moved.contiguous())
    assert torch.equal(t.cpu(), t_want) and t.dtype == torch.bfloat16 and t.ndim == 0
    assert codes.shape == (*moved.shape[:-1], moved.shape[-1] // 2) and codes.dtype == torch.uint8
    values, block_scales = vb.nvfp4.unpack_nvfp4(codes, scales)
    assert torch.equal(values.cpu().float(), codes_want.float())
    assert torch.equal(block_scales.cpu().float(), scale_want.float())
    # the linear, packed against its emulation through linear_mx
    n = 72
    w = C.randn(7, n, moved.shape[-1], std=0.02)
    w_codes, w_scales, tw = vb.nvfp4.quantize_nvfp4(w.cuda())
    alpha = (t * tw).float()
    bias = C.randn(8, n, std=0.1).cuda()
    one = torch.ones((), device="cuda")
    got = vb.nvfp4.nvfp4_linear(codes, scales, w_codes, w_scales, alpha, one, bias)
    want = vb.nvfp4.emulate_nvfp4_linear(codes, scales, w_codes, w_scales, alpha, one, bias)
    vb.ops.gemm_status()
    assert got.shape == (*moved.shape[:-1], n) and got.dtype == torch.bfloat16
    err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
    assert err <= 1e-2, err


def test_quantize_nvfp4_stochastic_uses_the_operator():
    vb = _vb()
    x = C.randn(31, 64, 128)
    seed = torch.tensor(99, dtype=torch.int64)
    codes, scales, t = vb.nvfp4.quantize_nvfp4(x.cuda(), -1, seed.cuda())
    values, block_scales = vb.nvfp4.unpack_nvfp4(codes, scales)
    levels = OT.grid_levels(OT.quantization_map("fp4_e2m1"))
    s_want, c_want = OQ.quantize_mx(x, levels, [-1], 16, 6.0, False, OT.quantization_map("fp8_e4m3"), None, seed,
                                    OQ.calculate_global_scale(x, 6.0, 448.0))
    assert torch.equal(values.cpu().float(), c_want.float())
    assert torch.equal(block_scales.cpu().float(), s_want.float())


def test_quantize_nvfp4_pair_is_the_two_casts():
    vb = _vb()
    g = torch.Generator().manual_seed(5)
    x = torch.randn(128, 192, generator=g).bfloat16().cuda()
    pair = vb.nvfp4.quantize_nvfp4_pair(x)
    rows, cols = vb.nvfp4.quantize_nvfp4(x, -1), vb.nvfp4.quantize_nvfp4(x.mT, -1)
    for got, want in zip(pair, (*rows, *cols)):
        assert torch.equal(got, want)
    assert pair[0].shape == (128, 96) and pair[3].shape == (192, 64)


def test_quantize_nvfp4_square_matches_the_oracle():
    vb = _vb()
    from oracle import tables as OT
    from oracle import training as oracle_training
    g = torch.Generator().manual_seed(6)
    w = (torch.randn(128, 256, generator=g) * 0.05).bfloat16()
    w[3, 7] = 1.5                                                     # an outlier sets the global scale
    values, scale, t = oracle_training.nvfp4_square_values(w, OT.quantization_map("fp4_e2m1"), OT.quantization_map("fp8_e4m3"))
    codes, scales, codes_t, scales_t, t_gpu = vb.nvfp4.quantize_nvfp4_square(w.cuda())
    assert torch.equal(t_gpu.cpu().reshape(()), t.reshape(()))
    got, got_scale = vb.nvfp4.unpack_nvfp4(codes, scales)
    assert torch.equal(got.cpu(), values)
    assert torch.equal(got_scale.cpu(), scale.repeat_interleave(16, 0))
    got_t, got_scale_t = vb.nvfp4.unpack_nvfp4(codes_t, scales_t)
    assert torch.equal(got_t.cpu(), values.mT)
    assert torch.equal(got_scale_t.cpu(), scale.mT.repeat_interleave(16, 0))


@pytest.mark.parametrize("merge,attention", [(True, "fused"), (True, "eager"), (False, "eager"), (True, "sdpa")])
def test_nvfp4_decoder_layer_matches_converted_graph(merge, attention):
    """Seven NVFP4 linears of a Llama-shaped layer (casts + native block-scaled GEMMs, merged QKV and
    gate/up with per-column alphas) against the converted microscaling graph on the CPU oracle."""
    from oracle import layers as OL

    vb = _vb()
    W = vb.workloads
    shape = W.LlamaShape(hidden=512, heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=1024)
    T = 256
    params = W.make_layer_params(3, shape)
    x = W.make_hidden_states(4, T, shape)
    want = OL.nvfp4_decoder_layer(x, params, shape, W.rope_tables(T, shape, "cpu"), W.causal_mask(T, "cpu")).float()
    layer = W.Nvfp4DecoderLayer({k: v.cuda() for k, v in params.items()}, shape, merge=merge, attention=attention)
    got = layer(x.cuda()).float().cpu()
    vb.ops.gemm_status()
    err = (got - want).abs()
    # 4-bit re-quantization after every block amplifies summation-order noise: a code that moves changes a
    # value by up to a third
    assert float(err.max()) <= 6e-2 * float(want.abs().max()), float(err.max() / want.abs().max())
    assert float(err.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) <= 2e-2


def test_silu_mul_cast_nvfp4_equals_the_separate_nodes():
    """SwiGLU + amax + cast against quantize_nvfp4(F.silu(gate) * up): the same global scale, and codes that
    agree except where the approximate exponential moves silu by one bfloat16 step."""
    import torch.nn.functional as F

    vb = _vb()
    g = torch.Generator().manual_seed(12)
    gu = torch.randn(256, 2 * 1024, generator=g).bfloat16().cuda()
    gate, up = gu[:, :1024], gu[:, 1024:]                      # strided halves of one matrix
    codes, scales, t = vb.nvfp4.silu_mul_cast_nvfp4(gate, up)
    want_codes, want_scales, want_t = vb.nvfp4.quantize_nvfp4(F.silu(gate) * up)
    assert torch.equal(t, want_t)
    got, _ = vb.nvfp4.unpack_nvfp4(codes, scales)
    want, _ = vb.nvfp4.unpack_nvfp4(want_codes, want_scales)
    assert float((got != want).float().mean()) < 2e-3
    assert float((scales != want_scales).float().mean()) < 2e-3
