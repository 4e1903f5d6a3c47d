"""The packed lookup-format weight and the decode-step linear that reads it, against the CPU oracle's
``linear_mx`` on the unpacked operands (golden case ``linear_mx_nf4`` pins that operator)."""

import pytest
import torch

import cases as C
from oracle import gemm as OG
from oracle import quantizers as OQ
from oracle import tables as OT

pytestmark = pytest.mark.gpu


def _vb():
    import voyager_b200

    return voyager_b200


def _nf4():
    nf4 = OT.quantization_map("lut4_to_int6")
    levels = torch.unique(nf4)
    index = torch.searchsorted(levels, nf4).to(torch.int64)
    mid = (levels[:-1] + levels[1:]) / 2
    return levels, index, mid, OT.quantization_map("fp8_e5m3")


def rel_err(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("m,n,k,bs", [(16, 256, 1024, 64), (1, 8, 128, 64), (5, 200, 384, 64), (16, 4096, 4096, 64),
                                      (32, 1000, 2176, 64), (17, 136, 256, 32), (16, 128, 14336, 128)])
def test_linear_lut4_matches_linear_mx(m, n, k, bs):
    vb = _vb()
    levels, index, mid, e5m3 = _nf4()
    x = C.randn(400 + m, m, k, outliers=0.002)
    w = C.randn(500 + n, n, k, std=0.02)
    bias = C.randn(7, n, std=0.1)
    sx, cx = OQ.quantize_mx(x, index, [-1], bs, 31.0, False, e5m3, mid)
    sw, cw = OQ.quantize_mx(w, index, [-1], bs, 31.0, False, e5m3, mid)
    alpha = torch.tensor(0.75, dtype=torch.bfloat16)
    want = OG.linear_mx(cx, cw, bias, input_scale=sx, weight_scale=sw, block_size=bs, input_code=levels,
                        weight_code=levels, alpha=alpha)
    P = vb.packed
    packed = P.pack_lut4_weight(cw.cuda(), sw.cuda(), levels.cuda(), bs)
    assert packed.codes.shape == (n, k // 2) and packed.nbytes <= (0.5 + 2.0 / bs) * n * k + 32
    assert torch.equal(P.unpack_lut4_weight(packed).cpu(), cw)
    got = P.linear_lut4(cx.cuda(), packed, bias.cuda(), input_scale=sx.cuda(), input_code=levels.cuda(),
                        alpha=alpha.cuda()).cpu()
    assert got.shape == want.shape and got.dtype == want.dtype
    assert rel_err(got, want) <= 1e-2, rel_err(got, want)
    # against a float64 product of the same bfloat16 operands: only the float32 summation order differs
    got32 = P.linear_lut4(cx.cuda(), packed, None, input_scale=sx.cuda(), input_code=levels.cuda(),
                          out_dtype=torch.float32).cpu()
    a = (levels[cx.long()] * OQ.expand_blocks(sx, cx, bs)).double()
    b = (levels[cw.long()] * OQ.expand_blocks(sw, cw, bs)).double()
    ref = a @ b.T
    assert rel_err(got32, ref) <= 2e-5, rel_err(got32, ref)
    # a second call finds the tile counters reset and gives the same bits
    again = P.linear_lut4(cx.cuda(), packed, None, input_scale=sx.cuda(), input_code=levels.cuda(),
                          out_dtype=torch.float32).cpu()
    assert torch.equal(again, got32)


def test_linear_lut4_takes_plain_activations_and_many_rows():
    vb = _vb()
    levels, index, mid, e5m3 = _nf4()
    P = vb.packed
    w = C.randn(601, 96, 256, std=0.02)
    sw, cw = OQ.quantize_mx(w, index, [-1], 64, 31.0, False, e5m3, mid)
    packed = P.pack_lut4_weight(cw.cuda(), sw.cuda(), levels.cuda(), 64)
    x = C.randn(602, 3, 4, 256)                                     # values, leading dimensions
    want = OG.linear_mx(x, cw, None, weight_scale=sw, block_size=64, weight_code=levels)
    got = P.linear_lut4(x.cuda(), packed).cpu()
    assert got.shape == (3, 4, 96) and rel_err(got, want) <= 1e-2
    big = C.randn(603, 200, 256)                                    # more than 32 rows: the tensor-core GEMM
    want = OG.linear_mx(big, cw, None, weight_scale=sw, block_size=64, weight_code=levels)
    got = P.linear_lut4(big.cuda(), packed).cpu()
    vb.ops.gemm_status()
    assert rel_err(got, want) <= 1e-2
    with pytest.raises(ValueError):
        P.pack_lut4_weight((cw + 20).cuda(), sw.cuda(), levels.cuda(), 64)
