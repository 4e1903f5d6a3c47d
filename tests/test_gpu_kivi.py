"""The packed KIVI cache: packing keeps every code, and the fused read from packed bytes is bit
for bit the ``dequantize`` of the unpacked codes (which the golden cases pin to the reference),
with and without the re-encoding table; codes and qparams themselves are checked against the
CPU oracle."""

import pytest
import torch

from golden_io import bits_equal, describe_mismatch
from oracle import quantizers as OQ
from oracle import tables as OT

pytestmark = pytest.mark.gpu


def _vb():
    import voyager_b200

    return voyager_b200


# (shape, axis): keys [B, kv, T, d] grouped along the sequence, values along the head dimension
GEOMETRIES = [((1, 2, 128, 64), -2), ((2, 2, 192, 128), -2), ((1, 2, 96, 128), -1), ((3, 130, 64), -1),
              ((1, 1, 100, 64), -2)]


@pytest.mark.parametrize("shape,axis", GEOMETRIES)
@pytest.mark.parametrize("bits", [2, 4])
def test_packed_cache_reads_what_the_operators_give(shape, axis, bits):
    vb = _vb()
    Q = torch.ops.quantized_ops
    g = torch.Generator().manual_seed(sum(shape) + bits)
    x = torch.randn(*shape, generator=g).bfloat16()
    qmap = OT.quantization_map(f"uint{bits}")
    scale_qmap = OT.quantization_map("fp8_e4m3")
    int6 = OT.quantization_map("int6")
    qmax = float(2 ** bits - 1)

    cache = vb.kivi.quantize_cache(x.cuda(), qmap.cuda(), axis, 64, bits, scale_qmap.cuda())
    # the oracle's codes and qparams
    s_want, z_want, c_want = OQ.quantize_affine(x, qmap, [axis], 64, 0.0, qmax, scale_qmap)
    assert bits_equal(cache.scale.cpu(), s_want) and bits_equal(cache.zero_point.cpu(), z_want)
    n = x.numel()
    per = 8 // bits
    packed = cache.packed.cpu()
    assert packed.numel() == (n * bits + 7) // 8
    idx = torch.arange(n)
    unpacked = (packed[idx // per].to(torch.int32) >> (bits * (idx % per)).to(torch.int32)) & (2 ** bits - 1)
    assert torch.equal(unpacked.reshape(shape).float(), c_want.float())

    # fused read == dequantize of the unpacked codes, plain and re-encoded through a table
    for table in (None, int6):
        want = OQ.dequantize(c_want, s_want, z_want, [axis], 64, None, table)
        got = cache.read(None if table is None else table.cuda()).cpu()
        assert got.dtype == want.dtype and got.shape == want.shape
        assert bits_equal(got, want), describe_mismatch(got, want)
        same = Q.dequantize(c_want.cuda(), s_want.cuda(), z_want.cuda(), [axis], 64, None,
                            None if table is None else table.cuda()).cpu()
        assert bits_equal(got, same)
    assert cache.nbytes < n * 2 // (3 if bits == 4 else 6)


def test_pack_codes_tail_and_dtypes():
    vb = _vb()
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        codes = torch.randint(0, 4, (37,)).to(dtype)
        packed = vb.kivi.pack_codes(codes.cuda(), 2).cpu()
        assert packed.numel() == 10
        idx = torch.arange(37)
        got = (packed[idx // 4].to(torch.int32) >> (2 * (idx % 4)).to(torch.int32)) & 3
        assert torch.equal(got.float(), codes.float())
    scale = torch.tensor(0.5, dtype=torch.bfloat16).cuda()
    out = vb.kivi.unpack_dequantize(vb.kivi.pack_codes(codes.cuda(), 2), 2, (37,), scale).cpu()
    assert torch.equal(out.float(), codes.float() * 0.5)
    assert vb.kivi.pack_codes(torch.empty(0, dtype=torch.bfloat16).cuda(), 2).numel() == 0


# ---------------------------------------------------------------------------
# decode-step attention straight from the packed cache
# ---------------------------------------------------------------------------
def _decode_problem(B, hkv, G, Tm, R, k_block, v_block, seed):
    vb = _vb()
    g = torch.Generator(device="cuda").manual_seed(seed)
    d = 128
    uint2 = vb.get_quantization_map("uint2").cuda()
    e4m3 = vb.get_quantization_map("fp8_e4m3").cuda()
    rnd = lambda *s: torch.randn(*s, generator=g, device="cuda").bfloat16()
    keys = vb.kivi.quantize_cache(rnd(B, hkv, Tm, d), uint2, -2, k_block, 2, e4m3)
    values = vb.kivi.quantize_cache(rnd(B, hkv, Tm, d), uint2, -1, v_block, 2, e4m3)
    return rnd(B, hkv, G, d), keys, values, rnd(B, hkv, R, d), rnd(B, hkv, R, d)


def _decode_by_operators(q, keys, values, k_res, v_res):
    """read() + the graph's matmul / scale / softmax / matmul nodes on bfloat16 tensors."""
    k_main, v_main = keys.read(), values.read()
    scores = torch.cat([torch.matmul(q, k_main.transpose(-1, -2)), torch.matmul(q, k_res.transpose(-1, -2))], -1)
    p = torch.softmax(scores * (1.0 / 128 ** 0.5), -1, dtype=torch.float32).to(q.dtype)
    tm = k_main.shape[-2]
    ctx = torch.matmul(p[..., :tm], v_main) + torch.matmul(p[..., tm:], v_res)
    return ctx.reshape(q.shape[0], -1)


@pytest.mark.parametrize("B,hkv,G,Tm,R,k_block,v_block", [
    (1, 1, 1, 64, 16, 64, 64), (2, 2, 4, 512, 128, 64, 64), (1, 2, 4, 1088, 32, 64, 32), (1, 1, 8, 640, 16, 128, 128),
    (16, 8, 4, 3968, 128, 64, 64), (1, 2, 3, 192, 144, 64, 64),
])
def test_decode_attention_matches_the_operators(B, hkv, G, Tm, R, k_block, v_block):
    vb = _vb()
    q, keys, values, k_res, v_res = _decode_problem(B, hkv, G, Tm, R, k_block, v_block, seed=Tm + R + G)
    got = vb.kivi.decode_attention(q, keys, values, k_res, v_res)
    assert got is not None and got.shape == (B, hkv * G * 128) and got.dtype == torch.bfloat16
    want = _decode_by_operators(q, keys, values, k_res, v_res)
    diff = (got.float() - want.float()).abs()
    # the dequantized operands are bit-identical; sums run in another order and a probability on a bfloat16
    # rounding boundary may move by one step
    assert float(diff.max()) <= 2e-2 * float(want.float().abs().max()), float(diff.max())
    assert float(diff.pow(2).mean().sqrt()) <= 3e-3 * float(want.float().pow(2).mean().sqrt())
    assert torch.equal(got, vb.kivi.decode_attention(q, keys, values, k_res, v_res))


def test_decode_attention_one_hot_rows_return_a_dequantized_value():
    """A query that puts all its weight on one cached position returns that position's dequantized values:
    the in-register decode equals read() bit for bit."""
    vb = _vb()
    q, keys, values, k_res, v_res = _decode_problem(1, 1, 4, 256, 16, 64, 64, seed=11)
    k_main, v_main = keys.read(), values.read()
    targets = [3, 77, 130, 255]
    for i, pos in enumerate(targets):
        q[0, 0, i] = k_main[0, 0, pos] * 64.0          # a huge score on its own key
    want = _decode_by_operators(q, keys, values, k_res, v_res).reshape(4, 128)
    got = vb.kivi.decode_attention(q, keys, values, k_res, v_res).reshape(4, 128)
    assert torch.equal(got, want)
    hit = sum(bool(torch.equal(got[i], v_main[0, 0, pos])) for i, pos in enumerate(targets))
    assert hit >= 3      # (a row whose own key is not its best match proves nothing)


def test_decode_attention_declines_other_layouts():
    vb = _vb()
    q, keys, values, k_res, v_res = _decode_problem(1, 1, 2, 96, 16, 32, 64, seed=5)   # key groups of 32 positions
    assert vb.kivi.decode_attention(q, keys, values, k_res, v_res) is None
    q, keys, values, k_res, v_res = _decode_problem(1, 1, 2, 128, 16, 64, 64, seed=5)
    assert vb.kivi.decode_attention(q, values, keys, k_res, v_res) is None              # keys / values swapped
    assert vb.kivi.decode_attention(q, keys, values, k_res[..., :8, :], v_res[..., :8, :]) is None   # R = 8


@pytest.mark.parametrize("per_sequence", [False, True])
def test_rope_append_equals_the_graph_nodes(per_sequence):
    vb = _vb()
    B, hq, hkv, d, R = 3, 8, 2, 128, 16
    g = torch.Generator(device="cuda").manual_seed(1)
    qkv = torch.randn(B, (hq + 2 * hkv) * d, generator=g, device="cuda").bfloat16()
    cos = torch.randn((B, d) if per_sequence else (d,), generator=g, device="cuda").bfloat16()
    sin = torch.randn((B, d) if per_sequence else (d,), generator=g, device="cuda").bfloat16()
    k_win = torch.randn(B, hkv, R, d, generator=g, device="cuda").bfloat16()
    v_win = torch.randn(B, hkv, R, d, generator=g, device="cuda").bfloat16()
    want_k, want_v = k_win.clone(), v_win.clone()
    c, s = (cos[:, None], sin[:, None]) if per_sequence else (cos, sin)
    rotate = lambda v: v * c + torch.cat([-v[..., d // 2:], v[..., :d // 2]], -1) * s
    want_q = rotate(qkv[:, :hq * d].reshape(B, hq, d))
    want_k[:, :, 5].copy_(rotate(qkv[:, hq * d:(hq + hkv) * d].reshape(B, hkv, d)))
    want_v[:, :, 5].copy_(qkv[:, (hq + hkv) * d:].reshape(B, hkv, d))
    got_q = vb.kivi.rope_append(qkv, cos, sin, hq, k_win, v_win, 5)
    assert torch.equal(got_q, want_q) and torch.equal(k_win, want_k) and torch.equal(v_win, want_v)
