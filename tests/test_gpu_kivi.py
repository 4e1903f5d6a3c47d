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
