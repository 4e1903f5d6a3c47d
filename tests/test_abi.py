"""The C-ABI library builds for sm_100a, loads without a GPU and exports every
symbol that include/vq_b200.h declares; host-side logic of the package."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import voyager_b200
from golden_io import bits_equal, describe_mismatch, golden_tables

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = []
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"^(?:int|int64_t|const char\*)\s+(vq_\w+)\s*\(", text, flags=re.M)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    voyager_b200.build()
    lib = ctypes.CDLL(voyager_b200._native.LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) >= 9
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    bound = set(voyager_b200._native.SIGNATURES) | {"vq_last_error"}
    assert set(declared) == bound, set(declared) ^ bound
    assert voyager_b200._native.lib().vq_version() >= 1


def test_argument_errors_are_reported_without_a_gpu():
    lib = voyager_b200._native.lib()
    rc = lib.vq_vmap(None, None, 0, None, 16, None)
    assert rc == -1
    assert b"null" in lib.vq_last_error()
    assert lib.vq_vmap(None, None, 0, None, 0, None) == 0  # empty input is a no-op


@pytest.mark.parametrize("name", sorted(golden_tables()))
def test_product_tables_match_reference(name):
    got = voyager_b200.get_quantization_map(name)
    want = golden_tables()[name]
    assert bits_equal(got, want), describe_mismatch(got, want)


def test_spec_strings():
    p = voyager_b200.parse_spec_fields("int8,qs=microscaling,bs=16,pot=1")
    assert p["dtype"] == "int8" and p["block_size"] == 16 and p["power_2_scale"] is True
    assert p["qscheme"] is voyager_b200.QScheme.MICROSCALING
    assert (p["quant_min"], p["quant_max"]) == (-128.0, 127.0)
    p = voyager_b200.parse_spec_fields("fp4_e2m1,qs=microscaling,bs=16,scale=fp8_e4m3,gs=1")
    assert p["quant_max"] == 6.0 and p["scale_dtype"] == "fp8_e4m3" and p["global_scale"] is True
    p = voyager_b200.parse_spec_fields("lut4_to_int6,qs=microscaling,bs=64,scale=fp8_e5m3,ax=(-2,-1)")
    assert p["quant_max"] == 31.0 and p["ch_axis"] == (-2, -1)
    p = voyager_b200.parse_spec_fields("fp8_e4m3,qs=per_tensor_symmetric")
    assert p["quant_max"] == 448.0 and p["amax_history_len"] == 64
    assert voyager_b200.parse_spec_fields("posit8_1,qs=microscaling")["quant_max"] == 4096.0
    assert voyager_b200.float_format("fp8_e5m3").signed is False
    assert voyager_b200.float_format("fp8_e4m3_ieee").max_norm == 240.0
    with pytest.raises(ValueError):
        voyager_b200.parse_spec_fields("int8,bogus=1")
    with pytest.raises(ValueError):
        voyager_b200.parse_spec_fields("")
    with pytest.raises(ValueError):
        voyager_b200.float_format("fp8_e4m2")
    with pytest.raises(ValueError):
        voyager_b200.parse_codebook_dtype("lut4_to_uint4")


def test_table_fingerprinting():
    R, N = voyager_b200.rounding, voyager_b200._native
    assert R.table_round(voyager_b200.get_quantization_map("int8")).mode == N.ROUND_INT
    spec = R.table_round(voyager_b200.get_quantization_map("fp8_e4m3"))
    assert spec.mode == N.ROUND_MINIFLOAT and spec.c.mbits == 3 and spec.c.emin == -6
    assert R.table_round(voyager_b200.get_quantization_map("fp8_e5m3")).mode == N.ROUND_MINIFLOAT
    assert R.table_round(voyager_b200.get_quantization_map("lut4_to_int6")).mode == N.ROUND_TABLE
    assert R.table_round(voyager_b200.get_quantization_map("posit8_1")).mode == N.ROUND_TABLE
    assert R.table_round(voyager_b200.get_quantization_map("fp8_e8m0")).mode == N.ROUND_TABLE
    # a perturbed int8 table is no longer recognised and is gathered
    t = voyager_b200.get_quantization_map("int8").clone()
    t[0x4000] = 3.0
    assert R.table_round(t).mode == N.ROUND_TABLE
    # the index form of a lookup format is a step function too
    idx, levels = voyager_b200.formats.index_table(voyager_b200.get_quantization_map("lut4_to_int6"))
    R.PREFER_STEPS = True
    try:
        R._table_cache.clear()
        s = R.table_round(idx)
        assert s.mode == N.ROUND_STEPS and s.c.n_steps <= 32
    finally:
        R.PREFER_STEPS = False
        R._table_cache.clear()


def test_steps_reproduce_table_on_host():
    """The step description rebuilt on the host equals the table entry for entry."""
    R = voyager_b200.rounding
    for name in ("lut4_to_int6", "fp4_e2m1", "uint2", "int4"):
        bits = voyager_b200.formats._table_bits(name)
        values, uppers, nan_value = R._steps_of(bits)
        patterns = np.arange(1 << 16)
        keys = R._ordered_key(patterns)
        idx = np.searchsorted(uppers[:-1].astype(np.int64), keys, side="right")
        rebuilt = values[idx]
        is_nan = (patterns & 0x7FFF) > 0x7F80
        assert np.array_equal(rebuilt[~is_nan], bits[~is_nan]), name
        both_nan = ((bits[is_nan] & 0x7FFF) > 0x7F80) & ((nan_value & 0x7FFF) > 0x7F80)
        assert np.all(both_nan | (bits[is_nan] == nan_value)), name


def test_broadcast_geometry():
    from voyager_b200.ops import _broadcast_geometry as geo

    g = geo((64, 256), torch.empty(64, 16), 16)
    assert g.ndim == 2 and list(g.size[:2]) == [64, 256] and list(g.div[:2]) == [1, 16] and list(g.stride[:2]) == [16, 1]
    g = geo((2, 64, 96), torch.empty(()), None)
    assert g.ndim == 1 and g.size[0] == 2 * 64 * 96 and g.stride[0] == 0
    g = geo((48, 64), torch.empty(48, 1), None)
    assert g.ndim == 2 and list(g.stride[:2]) == [1, 0]
    g = geo((1, 2, 128, 64), torch.empty(1, 2, 2, 64), 64)
    assert g.ndim == 3 and list(g.size[:3]) == [2, 128, 64] and list(g.div[:3]) == [1, 64, 1]
    g = geo((3, 40), torch.empty(3, 3), 16)
    assert list(g.div[:2]) == [1, 16]
    with pytest.raises(ValueError):
        geo((3, 40), torch.empty(3, 5), 16)


def test_fake_kernels_give_shapes():
    x = torch.empty(4, 40, dtype=torch.bfloat16, device="meta")
    t = torch.empty(65536, dtype=torch.bfloat16, device="meta")
    s, c = torch.ops.quantized_ops.quantize_mx(x, t, [-1], 16, 127.0, True)
    assert s.shape == (4, 3) and c.shape == (4, 40)
    s, z, c = torch.ops.quantized_ops.quantize_affine(x, t, [-1], 16, 0.0, 3.0)
    assert s.shape == z.shape == (4, 3)


def test_voyager_gpu_operator_schemas_are_the_references():
    """Names and schemas of the ``voyager_gpu`` call targets (reference ``backend/gpu/nvfp4.py:675-679,
    773-778, 851-854, 1094-1097``, ``fp8.py:311-314``, ``rmsnorm.py:132-136``), and their shape functions."""
    G = torch.ops.voyager_gpu
    want = {
        "cast_nvfp4": "voyager_gpu::cast_nvfp4(Tensor x, Tensor? hadamard, Tensor? seed, int axis) -> (Tensor, Tensor, Tensor)",
        "cast_nvfp4_pair": "voyager_gpu::cast_nvfp4_pair(Tensor x, Tensor? hadamard, Tensor? seed, Tensor? transpose_seed) "
                           "-> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)",
        "cast_nvfp4_square": "voyager_gpu::cast_nvfp4_square(Tensor x) -> (Tensor, Tensor, Tensor, Tensor, Tensor)",
        "nvfp4_linear": "voyager_gpu::nvfp4_linear(Tensor input, Tensor input_scale, Tensor weight, Tensor weight_scale, "
                        "Tensor alpha, Tensor one, Tensor? bias) -> Tensor",
        "cast_transpose_fp8": "voyager_gpu::cast_transpose_fp8(Tensor x, Tensor scale, ScalarType dtype) -> (Tensor, Tensor, Tensor)",
        "rmsnorm_backward": "voyager_gpu::rmsnorm_backward(Tensor[] gradients, Tensor x, Tensor rsqrt, Tensor weight, "
                            "Tensor? residual) -> (Tensor, Tensor)",
    }
    for name, schema in want.items():
        assert str(getattr(G, name).default._schema) == schema
    x = torch.empty(192, 128, dtype=torch.bfloat16, device="meta")
    codes, scales, t = G.cast_nvfp4(x, None, None, 1)
    assert codes.shape == (192, 64) and scales.shape == (256 * 8,) and t.shape == () and t.dtype == torch.bfloat16
    codes, scales, t = G.cast_nvfp4(x, None, None, 0)
    assert codes.shape == (128, 96) and scales.shape == (128 * 12,)
    assert [o.shape for o in G.cast_nvfp4_square(x)][2] == (128, 96)
    y = G.nvfp4_linear(codes, scales, codes, scales, t, t, None)
    assert y.shape == (128, 128) and y.dtype == torch.bfloat16
    c, ct, amax = G.cast_transpose_fp8(x, t, torch.float8_e4m3fn)
    assert c.shape == (192, 128) and ct.shape == (128, 192) and c.dtype == torch.float8_e4m3fn


def test_convolution_operator_schemas_are_the_references():
    """``conv2d_mx`` (reference ``ops/quantized.py:596-604``) and the layout twin ``conv2d`` (``ops/layout.py:175-181``)
    as the dispatcher normalises them, and their shape functions."""
    Q = torch.ops.quantized_ops
    assert str(Q.conv2d_mx.default._schema) == (
        "quantized_ops::conv2d_mx(Tensor input, Tensor weight, Tensor? bias=None, SymInt[2] stride=[1, 1], "
        "SymInt[2] padding=[0, 0], SymInt[2] dilation=[1, 1], SymInt groups=1, *, Tensor? input_scale=None, "
        "Tensor? weight_scale=None, int? block_size=None, Tensor? input_code=None, Tensor? weight_code=None, "
        'str layout="nchw", ScalarType? out_dtype=None) -> Tensor')
    assert str(Q.conv2d.default._schema) == (
        "quantized_ops::conv2d(Tensor input, Tensor weight, Tensor? bias=None, SymInt[2] stride=[1, 1], "
        'SymInt[2] padding=[0, 0], SymInt[2] dilation=[1, 1], SymInt groups=1, *, str layout="nchw", '
        "ScalarType? out_dtype=None) -> Tensor")
    x = torch.empty(2, 16, 10, 10, dtype=torch.bfloat16, device="meta")
    w = torch.empty(8, 16, 3, 3, dtype=torch.bfloat16, device="meta")
    assert Q.conv2d_mx(x, w, None, [1, 1], [1, 1]).shape == (2, 8, 10, 10)
    y = Q.conv2d(x.permute(0, 2, 3, 1), w.permute(2, 3, 1, 0), None, [2, 2], [1, 1], [1, 1], 1, layout="nhwc",
                 out_dtype=torch.float32)
    assert y.shape == (2, 5, 5, 8) and y.dtype == torch.float32
