"""The ``quantized_ops`` torch library, backed by sm_100a CUDA kernels.

Defines the same operator names and schemas as the reference's
``src/voyager_compiler/ops/quantized.py`` (``Library("quantized_ops", "DEF")``
at ``:97``) and ``ops/layout.py`` (the ``FRAGMENT`` at ``:140``), so a graph
produced by the reference's ``convert_pt2e`` runs unchanged.  Only the ``CUDA``
dispatch key gets kernels (calls into ``libvq_b200.so``) plus ``Meta`` shape
functions for tracing; there is deliberately no CPU implementation.

Do not import this module in a process that has imported the reference's
``voyager_compiler.ops``: both define the ``quantized_ops`` namespace.
"""

import math
from typing import List, Optional, Sequence, Tuple

import torch
from torch.library import Library

from . import _native as N
from . import rounding as R

LINEAR_LAYOUT = "xc,kc->xk"
MATMUL_LAYOUT = "xc,ck->xk"
DEFAULT_TENSOR_LAYOUT = "nchw"
QMAP_SIZE = 1 << 16
HADAMARD_SIZE = 16

quantized_ops_lib = Library("quantized_ops", "DEF")

_DTYPE_ID = {torch.bfloat16: N.VQ_BF16, torch.float16: N.VQ_F16, torch.float32: N.VQ_F32}


def _dtype_id(dtype):
    try:
        return _DTYPE_ID[dtype]
    except KeyError:
        raise TypeError(f"quantized_ops kernels take bfloat16, float16 or float32 tensors, not {dtype}") from None


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _is_dense(x):
    """True when ``x`` covers its storage range exactly once (any axis order)."""
    if x.is_contiguous():
        return True
    expected = 1
    for size, stride in sorted(zip(x.shape, x.stride()), key=lambda p: p[1]):
        if size == 1:
            continue
        if stride != expected:
            return False
        expected *= size
    return True


def _dense_like(x):
    """``x`` in a dense layout an elementwise kernel can walk in memory order,
    and an empty output with the same strides."""
    if not _is_dense(x):
        x = x.contiguous()
    return x, torch.empty_like(x)


# ---------------------------------------------------------------------------
# rounding selection from operator arguments
# ---------------------------------------------------------------------------
def _is_table(qmap):
    return qmap.numel() == QMAP_SIZE and qmap.dim() == 1


def _element_round(qmap, output_code, seed):
    if qmap is None:
        return R.none_round()
    if seed is not None:
        return R.stochastic_round(qmap, seed)
    if _is_table(qmap):
        return R.table_round(qmap)
    if qmap.dim() == 1:
        return R.search_round(qmap, output_code)
    raise NotImplementedError("region codebooks are handled by the caller")


# ---------------------------------------------------------------------------
# vmap
# ---------------------------------------------------------------------------
quantized_ops_lib.define("vmap(Tensor self, Tensor other) -> Tensor")


def vmap(input: torch.Tensor, qmap: torch.Tensor) -> torch.Tensor:
    """Round through a 65 536-entry table (reference ``quantized.py:151-184``)."""
    x, out = _dense_like(input)
    spec = R.table_round(qmap)
    N.check(N.lib().vq_vmap(x.data_ptr(), out.data_ptr(), _dtype_id(x.dtype), spec.ref, x.numel(), _stream()),
            "vq_vmap")
    return out


quantized_ops_lib.impl("vmap", N.device_guarded(vmap), "CUDA")


@torch.library.register_fake("quantized_ops::vmap")
def _(input, qmap):
    return torch.empty_like(input)


# ---------------------------------------------------------------------------
# broadcast geometry of scale / zero point against the input
# ---------------------------------------------------------------------------
def _broadcast_geometry(shape: Sequence[int], param: torch.Tensor, block_size: Optional[int]):
    """Collapse (input shape, parameter shape/strides, block size) into at most
    ``N.MAX_DIMS`` groups ``(size, div, stride)`` with
    ``param_index = sum (coord // div) * stride``."""
    nd = len(shape)
    pshape = list(param.shape)
    pstride = list(param.stride())
    if len(pshape) > nd:
        raise ValueError(f"parameter of shape {tuple(param.shape)} has more axes than the input {tuple(shape)}")
    pad = nd - len(pshape)
    pshape = [1] * pad + pshape
    pstride = [0] * pad + pstride
    dims = []
    for size, ps, st in zip(shape, pshape, pstride):
        if ps == size:
            dims.append((size, 1, st if size > 1 else 0))
        elif block_size is not None:
            blocks = -(-size // block_size)
            if ps != blocks and not (ps == 1 and size <= block_size):
                raise ValueError(
                    f"parameter extent {ps} does not match {size} elements in blocks of {block_size}")
            dims.append((size, block_size, st if ps > 1 else 0))
        elif ps == 1:
            dims.append((size, 1, 0))
        else:
            raise ValueError(f"parameter of shape {tuple(param.shape)} does not broadcast to {tuple(shape)}")
    # collapse: drop size-1 dims; merge neighbours that are both broadcast
    # (stride 0) or both dense-unblocked with compatible strides
    merged = []
    for size, div, st in dims:
        if size == 1:
            continue
        if merged:
            psize, pdiv, pst = merged[-1]
            if st == 0 and pst == 0:
                merged[-1] = (psize * size, 1, 0)
                continue
            if div == 1 and pdiv == 1 and st != 0 and pst == st * size:
                merged[-1] = (psize * size, 1, st)
                continue
        merged.append((size, div if st != 0 else 1, st))
    if not merged:
        merged = [(1, 1, 0)]
    if len(merged) > N.MAX_DIMS:
        raise NotImplementedError(f"parameter broadcast needs {len(merged)} index groups (max {N.MAX_DIMS})")
    g = N.VqBroadcast()
    g.ndim = len(merged)
    for i, (size, div, st) in enumerate(merged):
        g.size[i], g.div[i], g.stride[i] = size, div, st
    return g


def _prepare_params(x, scale, zero_point):
    """Compute dtype and parameter tensors for ``x (op) scale``: torch's type
    promotion, except that a single-element float32 scale next to 16-bit data
    is used at full precision without widening the result."""
    if zero_point is not None and (zero_point.shape != scale.shape or zero_point.dtype != scale.dtype):
        shape = torch.broadcast_shapes(scale.shape, zero_point.shape)
        dtype = torch.promote_types(scale.dtype, zero_point.dtype)
        scale = scale.to(dtype).expand(shape).contiguous()
        zero_point = zero_point.to(dtype).expand(shape).contiguous()
    out_dtype = torch.result_type(x, scale)
    if zero_point is not None:
        out_dtype = torch.promote_types(out_dtype, torch.result_type(x, zero_point))
    if x.dtype != out_dtype:
        x = x.to(out_dtype)
    if scale.dtype != out_dtype:
        if scale.dim() == 0 and scale.dtype == torch.float32 and scale.is_floating_point():
            pass  # used at float32 precision
        else:
            scale = scale.to(out_dtype)
            zero_point = None if zero_point is None else zero_point.to(out_dtype)
    return x, scale, zero_point


def _region_apply(input, codebook, fn):
    """Apply ``fn(flat_region_rows, region_index)`` per codebook region of a
    ``[*counts, k]`` codebook and put the results back in place."""
    counts = tuple(codebook.shape[:-1])
    if len(counts) != input.dim():
        raise ValueError(
            f"a {list(counts)} region codebook tiles {len(counts)} axes, but the tensor reaching it has "
            f"{input.dim()}")
    if any(extent % count for extent, count in zip(input.shape, counts)):
        raise ValueError(f"a {list(counts)} region codebook does not divide the {list(input.shape)} tensor reaching it")
    split = []
    for extent, count in zip(input.shape, counts):
        split += [count, extent // count]
    n = len(counts)
    order = list(range(0, 2 * n, 2)) + list(range(1, 2 * n, 2))
    inverse = [order.index(i) for i in range(2 * n)]
    moved = input.reshape(split).permute(order)
    regions = math.prod(counts)
    flat = moved.reshape(regions, -1).contiguous()
    out = torch.empty_like(flat)
    for r in range(regions):
        out[r] = fn(flat[r], r)
    return out.view(moved.shape).permute(inverse).reshape(input.shape)


# ---------------------------------------------------------------------------
# quantize / dequantize
# ---------------------------------------------------------------------------
quantized_ops_lib.define(
    "quantize(Tensor input, Tensor scale, Tensor? zero_point=None, "
    "SymInt[]? axes=None, int? block_size=None, Tensor? qmap=None, "
    "Tensor? output_code=None, Tensor? seed=None) -> Tensor"
)


def _quantize_with(x, scale, zero_point, block_size, spec):
    x, scale, zero_point = _prepare_params(x, scale, zero_point)
    x = x.contiguous()
    out = torch.empty_like(x)
    geom = _broadcast_geometry(x.shape, scale, block_size)
    N.check(N.lib().vq_quantize(x.data_ptr(), scale.data_ptr(), _ptr(zero_point), out.data_ptr(),
                                _dtype_id(x.dtype), _dtype_id(scale.dtype), geom, spec.ref, _stream()),
            "vq_quantize")
    return out


def quantize(input, scale, zero_point=None, axes=None, block_size=None, qmap=None, output_code=None, seed=None):
    """``round(input / scale [+ zero_point])`` (reference ``quantized.py:458-515``)."""
    if qmap is not None and seed is None and not _is_table(qmap) and qmap.dim() > 1:
        # One codebook per region (e.g. per attention head): scale first, then
        # search each region against its own entries.
        scaled = _quantize_with(input, scale, zero_point, block_size, R.none_round())
        tables = qmap.reshape(-1, qmap.shape[-1])
        bounds = None if output_code is None else output_code.reshape(tables.shape[0], -1)

        def per_region(rows, r):
            spec = R.search_round(tables[r], None if bounds is None else bounds[r])
            return _quantize_with(rows, rows.new_ones(()), None, None, spec)

        return _region_apply(scaled, qmap, per_region)
    return _quantize_with(input, scale, zero_point, block_size, _element_round(qmap, output_code, seed))


quantized_ops_lib.impl("quantize", N.device_guarded(quantize), "CUDA")


@torch.library.register_fake("quantized_ops::quantize")
def _(input, scale, zero_point=None, axes=None, block_size=None, qmap=None, output_code=None, seed=None):
    dtype = torch.result_type(input, scale)
    return torch.empty_like(input, dtype=dtype, memory_format=torch.contiguous_format)


quantized_ops_lib.define(
    "dequantize(Tensor input, Tensor scale, Tensor? zero_point=None, "
    "SymInt[]? axes=None, int? block_size=None, Tensor? input_qmap=None, "
    "Tensor? output_qmap=None) -> Tensor"
)


def dequantize(input, scale, zero_point=None, axes=None, block_size=None, input_qmap=None, output_qmap=None):
    """``round_out((round_in(input) - zero_point) * scale)`` (reference ``quantized.py:527-571``)."""
    x = input
    if input_qmap is not None and torch.result_type(x, scale) != x.dtype:
        x = vmap(x, input_qmap)  # rounds in the input's dtype before the promotion
        input_qmap = None
    x, scale, zero_point = _prepare_params(x, scale, zero_point)
    x = x.contiguous()
    out = torch.empty_like(x)
    geom = _broadcast_geometry(x.shape, scale, block_size)
    r_in = R.none_round() if input_qmap is None else R.table_round(input_qmap)
    r_out = R.none_round() if output_qmap is None else R.table_round(output_qmap)
    N.check(N.lib().vq_dequantize(x.data_ptr(), scale.data_ptr(), _ptr(zero_point), out.data_ptr(),
                                  _dtype_id(x.dtype), _dtype_id(scale.dtype), geom, r_in.ref, r_out.ref, _stream()),
            "vq_dequantize")
    return out


quantized_ops_lib.impl("dequantize", N.device_guarded(dequantize), "CUDA")


@torch.library.register_fake("quantized_ops::dequantize")
def _(input, scale, zero_point=None, axes=None, block_size=None, input_qmap=None, output_qmap=None):
    dtype = torch.result_type(input, scale)
    return torch.empty_like(input, dtype=dtype, memory_format=torch.contiguous_format)


# ---------------------------------------------------------------------------
# microscaling
# ---------------------------------------------------------------------------
def _block_geometry(shape, axes, block_size):
    """``(VqBlocks, scale_shape)`` for blocks of ``block_size`` along one or two axes."""
    nd = len(shape)
    axes = [axes] if isinstance(axes, int) else list(axes)
    axes = sorted({a + nd if a < 0 else a for a in axes})
    if not axes or len(axes) > 2 or any(a < 0 or a >= nd for a in axes):
        raise NotImplementedError(f"blocks along axes {axes} of a {nd}-d tensor")
    b = N.VqBlocks()
    prod = lambda xs: int(math.prod(xs))  # noqa: E731
    if len(axes) == 1:
        (a,) = axes
        b.O, b.A, b.M, b.B, b.I = prod(shape[:a]), 1, 1, shape[a], prod(shape[a + 1:])
        b.block_a, b.block_b = 1, block_size
    else:
        a0, a1 = axes
        b.O, b.A, b.M = prod(shape[:a0]), shape[a0], prod(shape[a0 + 1:a1])
        b.B, b.I = shape[a1], prod(shape[a1 + 1:])
        b.block_a, b.block_b = block_size, block_size
    scale_shape = list(shape)
    for a in axes:
        scale_shape[a] = -(-shape[a] // block_size)
    return b, scale_shape


def _scale_rule(x, quant_max, power_of_two, scale_qmap, global_scale):
    rule = N.VqScaleRule()
    rule.quant_max = float(quant_max)
    rule.power_of_two = int(bool(power_of_two))
    keep = []
    if global_scale is not None:
        if global_scale.numel() != 1:
            raise ValueError("global_scale must hold one element")
        gs = global_scale
        if gs.dtype not in _DTYPE_ID:
            gs = gs.to(x.dtype)
        if gs.dtype != x.dtype and not (gs.dim() == 0 and gs.dtype == torch.float32):
            gs = gs.to(torch.promote_types(gs.dtype, x.dtype))
        gs = gs.to(x.device)
        rule.global_scale = gs.data_ptr()
        rule.global_scale_dtype = _dtype_id(gs.dtype)
        keep.append(gs)
    if scale_qmap is not None and not power_of_two:
        spec = R.table_round(scale_qmap)
        rule.scale_round = spec.c
        keep.append(spec)
    else:
        rule.scale_round.mode = N.ROUND_NONE
    return rule, keep


quantized_ops_lib.define(
    "calculate_mx_qparam(Tensor self, SymInt[] axes, int block_size, "
    "float quant_max, bool force_scale_power_of_two=False, "
    "Tensor scale_qmap=None, Tensor? global_scale=None) -> Tensor"
)


def _mx_compute_dtype(x, global_scale):
    if global_scale is not None and global_scale.dim() > 0 and global_scale.is_floating_point():
        return torch.promote_types(x.dtype, global_scale.dtype)
    return x.dtype


def calculate_mx_qparam(input, axes, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None,
                        global_scale=None):
    """Per-block scale (reference ``quantized.py:966-1031``)."""
    assert block_size > 0
    x = input.contiguous()
    blocks, scale_shape = _block_geometry(x.shape, axes, block_size)
    rule, keep = _scale_rule(x, quant_max, force_scale_power_of_two, scale_qmap, global_scale)
    scale = torch.empty(scale_shape, dtype=x.dtype, device=x.device)
    N.check(N.lib().vq_mx_qparam(x.data_ptr(), scale.data_ptr(), _dtype_id(x.dtype), blocks, rule, _stream()),
            "vq_mx_qparam")
    del keep
    return scale


quantized_ops_lib.impl("calculate_mx_qparam", N.device_guarded(calculate_mx_qparam), "CUDA")


def _scale_shape(shape, axes, block_size):
    nd = len(shape)
    axes = [axes] if isinstance(axes, int) else list(axes)
    out = list(shape)
    for a in axes:
        out[a % nd] = -(-shape[a % nd] // block_size)
    return out


@torch.library.register_fake("quantized_ops::calculate_mx_qparam")
def _(input, axes, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None, global_scale=None):
    return input.new_empty(_scale_shape(input.shape, axes, block_size))


quantized_ops_lib.define(
    "quantize_mx(Tensor self, Tensor qmap, SymInt[] axes, int block_size, "
    "float quant_max, bool force_scale_power_of_two=False, "
    "Tensor scale_qmap=None, Tensor output_code=None, Tensor? seed=None, "
    "Tensor? global_scale=None) -> (Tensor, Tensor)"
)


def quantize_mx(input, qmap, axes, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None,
                output_code=None, seed=None, global_scale=None):
    """One pass: block amax -> scale -> codes (reference ``quantized.py:1080-1115``).
    Returns ``(scale, codes)``."""
    assert block_size > 0
    x = input.contiguous()
    if qmap is not None and seed is None and not _is_table(qmap) and qmap.dim() > 1:
        scale = calculate_mx_qparam(x, axes, block_size, quant_max, force_scale_power_of_two, scale_qmap,
                                    global_scale)
        element_scale = scale if global_scale is None else scale * global_scale
        return scale, quantize(x, element_scale, None, axes, block_size, qmap, output_code, None)
    blocks, scale_shape = _block_geometry(x.shape, axes, block_size)
    rule, keep = _scale_rule(x, quant_max, force_scale_power_of_two, scale_qmap, global_scale)
    spec = _element_round(qmap, output_code, seed)
    scale = torch.empty(scale_shape, dtype=x.dtype, device=x.device)
    codes = torch.empty_like(x)
    N.check(N.lib().vq_quantize_mx(x.data_ptr(), scale.data_ptr(), codes.data_ptr(), _dtype_id(x.dtype), blocks,
                                   rule, spec.ref, _stream()), "vq_quantize_mx")
    del keep
    return scale, codes


quantized_ops_lib.impl("quantize_mx", N.device_guarded(quantize_mx), "CUDA")


@torch.library.register_fake("quantized_ops::quantize_mx")
def _(input, qmap, axes, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None,
      output_code=None, seed=None, global_scale=None):
    return (input.new_empty(_scale_shape(input.shape, axes, block_size)),
            torch.empty_like(input, memory_format=torch.contiguous_format))


quantized_ops_lib.define(
    "dequantize_mx(Tensor self, Tensor scale, int block_size, "
    "Tensor? code=None, Tensor? global_scale=None) -> Tensor"
)


def _decode_and_scale(x, scale, code, block_size, global_scale=None):
    """``code[x] * scale [* global_scale]`` with each product rounded to the
    operand dtype (reference ``quantized.py:574-591``)."""
    if code is not None and code.dim() != 1:
        tables = code.reshape(-1, code.shape[-1])
        x = _region_apply(x.contiguous(), code,
                          lambda rows, r: _decode_and_scale(rows, None, tables[r].contiguous(), None))
        code = None
        if scale is None and global_scale is None:
            return x
    dtype = x.dtype
    if scale is not None:
        dtype = torch.promote_types(dtype, scale.dtype) if scale.dim() > 0 else dtype
    if global_scale is not None and global_scale.dim() > 0:
        dtype = torch.promote_types(dtype, global_scale.dtype)
    x = x.contiguous()
    if dtype != x.dtype:
        if code is not None:
            x = _decode_and_scale(x, None, code, None)  # entries are read in the code's dtype first
            code = None
        x = x.to(dtype)
    if scale is not None and scale.dtype != dtype:
        scale = scale.to(dtype)
    if code is not None and code.dtype != dtype:
        code = code.to(dtype)
    out = torch.empty_like(x)
    if scale is not None:
        geom = _broadcast_geometry(x.shape, scale, block_size)
    else:
        geom = N.VqBroadcast()
        geom.ndim = 1
        geom.size[0], geom.div[0], geom.stride[0] = x.numel(), 1, 0
    gs_dtype = 0
    if global_scale is not None:
        if global_scale.dtype != dtype and not (global_scale.dim() == 0 and global_scale.dtype == torch.float32):
            global_scale = global_scale.to(dtype)
        gs_dtype = _dtype_id(global_scale.dtype)
    N.check(N.lib().vq_dequantize_mx(x.data_ptr(), _ptr(scale), None if code is None else code.contiguous().data_ptr(),
                                     0 if code is None else code.numel(), _ptr(global_scale), gs_dtype,
                                     out.data_ptr(), _dtype_id(dtype), geom, _stream()), "vq_dequantize_mx")
    return out


def dequantize_mx(input, scale, block_size, code=None, global_scale=None):
    """Read codes back as values (reference ``quantized.py:1125-1149``)."""
    return _decode_and_scale(input, scale, code, block_size, global_scale)


quantized_ops_lib.impl("dequantize_mx", N.device_guarded(dequantize_mx), "CUDA")


@torch.library.register_fake("quantized_ops::dequantize_mx")
def _(input, scale, block_size, code=None, global_scale=None):
    dtype = torch.promote_types(input.dtype, scale.dtype)
    if global_scale is not None:
        dtype = torch.promote_types(dtype, global_scale.dtype)
    return input.new_empty(input.shape, dtype=dtype)


# ---------------------------------------------------------------------------
# group-wise affine (KIVI)
# ---------------------------------------------------------------------------
quantized_ops_lib.define(
    "quantize_affine(Tensor self, Tensor qmap, SymInt[] axes, int block_size, "
    "float quant_min, float quant_max, Tensor scale_qmap=None) "
    "-> (Tensor, Tensor, Tensor)"
)


def quantize_affine(input, qmap, axes, block_size, quant_min, quant_max, scale_qmap=None):
    """Per-block ``[min, max] -> [quant_min, quant_max]`` (reference
    ``quantized.py:1227-1283``).  Returns ``(scale, zero_point, codes)``."""
    assert block_size > 0
    (axis,) = axes
    x = input.contiguous()
    blocks, scale_shape = _block_geometry(x.shape, [axis], block_size)
    spec = R.table_round(qmap)
    sspec = R.none_round() if scale_qmap is None else R.table_round(scale_qmap)
    scale = torch.empty(scale_shape, dtype=x.dtype, device=x.device)
    zero = torch.empty_like(scale)
    codes = torch.empty_like(x)
    N.check(N.lib().vq_quantize_affine(x.data_ptr(), scale.data_ptr(), zero.data_ptr(), codes.data_ptr(),
                                       _dtype_id(x.dtype), blocks, float(quant_min), float(quant_max), sspec.ref,
                                       spec.ref, _stream()), "vq_quantize_affine")
    return scale, zero, codes


quantized_ops_lib.impl("quantize_affine", N.device_guarded(quantize_affine), "CUDA")


@torch.library.register_fake("quantized_ops::quantize_affine")
def _(input, qmap, axes, block_size, quant_min, quant_max, scale_qmap=None):
    shape = _scale_shape(input.shape, axes, block_size)
    return (input.new_empty(shape), input.new_empty(shape),
            torch.empty_like(input, memory_format=torch.contiguous_format))


# ---------------------------------------------------------------------------
# tensor amax and the NVFP4 global scale
# ---------------------------------------------------------------------------
@N.device_guarded
def tensor_amax(x: torch.Tensor) -> torch.Tensor:
    """``max |x|`` as a 0-d float32 tensor (one kernel, no host sync)."""
    x = x if _is_dense(x) else x.contiguous()
    out = torch.zeros((), dtype=torch.float32, device=x.device)
    N.check(N.lib().vq_amax(x.data_ptr(), _dtype_id(x.dtype), x.numel(), out.data_ptr(), _stream()), "vq_amax")
    return out


@N.device_guarded
def calculate_global_scale(input: torch.Tensor, quant_max: float, scale_max: float) -> torch.Tensor:
    """NVFP4's per-tensor scale ``amax / (quant_max * scale_max)`` in the
    input's dtype (reference ``fake_quantize.py:142-160``)."""
    return global_scale_of_amax(tensor_amax(input), input.dtype, quant_max, scale_max)


def global_scale_of_amax(amax: torch.Tensor, dtype, quant_max: float, scale_max: float) -> torch.Tensor:
    """``calculate_global_scale`` from a tensor's ``max |x|`` (a 0-d float32 tensor; a sharded tensor's after an
    all-reduce), in the tensor's ``dtype``."""
    amax = amax.to(dtype).reshape(1)
    # A correctly rounded division by the float32 divisor, as the CPU op does.
    divisor = torch.full((), float(quant_max * scale_max), dtype=torch.float32, device=amax.device)
    ratio = _quantize_with(amax, divisor, None, None, R.none_round()).reshape(())
    return ratio.clamp_min(torch.finfo(torch.float32).tiny)


# ---------------------------------------------------------------------------
# GEMMs
# ---------------------------------------------------------------------------
_ACT_LAYOUTS, _WGT_LAYOUTS, _OUT_LAYOUTS = ("xc", "cx"), ("kc", "ck"), ("xk", "kx")
_IN_KIND = {torch.bfloat16: N.IN_BF16, torch.float16: N.IN_F16}


def _parse_layout(layout: str):
    operands, out = layout.split("->")
    act, wgt = operands.split(",")
    assert act in _ACT_LAYOUTS, layout
    assert wgt in _WGT_LAYOUTS, layout
    assert out in _OUT_LAYOUTS, layout
    return act, wgt, out


@N.device_guarded
def gemm_tn(a: torch.Tensor, b: torch.Tensor, *, out_dtype=None, alpha=None, bias=None, in_kind=None,
            alpha_cols=None, residual=None, causal=None, gated_scale=None, round_acc=False, out=None):
    """``out[..., m, n] = alpha * sum_k a[..., m, k] * b[..., n, k] + bias[n]`` on the
    tensor cores (fp32 accumulation, one rounding to ``out_dtype``).

    ``alpha_cols [N]`` multiplies column ``n`` after ``alpha`` (per-output-channel scales);
    ``residual`` (the output's shape and dtype) is added after the rounding and the sum is
    rounded again, as ``residual + linear(...)`` would be.  ``causal=("scores", T)`` says
    that ``out[..., r, n]`` with ``n > r % T`` is never read (tiles of only such elements may
    stay unwritten); ``causal=("probabilities", T)`` that ``a[..., r, k]`` is zero for
    ``k > r % T`` (the contraction may stop early).  ``gated_scale`` selects the SwiGLU epilogue:
    ``b``'s rows interleave 32 gate rows with their 32 up rows and the result is the ``[..., N / 2]``
    e4m3 bytes of ``(silu(gate) * up) / gated_scale``.  ``round_acc`` rounds the accumulator to
    ``out_dtype`` before ``alpha`` / ``alpha_cols`` / ``bias`` (matmul, then dequantize: the two
    roundings of a converted per-tensor graph).

    ``a`` is ``[*batch, M, K]`` and ``b`` ``[*batch, N, K]`` or ``[N, K]``; both are
    used K-contiguous.  ``out``: a dense tensor to write the result into instead of a new one.  ``in_kind`` overrides the operand element kind for 8-bit
    operands stored as ``uint8``/``float8`` bytes.
    """
    if in_kind is None:
        if a.dtype != b.dtype or a.dtype not in _IN_KIND:
            raise NotImplementedError(
                f"the tensor-core GEMM takes bfloat16 or float16 operands of one dtype, not {a.dtype} x {b.dtype}")
        in_kind = _IN_KIND[a.dtype]
    elem = a.element_size()
    m, k = a.shape[-2], a.shape[-1]
    n = b.shape[-2]
    if b.shape[-1] != k:
        raise ValueError(f"contraction extents differ: {tuple(a.shape)} x {tuple(b.shape)}")
    pad = (-k) % (16 // elem)
    if pad:  # rows must be multiples of 16 bytes for the TMA descriptors
        a = torch.nn.functional.pad(a, (0, pad))
        b = torch.nn.functional.pad(b, (0, pad))
        k += pad
    batch_shape = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    if b.dim() == 2:
        # shared weight: fold the batch into the rows
        a2 = a.reshape(-1, k).contiguous()
        b2 = b.contiguous()
        batch, rows = 1, a2.shape[0]
        stride_a = stride_b = 0
    else:
        a2 = a.expand(*batch_shape, m, k).reshape(-1, m, k).contiguous()
        b2 = b.expand(*batch_shape, n, k).reshape(-1, n, k).contiguous()
        batch, rows = a2.shape[0], m
        stride_a, stride_b = m * k, n * k
    out_dtype = out_dtype or (a.dtype if a.dtype in _DTYPE_ID else torch.bfloat16)
    n_out = n
    if gated_scale is not None:
        if n % 64 or out_dtype != torch.bfloat16 or bias is not None or residual is not None or k == 0:
            raise NotImplementedError("the gated epilogue takes bfloat16 linears with N a multiple of 64, no bias, "
                                      "no residual")
        n_out = n // 2
        out = torch.empty((batch, rows, n_out), dtype=torch.uint8, device=a.device)
    elif out is not None:
        # the caller's buffer (e.g. memory its peers can read): dense, the result's size and dtype
        if out.dtype != out_dtype or out.numel() != batch * rows * n or not out.is_contiguous():
            raise ValueError("out must be a dense tensor of the result's size and dtype")
        out = out.view(batch, rows, n)
    else:
        out = torch.empty((batch, rows, n), dtype=out_dtype, device=a.device)
    if bias is not None:
        bias = bias.contiguous()
    epi = None
    if alpha_cols is not None or residual is not None or causal is not None or gated_scale is not None or round_acc:
        epi = N.VqGemmEpilogue()
        epi.round_acc = int(bool(round_acc))
        if gated_scale is not None:
            gated_scale = _as_scalar_param(gated_scale, a.device)
            epi.gate_scale, epi.gate_scale_dtype = gated_scale.data_ptr(), _dtype_id(gated_scale.dtype)
        if causal is not None:
            epi.causal_mode = {"scores": 1, "probabilities": 2}[causal[0]]
            epi.causal_period = int(causal[1])
        if alpha_cols is not None:
            alpha_cols = alpha_cols.reshape(-1).contiguous()
            if alpha_cols.numel() != n or alpha_cols.dtype not in _DTYPE_ID:
                raise ValueError(f"alpha_cols must hold {n} bfloat16/float16/float32 values")
            epi.alpha_cols, epi.alpha_cols_dtype = alpha_cols.data_ptr(), _dtype_id(alpha_cols.dtype)
        if residual is not None:
            if residual.dtype != out_dtype or residual.numel() != out.numel():
                raise ValueError("the residual must have the output's shape and dtype")
            residual = residual.contiguous()
            epi.residual, epi.ldr, epi.strideR = residual.data_ptr(), n, rows * n
    if out.numel():
        if k == 0:
            out.zero_()   # an empty sum; the epilogue's additions are all that is left
            if bias is not None:
                out += bias.to(out_dtype)
            if residual is not None:
                out += residual.reshape(out.shape)
        else:
            N.check(N.lib().vq_gemm_tn_ex(
                a2.data_ptr(), b2.data_ptr(), out.data_ptr(), in_kind, _dtype_id(out_dtype), rows, n, k, k, k, n_out,
                batch, stride_a, stride_b, rows * n_out, _ptr(alpha), 0 if alpha is None else _dtype_id(alpha.dtype),
                _ptr(bias), 0 if bias is None else _dtype_id(bias.dtype), epi, _stream()), "vq_gemm_tn_ex")
    return out.reshape(*batch_shape, m, n_out) if b.dim() > 2 else out.reshape(*a.shape[:-1], n_out)


def _as_scalar_param(t, device):
    if t is None:
        return None
    if t.numel() != 1:
        raise NotImplementedError("alpha must hold one element")
    if t.dtype not in _DTYPE_ID:
        t = t.float()
    return t.to(device).reshape(())


def _gemm_in_layout(native, activation, weight, layout, out_dtype, bias=None, alpha=None):
    act, wgt, out_l = _parse_layout(layout)
    n_act, n_wgt, n_out = _parse_layout(native)
    if act == "cx":
        activation = activation.mT
    # the kernel wants the weight [out, contraction]
    w = weight if wgt == "kc" else weight.mT
    y = gemm_tn(activation, w, out_dtype=out_dtype, alpha=alpha, bias=bias)
    return y.mT.contiguous() if out_l != n_out else y


quantized_ops_lib.define(
    f'linear(Tensor input, Tensor weight, Tensor? bias=None, *, str layout="{LINEAR_LAYOUT}", '
    "ScalarType? out_dtype=None) -> Tensor"
)
quantized_ops_lib.define(
    f'matmul(Tensor self, Tensor other, *, str layout="{MATMUL_LAYOUT}", ScalarType? out_dtype=None) -> Tensor'
)


def linear(input, weight, bias=None, *, layout=LINEAR_LAYOUT, out_dtype=None):
    """``aten.linear`` on operands stored as ``layout`` says (reference ``ops/layout.py:266-278``)."""
    return _gemm_in_layout(LINEAR_LAYOUT, input, weight, layout, out_dtype, bias)


def matmul(input, other, *, layout=MATMUL_LAYOUT, out_dtype=None):
    """``aten.matmul`` on operands stored as ``layout`` says (reference ``ops/layout.py:281-290``)."""
    return _gemm_in_layout(MATMUL_LAYOUT, input, other, layout, out_dtype)


quantized_ops_lib.impl("linear", N.device_guarded(linear), "CUDA")
quantized_ops_lib.impl("matmul", N.device_guarded(matmul), "CUDA")


def _gemm_out_shape(activation, weight, layout, weight_is_matrix):
    act, wgt, out_l = _parse_layout(layout)
    a_shape = list(activation.shape)
    if act == "cx":
        a_shape[-2], a_shape[-1] = a_shape[-1], a_shape[-2]
    n = weight.shape[-2] if wgt == "kc" else weight.shape[-1]
    if weight.dim() > 2:
        batch = torch.broadcast_shapes(tuple(a_shape[:-2]), tuple(weight.shape[:-2]))
        shape = [*batch, a_shape[-2], n]
    else:
        shape = [*a_shape[:-1], n]
    if out_l == "kx":
        shape[-2], shape[-1] = shape[-1], shape[-2]
    return shape


@torch.library.register_fake("quantized_ops::linear")
def _(input, weight, bias=None, *, layout=LINEAR_LAYOUT, out_dtype=None):
    return input.new_empty(_gemm_out_shape(input, weight, layout, True), dtype=out_dtype or input.dtype)


@torch.library.register_fake("quantized_ops::matmul")
def _(input, other, *, layout=MATMUL_LAYOUT, out_dtype=None):
    return input.new_empty(_gemm_out_shape(input, other, layout, False), dtype=out_dtype or input.dtype)


quantized_ops_lib.define(
    "linear_mx(Tensor input, Tensor weight, Tensor? bias=None, *, "
    "Tensor? input_scale=None, Tensor? weight_scale=None, "
    "int? block_size=None, Tensor? input_code=None, Tensor? weight_code=None, "
    "Tensor? alpha=None, Tensor? A_data=None, Tensor? A_indices=None, "
    f'Tensor? A_indptr=None, str layout="{LINEAR_LAYOUT}", '
    "ScalarType? out_dtype=None) -> Tensor"
)
quantized_ops_lib.define(
    "matmul_mx(Tensor self, Tensor other, *, Tensor? input_scale=None, "
    "Tensor? weight_scale=None, int? block_size=None, Tensor? input_code=None, "
    "Tensor? weight_code=None, Tensor? alpha=None, Tensor? A_data=None, "
    "Tensor? A_indices=None, Tensor? A_indptr=None, "
    f'str layout="{MATMUL_LAYOUT}", ScalarType? out_dtype=None) -> Tensor'
)


def _read_operand(x, scale, code, block_size):
    if scale is None and code is None:
        return x
    return _decode_and_scale(x, scale, code, block_size)


# "auto": apply block scales inside the GEMM's main loop when that is estimated to be faster than a
# read-back pass followed by the plain GEMM; "always" / "never" force the choice (tests, measurements).
MX_IN_MAINLOOP = "auto"


def _in_mainloop_pays(rows, n, k, batch, scaled_a, scaled_b, shared_weight):
    """Measured on a B200 (N = 4096 .. 28672, K = 4096 .. 14336, 16 .. 2048 rows): the transform warps
    add about 0.38 us per 64 elements of K to every wave of 74 CTA-pair tiles, while a separate read-back costs
    its bytes (2 read + 2 written per element of a scaled operand) at about 4.5 TB/s plus 3 us per launch,
    and at most 128 rows the plain GEMM falls back to its slower single-CTA tiles (about 15 us)."""
    tiles = -(-rows // 256) * -(-n // 256) * batch
    cost = 0.38 * -(-k // 64) * -(-tiles // 74)
    elements = (rows * batch if scaled_a else 0) + (n * (1 if shared_weight else batch) if scaled_b else 0)
    gain = 4.0 * elements * k / 4.5e6 + 3.0 * (int(scaled_a) + int(scaled_b)) + (15.0 if rows <= 128 else 0.0)
    return cost < gain


def _scales_per_row(x, scale, block_size):
    """True when ``scale`` is contiguous bfloat16 with one value per ``block_size`` elements of ``x``'s last dimension."""
    if scale is None:
        return True
    want = (*x.shape[:-1], -(-x.shape[-1] // block_size))
    return scale.dtype == torch.bfloat16 and tuple(scale.shape) == want and scale.is_contiguous()


def _mx_gemm_in_mainloop(native, a, b, bias, input_scale, weight_scale, block_size, alpha, layout, dtype):
    """The contraction straight from block-scaled bfloat16 codes (``vq_gemm_mx``), or ``None`` when the call is
    not of the shape that kernel takes (both operands K-contiguous with scales along K, a shared 2-D weight or
    equal batches) or a separate read-back is estimated to be faster (``_in_mainloop_pays``)."""
    act, wgt, out_l = _parse_layout(layout)
    if act != "xc" or wgt != "kc" or out_l != _parse_layout(native)[2]:
        return None
    if input_scale is None and weight_scale is None:
        return None
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.dim() < 2 or b.dim() < 2:
        return None
    if not isinstance(block_size, int) or block_size < 8 or block_size & (block_size - 1):
        return None
    k, n = a.shape[-1], b.shape[-2]
    if b.shape[-1] != k or k % 8 or k == 0:
        return None
    if not (_scales_per_row(a, input_scale, block_size) and _scales_per_row(b, weight_scale, block_size)):
        return None
    if b.dim() == 2:
        a2, b2 = a.reshape(-1, k), b
        batch, rows, stride_a, stride_b = 1, a2.shape[0], 0, 0
        out_shape = (*a.shape[:-1], n)
    else:
        if a.shape[:-2] != b.shape[:-2]:
            return None
        m = a.shape[-2]
        a2, b2 = a.reshape(-1, m, k), b.reshape(-1, n, k)
        batch, rows, stride_a, stride_b = a2.shape[0], m, m * k, n * k
        out_shape = (*a.shape[:-2], m, n)
    if batch == 0 or n == 0 or rows == 0 or MX_IN_MAINLOOP == "never":
        return None
    if MX_IN_MAINLOOP != "always" and not _in_mainloop_pays(rows, n, k, batch, input_scale is not None,
                                                            weight_scale is not None, b.dim() == 2):
        return None
    a2, b2 = a2.contiguous(), b2.contiguous()
    if bias is not None:
        bias = bias.contiguous()
    out = torch.empty((batch, rows, n), dtype=dtype, device=a.device)
    rc = N.lib().vq_gemm_mx(a2.data_ptr(), _ptr(input_scale), b2.data_ptr(), _ptr(weight_scale), block_size,
                            out.data_ptr(), _dtype_id(dtype), rows, n, k, k, k, n, batch, stride_a, stride_b, rows * n,
                            _ptr(alpha), 0 if alpha is None else _dtype_id(alpha.dtype), _ptr(bias),
                            0 if bias is None else _dtype_id(bias.dtype), _stream())
    if rc == -3:   # VQ_EUNSUPPORTED: no CTA pairs on this device
        return None
    N.check(rc, "vq_gemm_mx")
    return out.reshape(out_shape)


def _mx_gemm(native, a, b, bias, input_scale, weight_scale, block_size, input_code, weight_code, alpha, outliers,
             layout, out_dtype):
    if input_code is None and weight_code is None and all(t is None for t in outliers):
        dtype = a.dtype if out_dtype is None else out_dtype
        if dtype in _DTYPE_ID:
            y = _mx_gemm_in_mainloop(native, a, b, bias, input_scale, weight_scale, block_size,
                                     _as_scalar_param(alpha, a.device), layout, dtype)
            if y is not None:
                return y
    a = _read_operand(a, input_scale, input_code, block_size)
    b = _read_operand(b, weight_scale, weight_code, block_size)
    dtype = a.dtype if out_dtype is None else out_dtype
    if dtype not in _DTYPE_ID:
        raise NotImplementedError(f"output dtype {dtype}")
    if all(t is None for t in outliers):
        return _gemm_in_layout(native, a, b, layout, dtype, bias, _as_scalar_param(alpha, a.device))
    if any(t is None for t in outliers):
        raise ValueError("A_data, A_indices and A_indptr come together")
    # The outliers' product joins the float32 sum of product, alpha and bias before the one rounding
    # (reference quantized.py:688-722); it is computed [tokens, out] and stored as `layout` says last.
    act, wgt, out_l = _parse_layout(layout)
    n_out = _parse_layout(native)[2]
    y = _gemm_in_layout(native, a, b, f"{act},{wgt}->{n_out}", torch.float32, bias, _as_scalar_param(alpha, a.device))
    data, indices, indptr = outliers
    y = y + torch.ops.quantized_ops.spmm_csr(data, indices, indptr, b, None, None, None, wgt, out_dtype=torch.float32)
    y = y.to(dtype)
    return y.mT.contiguous() if out_l != n_out else y


# ---------------------------------------------------------------------------
# convolutions (a converted CNN graph's call targets; not a tuned path)
# ---------------------------------------------------------------------------
TENSOR_LAYOUT = "nchw"
quantized_ops_lib.define(
    "conv2d(Tensor input, Tensor weight, Tensor? bias=None, SymInt[2] stride=[1, 1], SymInt[2] padding=[0, 0], "
    f'SymInt[2] dilation=[1, 1], SymInt groups=1, *, str layout="{TENSOR_LAYOUT}", ScalarType? out_dtype=None) '
    "-> Tensor"
)
quantized_ops_lib.define(
    "conv2d_mx(Tensor input, Tensor weight, Tensor? bias=None, SymInt[2] stride=1, SymInt[2] padding=0, "
    "SymInt[2] dilation=1, SymInt groups=1, *, Tensor? input_scale=None, Tensor? weight_scale=None, "
    f'int? block_size=None, Tensor? input_code=None, Tensor? weight_code=None, str layout="{TENSOR_LAYOUT}", '
    "ScalarType? out_dtype=None) -> Tensor"
)


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def conv2d(input, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, *,
           layout=TENSOR_LAYOUT, out_dtype=None):
    """``aten.conv2d`` on feature maps stored as ``layout`` says (reference ``ops/layout.py:170-218``): under
    ``"nhwc"`` input and result are channels-last and a dense convolution's weight is ``[H, W, in, out]``;
    ``out_dtype`` sums in float32 and returns that dtype.  The convolution itself is the library's (cuDNN)."""
    if layout not in ("nchw", "nhwc"):
        raise ValueError(f"unknown tensor layout {layout!r}")
    nhwc = layout == "nhwc"
    if nhwc:
        input = input.permute(0, 3, 1, 2)
        if groups == 1:
            weight = weight.permute(3, 2, 0, 1)
    if out_dtype is not None:
        input, weight = input.float(), weight.float()
        bias = None if bias is None else bias.float()
    out = torch.nn.functional.conv2d(input, weight, bias, _pair(stride), _pair(padding), _pair(dilation), groups)
    if out_dtype is not None:
        out = out.to(out_dtype)
    return out.permute(0, 2, 3, 1) if nhwc else out


def conv2d_mx(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, *, input_scale=None,
              weight_scale=None, block_size=None, input_code=None, weight_code=None, layout=TENSOR_LAYOUT,
              out_dtype=None):
    """The convolution of block-scaled operands (reference ``ops/quantized.py:596-645``): both are read back
    (``code[x] * scale``, this package's kernel) and handed to ``conv2d``."""
    input = _read_operand(input, input_scale, input_code, block_size)
    weight = _read_operand(weight, weight_scale, weight_code, block_size)
    return conv2d(input, weight, bias, stride, padding, dilation, groups, layout=layout, out_dtype=out_dtype)


quantized_ops_lib.impl("conv2d", N.device_guarded(conv2d), "CUDA")
quantized_ops_lib.impl("conv2d_mx", N.device_guarded(conv2d_mx), "CUDA")


def _conv_out_shape(input, weight, stride, padding, dilation, groups, layout):
    nhwc = layout == "nhwc"
    n, h, w = (input.shape[0], input.shape[1], input.shape[2]) if nhwc else (input.shape[0], input.shape[2], input.shape[3])
    if nhwc and groups == 1:
        kh, kw, out_c = weight.shape[0], weight.shape[1], weight.shape[3]
    else:
        out_c, kh, kw = weight.shape[0], weight.shape[2], weight.shape[3]
    (sh, sw), (ph, pw), (dh, dw) = _pair(stride), _pair(padding), _pair(dilation)
    oh = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    ow = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    return (n, oh, ow, out_c) if nhwc else (n, out_c, oh, ow)


@torch.library.register_fake("quantized_ops::conv2d")
def _(input, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, *, layout=TENSOR_LAYOUT,
      out_dtype=None):
    return input.new_empty(_conv_out_shape(input, weight, stride, padding, dilation, groups, layout),
                           dtype=out_dtype or input.dtype)


@torch.library.register_fake("quantized_ops::conv2d_mx")
def _(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, *, input_scale=None, weight_scale=None,
      block_size=None, input_code=None, weight_code=None, layout=TENSOR_LAYOUT, out_dtype=None):
    return input.new_empty(_conv_out_shape(input, weight, stride, padding, dilation, groups, layout),
                           dtype=out_dtype or input.dtype)


def linear_mx(input, weight, bias=None, *, input_scale=None, weight_scale=None, block_size=None, input_code=None,
              weight_code=None, alpha=None, A_data=None, A_indices=None, A_indptr=None, layout=LINEAR_LAYOUT,
              out_dtype=None):
    """Microscaling linear: both operands are read back through their codebook
    and block scales (each product rounded to the operand dtype), multiplied
    with fp32 accumulation, scaled by ``alpha``, biased and rounded once
    (reference ``quantized.py:662-723``)."""
    return _mx_gemm(LINEAR_LAYOUT, input, weight, bias, input_scale, weight_scale, block_size, input_code,
                    weight_code, alpha, (A_data, A_indices, A_indptr), layout, out_dtype)


def matmul_mx(self, other, *, input_scale=None, weight_scale=None, block_size=None, input_code=None,
              weight_code=None, alpha=None, A_data=None, A_indices=None, A_indptr=None, layout=MATMUL_LAYOUT,
              out_dtype=None):
    """Microscaling matmul (reference ``quantized.py:752-805``)."""
    return _mx_gemm(MATMUL_LAYOUT, self, other, None, input_scale, weight_scale, block_size, input_code,
                    weight_code, alpha, (A_data, A_indices, A_indptr), layout, out_dtype)


quantized_ops_lib.impl("linear_mx", N.device_guarded(linear_mx), "CUDA")
quantized_ops_lib.impl("matmul_mx", N.device_guarded(matmul_mx), "CUDA")


@torch.library.register_fake("quantized_ops::linear_mx")
def _(input, weight, bias=None, **kwargs):
    layout = kwargs.get("layout", LINEAR_LAYOUT)
    return input.new_empty(_gemm_out_shape(input, weight, layout, True), dtype=kwargs.get("out_dtype") or input.dtype)


@torch.library.register_fake("quantized_ops::matmul_mx")
def _(self, other, **kwargs):
    layout = kwargs.get("layout", MATMUL_LAYOUT)
    return self.new_empty(_gemm_out_shape(self, other, layout, False), dtype=kwargs.get("out_dtype") or self.dtype)


def gemm_status(reset=True):
    """Raise if a tensor-core GEMM launched earlier gave up on a barrier wait
    (synchronises the device)."""
    torch.cuda.synchronize()
    N.check(N.lib().vq_gemm_status(int(reset)), "vq_gemm_status")


# ---------------------------------------------------------------------------
# Hadamard rotation, two-layout quantize, attention
# ---------------------------------------------------------------------------
HADAMARD_SIGNS = (1, 1, 1, -1, 1, -1, -1, -1, -1, -1, -1, 1, -1, 1, -1, -1)


def hadamard_matrix(device=None) -> torch.Tensor:
    """``diag(signs) @ H16 / 4``: Sylvester's 16x16 Hadamard matrix with Transformer
    Engine's fixed sign vector (reference ``fake_quantize.py:47-65``)."""
    h = torch.ones(1, 1)
    while h.shape[0] < HADAMARD_SIZE:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)])
    signs = torch.tensor(HADAMARD_SIGNS, dtype=torch.float32)
    return (signs[:, None] * h / math.sqrt(HADAMARD_SIZE)).to(device)


@N.device_guarded
def hadamard_rotate(x: torch.Tensor, axis: int, matrix: torch.Tensor) -> torch.Tensor:
    """Multiply each run of 16 elements along ``axis`` (the last or second-to-last) by
    ``matrix`` in fp32; the axis is zero padded to whole runs and keeps the padded
    length (reference ``quantized.py:1038-1067``)."""
    axis %= x.dim()
    if axis < x.dim() - 2:
        raise ValueError(f"cannot rotate along axis {axis} of {x.dim()}")
    x = x.contiguous()
    A = x.shape[axis]
    O = int(math.prod(x.shape[:axis]))
    I = int(math.prod(x.shape[axis + 1:]))
    padded = -(-A // HADAMARD_SIZE) * HADAMARD_SIZE
    out = torch.empty(*x.shape[:axis], padded, *x.shape[axis + 1:], dtype=x.dtype, device=x.device)
    m = matrix.to(device=x.device, dtype=torch.float32).contiguous()
    N.check(N.lib().vq_hadamard_rotate(x.data_ptr(), out.data_ptr(), _dtype_id(x.dtype), m.data_ptr(), O, A, I,
                                       _stream()), "vq_hadamard_rotate")
    return out


quantized_ops_lib.define(
    "quantize_mx_transpose(Tensor self, Tensor qmap, int block_size, "
    "float quant_max, bool force_scale_power_of_two=False, "
    "Tensor scale_qmap=None, Tensor output_code=None, Tensor? seed=None, "
    "Tensor? global_scale=None, Tensor? transpose_seed=None, "
    "Tensor? transpose_global_scale=None, Tensor? hadamard=None) "
    "-> (Tensor, Tensor, Tensor, Tensor)"
)


def quantize_mx_transpose(input, qmap, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None,
                          output_code=None, seed=None, global_scale=None, transpose_seed=None,
                          transpose_global_scale=None, hadamard=None):
    """``quantize_mx`` of the input along its last axis and of its transpose (optionally
    Hadamard-rotated) along the transpose's last axis (reference ``quantized.py:1171-1215``)."""
    t = input.mT.contiguous()
    if hadamard is not None:
        t = hadamard_rotate(t, -1, hadamard)
    common = (qmap, (-1,), block_size, quant_max, force_scale_power_of_two, scale_qmap, output_code)
    return (*quantize_mx(input, *common, seed, global_scale),
            *quantize_mx(t, *common, transpose_seed, transpose_global_scale))


quantized_ops_lib.impl("quantize_mx_transpose", N.device_guarded(quantize_mx_transpose), "CUDA")


@torch.library.register_fake("quantized_ops::quantize_mx_transpose")
def _(input, qmap, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None, output_code=None,
      seed=None, global_scale=None, transpose_seed=None, transpose_global_scale=None, hadamard=None):
    t_shape = list(input.shape)
    t_shape[-1], t_shape[-2] = t_shape[-2], t_shape[-1]
    if hadamard is not None:
        t_shape[-1] = -(-t_shape[-1] // HADAMARD_SIZE) * HADAMARD_SIZE
    return (input.new_empty(_scale_shape(input.shape, [-1], block_size)), torch.empty_like(input),
            input.new_empty(_scale_shape(t_shape, [-1], block_size)), input.new_empty(t_shape))


quantized_ops_lib.define(
    "sdpa_mx(Tensor query, Tensor key, Tensor value, Tensor? attn_mask=None, "
    "float dropout_p=0., bool is_causal=False, Tensor? query_residual=None, "
    "Tensor? key_residual=None, Tensor? value_residual=None, "
    "Tensor? residual_mask=None, *, float? scale=None, "
    "bool enable_gqa=False, Tensor? query_scale=None, Tensor? key_scale=None, "
    "Tensor? value_scale=None, int? block_size=None, Tensor? input_code=None, "
    "Tensor? weight_code=None, Tensor? probs_qmap=None, "
    "float? probs_quant_max=None, Tensor? probs_scale_qmap=None, "
    "Tensor? probs_code=None, bool force_scale_power_of_two=False) -> Tensor"
)


def _masked(scores, mask):
    if mask is None:
        return scores
    if mask.dtype == torch.bool:
        return scores.masked_fill(~mask, float("-inf"))
    return scores + mask


def sdpa_mx(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, query_residual=None,
            key_residual=None, value_residual=None, residual_mask=None, *, scale=None, enable_gqa=False,
            query_scale=None, key_scale=None, value_scale=None, block_size=None, input_code=None,
            weight_code=None, probs_qmap=None, probs_quant_max=None, probs_scale_qmap=None, probs_code=None,
            force_scale_power_of_two=False):
    """Attention over microscaling operands: read back q/k/v, scores and PV on the tensor
    cores, one softmax over main and residual keys, probabilities re-quantized with
    ``quantize_mx`` before the value matmul (reference ``quantized.py:836-928``)."""
    if is_causal and attn_mask is not None:
        raise ValueError("is_causal excludes an explicit attn_mask")
    q = _read_operand(query, query_scale, input_code, block_size)
    k = _read_operand(key, key_scale, weight_code, block_size)
    v = _read_operand(value, value_scale, weight_code, block_size)
    residual = key_residual is not None
    if enable_gqa:
        g = q.shape[-3] // k.shape[-3]
        k, v = k.repeat_interleave(g, dim=-3), v.repeat_interleave(g, dim=-3)
        if residual:
            key_residual = key_residual.repeat_interleave(g, dim=-3)
            value_residual = value_residual.repeat_interleave(g, dim=-3)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    scores = gemm_tn(q, k) * scale
    if is_causal:
        attn_mask = torch.ones(scores.shape[-2:], dtype=torch.bool, device=scores.device).tril()
    scores = _masked(scores, attn_mask)
    keys = scores.shape[-1]
    if residual:
        res = _masked(gemm_tn(query_residual, key_residual) * scale, residual_mask)
        scores = torch.cat([scores, res], dim=-1)
    probs = torch.softmax(scores, dim=-1)
    probs, res_probs = probs[..., :keys], probs[..., keys:]
    if probs_qmap is not None:
        p_scale, probs = quantize_mx(probs, probs_qmap, [-1], block_size, probs_quant_max,
                                     force_scale_power_of_two, probs_scale_qmap, probs_code)
        probs = _read_operand(probs, p_scale, input_code, block_size)
    out = gemm_tn(probs.contiguous(), v.mT)
    if residual:
        out = out + gemm_tn(res_probs.contiguous(), value_residual.mT)
    return out


quantized_ops_lib.impl("sdpa_mx", N.device_guarded(sdpa_mx), "CUDA")


@torch.library.register_fake("quantized_ops::sdpa_mx")
def _(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, query_residual=None, key_residual=None,
      value_residual=None, residual_mask=None, **kwargs):
    return query.new_empty(*query.shape[:-1], value.shape[-1])
