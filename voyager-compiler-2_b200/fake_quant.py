"""The fake-quant and calibration operators ``torch.ops.quantization.*`` on the CUDA kernels.

The reference defines them in ``src/voyager_compiler/quantization/ops.py`` (torch-op
references, Triton kernels for some calls on a GPU): quantize and scale straight back,
every intermediate rounded into the input's dtype, straight-through gradient.  Here each
is the matching ``quantized_ops`` kernel followed by the dequantizing kernel, so results are
bit-identical to the reference's CPU references (golden cases ``fq_*``, ``gwa_*``,
``mxfq_*``, ``hadamard_amax_*``).  Same names, schemas and argument meaning; CUDA key only.
"""

from typing import List, Optional

import torch
from torch.library import Library

from . import _native as N
from . import ops as O

# torch itself owns a "quantization" namespace (c10d); operators are added to it as a fragment,
# which is also what the reference's triton_op registrations do.
quantization_lib = Library("quantization", "FRAGMENT")
Q = torch.ops.quantized_ops

quantization_lib.define("fake_quant(Tensor input, Tensor qmap, Tensor scale) -> Tensor")
quantization_lib.define(
    "group_wise_affine_fake_quant(Tensor input, int[] axes, int block_size, float quant_min, float quant_max, "
    "Tensor? scale_qmap) -> (Tensor, Tensor, Tensor)")
quantization_lib.define(
    "mx_fake_quant(Tensor input, Tensor qmap, int[] axes, int block_size, float quant_max, bool power_of_two, "
    "Tensor? scale_qmap, Tensor? seed, Tensor? global_scale, Tensor? hadamard, int? hadamard_axis) -> Tensor")
quantization_lib.define("hadamard_amax(Tensor input, int axis, Tensor hadamard) -> Tensor")


def fake_quant(input: torch.Tensor, qmap: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``vmap(input / scale, qmap) * scale`` for a per-tensor or per-channel scale, which is
    cast to ``input``'s dtype first (reference ``quantization/ops.py:79-95``)."""
    scale = scale.to(input.dtype)
    codes = Q.quantize(input, scale, None, None, None, qmap)
    return Q.dequantize(codes, scale)


_ROUND_CLAMP_TABLES = {}


def _round_clamp_table(quant_min: float, quant_max: float, device) -> torch.Tensor:
    """``clamp(round(v), quant_min, quant_max)`` for every bfloat16 ``v``: the integer grid the
    reference's group-wise op rounds to (``quantization/ops.py:157-158``) as a lookup table."""
    key = (float(quant_min), float(quant_max), str(device))
    table = _ROUND_CLAMP_TABLES.get(key)
    if table is None:
        every = torch.arange(65536, dtype=torch.int32, device=device).to(torch.int16).view(torch.bfloat16)
        table = torch.clamp(torch.round(every), quant_min, quant_max)
        _ROUND_CLAMP_TABLES[key] = table
    return table


def group_wise_affine_fake_quant(input: torch.Tensor, axes: List[int], block_size: int, quant_min: float,
                                 quant_max: float, scale_qmap: Optional[torch.Tensor]):
    """Each block maps its own ``[min, max]`` onto ``[quant_min, quant_max]``: returns
    ``(output, scale, zero_point)`` (reference ``quantization/ops.py:109-160``)."""
    table = _round_clamp_table(quant_min, quant_max, input.device)
    scale, zero_point, codes = Q.quantize_affine(input, table, list(axes), block_size, quant_min, quant_max, scale_qmap)
    out = Q.dequantize(codes, scale, zero_point, list(axes), block_size)
    return out, scale, zero_point


def mx_fake_quant(input: torch.Tensor, qmap: torch.Tensor, axes: List[int], block_size: int, quant_max: float,
                  power_of_two: bool, scale_qmap: Optional[torch.Tensor], seed: Optional[torch.Tensor],
                  global_scale: Optional[torch.Tensor], hadamard: Optional[torch.Tensor],
                  hadamard_axis: Optional[int]) -> torch.Tensor:
    """Microscaling quantize-and-scale-back, optionally between a Hadamard rotation along
    ``hadamard_axis`` and its inverse; the rotated axis keeps its padding
    (reference ``quantization/ops.py:181-213``)."""
    x = input
    if hadamard is not None:
        x = O.hadamard_rotate(x, hadamard_axis, hadamard)
    scale, codes = Q.quantize_mx(x, qmap, list(axes), block_size, quant_max, power_of_two, scale_qmap, None, seed,
                                 global_scale)
    out = Q.dequantize(codes, scale, None, list(axes), block_size)
    if global_scale is not None:
        out = out * global_scale
    if hadamard is not None:
        out = O.hadamard_rotate(out, hadamard_axis, hadamard.T.contiguous())
    return out


def hadamard_amax(input: torch.Tensor, axis: int, hadamard: torch.Tensor) -> torch.Tensor:
    """Largest magnitude of ``hadamard_rotate(input, axis, hadamard)`` as a 0-d tensor of
    ``input``'s dtype: the global amax of a rotated ``mx_fake_quant``
    (reference ``quantization/ops.py:275-297``)."""
    return O.tensor_amax(O.hadamard_rotate(input, axis, hadamard)).to(input.dtype)


quantization_lib.impl("fake_quant", N.device_guarded(fake_quant), "CUDA")
quantization_lib.impl("group_wise_affine_fake_quant", N.device_guarded(group_wise_affine_fake_quant), "CUDA")
quantization_lib.impl("mx_fake_quant", N.device_guarded(mx_fake_quant), "CUDA")
quantization_lib.impl("hadamard_amax", N.device_guarded(hadamard_amax), "CUDA")


# ---- shapes for tracing ---------------------------------------------------------------
def _blocked_shape(shape, axes, block_size):
    shape = list(shape)
    for a in axes:
        shape[a] = -(-shape[a] // block_size)
    return shape


def _rotated_shape(shape, axis):
    shape = list(shape)
    shape[axis] = -(-shape[axis] // O.HADAMARD_SIZE) * O.HADAMARD_SIZE
    return shape


@torch.library.register_fake("quantization::fake_quant")
def _(input, qmap, scale):
    return torch.empty_like(input)


@torch.library.register_fake("quantization::group_wise_affine_fake_quant")
def _(input, axes, block_size, quant_min, quant_max, scale_qmap):
    param = input.new_empty(_blocked_shape(input.shape, axes, block_size))
    return torch.empty_like(input), param, torch.empty_like(param)


@torch.library.register_fake("quantization::mx_fake_quant")
def _(input, qmap, axes, block_size, quant_max, power_of_two, scale_qmap, seed, global_scale, hadamard,
      hadamard_axis):
    if hadamard is None:
        return torch.empty_like(input)
    return input.new_empty(_rotated_shape(input.shape, hadamard_axis))


@torch.library.register_fake("quantization::hadamard_amax")
def _(input, axis, hadamard):
    return input.new_empty(())


# ---- straight-through gradients (reference quantization/ops.py:54-76) -------------------
def _setup_straight_through(ctx, inputs, output):
    ctx.num_arguments = len(inputs)
    ctx.input_shape = inputs[0].shape
    if isinstance(output, tuple):
        ctx.mark_non_differentiable(*output[1:])


def _straight_through(ctx, grad, *unused):
    """The input takes the fake-quantized tensor's gradient unchanged, less the padding a
    rotation added; no other argument takes one."""
    if grad.shape != ctx.input_shape:
        grad = grad[tuple(slice(size) for size in ctx.input_shape)]
    return (grad,) + (None,) * (ctx.num_arguments - 1)


for _name in ("fake_quant", "group_wise_affine_fake_quant", "mx_fake_quant"):
    torch.library.register_autograd(f"quantization::{_name}", _straight_through,
                                    setup_context=_setup_straight_through, lib=quantization_lib)
