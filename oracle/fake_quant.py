"""CPU restatement of the reference's fake-quant ops (test infrastructure only).

``torch.ops.quantization.{fake_quant, group_wise_affine_fake_quant, mx_fake_quant,
hadamard_amax}`` of the reference (``src/voyager_compiler/quantization/ops.py``)
emulate quantization in calibration and training: quantize and scale straight
back, every intermediate rounded into the input's dtype.  Pinned by the golden
cases ``fq_*``, ``gwa_*``, ``mxfq_*`` and ``hadamard_amax_*`` that were produced
by running the reference's own CPU code.
"""

import torch

from . import quantizers as Q


def fake_quant(x, qmap, scale):
    """``vmap(x / scale, qmap) * scale`` with the scale cast to ``x``'s dtype first
    (reference ``quantization/ops.py:79-95``)."""
    scale = scale.to(x.dtype)
    return Q.vmap(x / scale, qmap) * scale


def group_wise_affine_fake_quant(x, axes, block_size, quant_min, quant_max, scale_qmap):
    """Per-block ``[min, max] -> [quant_min, quant_max]``: ``(output, scale, zero_point)``
    (reference ``quantization/ops.py:109-160``).  Codes are ``clamp(round(x / s + z))``,
    not a table lookup."""
    axes = [a % x.dim() for a in axes]
    low = Q.block_reduce(x, axes, block_size, "amin")
    high = Q.block_reduce(x, axes, block_size, "amax")
    one = torch.ones((), dtype=x.dtype)
    sf = (high - low) / (quant_max - quant_min)
    sf = torch.where(sf > 0.0, sf, one)
    if scale_qmap is not None:
        sf = Q.vmap(sf, scale_qmap)
        sf = torch.where(sf > 0.0, sf, one)
    zp = -low / sf + quant_min
    if scale_qmap is not None:
        zp = Q.vmap(zp, scale_qmap)
    esf = Q.expand_blocks(sf, x, block_size)
    ezp = Q.expand_blocks(zp, x, block_size)
    q = torch.clamp(torch.round(x / esf + ezp), quant_min, quant_max)
    return (q - ezp) * esf, sf, zp


def mx_fake_quant(x, qmap, axes, block_size, quant_max, power_of_two, scale_qmap, seed, global_scale,
                  hadamard, hadamard_axis):
    """Microscaling quantize-and-scale-back, optionally between a Hadamard rotation and its
    inverse (reference ``quantization/ops.py:181-213``)."""
    if hadamard is not None:
        x = Q.hadamard_rotate(x, hadamard_axis, hadamard)
    scale, out = Q.quantize_mx(x, qmap, axes, block_size, quant_max, power_of_two, scale_qmap=scale_qmap,
                               seed=seed, global_scale=global_scale)
    out = out * Q.expand_blocks(scale, out, block_size)
    if global_scale is not None:
        out = out * global_scale
    if hadamard is not None:
        out = Q.hadamard_rotate(out, hadamard_axis, hadamard.T)
    return out


def hadamard_amax(x, axis, hadamard):
    """``amax |hadamard_rotate(x)|`` as a 0-d tensor of ``x``'s dtype
    (reference ``quantization/ops.py:275-280``)."""
    return torch.amax(torch.abs(Q.hadamard_rotate(x, axis, hadamard)))
