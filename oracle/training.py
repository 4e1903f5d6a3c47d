"""CPU restatement of the reference's training-lowering kernels (test infrastructure only).

``rmsnorm_backward`` follows the decomposed backward that the reference runs wherever its
Triton kernel does not apply (``src/voyager_compiler/backend/gpu/rmsnorm.py:229-238``), which
its kernel reproduces "bit for bit" except for the order of its two sums
(``rmsnorm.py:14-20``).  Pinned by ``tests/golden/rmsnorm_backward.npz``, produced by calling
that reference function on CPU.
"""

import torch


def rmsnorm_backward(gradients, x, rsqrt, weight, residual):
    """``(dx, dw)`` of ``y = weight * bf16(x * rsqrt)``: the input gradient, plus ``residual``,
    and the weight gradient.  Tensor-dtype (bfloat16) products round once each; the chain
    through ``rsqrt`` is float32."""
    upstream = gradients[0]
    for extra in gradients[1:]:
        upstream = upstream + extra                     # rounded to the tensors' dtype each time
    cols = x.shape[-1]
    x32 = x.float()
    normalised = (x32 * rsqrt).to(x.dtype)
    leading = tuple(range(x.dim() - 1))
    weight_grad = (upstream * normalised).sum(leading)
    through_weight = (upstream * weight).float()
    # y depends on x directly (times rsqrt) and through rsqrt = (mean x^2 + eps)^-1/2
    row_dot = (through_weight * x32).sum(-1, keepdim=True)
    via_rsqrt = row_dot * -0.5 * rsqrt.pow(3)
    input_grad = (through_weight * rsqrt + via_rsqrt / cols * (x32 * 2.0)).to(x.dtype)
    if residual is not None:
        input_grad = residual + input_grad
    return input_grad, weight_grad


def nvfp4_square_values(weight, fp4_table, e4m3_table, block=16, fp4_max=6.0, e4m3_max=448.0):
    """``(values, block_scales, t)`` of the reference's 16x16-block NVFP4 weight cast before packing
    (``src/voyager_compiler/backend/gpu/nvfp4.py:1006-1012`` with ``_block_scales``, ``:170-179``):
    e2m1-valued elements ``[N, K]``, e4m3-valued scales ``[N / 16, K / 16]`` and the global scale.
    Parity unpinned: the reference's own CPU path needs torchao's packing helpers, which are not
    installed, so no vectors of it exist; the arithmetic is that of ``quantize_mx``, which is pinned."""
    from . import quantizers as Q

    t = Q.calculate_global_scale(weight, fp4_max, e4m3_max)
    n, k = weight.shape
    blocks = weight.reshape(n // block, block, k // block, block)
    amax = blocks.abs().amax((1, 3))
    scale = Q.vmap((amax / fp4_max / t).clamp(max=e4m3_max), e4m3_table)
    scale = torch.where(scale > 0, scale, torch.ones((), dtype=scale.dtype))
    element_scale = (scale * t)[:, None, :, None]
    values = Q.vmap((blocks / element_scale).reshape(n, k), fp4_table)
    return values, scale, t
