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
