"""Kernels of the reference's training lowering on the CUDA library.

``voyager_gpu::rmsnorm_backward`` is the operator the reference's ``fuse_rmsnorm_backward`` pass
puts in place of a captured ``LlamaRMSNorm``'s decomposed backward
(``backend/gpu/rmsnorm.py:133-238``): same name, schema and argument meaning, one CUDA kernel
for both gradients plus a small sum kernel instead of the reference's two Triton kernels.
"""

from typing import List, Optional, Sequence, Tuple

import torch
from torch.library import Library

from . import _native as N
from .ops import _ptr, _stream

__all__ = ["rmsnorm_backward", "MAX_GRADIENTS"]

# the most gradients one kernel sums into dy (reference ``rmsnorm.py:35``)
MAX_GRADIENTS = 3

# the reference's nvfp4 module defines this namespace; operators are added as a fragment, as
# its own rmsnorm module does
voyager_gpu_lib = Library("voyager_gpu", "FRAGMENT")
voyager_gpu_lib.define(
    "rmsnorm_backward(Tensor[] gradients, Tensor x, Tensor rsqrt, Tensor weight, Tensor? residual) -> (Tensor, Tensor)")


def _rmsnorm_backward_cuda(gradients: List[torch.Tensor], x: torch.Tensor, rsqrt: torch.Tensor, weight: torch.Tensor,
                           residual: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    cols = x.shape[-1]
    rows = x.numel() // max(cols, 1)
    dx = torch.empty_like(x)
    dw = torch.empty(cols, dtype=weight.dtype, device=x.device)
    programs = N.lib().vq_rmsnorm_backward_programs(rows, cols)
    partial = torch.empty((max(programs, 1), cols), dtype=torch.float32, device=x.device)
    grads = list(gradients) + [None] * (MAX_GRADIENTS - len(gradients))
    N.check(N.lib().vq_rmsnorm_backward(_ptr(grads[0]), _ptr(grads[1]), _ptr(grads[2]), len(gradients), x.data_ptr(),
                                        rsqrt.data_ptr(), weight.data_ptr(), _ptr(residual), dx.data_ptr(),
                                        partial.data_ptr(), dw.data_ptr(), rows, cols, _stream()),
            "vq_rmsnorm_backward")
    return dx, dw


voyager_gpu_lib.impl("rmsnorm_backward", N.device_guarded(_rmsnorm_backward_cuda), "CUDA")


@torch.library.register_fake("voyager_gpu::rmsnorm_backward")
def _(gradients, x, rsqrt, weight, residual):
    return torch.empty_like(x), weight.new_empty(x.shape[-1])


def rmsnorm_backward(gradients: Sequence[torch.Tensor], x: torch.Tensor, rsqrt: torch.Tensor, weight: torch.Tensor,
                     residual: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """RMSNorm's input gradient (plus ``residual``) and weight gradient
    (reference ``backend/gpu/rmsnorm.py:190-238``).  ``gradients`` sum to the norm's output gradient;
    ``rsqrt`` is the forward's ``rsqrt(mean(x.float() ** 2, -1) + eps)``, float32, shaped as ``x`` with a
    last dimension of 1.  Contiguous CUDA bfloat16 tensors of at most 8192 columns (a multiple of 8) run
    the kernel; anything else is refused: there is no other implementation here."""
    rows = [*gradients, x, *([] if residual is None else [residual])]
    ok = (x.is_cuda and 1 <= len(gradients) <= MAX_GRADIENTS and all(t.shape == x.shape for t in rows)
          and weight.shape == x.shape[-1:] and all(t.dtype is torch.bfloat16 for t in [*rows, weight])
          and rsqrt.dtype is torch.float32 and rsqrt.numel() * x.shape[-1] == x.numel()
          and all(t.is_contiguous() for t in [*rows, weight, rsqrt])
          and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192)
    if not ok:
        raise NotImplementedError("rmsnorm_backward takes one to three contiguous CUDA bfloat16 gradients shaped as x, "
                                  "a float32 rsqrt per row, and rows of a multiple of 8, at most 8192, columns")
    return torch.ops.voyager_gpu.rmsnorm_backward(list(gradients), x, rsqrt, weight, residual)
