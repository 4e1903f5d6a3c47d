"""GPTQ against the deployed block-scaled grid, solved on the device.

Mirrors the single-weight step of the reference's ``quantization/gptq.py``:
``hessian_inverse_chol`` (``:37-75``), ``salience_order`` (``:146-186``) and
``compensate_weight`` (``:223-308``).  The Hessian ``X^T X`` is accumulated on the
tensor cores (bf16 operands, fp32 accumulation, like the reference's CUDA
``addmm``, ``:697-704``); the Cholesky factorisations are torch.linalg calls, as
in the reference; the block scale, the column-by-column rounding with error
propagation and the trailing update are hand-written kernels (``csrc/gptq.cu``).

``compensate_weight_affine`` is the group-wise asymmetric variant (scale and
zero point per group); the reference has no such GPTQ, its rule is
``quantize_affine``'s.
"""

import logging
import types

import torch

from . import _native as N
from . import rounding as R
from .ops import _stream, gemm_tn

logger = logging.getLogger(__name__)

EPS = 1e-12


def accumulate_hessian(hessian, x):
    """``hessian += x^T x`` for a chunk ``x [tokens, K]`` of calibration activations
    (bfloat16 operands, fp32 accumulation)."""
    xt = x.to(torch.bfloat16).reshape(-1, x.shape[-1]).T.contiguous()
    update = gemm_tn(xt, xt, out_dtype=torch.float32)
    if hessian is None:
        return update
    return hessian.add_(update)


def hessian_inverse_chol(hessian, tokens, damping):
    """Upper Cholesky factor of ``inv(H / tokens + damp * mean(diag) * I)``; the damping is
    escalated x10 up to 1e4 if the matrix is not positive definite."""
    h = hessian / max(tokens, 1)
    damp = damping * h.diagonal().mean().clamp_min(EPS)
    applied = 0
    for escalation in (1, 10, 100, 1000, 10000):
        h.diagonal().add_((escalation - applied) * damp)
        applied = escalation
        lower, info = torch.linalg.cholesky_ex(h)
        if int(info) != 0:
            continue
        if escalation > 1:
            logger.warning("Hessian needed %dx the requested damping to invert: it is rank-deficient", escalation)
        return torch.linalg.cholesky(torch.cholesky_inverse(lower), upper=True)
    raise torch.linalg.LinAlgError("Hessian not positive-definite")


def salience_order(hessian, columns, within_block, block_size):
    """Permutation putting the most salient blocks (and, optionally, columns inside each
    block) first while keeping every block's columns together; None if the width is not a
    whole number of blocks."""
    if columns % block_size:
        return None
    blocks = columns // block_size
    diag = hessian.diagonal().reshape(blocks, block_size)
    block_order = torch.argsort(diag.mean(dim=1), descending=True)
    if within_block:
        rank = torch.argsort(diag, dim=1, descending=True)
    else:
        rank = torch.arange(block_size, device=hessian.device).expand(blocks, block_size)
    base = torch.arange(blocks, device=hessian.device).unsqueeze(1)
    return (base * block_size + rank)[block_order].reshape(-1)


@N.device_guarded
def sweep(weight, hinv_chol, block_size, qmap, scale_qmap=None, quant_max=None, salience=None, shrink=False,
          affine_range=None):
    """The blocked sweep given the inverse factor.  Returns the compensated weight (fp32,
    every value on the grid).  ``affine_range = (quant_min, quant_max)`` selects the
    group-wise affine rule."""
    work = weight.float().contiguous().clone()
    rows, K = work.shape
    U = hinv_chol.float().contiguous()
    out = torch.zeros_like(work)
    deltas = torch.empty(rows, min(block_size, K), dtype=torch.float32, device=work.device)
    spec = R.table_round(qmap)
    sspec = R.none_round() if scale_qmap is None else R.table_round(scale_qmap)
    sal = None if salience is None else salience.float().contiguous()
    affine = affine_range is not None
    qmin, qmax = (affine_range if affine else (0.0, float(quant_max)))
    lib, stream = N.lib(), _stream()
    for start in range(0, K, block_size):
        n = min(block_size, K - start)
        N.check(lib.vq_gptq_block(work.data_ptr(), out.data_ptr(), deltas.data_ptr(), U.data_ptr(),
                                  None if sal is None else sal.data_ptr(), rows, K, start, n, int(affine),
                                  float(qmin), float(qmax), int(bool(shrink)), sspec.ref, spec.ref, stream),
                "vq_gptq_block")
        if start + n < K:
            N.check(lib.vq_gptq_update(work.data_ptr(), deltas.data_ptr(), U.data_ptr(), rows, K, start, n, stream),
                    "vq_gptq_update")
    return out


def grid_of(qmap, scale_qmap, quant_max, block_size, ch_axis=-1):
    """The attributes ``compensate_weight`` reads from a fake-quant module."""
    return types.SimpleNamespace(qmap=qmap, scale_qmap=scale_qmap, quant_max=quant_max, block_size=block_size,
                                 ch_axis=ch_axis)


def compensate_weight(weight, hessian, tokens, fake_quant, damping, act_order=True, within_block=True,
                      shrink=False):
    """GPTQ-compensated reconstruction of ``weight [out, in]`` on the grid that
    ``fake_quant`` names (``qmap``, ``scale_qmap``, ``quant_max``, ``block_size``, ``ch_axis``)."""
    block_size = fake_quant.block_size
    axis = fake_quant.ch_axis
    axis = axis[0] if isinstance(axis, (tuple, list)) else axis
    if axis not in (-1, weight.dim() - 1):
        raise ValueError(
            f"weight blocks run along axis {axis}, but the compensation walks the input channels of a "
            f"{tuple(weight.shape)} weight")
    perm = salience_order(hessian, weight.shape[1], within_block, block_size) if act_order else None
    if act_order and perm is None:
        logger.warning("%d input channels is not a whole number of %d-channel blocks; salience ordering skipped",
                       weight.shape[1], block_size)
    if perm is not None:
        hessian = hessian[perm][:, perm]
        weight = weight[:, perm]
    salience = hessian.diagonal().clone()
    hinv = hessian_inverse_chol(hessian, tokens, damping)
    out = sweep(weight, hinv, block_size, fake_quant.qmap, fake_quant.scale_qmap, fake_quant.quant_max, salience,
                shrink)
    if perm is None:
        return out
    restored = torch.empty_like(out)
    restored[:, perm] = out
    return restored


def compensate_weight_affine(weight, hessian, tokens, qmap, quant_min, quant_max, group_size, damping):
    """Group-wise asymmetric GPTQ (act-order off): each group of ``group_size`` input channels maps
    its own [min, max] onto [quant_min, quant_max]."""
    hinv = hessian_inverse_chol(hessian, tokens, damping)
    return sweep(weight, hinv, group_size, qmap, affine_range=(float(quant_min), float(quant_max)))
