"""Oracle: the GPTQ column solve against the deployed microscaling grid.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Restates ``hessian_inverse_chol`` (reference
``src/voyager_compiler/quantization/gptq.py:37-75``), ``block_scale``
(``:85-143``), ``salience_order`` (``:146-186``), ``quantize_block``
(``:189-220``) and ``compensate_weight`` (``:223-308``).  The grid is passed
as plain arguments instead of a fake-quant module.  A second entry point,
``compensate_weight_affine``, substitutes the group-wise affine quantizer
(``quantize_affine``'s scale / zero-point rule, ``ops/quantized.py:1227-1283``)
for the microscaling block scale; the reference has no such variant, so that
one is composed from restated reference functions and is otherwise unpinned.
"""

import torch

from .quantizers import calculate_mx_qparam, quantize, vmap

EPS = 1e-12  # reference codebook_optimizer.py:51
SHRINK_GRID = (1.0, 0.93, 0.86, 0.79, 0.72)


def hessian_inverse_chol(hessian, tokens, damping):
    """Upper Cholesky factor of inv(H/tokens + damp*I), damping escalated x10 on failure."""
    h = hessian / max(tokens, 1)
    damp = damping * h.diagonal().mean().clamp_min(EPS)
    added = 0
    for mult in (1, 10, 100, 1000, 10000):
        h.diagonal().add_((mult - added) * damp)
        added = mult
        try:
            lower = torch.linalg.cholesky(h)
        except torch.linalg.LinAlgError:
            continue
        return torch.linalg.cholesky(torch.cholesky_inverse(lower), upper=True)
    raise torch.linalg.LinAlgError("Hessian not positive-definite")


def block_scale(block, weights, qmap, scale_qmap, quant_max, shrink):
    base = calculate_mx_qparam(block, -1, block.shape[-1], quant_max,
                               scale_qmap=scale_qmap).reshape(-1).clamp_min(EPS)
    if not shrink:
        return base
    best, best_err = base, None
    for factor in SHRINK_GRID:
        if factor == 1.0:
            s = base
        else:
            s = vmap((base * factor).bfloat16(), scale_qmap).float().clamp_min(EPS)
        q = quantize(block, s[:, None], qmap=qmap).float() * s[:, None]
        err = ((block - q).pow(2) * weights).sum(1)
        if best_err is None:
            best, best_err = s, err
        else:
            better = err < best_err
            best = torch.where(better, s, best)
            best_err = torch.where(better, err, best_err)
    return best


def salience_order(hessian, columns, within_block, block_size):
    if columns % block_size:
        return None
    nb = columns // block_size
    diag = hessian.diagonal().reshape(nb, block_size)
    block_order = torch.argsort(diag.mean(1), descending=True)
    if within_block:
        rank = torch.argsort(diag, dim=1, descending=True)
    else:
        rank = torch.arange(block_size).expand(nb, block_size)
    return (torch.arange(nb)[:, None] * block_size + rank)[block_order].reshape(-1)


def quantize_block(block, scale, hinv, qmap):
    """Column-by-column rounding with error propagation inside one block."""
    levels, deltas = [], []
    for c in range(block.shape[1]):
        w = block[:, c]
        q = quantize(w[:, None], scale[:, None], qmap=qmap)[:, 0] * scale
        d = (w - q) / hinv[c, c].clamp_min(EPS)
        block = block - d[:, None] * hinv[c]
        levels.append(q)
        deltas.append(d)
    return torch.stack(levels, 1), torch.stack(deltas, 1)


def sweep(weight, hinv_chol, salience, qmap, scale_qmap, quant_max, block_size, shrink=False):
    """The blocked sweep of ``compensate_weight`` given the inverse factor."""
    work = weight.float().clone()
    out = torch.zeros_like(work)
    cols = weight.shape[1]
    for start in range(0, cols, block_size):
        end = min(start + block_size, cols)
        s = block_scale(work[:, start:end], salience[start:end], qmap, scale_qmap,
                        quant_max, shrink)
        out[:, start:end], deltas = quantize_block(work[:, start:end], s,
                                                   hinv_chol[start:end, start:end], qmap)
        if end < cols:
            work[:, end:] -= deltas @ hinv_chol[start:end, end:]
    return out


def compensate_weight(weight, hessian, tokens, qmap, scale_qmap, quant_max, block_size,
                      damping, act_order=True, within_block=True, shrink=False):
    perm = salience_order(hessian, weight.shape[1], within_block, block_size) if act_order else None
    if perm is not None:
        hessian = hessian[perm][:, perm]
        weight = weight[:, perm]
    salience = hessian.diagonal().clone()
    hinv = hessian_inverse_chol(hessian, tokens, damping)
    out = sweep(weight, hinv, salience, qmap, scale_qmap, quant_max, block_size, shrink)
    if perm is None:
        return out
    restored = torch.empty_like(out)
    restored[:, perm] = out
    return restored


# ----------------------------------------------------------------------------
# group-wise affine variant (not in the reference; composed from its rules)
# ----------------------------------------------------------------------------
def affine_qparams(block, quant_min, quant_max):
    low = block.amin(1)
    high = block.amax(1)
    scale = (high - low) / (quant_max - quant_min)
    scale = torch.where(scale > 0.0, scale, torch.ones_like(scale))
    zero = -low / scale + quant_min
    return scale, zero


def sweep_affine(weight, hinv_chol, qmap, quant_min, quant_max, group):
    work = weight.float().clone()
    out = torch.zeros_like(work)
    cols = weight.shape[1]
    for start in range(0, cols, group):
        end = min(start + group, cols)
        block = work[:, start:end]
        scale, zero = affine_qparams(block, quant_min, quant_max)
        hinv = hinv_chol[start:end, start:end]
        levels, deltas = [], []
        for c in range(end - start):
            w = block[:, c]
            code = vmap(w / scale + zero, qmap)
            q = (code - zero) * scale
            d = (w - q) / hinv[c, c].clamp_min(EPS)
            block = block - d[:, None] * hinv[c]
            levels.append(q)
            deltas.append(d)
        out[:, start:end] = torch.stack(levels, 1)
        if end < cols:
            work[:, end:] -= torch.stack(deltas, 1) @ hinv_chol[start:end, end:]
    return out
