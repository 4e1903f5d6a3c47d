"""CPU restatement of the reference's outlier side stream (test infrastructure only).

``filter_outlier``, ``quantize_mx_outlier``, ``slice_csr_tensor`` and ``spmm_csr``
(reference ``src/voyager_compiler/ops/quantized.py:1286-1644``): elements whose magnitude
reaches a threshold leave the tensor as a fixed-capacity CSR matrix (padded data / column
indices, int32 row pointers) and are multiplied separately in float32.  Written with explicit
loops over rows; pinned by the golden cases ``outlier_*``.
"""

import math

import torch

from . import quantizers as Q


def _capacity(shape, max_pct):
    return int(math.prod(shape[-2:]) * max_pct)


def filter_outlier(x, threshold, max_pct=0.01):
    """``(data, indices, indptr, inlier)`` (reference ``quantized.py:1323-1373``).  The
    comparison happens in ``x``'s dtype (the threshold is rounded to it); zero-valued
    outliers are not stored; entries beyond the capacity are dropped in row-major order."""
    thr = torch.tensor(threshold, dtype=x.dtype)
    is_outlier = x.abs() >= thr
    inlier = torch.where(is_outlier, torch.zeros((), dtype=x.dtype), x)
    rows, cols = x.shape[-2:]
    cap = _capacity(x.shape, max_pct)
    flat = x.reshape(-1, rows, cols)
    mask = is_outlier.reshape(-1, rows, cols)
    data = torch.zeros(flat.shape[0], cap, dtype=x.dtype)
    indices = torch.full((flat.shape[0], cap), -1, dtype=torch.int32)
    indptr = torch.zeros(flat.shape[0], rows + 1, dtype=torch.int32)
    for b in range(flat.shape[0]):
        n = 0
        for r in range(rows):
            for c in range(cols):
                if mask[b, r, c] and flat[b, r, c] != 0:
                    if n < cap:
                        data[b, n] = flat[b, r, c]
                        indices[b, n] = c
                    n += 1
            indptr[b, r + 1] = min(n, cap)
    batch = x.shape[:-2]
    return data.reshape(*batch, cap), indices.reshape(*batch, cap), indptr.reshape(*batch, rows + 1), inlier


def quantize_mx_outlier(x, qmap, axes, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None,
                        output_code=None, threshold=None, max_pct=0.01, indptr_offset=0):
    """Outliers to a CSR, the rest through ``quantize_mx`` (reference ``quantized.py:1405-1455``)."""
    data, indices, indptr, inliers = filter_outlier(x, threshold, max_pct)
    if indptr_offset:
        indptr = indptr + indptr_offset
    scale, codes = Q.quantize_mx(inliers, qmap, axes, block_size, quant_max, force_scale_power_of_two, scale_qmap,
                                 output_code)
    return data, indices, indptr, scale, codes


def slice_csr_tensor(data, indices, indptr, dim=0, start=None, end=None, size_factor=1.0):
    """Rows ``[start, end)`` (``dim`` 0) or columns ``[start, end)`` (``dim`` 1) of one CSR matrix,
    re-padded to ``int(len(data) * size_factor)`` entries (reference ``quantized.py:1500-1541``)."""
    dim = dim + 2 if dim < 0 else dim
    cap = int(data.shape[0] * size_factor)
    vals, cols, ptr = [], [], [0]
    if dim == 0:
        for r in range(start, end):
            for e in range(int(indptr[r]), int(indptr[r + 1])):
                vals.append(data[e])
                cols.append(int(indices[e]))
            ptr.append(len(vals))
    else:
        for r in range(indptr.shape[0] - 1):
            for e in range(int(indptr[r]), int(indptr[r + 1])):
                if start <= int(indices[e]) < end:
                    vals.append(data[e])
                    cols.append(int(indices[e]) - start)
            ptr.append(len(vals))
    new_data = torch.zeros(cap, dtype=data.dtype)
    new_indices = torch.full((cap,), -1, dtype=indices.dtype)
    for i in range(min(cap, len(vals))):
        new_data[i] = vals[i]
        new_indices[i] = cols[i]
    return new_data, new_indices, torch.tensor(ptr, dtype=indptr.dtype).clamp(max=cap)


def spmm_csr(data, indices, indptr, B, B_scale=None, B_code=None, block_size=None, weight_layout="kc", *,
             out_dtype=None):
    """CSR x dense in float32 (reference ``quantized.py:1574-1644``); ``B`` is read back through
    its codebook and block scales first and is ``[out, contraction]`` for ``"kc"``."""
    if B_code is not None:
        B = Q.decode(B, B_code)
    if B_scale is not None:
        B = B * Q.expand_blocks(B_scale, B, block_size)
    if weight_layout == "kc":
        B = B.mT
    batch = indptr.shape[:-1]
    nb = int(math.prod(batch))
    indptr2 = indptr.reshape(nb, -1)
    indices2 = indices.reshape(nb, -1)
    data2 = data.reshape(nb, -1)
    Bb = B.reshape(nb, B.shape[-2], B.shape[-1]) if B.ndim > 2 else None
    rows = indptr2.shape[1] - 1
    out = torch.zeros(nb, rows, B.shape[-1], dtype=torch.float32)
    for b in range(nb):
        dense = (Bb[b] if Bb is not None else B).float()
        base = int(indptr2[b, 0])
        for r in range(rows):
            for e in range(int(indptr2[b, r]) - base, int(indptr2[b, r + 1]) - base):
                out[b, r] += data2[b, e].float() * dense[int(indices2[b, e])]
    return out.to(B.dtype if out_dtype is None else out_dtype).reshape(*batch, rows, B.shape[-1])
