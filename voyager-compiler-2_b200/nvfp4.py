"""NVFP4 on the tensor cores' native block-scaled MMA.

The counterpart of the reference's ``backend/gpu/nvfp4.py`` (``quantize_nvfp4:890``,
``pack_nvfp4:1045``, ``nvfp4_linear:1101``): an NVFP4 site of a converted graph
(``quantize_mx`` with an e2m1 table, block 16, e4m3 scales and a global scale,
feeding ``linear_mx`` with ``alpha``) is executed as one fused cast to packed
operands and one ``kind::mxf4nvf4`` GEMM.  The cast reproduces the operator's
codes and scales bit for bit; the GEMM accumulates the same products in fp32.
"""

from typing import NamedTuple, Optional

import torch

from . import _native as N
from .ops import _DTYPE_ID, _dtype_id, _ptr, _stream


class PackedNVFP4(NamedTuple):
    """``codes``: uint8 ``[*batch, rows, K/2]``; ``scales``: uint8 tiles; ``shape``: logical ``(*batch, rows, K)``."""

    codes: torch.Tensor
    scales: torch.Tensor
    shape: tuple


def _alloc(shape, device):
    *batch, rows, k = shape
    nb = 1
    for b in batch:
        nb *= b
    if k % 64:
        raise NotImplementedError("NVFP4 packing needs K to be a multiple of 64")
    codes = torch.empty(*batch, rows, k // 2, dtype=torch.uint8, device=device)
    per = int(N.lib().vq_nvfp4_scale_bytes(rows, k))
    scales = torch.zeros(nb, per, dtype=torch.uint8, device=device)
    return codes, scales, nb, rows, k, per


def quantize_nvfp4(x: torch.Tensor, global_scale: torch.Tensor) -> PackedNVFP4:
    """Cast bfloat16 ``x [*batch, rows, K]`` (blocks of 16 along K) to packed NVFP4."""
    if x.dtype != torch.bfloat16:
        raise NotImplementedError("quantize_nvfp4 takes bfloat16 input")
    x = x.contiguous()
    codes, scales, nb, rows, k, per = _alloc(tuple(x.shape), x.device)
    gs = global_scale if global_scale.dtype in _DTYPE_ID else global_scale.float()
    lib, stream = N.lib(), _stream()
    xb, cb = x.view(nb, rows, k), codes.view(nb, rows, k // 2)
    for b in range(nb):
        N.check(lib.vq_quantize_nvfp4(xb[b].data_ptr(), gs.data_ptr(), _dtype_id(gs.dtype), cb[b].data_ptr(),
                                      scales[b].data_ptr(), rows, k, stream), "vq_quantize_nvfp4")
    return PackedNVFP4(codes, scales, tuple(x.shape))


def pack_nvfp4(codes: torch.Tensor, scale: torch.Tensor, check: bool = True) -> PackedNVFP4:
    """Pack ``quantize_mx``'s outputs (bfloat16-valued e2m1 codes ``[*batch, rows, K]`` and e4m3-valued
    scales ``[*batch, rows, K/16]``).  ``check`` synchronises and raises if a value is not representable."""
    if codes.dtype != torch.bfloat16 or scale.dtype != torch.bfloat16:
        raise NotImplementedError("pack_nvfp4 takes bfloat16-valued codes and scales")
    codes, scale = codes.contiguous(), scale.contiguous()
    out, scales, nb, rows, k, per = _alloc(tuple(codes.shape), codes.device)
    bad = torch.zeros(1, dtype=torch.int32, device=codes.device)
    lib, stream = N.lib(), _stream()
    cin, sin, cb = codes.view(nb, rows, k), scale.view(nb, rows, k // 16), out.view(nb, rows, k // 2)
    for b in range(nb):
        N.check(lib.vq_pack_nvfp4(cin[b].data_ptr(), sin[b].data_ptr(), cb[b].data_ptr(), scales[b].data_ptr(), rows,
                                  k, bad.data_ptr(), stream), "vq_pack_nvfp4")
    if check and int(bad.item()):
        raise ValueError("pack_nvfp4: codes are not all e2m1 values or scales are not all e4m3 values")
    return PackedNVFP4(out, scales, tuple(codes.shape))


def nvfp4_gemm(a: PackedNVFP4, b: PackedNVFP4, alpha: Optional[torch.Tensor] = None,
               bias: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``alpha * (A @ B^T) + bias`` for packed operands ``a [*batch, M, K]`` and ``b [*batch, N, K]`` (equal
    batch shapes; a 2-D ``b`` with a batched ``a`` folds the batch into the rows)."""
    *abatch, m, k = a.shape
    *bbatch, n, kb = b.shape
    if k != kb:
        raise ValueError("contraction extents differ")
    if abatch and not bbatch:
        if m % 128 and len(abatch) and any(d != 1 for d in abatch):
            raise NotImplementedError("a shared weight with a batched activation needs M to be a multiple of 128")
        rows = m
        for d in abatch:
            rows *= d
        a_codes, a_scales, batch, m_eff = a.codes.reshape(rows, k // 2), a.scales.reshape(-1), 1, rows
    else:
        if list(abatch) != list(bbatch):
            raise NotImplementedError("batch shapes must match")
        batch = 1
        for d in abatch:
            batch *= d
        a_codes, a_scales, m_eff = a.codes, a.scales, m
    out = torch.empty((batch, m_eff, n), dtype=out_dtype, device=a.codes.device)
    if alpha is not None:
        alpha = alpha.reshape(()) if alpha.dtype in _DTYPE_ID else alpha.float().reshape(())
    if bias is not None:
        bias = bias.contiguous()
    N.check(N.lib().vq_gemm_nvfp4(a_codes.data_ptr(), a_scales.data_ptr(), b.codes.data_ptr(), b.scales.data_ptr(),
                                  out.data_ptr(), _dtype_id(out_dtype), m_eff, n, k, n, batch, m_eff * n,
                                  _ptr(alpha), 0 if alpha is None else _dtype_id(alpha.dtype), _ptr(bias),
                                  0 if bias is None else _dtype_id(bias.dtype), _stream()), "vq_gemm_nvfp4")
    return out.reshape(*abatch, m, n)


def nvfp4_linear(x: torch.Tensor, weight: PackedNVFP4, x_global_scale: torch.Tensor, w_global_scale: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """One NVFP4 linear: cast ``x`` and multiply; ``alpha = x_global_scale * w_global_scale`` in the scales'
    dtype, as the converted graph forms it."""
    alpha = x_global_scale * w_global_scale
    return nvfp4_gemm(quantize_nvfp4(x, x_global_scale), weight, alpha, bias, out_dtype)
