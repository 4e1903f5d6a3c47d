"""Microscaling weights kept packed in memory, and the decode-step linear that reads them.

A converted graph carries a lookup-format weight (``lut4_to_int6`` and friends) as a
bfloat16-valued tensor of codebook indices plus block scales (reference
``quantization/quantize_pt2e.py:754-856``): 2 bytes per parameter.  A decode step reads every
weight once for a handful of tokens, so its time is the weight bytes over HBM bandwidth.
``pack_lut4_weight`` bakes such a weight once into two indices per byte (0.53 bytes per
parameter with the bfloat16 block scales), and ``linear_lut4`` computes what
``quantized_ops::linear_mx`` computes on it (reference ``ops/quantized.py:662-723``): both
operands read back as ``bf16(level * scale)``, float32 products and sum, ``alpha``, bias, one
rounding.  Up to 32 activation rows run the weight-streaming kernel (``vq_gemm_lut4``); more rows
unpack the weight and take ``linear_mx``'s tensor-core GEMM.
"""

from typing import NamedTuple, Optional

import torch

from . import _native as N
from .ops import _DTYPE_ID, _dtype_id, _ptr, _stream

MAX_ROWS = 32


class PackedLUT4Weight(NamedTuple):
    """``codes``: uint8 ``[N, K / 2]``, element ``2 i`` in the low nibble of byte ``i``; ``scale``:
    bfloat16 ``[N, K / block_size]``; ``levels``: the 16 bfloat16 codebook entries."""

    codes: torch.Tensor
    scale: torch.Tensor
    levels: torch.Tensor
    block_size: int

    @property
    def shape(self):
        return (self.codes.shape[0], self.codes.shape[1] * 2)

    @property
    def nbytes(self) -> int:
        return self.codes.numel() + self.scale.numel() * 2 + self.levels.numel() * 2


@N.device_guarded
def pack_lut4_weight(codes: torch.Tensor, scale: torch.Tensor, levels: torch.Tensor, block_size: int,
                     check: bool = True) -> PackedLUT4Weight:
    """Pack ``quantize_mx``'s output for a 16-entry lookup format: ``codes [N, K]`` bfloat16-valued indices,
    ``scale [N, K / block_size]``.  ``check`` synchronises and raises if a code is not an index 0..15."""
    if codes.dim() != 2 or codes.dtype != torch.bfloat16:
        raise NotImplementedError("pack_lut4_weight takes a bfloat16-valued index matrix [N, K]")
    n, k = codes.shape
    if k % 128 or block_size < 32 or block_size & (block_size - 1) or k % block_size or levels.numel() != 16:
        raise NotImplementedError("packed lookup weights need K a multiple of 128, blocks of a power of two (at least "
                                  "32) dividing K, and a 16-entry codebook")
    if tuple(scale.shape) != (n, k // block_size):
        raise ValueError(f"scale of shape {tuple(scale.shape)} does not match {n} rows of {k // block_size} blocks")
    codes = codes.contiguous()
    out = torch.empty((n, k // 2), dtype=torch.uint8, device=codes.device)
    bad = torch.zeros(1, dtype=torch.int32, device=codes.device)
    N.check(N.lib().vq_pack_lut4(codes.data_ptr(), out.data_ptr(), n, k, bad.data_ptr(), _stream()), "vq_pack_lut4")
    if check and int(bad.item()):
        raise ValueError("pack_lut4_weight: the codes are not all codebook indices 0..15")
    return PackedLUT4Weight(out, scale.to(torch.bfloat16).contiguous(), levels.to(torch.bfloat16).contiguous(),
                            int(block_size))


def unpack_lut4_weight(weight: PackedLUT4Weight) -> torch.Tensor:
    """The bfloat16-valued index matrix ``[N, K]`` a packed weight was made from."""
    nib = torch.stack([weight.codes & 0xF, weight.codes >> 4], -1).flatten(-2)
    return nib.to(torch.bfloat16)


_counters = {}


def _scratch(device, m, n, k):
    """Float32 partial-sum workspace for this call and the device's tile counters (zero between calls)."""
    lib = N.lib()
    work = torch.empty(int(lib.vq_gemm_lut4_workspace_floats(m, n, k)), dtype=torch.float32, device=device)
    need = int(lib.vq_gemm_lut4_counters(n))
    have = _counters.get(device)
    if have is None or have.numel() < need:
        have = torch.zeros(max(need, 4096), dtype=torch.int32, device=device)
        _counters[device] = have
    return work, have


@N.device_guarded
def linear_lut4(input: torch.Tensor, weight: PackedLUT4Weight, bias: Optional[torch.Tensor] = None, *,
                input_scale: Optional[torch.Tensor] = None, input_code: Optional[torch.Tensor] = None,
                alpha: Optional[torch.Tensor] = None, out_dtype=None) -> torch.Tensor:
    """``linear_mx(input, W, bias, input_scale=, weight_scale=, block_size=, input_code=, weight_code=, alpha=)``
    for a packed ``W``.  ``input [..., K]`` is bfloat16: values, or codebook indices when ``input_code`` is given;
    ``input_scale [..., K / block_size]``."""
    n, k = weight.shape
    if input.dtype != torch.bfloat16 or input.shape[-1] != k:
        raise NotImplementedError(f"linear_lut4 takes bfloat16 activations of width {k}")
    lead = input.shape[:-1]
    x = input.reshape(-1, k)
    m = x.shape[0]
    dtype = out_dtype or torch.bfloat16
    if m > MAX_ROWS:
        # a prefill-sized product: unpack once and use the tensor-core GEMM behind linear_mx
        y = torch.ops.quantized_ops.linear_mx(x, unpack_lut4_weight(weight), bias, input_scale=input_scale,
                                              weight_scale=weight.scale, block_size=weight.block_size,
                                              input_code=input_code, weight_code=weight.levels, alpha=alpha,
                                              out_dtype=dtype)
        return y.reshape(*lead, n)
    x = x.contiguous()
    if x.data_ptr() % 16:
        x = x.clone()
    scale = None
    if input_scale is not None:
        scale = input_scale.reshape(m, -1).to(torch.bfloat16).contiguous()
        if scale.shape[1] != k // weight.block_size:
            raise ValueError("input_scale does not hold one value per block of the activation")
    code = None if input_code is None else input_code.to(torch.bfloat16).contiguous()
    if alpha is not None:
        alpha = alpha.reshape(()) if alpha.dtype in _DTYPE_ID else alpha.float().reshape(())
    if bias is not None:
        bias = bias.contiguous()
    out = torch.empty((m, n), dtype=dtype, device=x.device)
    work, counters = _scratch(x.device, m, n, k)
    N.check(N.lib().vq_gemm_lut4(x.data_ptr(), k, _ptr(scale), _ptr(code), 0 if code is None else code.numel(), m,
                                 weight.codes.data_ptr(), weight.scale.data_ptr(), weight.levels.data_ptr(),
                                 weight.block_size, out.data_ptr(), _dtype_id(dtype), n, k, _ptr(alpha),
                                 0 if alpha is None else _dtype_id(alpha.dtype), _ptr(bias),
                                 0 if bias is None else _dtype_id(bias.dtype), work.data_ptr(), counters.data_ptr(),
                                 _stream()), "vq_gemm_lut4")
    return out.reshape(*lead, n)
