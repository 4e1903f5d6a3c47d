"""A packed KIVI key/value cache on the CUDA kernels.

The reference quantizes a decode KV cache the KIVI way -- unsigned 2-bit (or 4-bit) codes
with one scale and zero point per group of 64, keys grouped along the sequence
(``ax=-2``), values along the head dimension (``ax=-1``), qparams rounded to FP8
(``examples/language_modeling/quantization_configs.py:171-207``) -- with
``quantized_ops::quantize_affine``, keeps the codes as bfloat16-valued tensors (2 bytes per
2-bit code) and reads them back through one fused ``quantized_ops::dequantize`` that also
re-encodes them for the attention matmul (``codegen/transform/quant_folding.py:2391-2547``).

Here the same codes are stored packed (four 2-bit codes per byte, an eighth of the bytes the
decode step reads), and ``read`` is that fused dequantize straight from the packed bytes:
bit for bit what the operators give on the unpacked codes.
"""

import dataclasses
from typing import List, Optional

import torch

from . import _native as N
from . import rounding as R
from .ops import _broadcast_geometry, _dtype_id, _prepare_params, _ptr, _stream

Q = torch.ops.quantized_ops


@N.device_guarded
def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Integer codes in ``[0, 2**bits)`` (values of a float tensor) as packed bytes: element ``i`` of
    the row-major tensor sits in byte ``i // (8 // bits)`` at bit ``bits * (i % (8 // bits))``."""
    codes = codes.contiguous()
    n = codes.numel()
    packed = torch.empty((n * bits + 7) // 8, dtype=torch.uint8, device=codes.device)
    N.check(N.lib().vq_pack_codes(codes.data_ptr(), _dtype_id(codes.dtype), packed.data_ptr(), bits, n, _stream()),
            "vq_pack_codes")
    return packed


@N.device_guarded
def unpack_dequantize(packed: torch.Tensor, bits: int, shape, scale: torch.Tensor,
                      zero_point: Optional[torch.Tensor] = None, block_size: Optional[int] = None,
                      output_qmap: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``round_out((code - zero_point) * scale)`` for packed codes of a tensor of ``shape``: what
    ``quantized_ops::dequantize(codes, scale, zero_point, axes, block_size, None, output_qmap)``
    returns for the unpacked codes (reference ``ops/quantized.py:527-571``)."""
    # the codes count as a tensor of the parameters' dtype, as the stored bfloat16-valued codes are
    like = torch.empty(0, dtype=scale.dtype, device=scale.device)
    _, scale, zero_point = _prepare_params(like, scale, zero_point)
    out = torch.empty(tuple(shape), dtype=scale.dtype, device=packed.device)
    geom = _broadcast_geometry(tuple(shape), scale, block_size)
    r_out = R.none_round() if output_qmap is None else R.table_round(output_qmap)
    N.check(N.lib().vq_unpack_dequantize(packed.data_ptr(), bits, scale.data_ptr(), _ptr(zero_point), out.data_ptr(),
                                         _dtype_id(out.dtype), _dtype_id(scale.dtype), geom, r_out.ref, _stream()),
            "vq_unpack_dequantize")
    return out


@dataclasses.dataclass
class PackedCache:
    """One quantized cache tensor: packed codes plus per-group scale and zero point."""

    packed: torch.Tensor          # uint8, ceil(numel * bits / 8) bytes
    scale: torch.Tensor           # one per group, the tensor's dtype
    zero_point: torch.Tensor
    shape: tuple
    axes: List[int]
    block_size: int
    bits: int

    @property
    def nbytes(self) -> int:
        return self.packed.numel() + self.scale.numel() * self.scale.element_size() * 2

    def read(self, output_qmap: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The cache's values, optionally re-encoded through ``output_qmap`` in the same pass."""
        fast = self._fast_layout() if output_qmap is None else None
        if fast is not None:
            return _read_2bit(self, *fast)
        return unpack_dequantize(self.packed, self.bits, self.shape, self.scale, self.zero_point, self.block_size,
                                 output_qmap)

    def _fast_layout(self):
        """``(outer, T, D, along_channels)`` when the streaming 2-bit kernel applies: bfloat16 parameters,
        groups along one of the last two axes, whole groups, channels a multiple of 8."""
        if self.bits != 2 or self.scale.dtype != torch.bfloat16 or self.zero_point.dtype != torch.bfloat16 \
                or len(self.shape) < 2 or len(self.axes) != 1:
            return None
        nd = len(self.shape)
        axis = self.axes[0] % nd
        T, D = self.shape[-2], self.shape[-1]
        outer = 1
        for extent in self.shape[:-2]:
            outer *= extent
        bs = self.block_size
        if D % 8 or not self.scale.is_contiguous() or not self.zero_point.is_contiguous():
            return None
        if axis == nd - 1 and bs >= 8 and bs & (bs - 1) == 0 and D % bs == 0:
            return outer, T, D, 1
        if axis == nd - 2 and T % bs == 0:
            return outer, T, D, 0
        return None


@N.device_guarded
def _read_2bit(cache: "PackedCache", outer, T, D, along_channels) -> torch.Tensor:
    out = torch.empty(cache.shape, dtype=torch.bfloat16, device=cache.packed.device)
    N.check(N.lib().vq_kivi_read_2bit(cache.packed.data_ptr(), cache.scale.data_ptr(), cache.zero_point.data_ptr(),
                                      out.data_ptr(), outer, T, D, along_channels, cache.block_size, _stream()),
            "vq_kivi_read_2bit")
    return out


def quantize_cache(x: torch.Tensor, qmap: torch.Tensor, axis: int, block_size: int, bits: int,
                   scale_qmap: Optional[torch.Tensor] = None) -> PackedCache:
    """Quantize ``x`` in groups of ``block_size`` along ``axis`` to unsigned ``bits``-bit codes
    (``quantize_affine``, reference ``ops/quantized.py:1227-1283``) and pack them."""
    axes = [axis]
    scale, zero_point, codes = Q.quantize_affine(x, qmap, axes, block_size, 0.0, float(2 ** bits - 1), scale_qmap)
    return PackedCache(pack_codes(codes, bits), scale, zero_point, tuple(x.shape), axes, block_size, bits)


def decode_attention(q: torch.Tensor, keys: PackedCache, values: PackedCache, k_recent: torch.Tensor,
                     v_recent: torch.Tensor, score_scale: Optional[float] = None) -> Optional[torch.Tensor]:
    """One decode step's attention over ``[packed cache | recent window]`` in one kernel.

    ``q [B, kv_heads, G, 128]`` (the query heads of each KV head); ``keys`` / ``values``: 2-bit caches of
    ``[B, kv_heads, Tm, 128]`` grouped along the positions / the channels; ``k_recent`` / ``v_recent``
    ``[B, kv_heads, R, 128]`` bfloat16.  Returns ``[B, kv_heads * G * 128]`` with the roundings of
    ``read()`` + ``matmul`` / ``softmax`` / ``matmul`` on bfloat16 tensors, or ``None`` when the kernel
    does not take this configuration (the caller then runs those operators)."""
    B, hkv, G, d = q.shape
    kf, vf = keys._fast_layout(), values._fast_layout()
    if kf is None or vf is None or kf[3] != 0 or vf[3] != 1 or q.dtype != torch.bfloat16:
        return None
    outer, Tm, D, _ = kf
    R = k_recent.shape[-2]
    if outer != B * hkv or vf[:3] != (outer, Tm, D) or d != D or tuple(k_recent.shape) != (B, hkv, R, D) \
            or tuple(v_recent.shape) != (B, hkv, R, D) or k_recent.dtype != torch.bfloat16 \
            or v_recent.dtype != torch.bfloat16:
        return None
    return _decode_attention(q.contiguous(), keys, values, k_recent.contiguous(), v_recent.contiguous(),
                             1.0 / d ** 0.5 if score_scale is None else float(score_scale))


@N.device_guarded
def _decode_attention(q, keys, values, k_recent, v_recent, score_scale):
    B, hkv, G, d = q.shape
    Tm, R = keys.shape[-2], k_recent.shape[-2]
    out = torch.empty((B, hkv * G * d), dtype=torch.bfloat16, device=q.device)
    rc = N.lib().vq_kivi_decode_attention(
        q.data_ptr(), keys.packed.data_ptr(), keys.scale.data_ptr(), keys.zero_point.data_ptr(),
        values.packed.data_ptr(), values.scale.data_ptr(), values.zero_point.data_ptr(), k_recent.data_ptr(),
        v_recent.data_ptr(), out.data_ptr(), B * hkv, G, Tm, R, d, keys.block_size, values.block_size, score_scale,
        _stream())
    if rc == -3:   # VQ_EUNSUPPORTED
        return None
    N.check(rc, "vq_kivi_decode_attention")
    return out


@N.device_guarded
def rope_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, q_heads: int, k_window: torch.Tensor,
                v_window: torch.Tensor, slot: int = -1) -> torch.Tensor:
    """RoPE on a decode step's merged projection ``qkv [B, (q_heads + 2 kv_heads) * d]`` and the cache append in
    one kernel: returns the rotated queries ``[B, q_heads, d]`` and writes the rotated keys and the values into
    position ``slot`` of the ``[B, kv_heads, R, d]`` windows.  ``cos`` / ``sin``: ``[d]`` or ``[B, d]``."""
    B, hkv, R, d = k_window.shape
    if qkv.shape != (B, (q_heads + 2 * hkv) * d) or v_window.shape != k_window.shape:
        raise ValueError("rope_append: shapes do not agree")
    if any(t.dtype != torch.bfloat16 for t in (qkv, cos, sin, k_window, v_window)):
        raise NotImplementedError("rope_append takes bfloat16 tensors")
    if not (k_window.is_contiguous() and v_window.is_contiguous()):
        raise ValueError("rope_append: the windows must be contiguous")
    qkv, cos, sin = qkv.contiguous(), cos.contiguous(), sin.contiguous()
    if cos.shape != sin.shape or cos.shape not in ((d,), (B, d)):
        raise ValueError("rope_append: cos / sin are [d] or [B, d]")
    slot = slot % R
    q_out = torch.empty((B, q_heads, d), dtype=torch.bfloat16, device=qkv.device)
    esz = 2
    N.check(N.lib().vq_rope_decode_append(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), q_out.data_ptr(),
                                          k_window.data_ptr() + slot * d * esz, v_window.data_ptr() + slot * d * esz,
                                          B, q_heads, hkv, d, R * d, d if cos.dim() == 2 else 0, _stream()),
            "vq_rope_decode_append")
    return q_out
