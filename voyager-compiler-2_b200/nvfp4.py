"""NVFP4 on the tensor cores' native block-scaled MMA.

The counterpart of the reference's ``backend/gpu/nvfp4.py``: an NVFP4 site of a converted
graph (``quantize_mx`` with an e2m1 table, block 16, e4m3 scales and a global scale, feeding
``linear_mx`` with ``alpha``) is executed as one fused cast to packed operands and one
``kind::mxf4nvf4`` GEMM.  The cast reproduces the operator's codes and scales bit for bit;
the GEMM accumulates the same products in fp32.

``quantize_nvfp4``, ``pack_nvfp4``, ``unpack_nvfp4``, ``nvfp4_linear`` and
``emulate_nvfp4_linear`` keep the reference's names, arguments and return values
(``backend/gpu/nvfp4.py:890-950, 1045-1091, 1101-1152, 1190-1227``); ``cast_nvfp4`` and
``nvfp4_gemm`` are the kernels underneath.
"""

from typing import NamedTuple, Optional

import torch

from . import _native as N
from .ops import _DTYPE_ID, _dtype_id, _ptr, _stream


BLOCK_SIZE = 16
FP4_MAX, E4M3_MAX = 6.0, 448.0


class PackedNVFP4(NamedTuple):
    """``codes``: uint8 ``[*batch, rows, K/2]`` (two e2m1 codes per byte, even element in the low
    nibble); ``scales``: uint8 e4m3 block scales in 128x4 tiles (512 bytes each, the layout the
    block-scaled MMA reads).  Unpacks as ``codes, scales = packed`` like the reference's pair."""

    codes: torch.Tensor
    scales: torch.Tensor

    @property
    def shape(self) -> tuple:
        """Logical ``(*batch, rows, K)``."""
        return (*self.codes.shape[:-1], self.codes.shape[-1] * 2)


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


@N.device_guarded
def cast_nvfp4(x: torch.Tensor, global_scale: torch.Tensor) -> PackedNVFP4:
    """Cast bfloat16 ``x [*batch, rows, K]`` (blocks of 16 along K) to packed NVFP4 against a given
    global scale, one pass (the role of the reference's ``cast_nvfp4`` kernels, ``nvfp4.py:683-739``)."""
    if x.dtype != torch.bfloat16:
        raise NotImplementedError("cast_nvfp4 takes bfloat16 input")
    x = x.contiguous()
    codes, scales, nb, rows, k, per = _alloc(tuple(x.shape), x.device)
    gs = global_scale if global_scale.dtype in _DTYPE_ID else global_scale.float()
    lib, stream = N.lib(), _stream()
    xb, cb = x.view(nb, rows, k), codes.view(nb, rows, k // 2)
    for b in range(nb):
        N.check(lib.vq_quantize_nvfp4(xb[b].data_ptr(), gs.data_ptr(), _dtype_id(gs.dtype), cb[b].data_ptr(),
                                      scales[b].data_ptr(), rows, k, stream), "vq_quantize_nvfp4")
    return PackedNVFP4(codes, scales)


@N.device_guarded
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
    return PackedNVFP4(out, scales)


@N.device_guarded
def nvfp4_gemm(a: PackedNVFP4, b: PackedNVFP4, alpha: Optional[torch.Tensor] = None,
               bias: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
               alpha_cols: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``alpha * alpha_cols[n] * (A @ B^T) + bias`` for packed operands ``a [*batch, M, K]`` and
    ``b [*batch, N, K]`` (equal batch shapes; a 2-D ``b`` with a batched ``a`` folds the batch into the rows)."""
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
    if out is None:
        out = torch.empty((batch, m_eff, n), dtype=out_dtype, device=a.codes.device)
    elif out.dtype != out_dtype or out.numel() != batch * m_eff * n or not out.is_contiguous():
        raise ValueError("out must be a dense tensor of the result's size and dtype")
    if alpha is not None:
        alpha = alpha.reshape(()) if alpha.dtype in _DTYPE_ID else alpha.float().reshape(())
    if bias is not None:
        bias = bias.contiguous()
    if alpha_cols is not None:
        alpha_cols = alpha_cols.reshape(-1).contiguous()
        if alpha_cols.numel() != n or alpha_cols.dtype not in _DTYPE_ID:
            raise ValueError(f"alpha_cols must hold {n} bfloat16/float16/float32 values")
    N.check(N.lib().vq_gemm_nvfp4_ex(a_codes.data_ptr(), a_scales.data_ptr(), b.codes.data_ptr(), b.scales.data_ptr(),
                                     out.data_ptr(), _dtype_id(out_dtype), m_eff, n, k, n, batch, m_eff * n,
                                     _ptr(alpha), 0 if alpha is None else _dtype_id(alpha.dtype), _ptr(bias),
                                     0 if bias is None else _dtype_id(bias.dtype), _ptr(alpha_cols),
                                     0 if alpha_cols is None else _dtype_id(alpha_cols.dtype), _stream()),
            "vq_gemm_nvfp4_ex")
    return out.reshape(*abatch, m, n)


@N.device_guarded
def silu_mul_cast_nvfp4(gate: torch.Tensor, up: torch.Tensor):
    """``quantize_nvfp4(silu(gate) * up)`` with the product and its tensor-wide amax made in one pass:
    ``(codes, scales, t)``.  ``gate`` / ``up``: ``[rows, cols]`` bfloat16, unit stride along the columns (the two
    halves of a merged gate/up projection are read in place)."""
    from . import ops as O

    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16 or gate.shape != up.shape or gate.dim() != 2:
        raise NotImplementedError("silu_mul_cast_nvfp4 takes two bfloat16 matrices of one shape")
    act, amax = silu_mul_amax(gate, up)
    t = O.global_scale_of_amax(amax, torch.bfloat16, FP4_MAX, E4M3_MAX)
    packed = cast_nvfp4(act, t)
    return packed.codes, packed.scales, t


@N.device_guarded
def silu_mul_amax(gate: torch.Tensor, up: torch.Tensor):
    """``(silu(gate) * up, max |.|)`` in one pass: the bfloat16 product and a 0-d float32 amax (what a tensor-parallel
    layer all-reduces before it casts its shard)."""
    rows, cols = gate.shape

    def strided(t):
        ok = t.stride(1) == 1 and t.stride(0) >= cols and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0
        return t if ok else t.contiguous()

    gate, up = strided(gate), strided(up)
    act = torch.empty((rows, cols), dtype=torch.bfloat16, device=gate.device)
    amax = torch.zeros((), dtype=torch.float32, device=gate.device)
    N.check(N.lib().vq_silu_mul_amax(gate.data_ptr(), up.data_ptr(), act.data_ptr(), amax.data_ptr(), rows, cols,
                                     gate.stride(0), up.stride(0), _stream()), "vq_silu_mul_amax")
    return act, amax


def nvfp4_linear_from_bf16(x: torch.Tensor, weight: PackedNVFP4, x_global_scale: torch.Tensor,
                           w_global_scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
                           out_dtype=torch.bfloat16) -> torch.Tensor:
    """One NVFP4 linear on a bfloat16 activation: cast ``x`` and multiply; ``alpha = x_global_scale *
    w_global_scale`` in the scales' dtype, as the converted graph forms it."""
    alpha = x_global_scale * w_global_scale
    return nvfp4_gemm(cast_nvfp4(x, x_global_scale), weight, alpha, bias, out_dtype)


# ---------------------------------------------------------------------------
# the reference's functions, by name and signature
# ---------------------------------------------------------------------------
_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def quantize_nvfp4(input: torch.Tensor, axis: int = -1, seed: Optional[torch.Tensor] = None,
                   hadamard: Optional[torch.Tensor] = None):
    """``(codes, scales, t)``: ``input`` quantized to NVFP4 along ``axis`` as the fake-quantizer does
    (optional random Hadamard transform, global scale ``t`` from the tensor's amax, e4m3 block
    scales, e2m1 elements), packed for ``nvfp4_linear``; codes have ``axis`` moved last; the axis must be a
    multiple of 64 long here (the reference pads its scale tiles and takes multiples of 16)
    (reference ``backend/gpu/nvfp4.py:890-950``)."""
    from . import ops as O

    axis %= input.ndim
    if hadamard is not None:
        input = O.hadamard_rotate(input, axis, hadamard)
    t = O.calculate_global_scale(input, FP4_MAX, E4M3_MAX)
    moved = input.movedim(axis, -1).contiguous()
    rows = moved.reshape(-1, moved.shape[-1])
    if seed is None:
        packed = cast_nvfp4(rows, t)
    else:
        from .formats import get_quantization_map, qmap_levels

        levels = qmap_levels(get_quantization_map("fp4_e2m1", input.device))
        scale_qmap = get_quantization_map("fp8_e4m3", input.device)
        # random bits are drawn for a tensor of the input's own shape, so quantize in place and move after
        scale, values = torch.ops.quantized_ops.quantize_mx(input, levels, [axis], BLOCK_SIZE, FP4_MAX, False,
                                                            scale_qmap, None, seed, t)
        packed = pack_nvfp4(values.movedim(axis, -1).reshape(rows.shape).contiguous(),
                            scale.movedim(axis, -1).reshape(rows.shape[0], -1).contiguous(), check=False)
    return packed.codes.view(*moved.shape[:-1], -1), packed.scales, t


def quantize_nvfp4_pair(input: torch.Tensor, seed: Optional[torch.Tensor] = None,
                        transpose_seed: Optional[torch.Tensor] = None, hadamard: Optional[torch.Tensor] = None):
    """``quantize_nvfp4`` of a matrix ``[M, K]`` along its last axis and of its transpose along its last
    axis (with ``hadamard`` and ``transpose_seed``): ``(codes, scales, t, codes_T, scales_T, t_T)``, what
    a training step needs of one operand for its forward and weight-gradient GEMMs
    (reference ``backend/gpu/nvfp4.py:953-980``).  Two casts here, each reading the matrix once."""
    if input.ndim != 2:
        raise ValueError("quantize_nvfp4_pair takes a matrix")
    return (*quantize_nvfp4(input, -1, seed), *quantize_nvfp4(input.mT, -1, transpose_seed, hadamard))


def quantize_nvfp4_square(weight: torch.Tensor):
    """A weight ``[N, K]`` quantized to NVFP4 in 16x16 blocks, packed along K for the forward GEMM and,
    transposed, along N for the input-gradient GEMM: ``(codes, scales, transposed_codes,
    transposed_scales, t)`` (reference ``backend/gpu/nvfp4.py:983-1017``).  ``quantize_nvfp4``'s
    arithmetic over square blocks: ``t`` from the weight's amax, a block's scale
    ``e4m3(amax / 6 / t)`` (1 where that is 0), every element divided by its block's scale times
    ``t`` and rounded to e2m1.  Both extents must be multiples of 64 here."""
    from . import ops as O
    from .formats import get_quantization_map

    if weight.ndim != 2 or weight.dtype != torch.bfloat16:
        raise NotImplementedError("quantize_nvfp4_square takes a bfloat16 matrix")
    n, k = weight.shape
    weight = weight.contiguous()
    t = O.calculate_global_scale(weight, FP4_MAX, E4M3_MAX)
    amax = weight.abs().view(n // BLOCK_SIZE, BLOCK_SIZE, k // BLOCK_SIZE, BLOCK_SIZE).amax((1, 3))
    scale = torch.ops.quantized_ops.vmap((amax / FP4_MAX / t).clamp(max=E4M3_MAX),
                                         get_quantization_map("fp8_e4m3", weight.device))
    scale = torch.where(scale > 0, scale, torch.ones((), dtype=scale.dtype, device=scale.device))
    values = torch.ops.quantized_ops.quantize(weight, scale * t, None, [0, 1], BLOCK_SIZE,
                                              get_quantization_map("fp4_e2m1", weight.device))
    rows = pack_nvfp4(values, scale.repeat_interleave(BLOCK_SIZE, 0), check=False)
    cols = pack_nvfp4(values.mT.contiguous(), scale.mT.repeat_interleave(BLOCK_SIZE, 0).contiguous(), check=False)
    return rows.codes, rows.scales, cols.codes, cols.scales, t


def unpack_nvfp4(codes: torch.Tensor, scales: torch.Tensor):
    """``(values, block_scales)`` in bfloat16, ``[..., K]`` and ``[..., K / 16]``: the inverse of
    ``pack_nvfp4`` (reference ``backend/gpu/nvfp4.py:1073-1091``)."""
    table = torch.tensor(_E2M1_VALUES, dtype=torch.bfloat16, device=codes.device)
    nibbles = torch.stack([codes & 0xF, codes >> 4], -1).flatten(-2).long()
    values = table[nibbles]
    *lead, k = values.shape
    rows = values.numel() // max(k, 1)
    r = torch.arange(rows, device=codes.device)[:, None]
    kb = torch.arange(k // BLOCK_SIZE, device=codes.device)[None, :]
    offset = ((r // 128) * (k // 64) + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    block_scales = scales.reshape(-1)[offset].view(torch.float8_e4m3fn).to(torch.bfloat16)
    return values, block_scales.reshape(*lead, -1)


def nvfp4_linear(input: torch.Tensor, input_scale: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                 alpha: torch.Tensor, one: Optional[torch.Tensor] = None,
                 bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``input @ weight.T * alpha + bias`` in bfloat16 on packed NVFP4 operands (``[..., K / 2]`` and
    ``[N, K / 2]`` codes with their packed block scales); ``alpha`` holds the product of the two
    global scales and is applied to the float32 product inside the GEMM; ``one`` is taken for the
    signature only (reference ``backend/gpu/nvfp4.py:1101-1152``)."""
    a = PackedNVFP4(input.reshape(-1, input.shape[-1]), input_scale)
    out = nvfp4_gemm(a, PackedNVFP4(weight, weight_scale), alpha, bias, torch.bfloat16)
    return out.reshape(*input.shape[:-1], -1)


def emulate_nvfp4_linear(input, input_scale, weight, weight_scale, alpha, one=None, bias=None) -> torch.Tensor:
    """``nvfp4_linear`` as the converted graph computes it: operands unpacked to bfloat16 and
    multiplied by ``linear_mx`` (reference ``backend/gpu/nvfp4.py:1190-1227``)."""
    input, input_scale = unpack_nvfp4(input, input_scale)
    weight, weight_scale = unpack_nvfp4(weight, weight_scale)
    return torch.ops.quantized_ops.linear_mx(input, weight, bias, input_scale=input_scale, weight_scale=weight_scale,
                                             block_size=BLOCK_SIZE, alpha=alpha)


# ---------------------------------------------------------------------------
# the ``voyager_gpu`` operators a lowered graph calls
# ---------------------------------------------------------------------------
# Same names and schemas as the reference registers (``backend/gpu/nvfp4.py:675-679, 773-778,
# 851-854, 1094-1097``), on the CUDA key only, so that a graph rewritten by the reference's
# ``backend.gpu.lower`` finds its call targets here.  Packed block scales are returned flat
# (``[ceil(rows/128) * 128 * ceil(K/64) * 4]`` bytes), as the reference's casts return them.
from torch.library import Library  # noqa: E402

voyager_gpu_lib = Library("voyager_gpu", "FRAGMENT")
voyager_gpu_lib.define("cast_nvfp4(Tensor x, Tensor? hadamard, Tensor? seed, int axis) -> (Tensor, Tensor, Tensor)")
voyager_gpu_lib.define("cast_nvfp4_pair(Tensor x, Tensor? hadamard, Tensor? seed, Tensor? transpose_seed) "
                       "-> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
voyager_gpu_lib.define("cast_nvfp4_square(Tensor x) -> (Tensor, Tensor, Tensor, Tensor, Tensor)")
voyager_gpu_lib.define("nvfp4_linear(Tensor input, Tensor input_scale, Tensor weight, Tensor weight_scale, "
                       "Tensor alpha, Tensor one, Tensor? bias) -> Tensor")


def _matrix(x):
    if x.ndim != 2 or x.dtype != torch.bfloat16:
        raise NotImplementedError("the voyager_gpu NVFP4 casts take a bfloat16 matrix")
    return x


def _cast_nvfp4_op(x, hadamard, seed, axis):
    codes, scales, t = quantize_nvfp4(_matrix(x), axis, seed, hadamard)
    return codes, scales.reshape(-1), t


def _cast_nvfp4_pair_op(x, hadamard, seed, transpose_seed):
    c, s, t, ct, st, tt = quantize_nvfp4_pair(_matrix(x), seed, transpose_seed, hadamard)
    return c, s.reshape(-1), t, ct, st.reshape(-1), tt


def _cast_nvfp4_square_op(x):
    c, s, ct, st, t = quantize_nvfp4_square(_matrix(x))
    return c, s.reshape(-1), ct, st.reshape(-1), t


voyager_gpu_lib.impl("cast_nvfp4", N.device_guarded(_cast_nvfp4_op), "CUDA")
voyager_gpu_lib.impl("cast_nvfp4_pair", N.device_guarded(_cast_nvfp4_pair_op), "CUDA")
voyager_gpu_lib.impl("cast_nvfp4_square", N.device_guarded(_cast_nvfp4_square_op), "CUDA")
voyager_gpu_lib.impl("nvfp4_linear", N.device_guarded(nvfp4_linear), "CUDA")


def _fake_cast_outputs(x, rows, cols):
    padded = -(-rows // 128) * 128 * (-(-(cols // BLOCK_SIZE) // 4) * 4)
    return (x.new_empty((rows, cols // 2), dtype=torch.uint8), x.new_empty((padded,), dtype=torch.uint8),
            x.new_empty((), dtype=torch.bfloat16))


@torch.library.register_fake("voyager_gpu::cast_nvfp4")
def _(x, hadamard, seed, axis):
    rows, cols = x.shape if axis % 2 == 1 else x.shape[::-1]
    return _fake_cast_outputs(x, rows, cols)


@torch.library.register_fake("voyager_gpu::cast_nvfp4_pair")
def _(x, hadamard, seed, transpose_seed):
    rows, cols = x.shape
    return (*_fake_cast_outputs(x, rows, cols), *_fake_cast_outputs(x, cols, rows))


@torch.library.register_fake("voyager_gpu::cast_nvfp4_square")
def _(x):
    rows, cols = x.shape
    c, s, t = _fake_cast_outputs(x, rows, cols)
    ct, st, _ = _fake_cast_outputs(x, cols, rows)
    return c, s, ct, st, t


@torch.library.register_fake("voyager_gpu::nvfp4_linear")
def _(input, input_scale, weight, weight_scale, alpha, one, bias):
    return input.new_empty((*input.shape[:-1], weight.shape[0]), dtype=torch.bfloat16)
