"""Oracle: quantize / dequantize / microscaling / affine ops on the CPU.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Restates the reference operators of ``src/voyager_compiler/ops/quantized.py``
(``vmap:151``, ``encode:232``, ``decode:290``, ``_philox:339``,
``_stochastic_round:418``, ``quantize:458``, ``dequantize:527``,
``calculate_mx_qparam:966``, ``hadamard_rotate:1038``, ``quantize_mx:1080``,
``dequantize_mx:1125``, ``quantize_mx_transpose:1171``,
``quantize_affine:1227``), the block geometry of
``quantization/mx_utils.py:16-125`` and ``calculate_global_scale``
(``quantization/fake_quantize.py:142-160``).

Numerics contract being restated: every intermediate is held in the input's
dtype, i.e. each arithmetic step is an exact float32 operation followed by
one round-to-nearest-even into that dtype (torch's CPU behaviour for
bfloat16/float16); Python-scalar divisors are used as float32 values.
"""

import math

import numpy as np
import torch

QMAP_SIZE = 1 << 16


# ----------------------------------------------------------------------------
# table / codebook lookups
# ----------------------------------------------------------------------------
def vmap(x, table):
    """Round through a 65 536-entry table indexed by the bfloat16 bit pattern."""
    bits = x.to(torch.bfloat16).contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
    return table[bits].to(x.dtype)


def _split_regions(x, counts):
    if len(counts) != x.dim():
        raise ValueError("codebook region grid rank does not match the tensor")
    if any(s % c for s, c in zip(x.shape, counts)):
        raise ValueError("codebook region grid does not divide the tensor")
    shape = []
    for s, c in zip(x.shape, counts):
        shape += [c, s // c]
    n = len(counts)
    order = list(range(0, 2 * n, 2)) + list(range(1, 2 * n, 2))
    back = [order.index(i) for i in range(2 * n)]
    return x.reshape(shape).permute(order), back


def encode(x, codebook, bounds=None):
    """Nearest codebook entry (or its index when ``bounds`` is given)."""
    edges = bounds if bounds is not None else (codebook[..., :-1] + codebook[..., 1:]) / 2
    if codebook.dim() == 1:
        idx = torch.searchsorted(edges, x.to(torch.bfloat16).float())
        return (idx if bounds is not None else codebook[idx]).to(x.dtype)
    moved, back = _split_regions(x, tuple(codebook.shape[:-1]))
    regions = codebook.numel() // codebook.shape[-1]
    flat = moved.reshape(regions, -1).to(torch.bfloat16).float().contiguous()
    idx = torch.searchsorted(edges.reshape(regions, -1).contiguous(), flat)
    got = idx if bounds is not None else codebook.reshape(regions, -1).gather(1, idx)
    return got.view(moved.shape).permute(back).reshape(x.shape).to(x.dtype)


def decode(indices, codebook):
    idx = indices.to(torch.long)
    if codebook.dim() == 1:
        return codebook[idx].to(indices.dtype)
    moved, back = _split_regions(idx, tuple(codebook.shape[:-1]))
    regions = codebook.numel() // codebook.shape[-1]
    got = codebook.reshape(regions, -1).gather(1, moved.reshape(regions, -1))
    return got.view(moved.shape).permute(back).reshape(idx.shape).to(indices.dtype)


# ----------------------------------------------------------------------------
# block geometry
# ----------------------------------------------------------------------------
def _norm_axes(axes, ndim):
    axes = [axes] if isinstance(axes, int) else list(axes)
    return sorted(a % ndim for a in axes)


def block_reduce(x, axes, block, how):
    """Reduce each block of ``block`` elements along every axis in ``axes``.

    A short last block is padded with zeros before the reduction (the
    reference pads before its amax/amin, ``mx_utils.py:85-105``); an axis
    shorter than the block is therefore one zero-padded block.
    """
    fn = {"amax": torch.amax, "amin": torch.amin}[how]
    for a in _norm_axes(axes, x.dim()):
        n = x.shape[a]
        if n % block:
            pad = [0, 0] * (x.dim() - 1 - a) + [0, block - n % block]
            x = torch.nn.functional.pad(x, pad)
            n = x.shape[a]
        x = fn(x.unflatten(a, (n // block, block)), dim=a + 1)
    return x


def expand_blocks(param, like, block):
    """One value per block repeated over the block, cut to ``like``'s shape."""
    while param.dim() < like.dim():
        param = param.unsqueeze(0)
    for d, n in enumerate(like.shape):
        if param.shape[d] != n:
            param = param.repeat_interleave(block, d)
    if list(param.shape) != list(like.shape):
        param = param[tuple(slice(n) for n in like.shape)]
    return param


# ----------------------------------------------------------------------------
# stochastic rounding (Philox4x32-10; quantized.py:318-446)
# ----------------------------------------------------------------------------
_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = np.uint64(0x9E3779B9), np.uint64(0xBB67AE85)
_LO = np.uint64(0xFFFFFFFF)


def philox4x32(counter, seed):
    """Four uint32 words per 64-bit counter under the 64-bit key ``seed``."""
    counter = np.asarray(counter, dtype=np.uint64)
    seed = np.uint64(int(seed) & 0xFFFFFFFFFFFFFFFF)
    c = [counter & _LO, counter >> np.uint64(32), np.zeros_like(counter), np.zeros_like(counter)]
    k0, k1 = seed & _LO, seed >> np.uint64(32)
    for _ in range(10):
        p0, p1 = c[0] * _M0, c[2] * _M1
        c = [
            (p1 >> np.uint64(32)) ^ c[1] ^ k0,
            p1 & _LO,
            (p0 >> np.uint64(32)) ^ c[3] ^ k1,
            p0 & _LO,
        ]
        k0, k1 = (k0 + _W0) & _LO, (k1 + _W1) & _LO
    return np.stack(c, -1)


def random_bytes(seed, shape):
    """Element ``i`` takes byte ``i%4`` of word ``(i%16)//4`` of draw ``i//16``."""
    n = math.prod(shape)
    words = philox4x32(np.arange(-(-n // 16), dtype=np.uint64), int(seed))
    shifts = np.arange(0, 32, 8, dtype=np.uint64)
    by = ((words[..., None] >> shifts) & np.uint64(0xFF)).reshape(-1)[:n]
    return torch.from_numpy(by.astype(np.int64)).view(shape)


def table_levels(table):
    t = table.float()
    return torch.unique(t[torch.isfinite(t)]) + 0.0


def stochastic_round(x, qmap, seed):
    levels = (table_levels(qmap) if qmap.numel() == QMAP_SIZE else qmap).float()
    v = x.float().clamp(levels[0], levels[-1])
    hi_i = torch.searchsorted(levels, v).clamp(max=levels.numel() - 1)
    hi = levels[hi_i]
    lo = torch.where(hi == v, hi, levels[(hi_i - 1).clamp(min=0)])
    noise = random_bytes(seed, x.shape) / 256
    near = torch.where(v < 0, hi, lo)
    far = torch.where(v < 0, lo, hi)
    away = v.abs() + noise * (hi - lo) >= far.abs()
    return torch.where(away, far, near).to(x.dtype)


# ----------------------------------------------------------------------------
# quantize / dequantize
# ----------------------------------------------------------------------------
def quantize(x, scale, zero_point=None, axes=None, block_size=None, qmap=None,
             output_code=None, seed=None):
    if block_size is not None:
        scale = expand_blocks(scale, x, block_size)
        if zero_point is not None:
            zero_point = expand_blocks(zero_point, x, block_size)
    y = x / scale if zero_point is None else x / scale + zero_point
    if qmap is None:
        return y
    if seed is not None:
        return stochastic_round(y, qmap, seed)
    if qmap.numel() == QMAP_SIZE and qmap.dim() == 1:
        return vmap(y, qmap)
    return encode(y, qmap, output_code)


def dequantize(x, scale, zero_point=None, axes=None, block_size=None,
               input_qmap=None, output_qmap=None):
    if input_qmap is not None:
        x = vmap(x, input_qmap)
    if block_size is not None:
        scale = expand_blocks(scale, x, block_size)
        if zero_point is not None:
            zero_point = expand_blocks(zero_point, x, block_size)
    y = x * scale if zero_point is None else (x - zero_point) * scale
    if output_qmap is not None:
        y = vmap(y, output_qmap)
    return y


def floor_log2(amax):
    """floor(log2(x)) of non-negative float32 values, zero read as 2**-126."""
    a = amax.float()
    a = torch.where(a == 0, torch.full_like(a, 2.0 ** -126), a)
    _, e = torch.frexp(a)  # a = m * 2**e with m in [0.5, 1)
    return (e - 1).to(torch.float32)


def calculate_mx_qparam(x, axes, block_size, quant_max, force_scale_power_of_two=False,
                        scale_qmap=None, global_scale=None):
    assert block_size > 0
    amax = block_reduce(x.abs(), axes, block_size, "amax")
    if force_scale_power_of_two:
        finite = torch.isfinite(amax)
        e = floor_log2(torch.where(finite, amax, torch.ones_like(amax)))
        e = e - math.floor(math.log2(quant_max))
        scale = torch.ldexp(torch.ones_like(e), e.to(torch.int32)).to(x.dtype)
        # An infinite amax gives an infinite scale; a NaN one gives NaN, which
        # the final ``> 0`` test replaces by one.
        scale = torch.where(finite, scale, amax.abs())
    else:
        scale = amax / quant_max
        if global_scale is not None:
            scale = scale / global_scale
        if scale_qmap is not None:
            scale = vmap(scale, scale_qmap)
    return torch.where(scale > 0.0, scale, torch.ones_like(scale))


def quantize_mx(x, qmap, axes, block_size, quant_max, force_scale_power_of_two=False,
                scale_qmap=None, output_code=None, seed=None, global_scale=None):
    scale = calculate_mx_qparam(x, axes, block_size, quant_max, force_scale_power_of_two,
                                scale_qmap, global_scale)
    element_scale = scale if global_scale is None else scale * global_scale
    codes = quantize(x, element_scale, None, axes, block_size, qmap, output_code, seed)
    return scale, codes


def decode_and_scale(x, scale, code, block_size):
    if code is not None:
        x = decode(x, code)
    if scale is not None:
        x = x * expand_blocks(scale, x, block_size)
    return x


def dequantize_mx(x, scale, block_size, code=None, global_scale=None):
    y = decode_and_scale(x, scale, code, block_size)
    return y if global_scale is None else y * global_scale


def quantize_affine(x, qmap, axes, block_size, quant_min, quant_max, scale_qmap=None):
    assert block_size > 0
    (axis,) = axes
    axis %= x.dim()
    low = block_reduce(x, [axis], block_size, "amin")
    high = block_reduce(x, [axis], block_size, "amax")
    one = torch.ones((), dtype=x.dtype)
    scale = (high - low) / (quant_max - quant_min)
    scale = torch.where(scale > 0.0, scale, one)
    if scale_qmap is not None:
        scale = vmap(scale, scale_qmap)
        scale = torch.where(scale > 0.0, scale, one)
    zero_point = -low / scale + quant_min
    if scale_qmap is not None:
        zero_point = vmap(zero_point, scale_qmap)
    codes = quantize(x, scale, zero_point, [axis], block_size, qmap)
    return scale, zero_point, codes


def calculate_global_scale(x, quant_max, scale_max):
    ratio = x.abs().amax() / (quant_max * scale_max)
    return ratio.clamp_min(torch.finfo(torch.float32).tiny)


# ----------------------------------------------------------------------------
# Hadamard rotation and the two-layout quantize
# ----------------------------------------------------------------------------
HADAMARD_SIZE = 16
HADAMARD_SIGNS = (1, 1, 1, -1, 1, -1, -1, -1, -1, -1, -1, 1, -1, 1, -1, -1)


def hadamard_matrix():
    """``diag(signs) @ H16 / 4`` (fake_quantize.py:47-65)."""
    h = torch.ones(1, 1)
    while h.shape[0] < HADAMARD_SIZE:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)])
    signs = torch.tensor(HADAMARD_SIGNS, dtype=torch.float32)
    return signs[:, None] * h / 4.0


def hadamard_rotate(x, axis, matrix):
    axis %= x.dim()
    if axis < x.dim() - 2:
        raise ValueError(f"cannot rotate along axis {axis} of {x.dim()}")
    pad = -x.shape[axis] % HADAMARD_SIZE
    if pad:
        x = torch.nn.functional.pad(x, (0, 0) * (x.dim() - 1 - axis) + (0, pad))
    runs = x.float().unflatten(axis, (-1, HADAMARD_SIZE))
    m = matrix.float()
    out = runs @ m if axis == x.dim() - 1 else m.T @ runs
    return out.flatten(axis, axis + 1).to(x.dtype)


def quantize_mx_transpose(x, qmap, block_size, quant_max, force_scale_power_of_two=False,
                          scale_qmap=None, output_code=None, seed=None, global_scale=None,
                          transpose_seed=None, transpose_global_scale=None, hadamard=None):
    t = x.mT
    if hadamard is not None:
        t = hadamard_rotate(t, -1, hadamard)
    common = (qmap, (-1,), block_size, quant_max, force_scale_power_of_two, scale_qmap,
              output_code)
    return (*quantize_mx(x, *common, seed, global_scale),
            *quantize_mx(t, *common, transpose_seed, transpose_global_scale))
