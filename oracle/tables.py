"""Oracle: the 65 536-entry lookup tables that define every format's grid.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Restates ``get_quantization_map`` and ``entry_levels``
(reference ``src/voyager_compiler/quantization/fake_quantize.py:69-139``),
the minifloat rounding of ``quantize_to_minifloat``
(``quantization/dtypes/fp8.py:69-135`` with ``round="even"`` and
``saturate_normals=True``), posit rounding (``quantization/dtypes/posit.py:8-73``)
and the NormalFloat levels (``quantization/dtypes/normal_float.py:4-62``),
plus the dtype-name grammar of ``quantization/qspec.py:87-227``.

A table has one entry per bfloat16 bit pattern: entry ``i`` is the value the
bfloat16 whose bits are ``i`` rounds to.  Everything here works in float32
on exact powers of two, so each step is exact.
"""

import functools
import re

import torch

QMAP_SIZE = 1 << 16


def all_bf16() -> torch.Tensor:
    """Every bfloat16 value, entry ``i`` having bit pattern ``i``."""
    bits = torch.arange(QMAP_SIZE, dtype=torch.int32).to(torch.int16)
    return bits.view(torch.bfloat16)


# ----------------------------------------------------------------------------
# dtype names (qspec.py:87-227)
# ----------------------------------------------------------------------------
def int_bounds(name):
    m = re.fullmatch(r"(u?)int(\d+)", name, re.IGNORECASE)
    if not m:
        return None
    n = int(m.group(2))
    return (0, (1 << n) - 1) if m.group(1) else (-(1 << (n - 1)), (1 << (n - 1)) - 1)


def float_params(name):
    """``(ebits, mbits, signed, max_norm)`` of ``fp<B>_e<X>m<Y>[_ieee]``."""
    m = re.fullmatch(r"fp(\d+)_e(\d+)m(\d+)(_ieee)?", name, re.IGNORECASE)
    if not m:
        return None
    total, ebits, mbits = int(m.group(1)), int(m.group(2)), int(m.group(3))
    if total not in (ebits + mbits, ebits + mbits + 1):
        raise ValueError(f"{name}: inconsistent bit counts")
    ieee = ebits > 4 or m.group(4) is not None
    emax = (1 << (ebits - 1)) - 1 if ieee else (1 << (ebits - 1))
    if name.lower() == "fp8_e4m3":
        top = 1.75
    else:
        top = 2.0 - 2.0 ** -mbits
    return ebits, mbits, total == ebits + mbits + 1, (2.0 ** emax) * top


def posit_params(name):
    m = re.fullmatch(r"posit(\d+)_(\d+)", name, re.IGNORECASE)
    return (int(m.group(1)), int(m.group(2))) if m else None


def lut_params(name):
    m = re.fullmatch(r"lut(\d+)(?:_to_(\w+))?", name)
    if not m:
        return None
    return int(m.group(1)), m.group(2)


def dtype_range(name):
    """``(quant_min, quant_max)`` a spec string defaults to (qspec.py:159-193)."""
    if (b := int_bounds(name)) is not None:
        return float(b[0]), float(b[1])
    if (f := float_params(name)) is not None:
        return -f[3], f[3]
    if (p := posit_params(name)) is not None:
        top = float((2 ** (2 ** p[1])) ** (p[0] - 2))
        return -top, top
    if (c := lut_params(name)) is not None:
        top = 1.0 if c[1] is None else dtype_range(c[1])[1]
        return -top, top
    raise ValueError(f"Unsupported dtype: {name}")


# ----------------------------------------------------------------------------
# grids
# ----------------------------------------------------------------------------
def _round_minifloat(values, ebits, mbits, max_norm):
    """Round float32 ``values`` (already clamped) half-to-even onto the grid."""
    mag = values.abs()
    # floor(log2 |v|), zero treated as one.
    exponent = torch.floor(torch.log2(torch.where(mag == 0, torch.ones_like(mag), mag)))
    emin = 2 - (1 << (ebits - 1))
    exponent = exponent.clamp(min=emin)
    step = torch.exp2(exponent - mbits)
    scaled = mag / step
    rounded = torch.round(scaled)  # half to even
    out = torch.sign(values) * rounded * step
    # sign(-0) is +0 and sign(tiny negative) is -1, so a negative value that
    # rounds to nothing stays -0 while -0 itself becomes +0, as in the reference.
    return out.clamp(-max_norm, max_norm)


def _posit_table(values, nbits, es):
    """Posit rounding by neighbour search over the decoded positive posits.

    A positive value between adjacent n-bit posits ``p[k] <= x < p[k+1]``
    rounds on the encoded bit string: the boundary is the (n+1)-bit posit
    whose pattern is ``2k+1``; a tie goes to the even pattern.  Magnitudes
    below ``2**floor(-(n-1)*2**es + 2**(es-1))`` become zero, magnitudes
    past maxpos saturate, and non-finite inputs become NaN.
    """

    def decode(pattern, width):
        # value of a positive posit bit pattern of ``width`` bits (sign bit 0)
        body = format(pattern, f"0{width - 1}b")
        lead = body[0]
        run = len(body) - len(body.lstrip(lead))
        k = run - 1 if lead == "1" else -run
        rest = body[run + 1:]  # skip the regime terminator
        ebits_str = rest[:es].ljust(es, "0")
        e = int(ebits_str, 2) if es else 0
        frac = rest[es:]
        f = int(frac, 2) / (1 << len(frac)) if frac else 0.0
        return (2.0 ** ((1 << es) * k + e)) * (1.0 + f)

    top = (1 << (nbits - 1)) - 1
    grid = torch.tensor([decode(p, nbits) for p in range(1, top + 1)], dtype=torch.float64)
    mids = torch.tensor(
        [decode(2 * p + 1, nbits + 1) for p in range(1, top)], dtype=torch.float64
    )
    x = values.double()
    mag = x.abs()
    below = torch.searchsorted(grid, mag, right=True) - 1  # grid[below] <= mag
    below = below.clamp(0, top - 1)
    pattern = below + 1
    has_next = below < top - 1
    mid = mids[below.clamp(max=top - 2)]
    up = has_next & ((mag > mid) | ((mag == mid) & (pattern % 2 == 1)))
    picked = torch.where(up, grid[(below + 1).clamp(max=top - 1)], grid[below])
    picked = torch.where(mag < grid[0], grid[0].expand_as(picked), picked)
    threshold = 2.0 ** ((-(nbits - 1) * (1 << es) + 2 ** (es - 1)) // 1)
    out = torch.sign(x) * picked
    out = torch.where((mag < threshold) | (x == 0), torch.zeros_like(out), out)
    out = torch.where(torch.isfinite(x), out, torch.full_like(out, float("nan")))
    return out.to(values.dtype)


def normal_float_levels(index_bits):
    """NormalFloat's ``2**k`` levels in [-1, 1], one more positive than negative."""
    from scipy.stats import norm

    half = 1 << (index_bits - 1)
    offset = 0.9677083
    pos = norm.ppf(torch.linspace(offset, 0.5, half + 1)[:-1]).tolist()
    neg = (-norm.ppf(torch.linspace(offset, 0.5, half)[:-1])).tolist()
    levels = torch.tensor(pos + [0] + neg, dtype=torch.float32).sort().values
    return levels / levels.max()


def grid_levels(table):
    """Distinct finite entries of a table, ascending float32, a single +0."""
    t = table.float()
    return torch.unique(t[torch.isfinite(t)]) + 0.0


def entry_levels(name):
    """Symmetric value grid of a LUT entry dtype (fake_quantize.py:125-139)."""
    levels = grid_levels(quantization_map(name))
    return levels[levels >= -levels.max()]


@functools.lru_cache(maxsize=None)
def quantization_map(name):
    """The bfloat16 table for ``name`` (``None`` = identity)."""
    v = all_bf16()
    if name is None:
        return v

    if (bounds := int_bounds(name)) is not None:
        return torch.clamp(torch.round(v), bounds[0], bounds[1])

    if (fmt := float_params(name)) is not None:
        ebits, mbits, signed, max_norm = fmt
        f = v.float()
        if not signed:
            f = f.abs()
        f = f.clamp(-max_norm, max_norm)
        return _round_minifloat(f, ebits, mbits, max_norm).to(torch.bfloat16)

    if (pos := posit_params(name)) is not None:
        return _posit_table(v, *pos)

    if (lut := lut_params(name)) is not None:
        index_bits, entry = lut
        levels = normal_float_levels(index_bits)
        if entry is not None:
            grid = entry_levels(entry)
            levels = levels.to(grid) * grid.max()
            levels = grid[(levels[:, None] - grid).abs().argmin(-1)]
        levels = levels.to(torch.bfloat16)
        x = v.clamp(levels.min(), levels.max())
        out = torch.empty_like(v)
        for start in range(0, QMAP_SIZE, 8192):
            chunk = x[start:start + 8192]
            nearest = (levels - chunk[:, None]).abs().argmin(-1)
            out[start:start + 8192] = levels[nearest]
        return out

    raise ValueError(f"Unsupported dtype: {name}")


def index_table(table):
    """The int64 index form of a LUT table (quantize_pt2e.py:767-771)."""
    values = torch.unique(table)
    return torch.searchsorted(values, table).to(torch.int64), values
