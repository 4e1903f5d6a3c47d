"""Number formats: dtype-name grammar, spec strings and the bfloat16 lookup tables.

Host-side set-up code.  The names and meanings follow the reference's
``quantization/qspec.py`` (``int_range:87``, ``float_format:122``,
``posit_format:159``, ``parse_codebook_dtype:196``, ``parse_spec_fields:230``)
and ``quantization/fake_quantize.py`` (``get_quantization_map:69``,
``entry_levels:125``), so spec strings such as
``"int8,qs=microscaling,bs=16,pot=1"`` mean the same thing here.

Tables are built with integer arithmetic on IEEE bit patterns (numpy), one
entry per bfloat16 bit pattern, and cached per (dtype, device).
"""

import enum
import functools
import re
from typing import NamedTuple, Optional, Tuple

import numpy as np
import torch

QMAP_SIZE = 1 << 16
DEFAULT_AMAX_HISTORY_LEN = 64


# ---------------------------------------------------------------------------
# dtype names
# ---------------------------------------------------------------------------
class QScheme(enum.Enum):
    PER_TENSOR_SYMMETRIC = "per_tensor_symmetric"
    PER_CHANNEL_SYMMETRIC = "per_channel_symmetric"
    MICROSCALING = "microscaling"
    GROUP_WISE_AFFINE = "group_wise_affine"


class FloatFormat(NamedTuple):
    bits: int
    ebits: int
    mbits: int
    ieee: bool
    max_norm: float

    @property
    def signed(self) -> bool:
        return self.bits == self.ebits + self.mbits + 1

    @property
    def emin(self) -> int:
        """Exponent of the smallest normal value (also of the subnormals' step)."""
        return 2 - (1 << (self.ebits - 1))


_INT_RE = re.compile(r"(u?)int(\d+)", re.IGNORECASE)
_FLOAT_RE = re.compile(r"fp(\d+)_e(\d+)m(\d+)(_ieee)?", re.IGNORECASE)
_POSIT_RE = re.compile(r"posit(\d+)_(\d+)", re.IGNORECASE)
_LUT_RE = re.compile(r"lut(\d+)(?:_to_(\w+))?")


def int_range(dtype: str) -> Optional[Tuple[int, int]]:
    m = _INT_RE.fullmatch(dtype)
    if m is None:
        return None
    width = int(m.group(2))
    if m.group(1):
        return 0, (1 << width) - 1
    return -(1 << (width - 1)), (1 << (width - 1)) - 1


def float_format(dtype: str) -> Optional[FloatFormat]:
    """``fp<B>_e<X>m<Y>[_ieee]``: B = X+Y+1 is signed, B = X+Y unsigned.  More
    than four exponent bits, or ``_ieee``, reserves the top exponent for
    inf/NaN; ``fp8_e4m3`` is torch's ``float8_e4m3fn`` (max 448)."""
    m = _FLOAT_RE.fullmatch(dtype)
    if m is None:
        return None
    bits, ebits, mbits = (int(m.group(i)) for i in (1, 2, 3))
    if bits - ebits - mbits not in (0, 1):
        raise ValueError(
            f"{dtype}: {bits} bits cannot hold {ebits} exponent and {mbits} mantissa bits "
            "with or without a sign bit")
    ieee = ebits > 4 or m.group(4) is not None
    emax = (1 << (ebits - 1)) - (1 if ieee else 0)
    if dtype.lower() == "fp8_e4m3":
        max_norm = 1.75 * 2.0 ** emax
    else:
        max_norm = (2.0 - 2.0 ** -mbits) * 2.0 ** emax
    return FloatFormat(bits, ebits, mbits, ieee, max_norm)


def posit_format(dtype: str) -> Optional[Tuple[int, int]]:
    m = _POSIT_RE.fullmatch(dtype)
    return None if m is None else (int(m.group(1)), int(m.group(2)))


def parse_codebook_dtype(dtype: str):
    """``lut<I>[_to_<E>]`` -> ``(index_bits, entry_dtype or None)``."""
    m = _LUT_RE.fullmatch(dtype)
    if m is None:
        return None
    index_bits, entry = int(m.group(1)), m.group(2)
    if entry is not None:
        ints, flt = int_range(entry), float_format(entry)
        signed_int = ints is not None and ints[0] != 0
        signed_float = flt is not None and flt.signed
        if not (signed_int or signed_float):
            raise ValueError(
                f"{dtype}: lookup-table entries must be int<N> or a signed fp<B>_e<X>m<Y>, not {entry}")
    return index_bits, entry


def quant_range(dtype: str) -> Tuple[float, float]:
    """The ``(quant_min, quant_max)`` a spec string defaults to."""
    if (r := int_range(dtype)) is not None:
        return float(r[0]), float(r[1])
    if (f := float_format(dtype)) is not None:
        return -f.max_norm, f.max_norm
    if (p := posit_format(dtype)) is not None:
        top = float((2 ** (2 ** p[1])) ** (p[0] - 2))
        return -top, top
    if (c := parse_codebook_dtype(dtype)) is not None:
        top = 1.0 if c[1] is None else quant_range(c[1])[1]
        return -top, top
    raise ValueError(f"Unsupported dtype: {dtype}")


# ---------------------------------------------------------------------------
# spec strings
# ---------------------------------------------------------------------------
_KEY_ALIASES = {
    "qmin": "quant_min", "qmax": "quant_max", "qs": "qscheme", "ahl": "amax_history_len",
    "ax": "ch_axis", "bs": "block_size", "pot": "power_2_scale", "scale": "scale_dtype",
    "othr": "outlier_threshold", "opct": "outlier_pct", "sr": "stochastic_rounding",
    "gs": "global_scale",
}


def _int_or_tuple(text: str):
    text = text.strip()
    if text.startswith("(") and text.endswith(")"):
        return tuple(int(t) for t in text[1:-1].split(","))
    return int(text)


def _flag(text: str) -> bool:
    if text not in ("0", "1", "false", "true"):
        raise ValueError(f"Expected 0, 1, false or true but got '{text}'")
    return text in ("1", "true")


_KEY_TYPES = {
    "quant_min": float, "quant_max": float, "qscheme": QScheme, "amax_history_len": int,
    "ch_axis": _int_or_tuple, "block_size": _int_or_tuple, "power_2_scale": _flag,
    "scale_dtype": str, "outlier_threshold": float, "outlier_pct": float,
    "stochastic_rounding": _flag, "global_scale": _flag,
}


def parse_spec_fields(spec: str) -> dict:
    """``"int8,qs=microscaling,bs=16"`` -> keyword arguments of a quantization spec."""
    if not spec:
        raise ValueError("String quantization_spec is None or empty")
    fields = re.split(r",(?![^()]*\))", spec)  # commas inside (...) belong to a tuple
    out = {"dtype": fields[0]}
    for field in fields[1:]:
        if "=" not in field:
            raise ValueError(f"Expected key=value format but got '{field}'")
        key, value = field.split("=")
        key = _KEY_ALIASES.get(key, key)
        if key not in _KEY_TYPES:
            raise ValueError(f"Unknown argument '{key}'. Valid keys: {', '.join(_KEY_TYPES)}")
        out[key] = _KEY_TYPES[key](value)
    scheme = out.get("qscheme")
    if scheme is not None:
        lo, hi = quant_range(out["dtype"])
        out.setdefault("quant_min", float(lo))
        out.setdefault("quant_max", float(hi))
        if scheme in (QScheme.PER_TENSOR_SYMMETRIC, QScheme.PER_CHANNEL_SYMMETRIC):
            out.setdefault("amax_history_len", DEFAULT_AMAX_HISTORY_LEN)
    return out


# ---------------------------------------------------------------------------
# bit-level helpers (numpy)
# ---------------------------------------------------------------------------
def _bf16_patterns() -> np.ndarray:
    return np.arange(QMAP_SIZE, dtype=np.uint32)


def _bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (NaN -> 0x7FC0 | sign)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    nan = np.isnan(x)
    return np.where(nan, ((u >> 16) & 0x8000) | 0x7FC0, rounded).astype(np.uint16)


def _rne_shift(sig: np.ndarray, shift: np.ndarray) -> np.ndarray:
    """``sig >> shift`` rounded half to even (int64 arrays, shift >= 0)."""
    shift = np.minimum(shift, 62)
    kept = sig >> shift
    rem = sig - (kept << shift)
    half = np.where(shift > 0, np.int64(1) << np.maximum(shift - 1, 0), np.int64(0))
    up = (rem > half) | ((rem == half) & (shift > 0) & ((kept & 1) == 1))
    return kept + up.astype(np.int64)


def _int_table(lo: int, hi: int) -> np.ndarray:
    v = _bf16_to_f32(_bf16_patterns())
    with np.errstate(invalid="ignore"):
        r = np.rint(v)  # half to even, keeps -0
        clipped = np.minimum(np.maximum(r, np.float32(lo)), np.float32(hi))
    out = np.where((r == 0) | np.isnan(r), r, clipped)
    return _f32_to_bf16_bits(out.astype(np.float32))


def _minifloat_table(fmt: FloatFormat) -> np.ndarray:
    bits = _bf16_patterns()
    sign = (bits >> 15) & 1
    mag_bits = (bits & 0x7FFF).astype(np.int64) << 16          # float32 pattern of |v|
    is_nan = (bits & 0x7FFF) > 0x7F80
    exp_field = mag_bits >> 23
    frac = mag_bits & 0x7FFFFF
    # 24-bit significand and its exponent: value = sig * 2^(e - 23)
    sig = np.where(exp_field > 0, frac | (1 << 23), frac)
    e = np.where(exp_field > 0, exp_field - 127, -126)
    # saturate before rounding
    max_sig, max_e = np.frexp(np.float64(fmt.max_norm))        # max = max_sig * 2^max_e
    over = (sig.astype(np.float64) * np.exp2((e - 23).astype(np.float64))) > fmt.max_norm
    # grid step exponent: 2^(max(e, emin) - mbits); drop = bits of sig below the step
    step_e = np.maximum(e, fmt.emin) - fmt.mbits
    drop = step_e - (e - 23)
    q = _rne_shift(sig, np.maximum(drop, 0)) << np.maximum(-drop, 0)
    step_e = np.where(drop < 0, e - 23, step_e)
    value = q.astype(np.float64) * np.exp2(step_e.astype(np.float64))
    value = np.where(over, fmt.max_norm, np.minimum(value, fmt.max_norm))
    if fmt.signed:
        # sign(v) * q: -0 itself becomes +0, a negative that rounds to nothing stays -0
        neg = (sign == 1) & ((bits & 0x7FFF) != 0)
        value = np.where(neg, -value, value)
    out = value.astype(np.float32)
    out = np.where(is_nan, np.float32(np.nan), out)
    return _f32_to_bf16_bits(out)


def _posit_value(pattern: int, nbits: int, es: int) -> float:
    """Value of a positive posit body (the nbits-1 bits after the sign)."""
    width = nbits - 1
    lead = (pattern >> (width - 1)) & 1
    run = 0
    while run < width and ((pattern >> (width - 1 - run)) & 1) == lead:
        run += 1
    k = run - 1 if lead else -run
    used = min(run + 1, width)
    rest_bits = width - used
    rest = pattern & ((1 << rest_bits) - 1)
    e_have = min(es, rest_bits)
    exponent = (rest >> (rest_bits - e_have)) << (es - e_have) if es else 0
    f_bits = rest_bits - e_have
    fraction = (rest & ((1 << f_bits) - 1)) / (1 << f_bits) if f_bits else 0.0
    return 2.0 ** (k * (1 << es) + exponent) * (1.0 + fraction)


def _posit_table(nbits: int, es: int) -> np.ndarray:
    """Round every bfloat16 to posit<nbits, es>: encode as regime|exponent|fraction,
    cut to nbits-1 bits with round-half-even on the bit string, saturate at maxpos;
    magnitudes below 2^floor(-(n-1)*2^es + 2^(es-1)) become 0, non-finite -> NaN."""
    width = nbits - 1
    top = (1 << width) - 1
    import math
    threshold = 2.0 ** math.floor(-(nbits - 1) * (1 << es) + 2 ** (es - 1))
    out = np.zeros(QMAP_SIZE, dtype=np.float32)
    cache = {}
    for b in range(0x0001, 0x7F80):
        x = float(_bf16_to_f32(np.array([b], dtype=np.uint32))[0])
        if x < threshold:
            continue
        mant, ex = math.frexp(x)           # x = mant * 2^ex, mant in [0.5, 1)
        scale = ex - 1
        frac7 = int(round((mant * 2 - 1) * 128))  # bf16 has 7 fraction bits (exact)
        k, exponent = scale >> es, scale & ((1 << es) - 1)
        if k >= 0:
            regime, rlen = ((1 << (k + 1)) - 1) << 1, k + 2
        else:
            regime, rlen = 1, -k + 1
        body = (((regime << es) | exponent) << 7) | frac7
        blen = rlen + es + 7
        if blen > width:
            cut = blen - width
            kept, rem = body >> cut, body & ((1 << cut) - 1)
            half = 1 << (cut - 1)
            if rem > half or (rem == half and (kept & 1)):
                kept += 1
        else:
            kept = body << (width - blen)
        kept = min(max(kept, 1), top)
        if kept not in cache:
            cache[kept] = _posit_value(kept, nbits, es)
        out[b] = cache[kept]
        out[b | 0x8000] = -cache[kept]
    out[0x7F80:0x8000] = np.nan
    out[0xFF80:] = np.nan
    return _f32_to_bf16_bits(out)


def _normal_float_levels(index_bits: int) -> np.ndarray:
    """NormalFloat levels in [-1, 1] (float32): quantiles of N(0,1), one more
    positive level than negative, a zero, normalised by the largest."""
    from scipy.stats import norm

    half = 1 << (index_bits - 1)
    offset = 0.9677083
    upper = norm.ppf(torch.linspace(offset, 0.5, half + 1)[:-1].numpy())
    lower = -norm.ppf(torch.linspace(offset, 0.5, half)[:-1].numpy())
    levels = np.sort(np.concatenate([upper, [0.0], lower]).astype(np.float32))
    return levels / levels.max()


def _levels_of(table_bits: np.ndarray) -> np.ndarray:
    v = _bf16_to_f32(table_bits.astype(np.uint32))
    return np.unique(v[np.isfinite(v)]) + np.float32(0.0)


def _lut_table(index_bits: int, entry: Optional[str]) -> np.ndarray:
    levels = _normal_float_levels(index_bits)
    if entry is not None:
        grid = _levels_of(_table_bits(entry))
        grid = grid[grid >= -grid.max()]
        scaled = levels * grid.max()
        levels = grid[np.abs(scaled[:, None] - grid[None, :]).argmin(-1)]
    levels = _bf16_to_f32(_f32_to_bf16_bits(levels.astype(np.float32)).astype(np.uint32))
    v = _bf16_to_f32(_bf16_patterns())
    with np.errstate(invalid="ignore"):
        x = np.minimum(np.maximum(v, levels.min()), levels.max())
        # |level - x| evaluated in bfloat16, first minimum wins (NaN -> index 0)
        diff = _bf16_to_f32(_f32_to_bf16_bits(np.abs(levels[None, :] - x[:, None])).astype(np.uint32))
    diff = np.where(np.isnan(diff), -1.0, diff)
    return _f32_to_bf16_bits(levels[diff.argmin(-1)])


@functools.lru_cache(maxsize=None)
def _table_bits(dtype: Optional[str]) -> np.ndarray:
    if dtype is None:
        return _bf16_patterns().astype(np.uint16)
    if (r := int_range(dtype)) is not None:
        return _int_table(*r)
    if (f := float_format(dtype)) is not None:
        return _minifloat_table(f)
    if (p := posit_format(dtype)) is not None:
        return _posit_table(*p)
    if (c := parse_codebook_dtype(dtype)) is not None:
        return _lut_table(*c)
    raise ValueError(f"Unsupported dtype: {dtype}")


@functools.lru_cache(maxsize=None)
def get_quantization_map(dtype: Optional[str], device=None) -> torch.Tensor:
    """The 65 536-entry bfloat16 table rounding a bfloat16 value to ``dtype``
    (``None`` = identity).  Shared by all callers: do not modify in place."""
    bits = _table_bits(dtype)
    t = torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
    return t if device is None else t.to(device)


def qmap_levels(qmap: torch.Tensor) -> torch.Tensor:
    """Distinct finite entries of a table, ascending float32, a single +0."""
    t = qmap.float()
    return torch.unique(t[torch.isfinite(t)]) + 0.0


def entry_levels(dtype: str, device=None) -> torch.Tensor:
    levels = qmap_levels(get_quantization_map(dtype, device))
    return levels[levels >= -levels.max()]


def index_table(table: torch.Tensor):
    """``(int64 index table, levels)`` for a lookup-table dtype, the form a
    converted graph stores (reference ``quantize_pt2e.py:754-771``)."""
    levels = torch.unique(table)
    return torch.searchsorted(levels, table).to(torch.int64), levels
