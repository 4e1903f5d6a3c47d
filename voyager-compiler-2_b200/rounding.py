"""Choose how a kernel rounds onto the grid that an operator's ``qmap`` defines.

An operator receives its format as data: a 65 536-entry table indexed by the
bfloat16 bit pattern (values, or int64 indices after conversion of a lookup
format), or a small codebook that is searched.  Gathering from a 128 KB table
is correct for any table but costs one scattered load per element, so the
table is fingerprinted once (one device-to-host copy, cached per tensor) and
an arithmetic form is used only when the table is bit-for-bit the canonical
table of an integer or minifloat format, or when it is a step function with at
most 32 runs (NF4-style codebooks, 4-bit and 2-bit integers, e2m1).  Anything
else is gathered.
"""

import ctypes
import hashlib
import math

import numpy as np
import torch

from . import _native as N
from . import formats

_ARITHMETIC_DTYPES = (
    [f"int{n}" for n in range(2, 9)] + [f"uint{n}" for n in range(1, 9)]
    + ["fp8_e4m3", "fp8_e5m2", "fp8_e5m3", "fp8_e4m3_ieee", "fp6_e3m2", "fp6_e2m3", "fp4_e2m1", "fp4_e3m0",
       "fp8_e3m4", "fp8_e2m5", "fp7_e4m3", "fp7_e3m4"]
)

_fingerprints = None

# A step search costs several dependent shared-memory reads per element and
# measured slower than gathering from the table (0.8 vs 1.6 TB/s for a 16-level
# codebook), so unrecognised tables are gathered.
PREFER_STEPS = False


def _digest(bits: np.ndarray) -> bytes:
    return hashlib.blake2b(np.ascontiguousarray(bits, dtype=np.uint16).tobytes(), digest_size=16).digest()


def _canonical_fingerprints():
    global _fingerprints
    if _fingerprints is None:
        table = {}
        for name in _ARITHMETIC_DTYPES:
            try:
                bits = formats._table_bits(name)
            except ValueError:
                continue
            table[_digest(bits)] = name
        _fingerprints = table
    return _fingerprints


def _minifloat_fits_kernel(fmt: formats.FloatFormat) -> bool:
    top = math.frexp(fmt.max_norm)[1] - 1
    return fmt.mbits <= 10 and fmt.emin - fmt.mbits >= -126 and top - fmt.mbits <= 126 and top >= fmt.emin


def _ordered_key(bits: np.ndarray) -> np.ndarray:
    bits = bits.astype(np.int64)
    return np.where(bits & 0x8000, 0x7FFF - (bits & 0x7FFF), 0x8000 + bits)


def _steps_of(bits: np.ndarray):
    """Describe a table as runs of equal entries over value-ordered inputs, or
    return None when there are more than 32 runs or NaN inputs disagree."""
    patterns = np.arange(1 << 16, dtype=np.int64)
    is_nan = (patterns & 0x7FFF) > 0x7F80
    nan_entries = np.unique(bits[is_nan])
    if nan_entries.size != 1:
        # NaN inputs may map to NaNs of either sign; any NaN stands for them.
        if not np.all((nan_entries & 0x7FFF) > 0x7F80):
            return None
        nan_entries = np.array([0x7FC0], dtype=bits.dtype)
    keys = _ordered_key(patterns[~is_nan])
    order = np.argsort(keys, kind="stable")
    keys, vals = keys[order], bits[~is_nan][order]
    change = np.flatnonzero(vals[1:] != vals[:-1]) + 1
    if change.size + 1 > N.MAX_STEPS:
        return None
    starts = np.concatenate([[0], change])
    values = vals[starts]
    uppers = np.concatenate([keys[change], [0xFFFF]])
    return values.astype(np.uint16), uppers.astype(np.uint16), int(nan_entries[0])


class RoundSpec:
    """A ``VqRound`` plus the tensors it points into (kept alive with it)."""

    __slots__ = ("c", "keep", "mode", "returns_index")

    def __init__(self, c, keep=(), returns_index=False):
        self.c = c
        self.keep = keep
        self.mode = c.mode
        self.returns_index = returns_index

    @property
    def ref(self):
        return ctypes.byref(self.c)


def none_round() -> RoundSpec:
    c = N.VqRound()
    c.mode = N.ROUND_NONE
    return RoundSpec(c)


_NONE = None
_table_cache = {}


def _classify_table(table_bf16: torch.Tensor, allow_arithmetic=True) -> RoundSpec:
    c = N.VqRound()
    c.mode = N.ROUND_TABLE
    c.table = table_bf16.data_ptr()
    if not allow_arithmetic:
        return RoundSpec(c, (table_bf16,))
    bits = table_bf16.view(torch.int16).cpu().numpy().view(np.uint16)
    name = _canonical_fingerprints().get(_digest(bits))
    if name is not None:
        if (r := formats.int_range(name)) is not None:
            c.mode = N.ROUND_INT
            c.lo, c.hi = float(r[0]), float(r[1])
            return RoundSpec(c, (table_bf16,))
        fmt = formats.float_format(name)
        if fmt is not None and _minifloat_fits_kernel(fmt):
            c.mode = N.ROUND_MINIFLOAT
            c.emin, c.mbits = fmt.emin, fmt.mbits
            c.max_norm = float(fmt.max_norm)
            c.is_signed = int(fmt.signed)
            return RoundSpec(c, (table_bf16,))
    steps = _steps_of(bits) if PREFER_STEPS else None
    if steps is not None:
        values, uppers, nan_value = steps
        packed = np.concatenate([uppers, values]).astype(np.uint16).view(np.int16)
        steps = torch.from_numpy(packed.copy()).to(table_bf16.device)
        c.mode = N.ROUND_STEPS
        c.n_steps = len(values)
        c.steps = steps.data_ptr()
        c.nan_value = nan_value
        return RoundSpec(c, (table_bf16, steps))
    return RoundSpec(c, (table_bf16,))


def table_round(qmap: torch.Tensor, allow_arithmetic=True) -> RoundSpec:
    """Rounding through a 65 536-entry table (bfloat16 values or int64 indices).

    The first use of a table copies it to the host once to fingerprint it;
    make that first call outside any CUDA-graph capture.
    """
    key = (qmap.data_ptr(), qmap.device, qmap.dtype, qmap._version, allow_arithmetic)
    hit = _table_cache.get(key)
    if hit is not None:
        return hit
    table = qmap if qmap.dtype == torch.bfloat16 else qmap.to(torch.bfloat16)
    table = table.contiguous()
    spec = _classify_table(table, allow_arithmetic)
    spec.keep = (qmap, table) + tuple(spec.keep)
    if len(_table_cache) > 256:
        _table_cache.clear()
    _table_cache[key] = spec
    return spec


_levels_cache = {}


def stochastic_round(qmap: torch.Tensor, seed: torch.Tensor) -> RoundSpec:
    key = (qmap.data_ptr(), qmap.device, qmap.dtype, qmap._version)
    hit = _levels_cache.get(key)
    if hit is None:
        levels = formats.qmap_levels(qmap) if qmap.numel() == formats.QMAP_SIZE else qmap.float()
        levels = levels.contiguous()
        if len(_levels_cache) > 256:
            _levels_cache.clear()
        # the entry holds the table itself: its address cannot be handed to another tensor while it is cached
        _levels_cache[key] = (qmap, levels)
    else:
        levels = hit[1]
    if seed.dtype != torch.int64 or seed.device != qmap.device:
        seed = seed.to(device=qmap.device, dtype=torch.int64)
    c = N.VqRound()
    c.mode = N.ROUND_STOCHASTIC
    c.levels = levels.data_ptr()
    c.n_levels = levels.numel()
    c.seed = seed.data_ptr()
    return RoundSpec(c, (levels, seed))


def search_round(codebook: torch.Tensor, bounds) -> RoundSpec:
    """Nearest entry of a 1-D ascending codebook: the element falls between the
    midpoints of neighbouring entries (``bounds`` when given, in which case the
    result is the entry's index instead of its value)."""
    if bounds is not None:
        edges = bounds.float().contiguous()
        levels = None
    else:
        edges = ((codebook[:-1] + codebook[1:]) / 2).float().contiguous()
        levels = codebook.float().contiguous()
    c = N.VqRound()
    c.mode = N.ROUND_SEARCH
    c.edges = edges.data_ptr() if edges.numel() else None
    c.n_edges = edges.numel()
    if levels is not None:
        c.levels = levels.data_ptr()
        c.n_levels = levels.numel()
    return RoundSpec(c, (edges, levels), returns_index=bounds is not None)
