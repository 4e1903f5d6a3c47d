"""Real-FP8 execution of per-tensor / per-channel quantized GEMMs.

A converted per-tensor graph runs ``quantize -> aten.linear / aten.matmul ->
dequantize`` on bfloat16 tensors that merely hold FP8 values.  The reference's
GPU backend replaces each such site by a cast to FP8 bytes and one scaled FP8
GEMM (``backend/gpu/fp8.py``: ``quantize_fp8:253``, ``fp8_linear:372``,
``fp8_bmm:403``).  These functions are that replacement on hand-written
sm_100a kernels: the cast writes the exact byte encoding of the value the
``quantize`` op would have produced, and the GEMM is a tcgen05 ``kind::f8f6f4``
MMA with fp32 accumulation whose epilogue applies ``scale_a * scale_b`` and the
bias before a single rounding.
"""

import math
from typing import Optional

import torch

from . import _native as N
from .ops import _DTYPE_ID, _dtype_id, _ptr, _stream, gemm_tn

_FORMATS = {"fp8_e4m3": N.IN_E4M3, "fp8_e5m2": N.IN_E5M2,
            torch.float8_e4m3fn: N.IN_E4M3, torch.float8_e5m2: N.IN_E5M2}


def _typed(codes: torch.Tensor, dtype):
    """Bytes for a format named by a string; the torch FP8 dtype when that is what was asked for
    (the reference's casts return float8 tensors)."""
    return codes.view(dtype) if isinstance(dtype, torch.dtype) else codes


@N.device_guarded
def quantize_fp8(x: torch.Tensor, scale: torch.Tensor, dtype="fp8_e4m3") -> torch.Tensor:
    """Cast ``x / scale`` to FP8 (reference ``backend/gpu/fp8.py:253-261``): a ``uint8`` tensor of
    ``x``'s shape for ``dtype`` ``"fp8_e4m3"`` / ``"fp8_e5m2"``, a float8 tensor for a torch dtype.

    ``scale`` holds one element, or one per row of the last axis
    (shape ``[..., 1]``, per-channel weights).
    """
    if x.dtype != torch.bfloat16:
        raise NotImplementedError("quantize_fp8 takes bfloat16 input")
    x = x.contiguous()
    n = x.numel()
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    if scale.numel() == 1:
        per = 0
    else:
        rows = n // x.shape[-1]
        if scale.numel() != rows:
            raise ValueError(f"scale of shape {tuple(scale.shape)} is neither one value nor one per row of {tuple(x.shape)}")
        per = x.shape[-1]
        scale = scale.contiguous()
    if scale.dtype not in _DTYPE_ID:
        scale = scale.float()
    if n % 16 or (per % 16):
        raise NotImplementedError("quantize_fp8 needs element counts that are multiples of 16")
    N.check(N.lib().vq_quantize_fp8(x.data_ptr(), scale.data_ptr(), _dtype_id(scale.dtype), out.data_ptr(),
                                    _FORMATS[dtype], n, per, _stream()), "vq_quantize_fp8")
    return _typed(out, dtype)


def fp8_gemm(a: torch.Tensor, b: torch.Tensor, alpha: Optional[torch.Tensor] = None,
             bias: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, dtype: str = "fp8_e4m3",
             alpha_cols: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
             causal=None, gated_scale: Optional[torch.Tensor] = None, round_acc: bool = False,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``alpha * alpha_cols[n] * (a @ b^T) + bias`` (+ ``residual`` after the rounding) for FP8 byte
    operands ``a [*batch, M, K]`` and ``b [*batch, N, K]`` (or ``[N, K]``), fp32 accumulation;
    ``causal``, ``gated_scale``, ``round_acc`` and ``out`` as for ``ops.gemm_tn``."""
    return gemm_tn(a, b, out_dtype=out_dtype, alpha=alpha, bias=bias, in_kind=_FORMATS[dtype],
                   alpha_cols=alpha_cols, residual=residual, causal=causal, gated_scale=gated_scale,
                   round_acc=round_acc, out=out)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, chunk: int = 32) -> torch.Tensor:
    """Rows of two ``[I, ...]`` tensors (weights, or per-row scales) alternating in runs of ``chunk``:
    the row order the gated GEMM epilogue expects of its B operand and of ``alpha_cols``."""
    if gate.shape != up.shape or gate.shape[0] % chunk:
        raise ValueError("gate and up must have one shape with a multiple of 32 rows")
    g = gate.reshape(gate.shape[0] // chunk, 1, chunk, *gate.shape[1:])
    u = up.reshape(up.shape[0] // chunk, 1, chunk, *up.shape[1:])
    return torch.cat([g, u], 1).reshape(2 * gate.shape[0], *gate.shape[1:]).contiguous()


def _as_bytes(t: torch.Tensor):
    """FP8 tensors (torch float8 dtypes or raw bytes) as ``(uint8 view, format name)``."""
    if t.dtype == torch.float8_e5m2:
        return t.view(torch.uint8), "fp8_e5m2"
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8), "fp8_e4m3"
    if t.dtype == torch.uint8:
        return t, "fp8_e4m3"
    raise NotImplementedError(f"FP8 operands are float8 tensors or their bytes, not {t.dtype}")


def fp8_linear(input: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor,
               bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``input @ weight.T * scale + bias`` in bfloat16 as one FP8 GEMM (reference
    ``backend/gpu/fp8.py:372-400``).  ``input [..., K]`` and ``weight [N, K]`` are FP8;
    ``scale`` is a float32 scalar or ``[1, N]`` per output channel; ``bias [N]`` bfloat16."""
    a, fmt = _as_bytes(input)
    w, fmt_w = _as_bytes(weight)
    if fmt != fmt_w:
        raise NotImplementedError("both operands of the FP8 GEMM share one format")
    if scale.dim() == 0 or scale.numel() == 1 and scale.dim() < 2:
        return fp8_gemm(a, w, scale.reshape(()), bias, dtype=fmt)
    if scale.numel() != w.shape[0]:
        raise ValueError(f"scale of shape {tuple(scale.shape)} is neither a scalar nor one per output channel")
    return fp8_gemm(a, w, None, bias, dtype=fmt, alpha_cols=scale)


def fp8_bmm(input: torch.Tensor, other: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``input @ other * scale`` in bfloat16 over shared batch dimensions (reference
    ``backend/gpu/fp8.py:403-429``): ``input [..., M, K]``, ``other [..., K, N]``, float32 scalar."""
    a, fmt = _as_bytes(input)
    b, fmt_b = _as_bytes(other)
    if fmt != fmt_b:
        raise NotImplementedError("both operands of the FP8 GEMM share one format")
    if a.shape[:-2] != b.shape[:-2]:
        raise ValueError("fp8_bmm operands share their batch dimensions")
    return fp8_gemm(a, b.transpose(-2, -1).contiguous(), scale.reshape(()), dtype=fmt)


@N.device_guarded
def softmax_quantize_fp8(scores: torch.Tensor, score_scale: float, out_scale: torch.Tensor,
                         mask: Optional[torch.Tensor] = None, causal_period: int = 0,
                         dtype: str = "fp8_e4m3") -> torch.Tensor:
    """FP8 codes of ``softmax(scores * score_scale + mask)`` along the last axis in one pass
    (every intermediate rounded to bfloat16 as the unfused graph does).  ``mask`` is a
    ``[rows, cols]`` bfloat16 tensor applied cyclically over the score rows; ``causal_period``
    ``T`` masks columns beyond ``row % T``."""
    if scores.dtype != torch.bfloat16:
        raise NotImplementedError("softmax_quantize_fp8 takes bfloat16 scores")
    scores = scores.contiguous()
    cols = scores.shape[-1]
    rows = scores.numel() // max(cols, 1)
    out = torch.empty(scores.shape, dtype=torch.uint8, device=scores.device)
    mask_rows = 0
    if mask is not None:
        mask = mask.to(torch.bfloat16).reshape(-1, cols).contiguous()
        mask_rows = mask.shape[0]
    if out_scale.dtype not in _DTYPE_ID:
        out_scale = out_scale.float()
    N.check(N.lib().vq_softmax_quantize_fp8(scores.data_ptr(), out.data_ptr(), rows, cols, float(score_scale),
                                            _ptr(mask), mask_rows, int(causal_period), out_scale.data_ptr(),
                                            _dtype_id(out_scale.dtype), _FORMATS[dtype], _stream()),
            "vq_softmax_quantize_fp8")
    return out


@N.device_guarded
def attention_fp8(q8: torch.Tensor, k8: torch.Tensor, vt8: torch.Tensor, alpha_qk: torch.Tensor, score_scale: float,
                  p_scale: torch.Tensor, alpha_pv: torch.Tensor, ctx_scale: Optional[torch.Tensor] = None,
                  round_acc: bool = False):
    """Causal attention on FP8 operands in one kernel: ``fp8_gemm(q8, k8, alpha_qk)``,
    ``softmax_quantize_fp8(.., score_scale, p_scale, causal_period=T)``, ``fp8_gemm(p8, vt8, alpha_pv)``
    and, with ``ctx_scale``, the cast of the context, with the same rounding steps.
    ``q8``: ``[kv_heads, groups * T, 128]`` (a KV group's query heads stacked along the rows),
    ``k8``: ``[kv_heads, T, 128]``, ``vt8``: ``[kv_heads, 128, T]``, all e4m3 codes.
    Returns the e4m3 context ``[T, heads * 128]`` when ``ctx_scale`` is given, else the
    bfloat16 context ``[kv_heads, groups * T, 128]``.  ``round_acc``: both GEMMs as
    ``fp8_gemm(..., round_acc=True)``."""
    kv, rows, d = q8.shape
    T = k8.shape[1]
    groups = rows // T
    if k8.shape != (kv, T, d) or vt8.shape != (kv, d, T) or groups * T != rows:
        raise ValueError("attention_fp8: operand shapes do not agree")
    q8, k8, vt8 = q8.contiguous(), k8.contiguous(), vt8.contiguous()
    scalars = [_scale_arg(t) for t in (alpha_qk, p_scale, alpha_pv)]
    out8 = out16 = None
    if ctx_scale is not None:
        ctx_scale = _scale_arg(ctx_scale)
        out8 = torch.empty((T, kv * groups * d), dtype=torch.uint8, device=q8.device)
    else:
        out16 = torch.empty((kv, rows, d), dtype=torch.bfloat16, device=q8.device)
    N.check(N.lib().vq_attention_fp8(q8.data_ptr(), k8.data_ptr(), vt8.data_ptr(), _ptr(out8), kv * groups * d,
                                     _ptr(out16), T, kv, groups, d, scalars[0].data_ptr(), _dtype_id(scalars[0].dtype),
                                     float(score_scale), scalars[1].data_ptr(), _dtype_id(scalars[1].dtype),
                                     scalars[2].data_ptr(), _dtype_id(scalars[2].dtype), _ptr(ctx_scale),
                                     _dtype_id(ctx_scale.dtype) if ctx_scale is not None else 0, int(bool(round_acc)),
                                     _stream()),
            "vq_attention_fp8")
    return out8 if out8 is not None else out16


@N.device_guarded
def roundtrip_add(x: torch.Tensor, scale: torch.Tensor, y: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dequantize(quantize(x, scale, qmap=fp8_e4m3), scale) [+ y]`` in one kernel, each node's bfloat16
    rounding kept: what a per-tensor e4m3 cast leaves of a residual stream, added to the branch output."""
    x = _bf16_input("x", x)
    scale = _scale_arg(scale)
    if y is not None:
        y = _bf16_input("y", y)
        if y.shape != x.shape:
            raise ValueError("roundtrip_add: x and y differ in shape")
    if x.numel() % 8:
        raise NotImplementedError("roundtrip_add takes a multiple of 8 elements")
    out = torch.empty_like(x)
    N.check(N.lib().vq_fp8_roundtrip_add(x.data_ptr(), _ptr(y), out.data_ptr(), x.numel(), scale.data_ptr(),
                                         _dtype_id(scale.dtype), _stream()), "vq_fp8_roundtrip_add")
    return out


@N.device_guarded
def rope_heads_bf16(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE of ``x [T, heads, d]`` (any row stride: a slice of a merged projection) in one kernel, with
    the elementwise graph's roundings, written head-major ``[heads, T, d]`` as the attention kernel reads it."""
    T, heads, d = x.shape
    if x.dtype != torch.bfloat16:
        raise NotImplementedError("rope_heads_bf16 takes bfloat16 input")
    x, ldx = _heads_view("rope_heads_bf16", x)
    cos, sin = _bf16_input("rope_heads_bf16", cos), _bf16_input("rope_heads_bf16", sin)
    if tuple(cos.shape) != (T, d) or tuple(sin.shape) != (T, d):
        raise ValueError("cos / sin must be [T, head_dim]")
    out = torch.empty((heads, T, d), dtype=torch.bfloat16, device=x.device)
    N.check(N.lib().vq_rope_heads_bf16(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), out.data_ptr(), T, heads, d, ldx, d,
                                       d, T * d, _stream()), "vq_rope_heads_bf16")
    return out


@N.device_guarded
def attention_bf16_heads(q_heads: torch.Tensor, k_heads: torch.Tensor, vt: torch.Tensor,
                         score_scale: Optional[float] = None, round_acc: bool = True) -> torch.Tensor:
    """``attention_bf16`` on operands already in the kernel's layout: ``q_heads [heads, T, 128]``, ``k_heads
    [kv_heads, T, 128]`` (what ``rope_heads_bf16`` writes) and ``vt [kv_heads, 128, T]`` -> ``[T, heads * 128]``."""
    heads, T, d = q_heads.shape
    kv = k_heads.shape[0]
    if k_heads.shape != (kv, T, d) or vt.shape != (kv, d, T) or heads % kv:
        raise ValueError("attention_bf16_heads: operand shapes do not agree")
    if any(t.dtype != torch.bfloat16 for t in (q_heads, k_heads, vt)):
        raise NotImplementedError("attention_bf16_heads takes bfloat16 operands")
    q_heads, k_heads, vt = q_heads.contiguous(), k_heads.contiguous(), vt.contiguous()
    out = torch.empty((T, heads * d), dtype=torch.bfloat16, device=q_heads.device)
    scale = 1.0 / math.sqrt(d) if score_scale is None else float(score_scale)
    N.check(N.lib().vq_attention_bf16(q_heads.data_ptr(), k_heads.data_ptr(), vt.data_ptr(), out.data_ptr(), heads * d, T,
                                      kv, heads // kv, d, scale, int(bool(round_acc)), _stream()), "vq_attention_bf16")
    return out


@N.device_guarded
def attention_bf16(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, score_scale: Optional[float] = None,
                   round_acc: bool = True) -> torch.Tensor:
    """Causal self-attention on bfloat16 operands in one kernel, with the roundings of the eager graph
    (``matmul`` -> scale + mask -> ``softmax`` -> ``matmul``, every intermediate a bfloat16 tensor):
    ``q [T, heads, 128]``, ``k`` / ``v`` ``[T, kv_heads, 128]`` -> ``[T, heads * 128]``.  ``round_acc=False``
    keeps the scores in float32 until they are scaled (a fused-attention library's semantics)."""
    T, heads, d = q.shape
    kv = k.shape[1]
    if k.shape != (T, kv, d) or v.shape != (T, kv, d) or heads % kv:
        raise ValueError("attention_bf16: operand shapes do not agree")
    if any(t.dtype != torch.bfloat16 for t in (q, k, v)):
        raise NotImplementedError("attention_bf16 takes bfloat16 operands")
    groups = heads // kv
    # a KV group's query heads stacked along the rows; V transposed (the P V product contracts over keys)
    qg = q.reshape(T, kv, groups, d).permute(1, 2, 0, 3).contiguous()
    kk = k.permute(1, 0, 2).contiguous()
    vt = v.permute(1, 2, 0).contiguous()
    out = torch.empty((T, heads * d), dtype=torch.bfloat16, device=q.device)
    scale = 1.0 / math.sqrt(d) if score_scale is None else float(score_scale)
    N.check(N.lib().vq_attention_bf16(qg.data_ptr(), kk.data_ptr(), vt.data_ptr(), out.data_ptr(), heads * d, T, kv,
                                      groups, d, scale, int(bool(round_acc)), _stream()), "vq_attention_bf16")
    return out


def attention_status(reset: bool = True) -> int:
    """0, or the timeout code if a bounded wait inside ``attention_fp8`` / ``attention_bf16`` ran out since the last reset."""
    return N.lib().vq_attention_status(int(reset))


def _scale_arg(scale: torch.Tensor) -> torch.Tensor:
    if scale.numel() != 1:
        raise ValueError("the fused FP8 casts take one per-tensor scale")
    return scale if scale.dtype in _DTYPE_ID else scale.float()


def _bf16_input(name: str, t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.bfloat16:
        raise NotImplementedError(f"{name} takes bfloat16 input")
    return t.contiguous()


@N.device_guarded
def rmsnorm_quantize_fp8(x: torch.Tensor, weight: torch.Tensor, eps: float, scale: torch.Tensor,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """e4m3 bytes of ``rms_norm(x, weight, eps) / scale`` in one pass over ``x [..., H]`` (into ``out``, a dense
    uint8 tensor of that many bytes, when given)."""
    x, weight, scale = _bf16_input("rmsnorm_quantize_fp8", x), _bf16_input("rmsnorm_quantize_fp8", weight), _scale_arg(scale)
    cols = x.shape[-1]
    if out is None:
        out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    elif out.dtype != torch.uint8 or out.numel() != x.numel() or not out.is_contiguous():
        raise ValueError("out must be a dense uint8 tensor with one byte per element")
    else:
        out = out.view(x.shape)
    N.check(N.lib().vq_rmsnorm_quantize_fp8(x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.numel() // max(cols, 1),
                                            cols, float(eps), scale.data_ptr(), _dtype_id(scale.dtype), _stream()),
            "vq_rmsnorm_quantize_fp8")
    return out


def _rows_view(name: str, t: torch.Tensor):
    """``t`` as ``(tensor, rows, cols, row stride)``: dense, or a column slice of a wider matrix."""
    if t.dtype != torch.bfloat16:
        raise NotImplementedError(f"{name} takes bfloat16 input")
    if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1] and t.stride(0) % 8 == 0 \
            and t.data_ptr() % 16 == 0:
        return t, t.shape[0], t.shape[1], t.stride(0)
    t = t.contiguous()
    cols = t.shape[-1] if t.dim() else 1
    return t, t.numel() // max(cols, 1), cols, cols


@N.device_guarded
def silu_mul_quantize_fp8(gate: torch.Tensor, up: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3 bytes of ``(silu(gate) * up) / scale`` in one pass.  ``gate`` and ``up`` may be
    column slices of one wider matrix (the two halves of a merged projection)."""
    if gate.shape != up.shape:
        raise ValueError("gate and up differ in shape")
    scale = _scale_arg(scale)
    g, rows, cols, ldg = _rows_view("silu_mul_quantize_fp8", gate)
    u, _, _, ldu = _rows_view("silu_mul_quantize_fp8", up)
    out = torch.empty(gate.shape, dtype=torch.uint8, device=gate.device)
    N.check(N.lib().vq_silu_mul_quantize_fp8(g.data_ptr(), u.data_ptr(), out.data_ptr(), rows, cols, ldg, ldu,
                                             scale.data_ptr(), _dtype_id(scale.dtype), _stream()),
            "vq_silu_mul_quantize_fp8")
    return out


def _heads_view(name: str, x: torch.Tensor):
    """``x [T, heads, d]`` as ``(tensor, token stride)``: dense, or head columns sliced out of a
    wider ``[T, *]`` matrix (unit stride along d, d between heads)."""
    if x.dtype != torch.bfloat16:
        raise NotImplementedError(f"{name} takes bfloat16 input")
    T, heads, d = x.shape
    if x.stride(2) == 1 and x.stride(1) == d and x.stride(0) >= heads * d and x.stride(0) % 8 == 0 \
            and x.data_ptr() % 16 == 0:
        return x, x.stride(0)
    return x.contiguous(), heads * d


@N.device_guarded
def rope_quantize_fp8(x: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                      scale: torch.Tensor) -> torch.Tensor:
    """e4m3 bytes of the rotary embedding of ``x [T, heads, d]`` (rotate-half form, ``cos`` /
    ``sin`` ``[T, d]``; ``None`` skips the rotation), laid out head-major ``[heads, T, d]``."""
    scale = _scale_arg(scale)
    T, heads, d = x.shape
    x, ldx = _heads_view("rope_quantize_fp8", x)
    if cos is not None:
        cos, sin = _bf16_input("rope_quantize_fp8", cos), _bf16_input("rope_quantize_fp8", sin)
        if tuple(cos.shape) != (T, d) or tuple(sin.shape) != (T, d):
            raise ValueError("cos / sin must be [T, head_dim]")
    out = torch.empty((heads, T, d), dtype=torch.uint8, device=x.device)
    N.check(N.lib().vq_rope_quantize_fp8(x.data_ptr(), _ptr(cos), _ptr(sin), out.data_ptr(), T, heads, d,
                                         ldx, d, d, T * d, scale.data_ptr(), _dtype_id(scale.dtype), _stream()),
            "vq_rope_quantize_fp8")
    return out


@N.device_guarded
def qkv_post_fp8(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 q_scale: torch.Tensor, k_scale: torch.Tensor, v_scale: torch.Tensor):
    """``rope_quantize_fp8(q)``, ``rope_quantize_fp8(k)`` and ``transpose_quantize_fp8(v)`` as one launch, for
    ``q [T, heads, d]``, ``k`` / ``v [T, kv_heads, d]`` that are column slices of one ``[T, *]`` matrix (the output
    of a merged q/k/v projection).  Returns ``(q8 [heads, T, d], k8 [kv_heads, T, d], vt8 [kv_heads, d, T])``, equal
    to the separate calls bit for bit; operands that are not such slices take the separate calls."""
    T, heads, d = q.shape
    kv = k.shape[1]
    views = [_heads_view("qkv_post_fp8", t) for t in (q, k, v)]
    same = all(t is o for (t, _), o in zip(views, (q, k, v))) and len({ld for _, ld in views}) == 1
    if not same or d % 16 != 0 or tuple(k.shape) != (T, kv, d) or tuple(v.shape) != (T, kv, d):
        return rope_quantize_fp8(q, cos, sin, q_scale), rope_quantize_fp8(k, cos, sin, k_scale), \
            transpose_quantize_fp8(v, v_scale)
    cos, sin = _bf16_input("qkv_post_fp8", cos), _bf16_input("qkv_post_fp8", sin)
    if tuple(cos.shape) != (T, d) or tuple(sin.shape) != (T, d):
        raise ValueError("cos / sin must be [T, head_dim]")
    scales = [_scale_arg(t) for t in (q_scale, k_scale, v_scale)]
    q8 = torch.empty((heads, T, d), dtype=torch.uint8, device=q.device)
    k8 = torch.empty((kv, T, d), dtype=torch.uint8, device=q.device)
    vt8 = torch.empty((kv, d, T), dtype=torch.uint8, device=q.device)
    N.check(N.lib().vq_qkv_post_fp8(q.data_ptr(), k.data_ptr(), v.data_ptr(), views[0][1], cos.data_ptr(), sin.data_ptr(),
                                    q8.data_ptr(), k8.data_ptr(), vt8.data_ptr(), T, heads, kv, d,
                                    scales[0].data_ptr(), _dtype_id(scales[0].dtype), scales[1].data_ptr(),
                                    _dtype_id(scales[1].dtype), scales[2].data_ptr(), _dtype_id(scales[2].dtype), _stream()),
            "vq_qkv_post_fp8")
    return q8, k8, vt8


@N.device_guarded
def transpose_heads_quantize_fp8(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3 bytes of a head-major ``x [heads, T, d] / scale`` laid out token-major ``[T, heads * d]``."""
    x, scale = _bf16_input("transpose_heads_quantize_fp8", x), _scale_arg(scale)
    heads, T, d = x.shape
    out = torch.empty((T, heads * d), dtype=torch.uint8, device=x.device)
    N.check(N.lib().vq_rope_quantize_fp8(x.data_ptr(), None, None, out.data_ptr(), T, heads, d, d, T * d,
                                         heads * d, d, scale.data_ptr(), _dtype_id(scale.dtype), _stream()),
            "vq_rope_quantize_fp8")
    return out


@N.device_guarded
def transpose_quantize_fp8(x: torch.Tensor, scale: torch.Tensor, dtype="fp8_e4m3") -> torch.Tensor:
    """FP8 bytes of ``x [T, heads, d] / scale`` laid out ``[heads, d, T]``."""
    scale = _scale_arg(scale)
    T, heads, d = x.shape
    x, ldx = _heads_view("transpose_quantize_fp8", x)
    out = torch.empty((heads, d, T), dtype=torch.uint8, device=x.device)
    N.check(N.lib().vq_transpose_quantize_fp8(x.data_ptr(), out.data_ptr(), None, None, _FORMATS[dtype], T, heads, d,
                                              ldx, scale.data_ptr(), _dtype_id(scale.dtype), _stream()),
            "vq_transpose_quantize_fp8")
    return _typed(out, dtype)


@N.device_guarded
def quantize_fp8_transpose(input: torch.Tensor, scale: torch.Tensor, dtype="fp8_e4m3"):
    """``(codes [M, N], transpose [N, M], amax)`` of a matrix in one pass over it: the FP8 bytes
    of ``input / scale`` in both layouts and ``amax(|input|)`` as a 0-d tensor of ``input``'s dtype
    (reference ``backend/gpu/fp8.py:342-369``)."""
    x, scale = _bf16_input("quantize_fp8_transpose", input), _scale_arg(scale)
    if x.ndim != 2:
        raise ValueError("quantize_fp8_transpose takes a matrix")
    rows, cols = x.shape
    codes = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    transpose = torch.empty((cols, rows), dtype=torch.uint8, device=x.device)
    amax = torch.zeros((), dtype=torch.int32, device=x.device)
    N.check(N.lib().vq_transpose_quantize_fp8(x.data_ptr(), transpose.data_ptr(), codes.data_ptr(), amax.data_ptr(),
                                              _FORMATS[dtype], rows, 1, cols, cols, scale.data_ptr(),
                                              _dtype_id(scale.dtype), _stream()),
            "vq_transpose_quantize_fp8")
    return _typed(codes, dtype), _typed(transpose, dtype), amax.to(torch.int16).view(torch.bfloat16)


# ---------------------------------------------------------------------------
# ``voyager_gpu::cast_transpose_fp8``: the operator the reference's training lowering calls
# (``backend/gpu/fp8.py:311-340``), same name and schema, CUDA key only
# ---------------------------------------------------------------------------
from torch.library import Library  # noqa: E402

voyager_gpu_lib = Library("voyager_gpu", "FRAGMENT")
voyager_gpu_lib.define("cast_transpose_fp8(Tensor x, Tensor scale, ScalarType dtype) -> (Tensor, Tensor, Tensor)")


def _cast_transpose_fp8_op(x, scale, dtype):
    if dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise NotImplementedError(f"cast_transpose_fp8 casts to float8_e4m3fn or float8_e5m2, not {dtype}")
    return quantize_fp8_transpose(x, scale, dtype)


voyager_gpu_lib.impl("cast_transpose_fp8", N.device_guarded(_cast_transpose_fp8_op), "CUDA")


@torch.library.register_fake("voyager_gpu::cast_transpose_fp8")
def _(x, scale, dtype):
    rows, cols = x.shape
    return (x.new_empty((rows, cols), dtype=dtype), x.new_empty((cols, rows), dtype=dtype),
            x.new_empty((), dtype=x.dtype))
