"""Oracle: the quantized GEMMs (decode, scale, float32 product, one rounding).

TEST INFRASTRUCTURE ONLY (see the package docstring).

Restates ``linear_mx`` / ``matmul_mx`` / ``sdpa_mx``
(reference ``src/voyager_compiler/ops/quantized.py:662-723, 752-805, 836-928``)
and the layout GEMMs ``quantized_ops.linear`` / ``matmul``
(``src/voyager_compiler/ops/layout.py:231-284``): operands are read back
through their codebooks, multiplied by their per-block scales (rounded to the
operand dtype), multiplied in float32, scaled by ``alpha``, biased, and
rounded once to the output dtype.  Outlier CSR side streams are not restated.
"""

import math

import torch

from .quantizers import decode_and_scale, quantize_mx

_ACT, _WGT, _OUT = ("xc", "cx"), ("kc", "ck"), ("xk", "kx")


def parse_layout(layout):
    operands, out = layout.split("->")
    act, wgt = operands.split(",")
    assert act in _ACT and wgt in _WGT and out in _OUT, layout
    return act, wgt, out


def _gemm(native, a, b, layout, out_dtype, bias=None):
    act, wgt, out = parse_layout(layout)
    n_act, n_wgt, n_out = parse_layout(native)
    if act != n_act:
        a = a.mT
    if wgt != n_wgt:
        b = b.mT
    if out_dtype is not None:
        a, b = a.float(), b.float()
        bias = None if bias is None else bias.float()
    if native == "xc,kc->xk":
        y = torch.nn.functional.linear(a, b, bias)
    else:
        y = torch.matmul(a, b)
    if out_dtype is not None:
        y = y.to(out_dtype)
    return y.mT.contiguous() if out != n_out else y


def linear(x, w, bias=None, *, layout="xc,kc->xk", out_dtype=None):
    return _gemm("xc,kc->xk", x, w, layout, out_dtype, bias)


def matmul(a, b, *, layout="xc,ck->xk", out_dtype=None):
    return _gemm("xc,ck->xk", a, b, layout, out_dtype)


def _read(x, scale, code, block_size):
    if scale is None and code is None:
        return x
    return decode_and_scale(x, scale, code, block_size)


def linear_mx(x, w, bias=None, *, input_scale=None, weight_scale=None, block_size=None,
              input_code=None, weight_code=None, alpha=None, A_data=None, A_indices=None, A_indptr=None,
              layout="xc,kc->xk", out_dtype=None):
    act, wgt, out = parse_layout(layout)
    a = _read(x, input_scale, input_code, block_size)
    b = _read(w, weight_scale, weight_code, block_size)
    dtype = a.dtype if out_dtype is None else out_dtype
    acc = torch.promote_types(dtype, torch.float32)
    y = linear(a, b, bias if alpha is None else None, layout=f"{act},{wgt}->xk", out_dtype=acc)
    if alpha is not None:
        y = y * alpha
        if bias is not None:
            y = y + bias
    if A_data is not None:   # the outliers' product joins the float32 sum before the one rounding
        from .outliers import spmm_csr

        y = y + spmm_csr(A_data, A_indices, A_indptr, w, weight_scale, weight_code, block_size, wgt, out_dtype=acc)
    y = y.to(dtype)
    return y.mT.contiguous() if out != "xk" else y


def matmul_mx(a, b, *, input_scale=None, weight_scale=None, block_size=None,
              input_code=None, weight_code=None, alpha=None, layout="xc,ck->xk",
              out_dtype=None):
    act, wgt, out = parse_layout(layout)
    a = _read(a, input_scale, input_code, block_size)
    b = _read(b, weight_scale, weight_code, block_size)
    dtype = a.dtype if out_dtype is None else out_dtype
    acc = torch.promote_types(dtype, torch.float32)
    y = matmul(a, b, layout=f"{act},{wgt}->xk", out_dtype=acc)
    if alpha is not None:
        y = y * alpha
    y = y.to(dtype)
    return y.mT.contiguous() if out != "xk" else y


def _mask(scores, mask):
    if mask is None:
        return scores
    if mask.dtype == torch.bool:
        return scores.masked_fill(~mask, float("-inf"))
    return scores + mask


def sdpa_mx(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, query_residual=None,
            key_residual=None, value_residual=None, residual_mask=None, *, scale=None,
            enable_gqa=False, query_scale=None, key_scale=None, value_scale=None,
            block_size=None, input_code=None, weight_code=None, probs_qmap=None,
            probs_quant_max=None, probs_scale_qmap=None, probs_code=None,
            force_scale_power_of_two=False):
    if is_causal and attn_mask is not None:
        raise ValueError("is_causal excludes an explicit attn_mask")
    q = _read(q, query_scale, input_code, block_size)
    k = _read(k, key_scale, weight_code, block_size)
    v = _read(v, value_scale, weight_code, block_size)
    has_res = key_residual is not None
    if enable_gqa:
        g = q.shape[-3] // k.shape[-3]
        k, v = k.repeat_interleave(g, -3), v.repeat_interleave(g, -3)
        if has_res:
            key_residual = key_residual.repeat_interleave(g, -3)
            value_residual = value_residual.repeat_interleave(g, -3)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if is_causal:
        attn_mask = torch.ones(s.shape[-2:], dtype=torch.bool).tril()
    s = _mask(s, attn_mask)
    n_main = s.shape[-1]
    if has_res:
        r = _mask(query_residual @ key_residual.transpose(-1, -2) * scale, residual_mask)
        s = torch.cat([s, r], -1)
    p = torch.softmax(s, -1)
    p, p_res = p[..., :n_main], p[..., n_main:]
    if probs_qmap is not None:
        p_scale, p = quantize_mx(p, probs_qmap, [-1], block_size, probs_quant_max,
                                 force_scale_power_of_two, probs_scale_qmap, probs_code)
        p = _read(p, p_scale, input_code, block_size)
    o = torch.matmul(p, v)
    if has_res:
        o = o + torch.matmul(p_res, value_residual)
    return o
