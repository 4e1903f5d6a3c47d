"""Oracle: a per-tensor FP8 quantized Llama decoder layer as its converted graph computes it.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Restates, with the oracle's CPU operators, the node pattern that the reference's
``convert_pt2e`` emits for per-tensor symmetric quantization
(``src/voyager_compiler/quantization/quantize_pt2e.py:526-626``):
``quantize(x, s_a, qmap)`` -> ``aten.linear / aten.matmul`` on the bfloat16-valued
codes -> ``dequantize(y, s_a * s_w, output_qmap=identity)``, applied to the seven
linears and the two attention matmuls of a Llama layer with HF eager attention
(``scripts/models/clm.py:286-331`` prepares that graph).  RMSNorm, RoPE, softmax
and SwiGLU are plain bfloat16 torch ops, as in the graph.
"""

import math

import torch
import torch.nn.functional as F

from . import quantizers as OQ
from . import tables as OT


def fp8_decoder_layer(x, params, scales, shape, rope, mask, record=None):
    """x: [T, hidden] bfloat16 on the CPU.  ``scales``: bfloat16 0-d tensors keyed
    'h','q','k','v','p','ctx','h2','act' and 'w_<linear>'.  ``rope`` = (cos, sin).
    ``record(name, tensor)`` sees the graph's intermediate tensors (codes are bfloat16-valued):
    'h8', 'q_lin'/'k_lin'/'v_lin' [T, heads, d], 'q8' [heads, T, d], 'k8' [kv, T, d], 'v8' [kv, d, T],
    'ctx' [T, heads * d], 'ctx8', 'x1', 'h28', 'act8'."""
    rec = record or (lambda name, t: None)
    e4m3 = OT.quantization_map("fp8_e4m3")
    ident = OT.quantization_map(None)
    T = x.shape[0]
    cos, sin = rope

    def quant(t, name):
        return OQ.quantize(t, scales[name], None, None, None, e4m3)

    weights = {n: quant(params[n], "w_" + n) for n in ("q", "k", "v", "o", "gate", "up", "down")}

    def qlinear(codes, act_name, w_name):
        y = F.linear(codes, weights[w_name])
        return OQ.dequantize(y, scales[act_name] * scales["w_" + w_name], None, None, None, None, ident)

    def rope_apply(t):
        half = t.shape[-1] // 2
        rot = torch.cat([-t[..., half:], t[..., :half]], -1)
        return t * cos[:, None, :] + rot * sin[:, None, :]

    h = quant(F.rms_norm(x, (shape.hidden,), params["ln1"], shape.eps), "h")
    rec("h8", h)
    q = qlinear(h, "h", "q").view(T, shape.heads, shape.head_dim)
    k = qlinear(h, "h", "k").view(T, shape.kv_heads, shape.head_dim)
    v = qlinear(h, "h", "v").view(T, shape.kv_heads, shape.head_dim)
    rec("q_lin", q), rec("k_lin", k), rec("v_lin", v)
    q, k = rope_apply(q), rope_apply(k)
    g = shape.heads // shape.kv_heads
    qh = quant(q.transpose(0, 1), "q")                                # [heads, T, d]
    rec("q8", qh), rec("k8", quant(k.transpose(0, 1), "k")), rec("v8", quant(v.permute(1, 2, 0), "v"))
    kt = quant(k.repeat_interleave(g, 1).permute(1, 2, 0), "k")       # [heads, d, T]
    vh = quant(v.repeat_interleave(g, 1).transpose(0, 1), "v")        # [heads, T, d]
    scores = OQ.dequantize(torch.matmul(qh, kt), scales["q"] * scales["k"], None, None, None, None, ident)
    scores = scores * (1.0 / math.sqrt(shape.head_dim)) + mask
    p = quant(torch.softmax(scores.float(), -1).to(x.dtype), "p")
    ctx = OQ.dequantize(torch.matmul(p, vh), scales["p"] * scales["v"], None, None, None, None, ident)
    ctx = ctx.transpose(0, 1).reshape(T, shape.heads * shape.head_dim)
    ctx8 = quant(ctx, "ctx")
    rec("ctx", ctx), rec("ctx8", ctx8)
    x1 = x + qlinear(ctx8, "ctx", "o")
    h2 = quant(F.rms_norm(x1, (shape.hidden,), params["ln2"], shape.eps), "h2")
    rec("x1", x1), rec("h28", h2)
    act = F.silu(qlinear(h2, "h2", "gate")) * qlinear(h2, "h2", "up")
    act8 = quant(act, "act")
    rec("act8", act8)
    return x1 + qlinear(act8, "act", "down")


def nvfp4_decoder_layer(x, params, shape, rope, mask):
    """A Llama decoder layer whose seven linears are NVFP4 sites of a converted microscaling graph
    (reference ``quantization/quantize_pt2e.py:700-1142``): the activation goes through the in-graph
    global scale ``clamp_min(amax(abs(x)) / (6 * 448), tiny)`` (``:881-901``) and
    ``quantize_mx(x, e2m1, (-1,), 16, 6.0, False, e4m3, None, None, t)``; the weight is quantized the same
    way once (``:805-856``); the consumer is ``linear_mx(codes, w_codes, input_scale=, weight_scale=,
    block_size=16, alpha=t_x * t_w)`` (``:1025-1057``).  The attention matmuls are not annotated in that
    recipe and run as HF eager attention in bfloat16; RMSNorm, RoPE and SwiGLU are plain bfloat16 ops."""
    from . import gemm as OG

    e2m1, e4m3 = OT.quantization_map("fp4_e2m1"), OT.quantization_map("fp8_e4m3")
    T = x.shape[0]
    cos, sin = rope

    def quant(t):
        g = OQ.calculate_global_scale(t, 6.0, 448.0)
        s, c = OQ.quantize_mx(t, e2m1, [-1], 16, 6.0, False, e4m3, None, None, g)
        return s, c, g

    weights = {n: quant(params[n]) for n in ("q", "k", "v", "o", "gate", "up", "down")}

    def qlinear(act, name):
        s, c, g = act
        sw, cw, gw = weights[name]
        return OG.linear_mx(c, cw, None, input_scale=s, weight_scale=sw, block_size=16, alpha=g * gw)

    def rope_apply(t):
        half = t.shape[-1] // 2
        rot = torch.cat([-t[..., half:], t[..., :half]], -1)
        return t * cos[:, None, :] + rot * sin[:, None, :]

    h = quant(F.rms_norm(x, (shape.hidden,), params["ln1"], shape.eps))      # one quantize node feeds q, k and v
    q = rope_apply(qlinear(h, "q").view(T, shape.heads, shape.head_dim))
    k = rope_apply(qlinear(h, "k").view(T, shape.kv_heads, shape.head_dim))
    v = qlinear(h, "v").view(T, shape.kv_heads, shape.head_dim)
    g = shape.heads // shape.kv_heads
    scores = torch.matmul(q.transpose(0, 1), k.repeat_interleave(g, 1).permute(1, 2, 0))
    scores = scores * (1.0 / math.sqrt(shape.head_dim)) + mask
    p = torch.softmax(scores.float(), -1).to(x.dtype)
    ctx = torch.matmul(p, v.repeat_interleave(g, 1).transpose(0, 1)).transpose(0, 1).reshape(T, -1)
    x1 = x + qlinear(quant(ctx), "o")
    h2 = quant(F.rms_norm(x1, (shape.hidden,), params["ln2"], shape.eps))
    act = F.silu(qlinear(h2, "gate")) * qlinear(h2, "up")
    return x1 + qlinear(quant(act), "down")


def mxnf4_decode_layer(x, weights, tables, cache, rope, residual_scale, shape):
    """One decode step of a Llama decoder layer in the MXNF4 recipe with a KIVI cache, as the converted
    graph's operators compute it (batch ``B``, one new token per sequence).

    Linears (``quantize_pt2e.py:700-1142``): the activation goes through ``quantize_mx(x, index_table,
    (-1,), 64, 31.0, False, e5m3, midpoints)``, the weight is baked as codebook indices + block scales, the
    consumer is ``linear_mx(..., block_size=64, input_code=levels, weight_code=levels)``.  q/k/v (and
    gate/up) read one shared quantize node.  Residual adds take their earlier operand through a per-tensor
    ``fp8_e4m3`` quantize / dequantize.  The cached keys and values are KIVI codes (``quantize_affine``,
    uint2, groups of 64: keys along the sequence, values along the head dimension) read back with
    ``dequantize(codes, scale, zero_point, axes, 64)``; the newest ``R`` positions (the last one is this
    step's token) are kept in bfloat16.  Attention is eager bfloat16 over [main | residual] keys.

    ``weights``: name -> (index codes [N, K], scale [N, K / 64]) for 'qkv', 'o', 'gate_up', 'down' and
    'ln1', 'ln2' gains.  ``tables``: dict with 'levels', 'index', 'mid', 'e5m3', 'e4m3'.  ``cache``: dict
    with 'k' / 'v' -> (codes, scale, zero_point) of shape [B, kv, Tm, d] and 'k_res' / 'v_res'
    [B, kv, R, d] whose last position is overwritten by this step.  ``rope`` = (cos, sin) [d] of the new position."""
    from . import gemm as OG

    t = tables
    B = x.shape[0]
    d, hq, hkv = shape.head_dim, shape.heads, shape.kv_heads
    cos, sin = rope

    def qlinear(act, name):
        s, c = OQ.quantize_mx(act, t["index"], [-1], 64, 31.0, False, t["e5m3"], t["mid"])
        cw, sw = weights[name]
        return OG.linear_mx(c, cw, None, input_scale=s, weight_scale=sw, block_size=64, input_code=t["levels"],
                            weight_code=t["levels"])

    def through_fp8(v):
        q = OQ.quantize(v, residual_scale, None, None, None, t["e4m3"])
        return OQ.dequantize(q, residual_scale)

    def rope_apply(v):
        half = d // 2
        rot = torch.cat([-v[..., half:], v[..., :half]], -1)
        return v * cos + rot * sin

    qkv = qlinear(F.rms_norm(x, (shape.hidden,), weights["ln1"], shape.eps), "qkv")
    q = rope_apply(qkv[:, :hq * d].reshape(B, hq, d))
    k = rope_apply(qkv[:, hq * d:(hq + hkv) * d].reshape(B, hkv, d))
    v = qkv[:, (hq + hkv) * d:].reshape(B, hkv, d)
    k_res, v_res = cache["k_res"].clone(), cache["v_res"].clone()
    k_res[:, :, -1] = k
    v_res[:, :, -1] = v
    k_main = OQ.dequantize(*cache["k"], [-2], 64)
    v_main = OQ.dequantize(*cache["v"], [-1], 64)
    qg = q.reshape(B, hkv, hq // hkv, d)
    scale = 1.0 / math.sqrt(d)
    scores = torch.cat([torch.matmul(qg, k_main.transpose(-1, -2)), torch.matmul(qg, k_res.transpose(-1, -2))], -1)
    p = torch.softmax((scores * scale).float(), -1).to(x.dtype)
    tm = k_main.shape[-2]
    ctx = torch.matmul(p[..., :tm], v_main) + torch.matmul(p[..., tm:], v_res)
    x1 = through_fp8(x) + qlinear(ctx.reshape(B, hq * d), "o")
    gu = qlinear(F.rms_norm(x1, (shape.hidden,), weights["ln2"], shape.eps), "gate_up")
    inter = gu.shape[-1] // 2
    act = F.silu(gu[:, :inter]) * gu[:, inter:]
    return through_fp8(x1) + qlinear(act, "down")
