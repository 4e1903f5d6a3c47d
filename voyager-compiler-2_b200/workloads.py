"""Synthetic Llama-shaped decoder layers that exercise the quantized hot path.

These are the callers the benchmark and the tests drive: random-init weights
of a Llama-3.1-8B-shaped layer (hidden 4096, 32 query / 8 KV heads of 128,
SwiGLU 14336, RMSNorm, RoPE theta 5e5), quantized the way the reference's
converted graphs are (``scripts/models/clm.py:353-389`` builds them;
``quantization/quantize_pt2e.py:526-626`` emits the per-tensor node pattern).

``Fp8DecoderLayer`` is the FP8 per-tensor layer: every linear and both attention
matmuls run as FP8 casts + tcgen05 FP8 GEMMs (the replacement the reference's
``backend/gpu`` makes for ``quantize -> aten.linear -> dequantize`` sites);
RMSNorm, RoPE, softmax and SwiGLU stay bfloat16 torch ops, as in the graph.
"""

import dataclasses
import math

import torch
import torch.nn.functional as F

from . import fp8 as FP8
from . import formats

E4M3_MAX = 448.0


@dataclasses.dataclass(frozen=True)
class LlamaShape:
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 14336
    rope_theta: float = 5e5
    eps: float = 1e-5
    vocab: int = 128256

    @property
    def groups(self):
        return self.heads // self.kv_heads


LLAMA_8B = LlamaShape()
TINY = LlamaShape(hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512, vocab=1024)

LINEARS = ("q", "k", "v", "o", "gate", "up", "down")


def linear_shapes(shape: LlamaShape):
    h, d = shape.hidden, shape.head_dim
    return {"q": (shape.heads * d, h), "k": (shape.kv_heads * d, h), "v": (shape.kv_heads * d, h),
            "o": (h, shape.heads * d), "gate": (shape.intermediate, h), "up": (shape.intermediate, h),
            "down": (h, shape.intermediate)}


def make_layer_params(seed: int, shape: LlamaShape, device="cpu"):
    """Random-init weights ~N(0, 0.02) and unit RMSNorm gains, generated on the CPU."""
    g = torch.Generator().manual_seed(seed)
    params = {name: (torch.randn(*dims, generator=g) * 0.02).bfloat16().to(device)
              for name, dims in linear_shapes(shape).items()}
    params["ln1"] = torch.ones(shape.hidden, dtype=torch.bfloat16, device=device)
    params["ln2"] = torch.ones(shape.hidden, dtype=torch.bfloat16, device=device)
    return params


def make_hidden_states(seed: int, tokens: int, shape: LlamaShape, device="cpu"):
    """Layer input for ``tokens`` random token ids: embedding rows of distinct ids
    drawn from an N(0,1) table are i.i.d. normal rows, which is what is generated
    (no vocabulary-sized table is materialised)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(tokens, shape.hidden, generator=g).bfloat16().to(device)


def rope_tables(tokens: int, shape: LlamaShape, device):
    inv = 1.0 / (shape.rope_theta ** (torch.arange(0, shape.head_dim, 2, dtype=torch.float32) / shape.head_dim))
    angle = torch.arange(tokens, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([angle, angle], -1)
    return emb.cos().bfloat16().to(device), emb.sin().bfloat16().to(device)


def apply_rope(x, cos, sin):
    """x: [T, heads, head_dim]; HF Llama's rotate-half form."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], -1)
    return x * cos[:, None, :] + rot * sin[:, None, :]


def causal_mask(tokens: int, device, dtype=torch.bfloat16):
    m = torch.full((tokens, tokens), float("-inf"), dtype=dtype, device=device)
    return torch.triu(m, 1)


def _amax_scale(t, qmax=E4M3_MAX):
    return (t.abs().amax() / qmax).to(torch.bfloat16)


def bf16_layer_forward(x, params, shape: LlamaShape, record=None):
    """The unquantized bfloat16 layer (calibration pass).  ``record(name, tensor)``
    sees every tensor that the quantized layer quantizes."""
    T = x.shape[0]
    rec = record or (lambda name, t: None)
    cos, sin = rope_tables(T, shape, x.device)
    h = F.rms_norm(x, (shape.hidden,), params["ln1"], shape.eps)
    rec("h", h)
    q = F.linear(h, params["q"]).view(T, shape.heads, shape.head_dim)
    k = F.linear(h, params["k"]).view(T, shape.kv_heads, shape.head_dim)
    v = F.linear(h, params["v"]).view(T, shape.kv_heads, shape.head_dim)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    rec("q", q), rec("k", k), rec("v", v)
    kk = k.repeat_interleave(shape.groups, 1)
    vv = v.repeat_interleave(shape.groups, 1)
    scores = torch.matmul(q.transpose(0, 1), kk.permute(1, 2, 0)) * (1.0 / math.sqrt(shape.head_dim))
    scores = scores + causal_mask(T, x.device)
    p = torch.softmax(scores.float(), -1).to(x.dtype)
    rec("p", p)
    ctx = torch.matmul(p, vv.transpose(0, 1)).transpose(0, 1).reshape(T, shape.heads * shape.head_dim)
    rec("ctx", ctx)
    x1 = x + F.linear(ctx, params["o"])
    h2 = F.rms_norm(x1, (shape.hidden,), params["ln2"], shape.eps)
    rec("h2", h2)
    act = F.silu(F.linear(h2, params["gate"])) * F.linear(h2, params["up"])
    rec("act", act)
    return x1 + F.linear(act, params["down"])


def calibrate_fp8_scales(x, params, shape: LlamaShape):
    """Per-tensor scales ``amax / 448`` in bfloat16 for every quantized tensor
    (activations from one bfloat16 forward of ``x``; weights from their own amax)."""
    scales = {}
    bf16_layer_forward(x, params, shape, lambda name, t: scales.__setitem__(name, _amax_scale(t)))
    for name in LINEARS:
        scales["w_" + name] = _amax_scale(params[name])
    return scales


class Fp8DecoderLayer:
    """FP8 per-tensor decoder layer on the CUDA kernels (prefill, batch 1)."""

    def __init__(self, params, scales, shape: LlamaShape, merge_qkv=True, merge_gate_up=True, fuse_residual=True,
                 fuse_swiglu=True, fuse_attention=True, graph_rounding=True):
        self.shape = shape
        # The converted graph rounds each matmul to bfloat16 and then multiplies by s_a * s_w in its
        # dequantize (two roundings); ``graph_rounding`` keeps both inside the GEMM epilogues.  Without
        # it every product is rounded once, as the reference's scaled-GEMM replacement does.
        self.ra = bool(graph_rounding)
        self.merge_qkv, self.merge_gate_up, self.fuse_residual = merge_qkv, merge_gate_up, fuse_residual
        self.fuse_swiglu = fuse_swiglu
        # one kernel for Q K^T, softmax, P V and the cast of the context (head_dim 128)
        self.fuse_attention = fuse_attention and shape.head_dim == 128
        self.scales = scales
        self.ln1, self.ln2 = params["ln1"], params["ln2"]
        # weights are cast once, as convert_pt2e bakes them
        self.w8 = {name: FP8.quantize_fp8(params[name], scales["w_" + name]) for name in LINEARS}
        s = scales
        self.alpha = {name: (s[src] * s["w_" + name]).reshape(()) for name, src in
                      (("q", "h"), ("k", "h"), ("v", "h"), ("o", "ctx"), ("gate", "h2"), ("up", "h2"), ("down", "act"))}
        self.alpha_qk = (s["q"] * s["k"]).reshape(())
        self.alpha_pv = (s["p"] * s["v"]).reshape(())
        # linears that read one quantized input run as one GEMM; each keeps its own scale per column
        def merged(names):
            w = torch.cat([self.w8[n] for n in names], 0)
            a = torch.cat([self.alpha[n].float().expand(self.w8[n].shape[0]) for n in names]).contiguous()
            return w, a
        self.w8_qkv, self.alpha_qkv = merged(("q", "k", "v"))
        self.w8_gate_up, self.alpha_gate_up = merged(("gate", "up"))
        # the same two linears with rows interleaved in runs of 32, for the GEMM whose epilogue is SiLU * up + cast
        inter = shape.intermediate
        self.w8_swiglu = FP8.interleave_gate_up(self.w8["gate"], self.w8["up"])
        self.alpha_swiglu = FP8.interleave_gate_up(self.alpha_gate_up[:inter], self.alpha_gate_up[inter:])
        self._rope = None
        self._mask = None
        self._side = None

    @property
    def LAUNCHES(self):
        """Kernels of this package launched per forward: 3 fused casts (5 when q, k and v come from separate
        GEMMs), 4 GEMMs and the attention kernel, or one cast, the softmax and 2 GEMMs more when the attention runs
        as separate kernels."""
        casts = 2 + (1 if self.merge_qkv else 3) + (0 if self.merge_gate_up else 1)
        gemms = 2 + (1 if self.merge_qkv else 3) + (1 if self.merge_gate_up else 2)
        return casts + gemms + (1 if self.fuse_attention else 4)   # else: two GEMMs, the softmax, the context cast

    def _tables(self, T, device):
        if self._rope is None or self._rope[0].shape[0] != T:
            self._rope = rope_tables(T, self.shape, device)
            self._mask = causal_mask(T, device)
        return self._rope, self._mask

    def forward(self, x):
        """Every FP8 cast is fused with the bfloat16 operation that produces its input."""
        sh, s = self.shape, self.scales
        T = x.shape[0]
        (cos, sin), _ = self._tables(T, x.device)
        nq, nkv = sh.heads * sh.head_dim, sh.kv_heads * sh.head_dim
        h8 = FP8.rmsnorm_quantize_fp8(x, self.ln1, sh.eps, s["h"])
        if self.merge_qkv:
            qkv = FP8.fp8_gemm(h8, self.w8_qkv, alpha_cols=self.alpha_qkv, round_acc=self.ra)  # [T, (heads + 2 kv) * d]
            q, k, v = qkv[:, :nq], qkv[:, nq:nq + nkv], qkv[:, nq + nkv:]
        else:
            q, k, v = (FP8.fp8_gemm(h8, self.w8[n], self.alpha[n], round_acc=self.ra) for n in ("q", "k", "v"))
        q = q.unflatten(1, (sh.heads, sh.head_dim))
        k = k.unflatten(1, (sh.kv_heads, sh.head_dim))
        v = v.unflatten(1, (sh.kv_heads, sh.head_dim))
        # query heads of one KV group are stacked along the rows: [kv, groups*T, d]
        if self.merge_qkv:
            # slices of one matrix: the two RoPE casts and the value transpose are one launch
            q8, k8, vt8 = FP8.qkv_post_fp8(q, k, v, cos, sin, s["q"], s["k"], s["v"])
            q8 = q8.view(sh.kv_heads, sh.groups * T, sh.head_dim)
        else:
            # the small K and V casts run beside the Q cast on a second stream (a fork and join that a
            # CUDA graph capture records as parallel branches)
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream(device=x.device)
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                k8 = FP8.rope_quantize_fp8(k, cos, sin, s["k"])                 # [kv, T, d]
                vt8 = FP8.transpose_quantize_fp8(v, s["v"])                     # [kv, d, T]
            q8 = FP8.rope_quantize_fp8(q, cos, sin, s["q"]).view(sh.kv_heads, sh.groups * T, sh.head_dim)
            main.wait_stream(self._side)
            for t in (k8, vt8):
                t.record_stream(main)
            k.record_stream(self._side)
        if self.fuse_attention and T % 128 == 0:
            ctx8 = FP8.attention_fp8(q8, k8, vt8, self.alpha_qk, 1.0 / math.sqrt(sh.head_dim), s["p"], self.alpha_pv,
                                     s["ctx"], round_acc=self.ra)            # [T, heads*d]
            return self._after_attention(x, ctx8)
        # masked scores are neither computed nor read; masked probabilities are zero codes
        scores = FP8.fp8_gemm(q8, k8, self.alpha_qk, causal=("scores", T), round_acc=self.ra)  # [kv, groups*T, T]
        # scale, causal mask, softmax and the FP8 cast of the probabilities in one pass
        p8 = FP8.softmax_quantize_fp8(scores, 1.0 / math.sqrt(sh.head_dim), s["p"], causal_period=T)
        ctx = FP8.fp8_gemm(p8, vt8, self.alpha_pv, causal=("probabilities", T), round_acc=self.ra)   # [kv, groups*T, d]
        # the cast of the context undoes the head-major layout: [kv*groups, T, d] -> [T, heads*d]
        ctx8 = FP8.transpose_heads_quantize_fp8(ctx.view(sh.heads, T, sh.head_dim), s["ctx"])
        return self._after_attention(x, ctx8)

    def _after_attention(self, x, ctx8):
        """Output projection, residual, and the MLP block."""
        sh, s = self.shape, self.scales
        if self.fuse_residual:
            x1 = FP8.fp8_gemm(ctx8, self.w8["o"], self.alpha["o"], residual=x, round_acc=self.ra)   # x + o_proj(ctx)
        else:
            x1 = x + FP8.fp8_gemm(ctx8, self.w8["o"], self.alpha["o"], round_acc=self.ra)
        h28 = FP8.rmsnorm_quantize_fp8(x1, self.ln2, sh.eps, s["h2"])
        if self.fuse_swiglu and sh.intermediate % 32 == 0:
            # gate and up linears, SiLU, product and the cast of down_proj's input in one GEMM
            act8 = FP8.fp8_gemm(h28, self.w8_swiglu, alpha_cols=self.alpha_swiglu, gated_scale=s["act"],
                                round_acc=self.ra)
        else:
            if self.merge_gate_up:
                gu = FP8.fp8_gemm(h28, self.w8_gate_up, alpha_cols=self.alpha_gate_up, round_acc=self.ra)   # [T, 2 * intermediate]
                gate, up = gu[:, :sh.intermediate], gu[:, sh.intermediate:]
            else:
                gate, up = (FP8.fp8_gemm(h28, self.w8[n], self.alpha[n], round_acc=self.ra) for n in ("gate", "up"))
            act8 = FP8.silu_mul_quantize_fp8(gate, up, s["act"])
        if self.fuse_residual:
            return FP8.fp8_gemm(act8, self.w8["down"], self.alpha["down"], residual=x1, round_acc=self.ra)
        return x1 + FP8.fp8_gemm(act8, self.w8["down"], self.alpha["down"], round_acc=self.ra)

    def forward_unfused(self, x):
        """The same layer with every producer run by torch and a plain cast after it."""
        sh, s = self.shape, self.scales
        T = x.shape[0]
        (cos, sin), mask = self._tables(T, x.device)
        h8 = FP8.quantize_fp8(F.rms_norm(x, (sh.hidden,), self.ln1, sh.eps), s["h"])
        q = FP8.fp8_gemm(h8, self.w8["q"], self.alpha["q"], round_acc=self.ra).view(T, sh.heads, sh.head_dim)
        k = FP8.fp8_gemm(h8, self.w8["k"], self.alpha["k"], round_acc=self.ra).view(T, sh.kv_heads, sh.head_dim)
        v = FP8.fp8_gemm(h8, self.w8["v"], self.alpha["v"], round_acc=self.ra).view(T, sh.kv_heads, sh.head_dim)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        q8 = FP8.quantize_fp8(q.view(T, sh.kv_heads, sh.groups, sh.head_dim).permute(1, 2, 0, 3)
                              .reshape(sh.kv_heads, sh.groups * T, sh.head_dim), s["q"])
        k8 = FP8.quantize_fp8(k.transpose(0, 1), s["k"])                    # [kv, T, d]
        vt8 = FP8.quantize_fp8(v.permute(1, 2, 0), s["v"])                  # [kv, d, T]
        scores = FP8.fp8_gemm(q8, k8, self.alpha_qk, round_acc=self.ra)     # [kv, groups*T, T]
        p8 = FP8.softmax_quantize_fp8(scores, 1.0 / math.sqrt(sh.head_dim), s["p"], causal_period=T)
        ctx = FP8.fp8_gemm(p8, vt8, self.alpha_pv, round_acc=self.ra)       # [kv, groups*T, d]
        ctx = ctx.view(sh.kv_heads, sh.groups, T, sh.head_dim).permute(2, 0, 1, 3).reshape(T, sh.heads * sh.head_dim)
        x1 = x + FP8.fp8_gemm(FP8.quantize_fp8(ctx, s["ctx"]), self.w8["o"], self.alpha["o"], round_acc=self.ra)
        h28 = FP8.quantize_fp8(F.rms_norm(x1, (sh.hidden,), self.ln2, sh.eps), s["h2"])
        act = F.silu(FP8.fp8_gemm(h28, self.w8["gate"], self.alpha["gate"], round_acc=self.ra)) * \
            FP8.fp8_gemm(h28, self.w8["up"], self.alpha["up"], round_acc=self.ra)
        return x1 + FP8.fp8_gemm(FP8.quantize_fp8(act, s["act"]), self.w8["down"], self.alpha["down"],
                                 round_acc=self.ra)

    __call__ = forward


# ---------------------------------------------------------------------------
# NVFP4 decoder layer (e2m1, blocks of 16 along K, e4m3 block scales, one global scale per tensor)
# ---------------------------------------------------------------------------
class Nvfp4DecoderLayer:
    """A Llama-shaped decoder layer whose seven linears run as NVFP4 casts + native block-scaled
    GEMMs -- the sites the reference's ``backend/gpu/nvfp4.py`` rewrites (``quantize_mx`` with an
    e2m1 table, block 16, e4m3 scales and a global scale, feeding ``linear_mx`` with ``alpha``).
    Everything else (RMSNorm, RoPE, attention, SiLU, residual adds) is not quantized in that graph
    and stays bfloat16 torch operators.

    Weights are quantized once, each with its own global scale, exactly as ``convert_pt2e`` bakes
    them (``quantization/quantize_pt2e.py:805-856``).  Linears that read one activation share one
    cast and one GEMM (q/k/v, gate/up): the activation is quantized once in the graph as well
    (shared fake-quantizer), and column ``n`` of the merged product is scaled by its own linear's
    ``alpha = bf16(t_activation * t_weight)``.
    """

    def __init__(self, params, shape: LlamaShape, merge=True, attention="fused"):
        from . import nvfp4 as NV

        self.NV, self.shape, self.merge = NV, shape, merge
        # "eager": the graph's own attention operators (matmul, scale + mask, softmax, matmul: HF eager
        # attention, every intermediate a bfloat16 tensor).  "fused": the same roundings inside this package's
        # one-kernel attention (head_dim 128, T a multiple of 128; other shapes run "eager").  "sdpa": torch's
        # fused kernel, which keeps the scores in float32; it differs from the other two by the bfloat16
        # rounding of the scores (half a unit at 64..128), which the 4-bit casts downstream amplify to
        # quantization-noise level.
        if attention not in ("eager", "fused", "sdpa"):
            raise ValueError(attention)
        self.attention = attention
        self.ln1, self.ln2 = params["ln1"], params["ln2"]
        packed = {n: NV.quantize_nvfp4(params[n]) for n in LINEARS}
        self.w = {n: (c, s) for n, (c, s, t) in packed.items()}
        self.tw = {n: t for n, (c, s, t) in packed.items()}
        self.one = torch.ones((), device=self.ln1.device)

        def merged(names):
            # scale tiles cover 128 rows each: whole tiles concatenate along the rows
            assert all(self.w[n][0].shape[0] % 128 == 0 for n in names)
            codes = torch.cat([self.w[n][0] for n in names], 0)
            scales = torch.cat([self.w[n][1].reshape(-1) for n in names])
            tw = torch.cat([self.tw[n].reshape(1).expand(self.w[n][0].shape[0]) for n in names]).contiguous()
            return codes, scales, tw

        self.merged = {"qkv": merged(("q", "k", "v")), "gate_up": merged(("gate", "up"))} if merge else {}
        self._rope = None
        self._mask = None

    # kernels of this package per forward (merged): 4 x (amax + cast), 4 GEMMs, 2 RoPE, the attention
    LAUNCHES = 15

    def _linear(self, x, names):
        """``[linear(x, W_n) for n in names]`` through one cast of ``x``."""
        NV = self.NV
        codes, scales, t = NV.quantize_nvfp4(x)
        if len(names) > 1 and self.merge:
            wc, ws, tw = self.merged["qkv" if names[0] == "q" else "gate_up"]
            alpha_cols = (t * tw).float()                     # bf16(t_x * t_w) per column, widened
            y = NV.nvfp4_gemm(NV.PackedNVFP4(codes, scales), NV.PackedNVFP4(wc, ws), None, None, torch.bfloat16,
                              alpha_cols=alpha_cols)
            sizes = [self.w[n][0].shape[0] for n in names]
            return list(torch.split(y, sizes, dim=-1))
        return [NV.nvfp4_linear(codes, scales, *self.w[n], (t * self.tw[n]).float(), self.one, None) for n in names]

    def _attention(self, q, k, v):
        """Causal attention of ``q [T, heads, d]``, ``k`` / ``v`` ``[T, kv_heads, d]`` -> ``[T, heads * d]``."""
        sh = self.shape
        T = q.shape[0]
        if self.attention == "sdpa":
            ctx = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None],
                                                 v.transpose(0, 1)[None], is_causal=True, enable_gqa=True)[0]
            return ctx.transpose(0, 1).reshape(T, sh.heads * sh.head_dim)
        if self.attention == "fused" and sh.head_dim == 128 and T % 128 == 0:
            from . import fp8 as F8

            return F8.attention_bf16(q, k, v)
        if self._mask is None or self._mask.shape[0] != T:
            self._mask = causal_mask(T, q.device)
        # a KV group's query heads share its keys: [kv, groups, T, d] x [kv, 1, d, T], no repeated K / V
        qg = q.reshape(T, sh.kv_heads, sh.groups, sh.head_dim).permute(1, 2, 0, 3)
        scores = torch.matmul(qg, k.permute(1, 2, 0)[:, None])                       # [kv, groups, T, T] bfloat16
        # mask + scores / sqrt(d): the mask is 0 or -inf, so one rounding here equals the graph's two
        scores = torch.add(self._mask, scores, alpha=1.0 / math.sqrt(sh.head_dim))
        p = torch.softmax(scores, -1)                                                # float32 inside, rounded once
        ctx = torch.matmul(p, v.transpose(0, 1)[:, None])                            # [kv, groups, T, d]
        return ctx.permute(2, 0, 1, 3).reshape(T, sh.heads * sh.head_dim)

    def forward(self, x):
        sh = self.shape
        T = x.shape[0]
        if self._rope is None or self._rope[0].shape[0] != T:
            self._rope = rope_tables(T, sh, x.device)
        cos, sin = self._rope
        h = F.rms_norm(x, (sh.hidden,), self.ln1, sh.eps)
        q, k, v = self._linear(h, ("q", "k", "v"))
        if self.attention == "fused" and sh.head_dim == 128 and T % 128 == 0:
            # RoPE straight into the attention kernel's head-major layout (slices of the merged projection are
            # read in place), V transposed for the P V contraction
            from . import fp8 as F8

            ctx = F8.attention_bf16_heads(F8.rope_heads_bf16(q.unflatten(1, (sh.heads, sh.head_dim)), cos, sin),
                                          F8.rope_heads_bf16(k.unflatten(1, (sh.kv_heads, sh.head_dim)), cos, sin),
                                          v.unflatten(1, (sh.kv_heads, sh.head_dim)).permute(1, 2, 0).contiguous())
        else:
            q = apply_rope(q.reshape(T, sh.heads, sh.head_dim), cos, sin)
            k = apply_rope(k.reshape(T, sh.kv_heads, sh.head_dim), cos, sin)
            v = v.reshape(T, sh.kv_heads, sh.head_dim)
            ctx = self._attention(q, k, v)
        x1 = x + self._linear(ctx, ("o",))[0]
        h2 = F.rms_norm(x1, (sh.hidden,), self.ln2, sh.eps)
        gate, up = self._linear(h2, ("gate", "up"))
        if self.attention == "fused":
            # SwiGLU, its amax and the NVFP4 cast without a separate amax pass
            NV = self.NV
            codes, scales, t = NV.silu_mul_cast_nvfp4(gate, up)
            down = NV.nvfp4_linear(codes, scales, *self.w["down"], (t * self.tw["down"]).float(), self.one, None)
            return x1 + down
        return x1 + self._linear(F.silu(gate) * up, ("down",))[0]

    __call__ = forward


def make_layer_params_on_device(seed: int, shape: LlamaShape, device):
    """``make_layer_params`` drawn by the device's generator (for many-layer benchmarks, where drawing
    billions of normals on the host would dominate set-up; the values differ from the host generator's)."""
    g = torch.Generator(device=device).manual_seed(seed)
    params = {name: (torch.randn(*dims, generator=g, device=device) * 0.02).bfloat16()
              for name, dims in linear_shapes(shape).items()}
    params["ln1"] = torch.ones(shape.hidden, dtype=torch.bfloat16, device=device)
    params["ln2"] = torch.ones(shape.hidden, dtype=torch.bfloat16, device=device)
    return params


class Nvfp4Model:
    """``layers`` NVFP4 decoder layers, a final RMSNorm and an NVFP4 ``lm_head`` applied to the last position
    (what a prefill hands to sampling): the shape of a converted Llama-3.1-8B graph with
    ``fp4_e2m1,qs=microscaling,bs=16,scale=fp8_e4m3,gs=1`` on activations and weights of every linear."""

    def __init__(self, layers: int, shape: LlamaShape, device, seed: int = 0, layer_cls=None, **layer_args):
        from . import nvfp4 as NV

        self.NV, self.shape = NV, shape
        cls = layer_cls or Nvfp4DecoderLayer
        self.layers = []
        for i in range(layers):
            params = make_layer_params_on_device(seed + i, shape, device)
            self.layers.append(cls(params, shape, **layer_args))
            del params
        g = torch.Generator(device=device).manual_seed(seed + layers)
        head = (torch.randn(shape.vocab, shape.hidden, generator=g, device=device) * 0.02).bfloat16()
        self.head = NV.quantize_nvfp4(head)
        del head
        self.norm = torch.ones(shape.hidden, dtype=torch.bfloat16, device=device)
        self.one = torch.ones((), device=device)

    @property
    def LAUNCHES(self):
        return sum(layer.LAUNCHES for layer in self.layers) + 3

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return self.logits(x[-1:])

    def logits(self, last):
        """``last``: the final position's hidden state ``[1, hidden]`` -> ``[1, vocab]``."""
        NV = self.NV
        codes, scales, t = NV.quantize_nvfp4(F.rms_norm(last, (self.shape.hidden,), self.norm, self.shape.eps))
        wc, ws, tw = self.head
        return NV.nvfp4_linear(codes, scales, wc, ws, (t * tw).float(), self.one, None)

    __call__ = forward


# ---------------------------------------------------------------------------
# MXNF4 decode step with a KIVI cache
# ---------------------------------------------------------------------------
class Mxnf4DecodeLayer:
    """One decode step of a decoder layer in the MXNF4 recipe (``lut4_to_int6`` with NF4 levels, blocks
    of 64, ``fp8_e5m3`` scales on weights and activations; residual adds through a per-tensor
    ``fp8_e4m3`` cast; KIVI 2-bit cache with the newest positions in bfloat16) for a batch of sequences
    that each add one token.

    Weights live packed (``packed.PackedLUT4Weight``, q/k/v and gate/up merged row-wise: microscaling
    weights carry only per-block scales, so stacking rows changes nothing) and every linear is one
    activation ``quantize_mx`` plus the weight-streaming ``linear_lut4``.  The cached keys and values
    are packed 2-bit codes; the attention over [cache | recent] keys is one kernel that decodes them in
    registers (``kivi.decode_attention``; ``fused_attention=False`` reads the cache back to bfloat16 and runs
    the graph's matmul / softmax / matmul as torch operators).
    """

    def __init__(self, weights, tables, cache, residual_scale, shape: LlamaShape, fused_attention=True):
        self.w, self.t, self.cache, self.shape = weights, tables, cache, shape
        self.fused_attention = fused_attention
        self.fused_residual = fused_attention      # the three residual nodes (quantize, dequantize, add) as one kernel
        self.residual_scale = residual_scale
        self.ln1, self.ln2 = weights["ln1"], weights["ln2"]

    # kernels of this package per step: 4 quantize_mx, 4 linears, RoPE + append, the attention, 2 residual casts + adds
    LAUNCHES = 12

    def _linear(self, x, name):
        from . import packed as P

        t = self.t
        s, c = torch.ops.quantized_ops.quantize_mx(x, t["index"], [-1], 64, 31.0, False, t["e5m3"], t["mid"])
        return P.linear_lut4(c, self.w[name], input_scale=s, input_code=t["levels"])

    def _through_fp8(self, x):
        q = torch.ops.quantized_ops.quantize(x, self.residual_scale, None, None, None, self.t["e4m3"])
        return torch.ops.quantized_ops.dequantize(q, self.residual_scale)

    def _residual_add(self, x, branch):
        """``dequantize(quantize(x)) + branch``: the residual stream through its per-tensor e4m3 cast."""
        if self.fused_residual:
            from . import fp8 as F8

            return F8.roundtrip_add(x, self.residual_scale, branch)
        return self._through_fp8(x) + branch

    def forward(self, x, rope):
        """``x [B, hidden]``; ``rope = (cos, sin)`` of the new position, ``[head_dim]`` each."""
        sh = self.shape
        B, d, hq, hkv = x.shape[0], sh.head_dim, sh.heads, sh.kv_heads
        cos, sin = rope
        half = d // 2

        def rotate(v):
            return v * cos + torch.cat([-v[..., half:], v[..., :half]], -1) * sin

        qkv = self._linear(F.rms_norm(x, (sh.hidden,), self.ln1, sh.eps), "qkv")
        k_res, v_res = self.cache["k_res"], self.cache["v_res"]
        if self.fused_attention:
            from . import kivi as KV

            q = KV.rope_append(qkv, cos, sin, hq, k_res, v_res, -1)   # this step's token takes the last recent slot
        else:
            q = rotate(qkv[:, :hq * d].reshape(B, hq, d))
            k = rotate(qkv[:, hq * d:(hq + hkv) * d].reshape(B, hkv, d))
            v = qkv[:, (hq + hkv) * d:].reshape(B, hkv, d)
            k_res[:, :, -1].copy_(k)
            v_res[:, :, -1].copy_(v)
        qg = q.reshape(B, hkv, hq // hkv, d)
        ctx = None
        if self.fused_attention:
            from . import kivi as KV

            ctx = KV.decode_attention(qg, self.cache["k"], self.cache["v"], k_res, v_res)
        if ctx is None:
            k_main, v_main = self.cache["k"].read(), self.cache["v"].read()
            scores = torch.cat([torch.matmul(qg, k_main.transpose(-1, -2)), torch.matmul(qg, k_res.transpose(-1, -2))], -1)
            p = torch.softmax(scores * (1.0 / math.sqrt(d)), -1, dtype=torch.float32).to(x.dtype)
            tm = k_main.shape[-2]
            ctx = torch.matmul(p[..., :tm], v_main) + torch.matmul(p[..., tm:], v_res)
        x1 = self._residual_add(x, self._linear(ctx.reshape(B, hq * d), "o"))
        gu = self._linear(F.rms_norm(x1, (sh.hidden,), self.ln2, sh.eps), "gate_up")
        inter = gu.shape[-1] // 2
        return self._residual_add(x1, self._linear(F.silu(gu[:, :inter]) * gu[:, inter:], "down"))

    __call__ = forward


def nf4_tables(device):
    """The lookup tables of ``lut4_to_int6`` as a converted graph holds them (``quantize_pt2e.py:754-791``):
    the 16 levels, the 65 536-entry index table, the midpoints, plus the scale and residual tables."""
    nf4 = formats.get_quantization_map("lut4_to_int6", device)
    index, levels = formats.index_table(nf4)
    return {"levels": levels, "index": index, "mid": (levels[:-1] + levels[1:]) / 2,
            "e5m3": formats.get_quantization_map("fp8_e5m3", device),
            "e4m3": formats.get_quantization_map("fp8_e4m3", device),
            "uint2": formats.get_quantization_map("uint2", device)}
