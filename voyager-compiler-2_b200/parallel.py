"""Tensor-parallel microscaling linears over one multi-GPU box.

The reference has no distributed execution (its ``modeling.py`` only places
layers on devices).  This module shards the quantized linears of a Llama-shaped
layer the Megatron way, one process per GPU with ``torch.distributed``:

* **column-parallel** (q/k/v, gate/up): the weight's codes and block scales are
  split along the output features; blocks run along K, so a shard is a row
  slice.  The activation is quantized once (or its codes and scales are
  all-gathered from token shards, 2.1 B/element instead of 2 + 2).
* **row-parallel** (o_proj, down_proj): weight and activation are split along K
  in whole blocks, so each rank's block scales and codes are exactly those of
  the unsharded tensor; ranks produce fp32 partial products that are
  reduce-scattered over token rows (or all-reduced) and rounded once, which is
  the single-GPU result up to fp32 summation order.
* a per-tensor global scale (NVFP4) on a K-sharded activation needs the global
  amax: one scalar all-reduce(max) keeps it, and therefore every code, identical
  to the single-GPU run.

Collectives are NCCL on GPUs (NVLink/NVSwitch); the same code runs on the gloo
backend for the CPU tests, where the operator namespace is injected.
"""

import dataclasses
from typing import Optional

import torch
import torch.distributed as dist


@dataclasses.dataclass(frozen=True)
class MXSpec:
    """Arguments of ``quantize_mx`` / ``linear_mx`` for one tensor."""

    qmap: torch.Tensor
    block_size: int
    quant_max: float
    power_of_two: bool = False
    scale_qmap: Optional[torch.Tensor] = None
    output_code: Optional[torch.Tensor] = None
    code: Optional[torch.Tensor] = None          # codebook for read-back (lookup formats)
    global_scale_max: Optional[float] = None     # NVFP4: largest value of the scale dtype (448)


def _ops(ops):
    return torch.ops.quantized_ops if ops is None else ops


def shard_bounds(extent: int, rank: int, world: int, multiple: int = 1):
    """Contiguous shard ``[lo, hi)`` of ``extent`` for ``rank``; every shard is a whole
    number of ``multiple`` (blocks must not straddle ranks)."""
    if extent % (world * multiple):
        raise ValueError(f"{extent} does not split into {world} shards of whole {multiple}-element blocks")
    per = extent // world
    return rank * per, (rank + 1) * per


def shard_weight(codes, scale, mode: str, rank: int, world: int, block_size: int):
    """Slice a quantized weight ``codes [N, K]`` / ``scale [N, K/bs]`` for ``rank``.
    ``mode`` is ``"column"`` (split N) or ``"row"`` (split K)."""
    if mode == "column":
        lo, hi = shard_bounds(codes.shape[0], rank, world)
        return codes[lo:hi].contiguous(), scale[lo:hi].contiguous()
    if mode == "row":
        lo, hi = shard_bounds(codes.shape[1], rank, world, block_size)
        return codes[:, lo:hi].contiguous(), scale[:, lo // block_size:hi // block_size].contiguous()
    raise ValueError(mode)


def global_amax_scale(x, spec: MXSpec, group=None):
    """NVFP4's per-tensor scale ``amax / (quant_max * scale_max)`` of a tensor whose K
    axis is sharded over ``group``: the amax is all-reduced so that every rank gets the
    value the unsharded tensor would give."""
    if x.is_cuda:
        from .ops import tensor_amax  # one pass, no intermediate |x| tensor

        amax = tensor_amax(x)
    else:
        amax = x.abs().amax().float()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    ratio = (amax.to(x.dtype) / (spec.quant_max * spec.global_scale_max))
    return ratio.clamp_min(torch.finfo(torch.float32).tiny)


def quantize_activation(x, spec: MXSpec, ops=None, group=None):
    """``(scale, codes, global_scale)`` of an activation blocked along its last axis."""
    gs = None if spec.global_scale_max is None else global_amax_scale(x, spec, group)
    scale, codes = _ops(ops).quantize_mx(x, spec.qmap, [-1], spec.block_size, spec.quant_max, spec.power_of_two,
                                         spec.scale_qmap, spec.output_code, None, gs)
    return scale, codes, gs


def all_gather_rows(t, group=None):
    """Concatenate every rank's token rows (first axis)."""
    world = dist.get_world_size(group)
    if world == 1:
        return t
    out = torch.empty((world * t.shape[0], *t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out


def reduce_scatter_rows(t, group=None):
    """Sum over ranks and keep this rank's slice of the token rows (first axis)."""
    world = dist.get_world_size(group)
    if world == 1:
        return t
    if t.shape[0] % world:
        raise ValueError(f"{t.shape[0]} token rows do not split over {world} ranks")
    out = torch.empty((t.shape[0] // world, *t.shape[1:]), dtype=t.dtype, device=t.device)
    if dist.get_backend(group) == "gloo":  # gloo has no reduce_scatter_tensor
        full = t.contiguous().clone()
        dist.all_reduce(full, group=group)
        rank = dist.get_rank(group)
        return full[rank * out.shape[0]:(rank + 1) * out.shape[0]].contiguous()
    dist.reduce_scatter_tensor(out, t.contiguous(), group=group)
    return out


def column_parallel_linear(x, w_codes, w_scale, act: MXSpec, wgt: MXSpec, *, weight_global_scale=None,
                           gather_input=False, group=None, ops=None, quantized=None):
    """``x @ W[shard]^T`` for a weight split along its output features.  ``x`` is the full
    activation ``[T, K]`` (or this rank's token rows when ``gather_input``: codes and scales
    are gathered, not the bfloat16 values).  ``quantized`` reuses an activation already
    quantized by ``quantize_activation`` (linears sharing one input).  Returns ``[T, N / world]``."""
    scale, codes, gs = quantized if quantized is not None else quantize_activation(x, act, ops, None)
    if gather_input:
        if gs is not None:
            raise ValueError("a global scale must be computed over the gathered activation")
        scale, codes = all_gather_rows(scale, group), all_gather_rows(codes, group)
    alpha = None if gs is None else gs * weight_global_scale
    return _ops(ops).linear_mx(codes, w_codes, None, input_scale=scale, weight_scale=w_scale,
                               block_size=act.block_size, input_code=act.code, weight_code=wgt.code, alpha=alpha)


def row_parallel_linear(x_shard, w_codes, w_scale, act: MXSpec, wgt: MXSpec, *, weight_global_scale=None,
                        scatter_output=True, group=None, ops=None):
    """``x @ W^T`` for activation and weight split along K: fp32 partial products are
    reduce-scattered over token rows (or all-reduced) and rounded once to ``x``'s dtype."""
    scale, codes, gs = quantize_activation(x_shard, act, ops, group)
    alpha = None if gs is None else gs * weight_global_scale
    partial = _ops(ops).linear_mx(codes, w_codes, None, input_scale=scale, weight_scale=w_scale,
                                  block_size=act.block_size, input_code=act.code, weight_code=wgt.code,
                                  alpha=alpha, out_dtype=torch.float32)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        if scatter_output:
            partial = reduce_scatter_rows(partial, group)
        else:
            dist.all_reduce(partial, group=group)
    return partial.to(x_shard.dtype)


class TensorParallelMLP:
    """SwiGLU MLP with gate/up column-parallel and down row-parallel.  Weights are
    quantized once on the full tensors (so block and global scales are the single-GPU
    ones) and then sliced per rank."""

    def __init__(self, gate, up, down, act: MXSpec, wgt: MXSpec, group=None, ops=None):
        self.act, self.wgt, self.group, self.ops = act, wgt, group, ops
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        q = _ops(ops)
        self.shards = {}
        for name, w, mode in (("gate", gate, "column"), ("up", up, "column"), ("down", down, "row")):
            gs = None
            if wgt.global_scale_max is not None:
                gs = global_amax_scale(w, wgt, None)  # the full weight is present on every rank here
            s, c = q.quantize_mx(w, wgt.qmap, [-1], wgt.block_size, wgt.quant_max, wgt.power_of_two, wgt.scale_qmap,
                                 wgt.output_code, None, gs)
            cs, ss = shard_weight(c, s, mode, self.rank, self.world, wgt.block_size)
            self.shards[name] = (cs, ss, gs)

    def forward(self, x, scatter_output=False):
        a, w = self.act, self.wgt
        xq = quantize_activation(x, a, self.ops, None)           # gate and up read one quantized input
        g = column_parallel_linear(x, *self.shards["gate"][:2], a, w, weight_global_scale=self.shards["gate"][2],
                                   group=self.group, ops=self.ops, quantized=xq)
        u = column_parallel_linear(x, *self.shards["up"][:2], a, w, weight_global_scale=self.shards["up"][2],
                                   group=self.group, ops=self.ops, quantized=xq)
        h = torch.nn.functional.silu(g) * u                      # [T, I / world]: already K-sharded for down
        return row_parallel_linear(h, *self.shards["down"][:2], a, w, weight_global_scale=self.shards["down"][2],
                                   scatter_output=scatter_output, group=self.group, ops=self.ops)

    __call__ = forward


# ---------------------------------------------------------------------------
# GPTQ over several GPUs: the linears of a model are independent problems
# ---------------------------------------------------------------------------
def gptq_cost(tokens: int, out_features: int, in_features: int) -> float:
    """Relative cost of one GPTQ problem: the Hessian ``X^T X`` (tokens * K^2), its Cholesky
    factorisations (K^3) and the column sweep with its trailing updates (out * K^2)."""
    k = float(in_features)
    return float(tokens) * k * k + k ** 3 + float(out_features) * k * k


def lpt_schedule(costs, world: int):
    """Longest-processing-time assignment of problems to ``world`` ranks: problems in descending
    cost, each to the rank with the least work so far (ties to the lower rank, so every rank
    computes the same table without communicating).  Returns one list of problem indices per rank."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0.0] * world
    assignment = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda q: (load[q], q))
        assignment[r].append(i)
        load[r] += costs[i]
    return assignment


def gptq_layer_parallel(problems, solve, group=None):
    """Run independent GPTQ problems across the ranks of ``group`` and give every rank all results.

    ``problems`` is the same list on every rank, each item a dict with ``weight [out, in]``,
    ``tokens`` and whatever ``solve(problem) -> Tensor`` needs (its Hessian or calibration
    activations); ``solve`` is called only for the problems this rank owns under the LPT schedule
    (cost ``gptq_cost``).  The reference walks a model's linears one after another
    (``quantization/gptq.py:560-707``); with calibration activations given per linear they do not
    depend on each other, and the only exchange is handing the compensated weights round at the end."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    costs = [gptq_cost(p["tokens"], p["weight"].shape[0], p["weight"].shape[1]) for p in problems]
    mine = lpt_schedule(costs, world)[rank]
    local = {i: solve(problems[i]) for i in mine}
    if world == 1:
        return [local[i].to(problems[i]["weight"].dtype) for i in range(len(problems))]
    owner = {}
    for r, indices in enumerate(lpt_schedule(costs, world)):
        for i in indices:
            owner[i] = r
    # One wire format on every rank: float32 (what the solve computes in, whatever the weight's dtype),
    # the weight's shape, contiguous.  Receivers cannot know what dtype ``solve`` returned on the owner.
    results = []
    for i, p in enumerate(problems):
        weight = p["weight"]
        if owner[i] == rank:
            if local[i].shape != weight.shape:
                raise ValueError(f"solve() returned shape {tuple(local[i].shape)} for a weight of {tuple(weight.shape)}")
            out = local[i].to(torch.float32).contiguous()
        else:
            out = torch.empty(weight.shape, dtype=torch.float32, device=weight.device)
        dist.broadcast(out, src=dist.get_global_rank(group, owner[i]) if group is not None else owner[i], group=group)
        results.append(out.to(weight.dtype))
    return results


# ---------------------------------------------------------------------------
# The per-tensor FP8 decoder layer, tensor- and sequence-parallel
# ---------------------------------------------------------------------------
class PeerExchange:
    """All-gather and reduce-scatter over token rows by plain loads from the peers' memory (NVLink) instead of
    NCCL: each rank writes into its own symmetric-memory buffer, a cross-rank barrier orders the writes, and
    ``vq_peer_gather`` / ``vq_peer_reduce_rows`` pull what this rank needs.  One buffer serves the gathers and one
    the partial sums; a layer alternates gather, reduce, gather, reduce, so the barrier of the next exchange
    also tells every rank that its peers have finished reading the buffer it is about to rewrite.

    ``gather_bytes`` / ``reduce_floats``: the largest per-rank chunk of each kind.  Needs peer access between
    the group's GPUs (``torch.distributed._symmetric_memory``)."""

    def __init__(self, gather_bytes: int, reduce_floats: int, device, group=None):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.gather_buf = symm.empty(max(gather_bytes, 16), dtype=torch.uint8, device=device)
        self.reduce_buf = symm.empty(max(reduce_floats, 4), dtype=torch.float32, device=device)
        self.scalar_buf = symm.empty(4, dtype=torch.float32, device=device)
        self.gather_hdl = symm.rendezvous(self.gather_buf, self.group)
        self.reduce_hdl = symm.rendezvous(self.reduce_buf, self.group)
        self.scalar_hdl = symm.rendezvous(self.scalar_buf, self.group)
        self._scalar_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self.scalar_hdl.buffer_ptrs])
        array = ctypes.c_void_p * self.world
        self._gather_ptrs = array(*[int(p) for p in self.gather_hdl.buffer_ptrs])
        self._reduce_ptrs = array(*[int(p) for p in self.reduce_hdl.buffer_ptrs])
        self._channel = 0

    def gather_slot(self, nbytes: int) -> torch.Tensor:
        """This rank's chunk of the next all-gather, to be written by the producer kernel."""
        return self.gather_buf[:nbytes]

    def reduce_slot(self, shape) -> torch.Tensor:
        """This rank's float32 partial sums (all token rows) of the next reduce-scatter, the GEMM's output."""
        n = 1
        for extent in shape:
            n *= extent
        return self.reduce_buf[:n].view(shape)

    def all_gather_rows(self, mine: torch.Tensor) -> torch.Tensor:
        """``mine``: a view of ``gather_slot`` already written on the current stream.  Returns every rank's rows."""
        from ._native import check, lib
        from .ops import _stream

        nbytes = mine.numel() * mine.element_size()
        if nbytes % 16:
            raise ValueError("a rank's chunk must be a multiple of 16 bytes")
        out = torch.empty((self.world * mine.shape[0], *mine.shape[1:]), dtype=mine.dtype, device=mine.device)
        self.gather_hdl.barrier(channel=0)
        check(lib().vq_peer_gather(self._gather_ptrs, self.world, nbytes, out.data_ptr(), _stream()), "vq_peer_gather")
        return out

    def all_reduce_max(self, value: torch.Tensor) -> torch.Tensor:
        """Max over ranks of a non-negative float32 scalar (a tensor's amax).  Uses of the scalar buffer are
        separated by a gather or a reduce, like those of the other two buffers."""
        from ._native import check, lib
        from .ops import _stream

        self.scalar_buf[:1].copy_(value.reshape(1))
        out = torch.empty((), dtype=torch.float32, device=value.device)
        self.scalar_hdl.barrier(channel=0)
        check(lib().vq_peer_max(self._scalar_ptrs, self.world, out.data_ptr(), _stream()), "vq_peer_max")
        return out

    def all_gather_parts(self, parts):
        """After ONE barrier, gather several byte ranges ``(offset, nbytes)`` of every rank's ``gather_slot``
        (each a multiple of 16 bytes at a 16-byte aligned offset): a list of flat uint8 tensors, rank-major."""
        import ctypes

        from ._native import check, lib
        from .ops import _stream

        self.gather_hdl.barrier(channel=0)
        outs = []
        for offset, nbytes in parts:
            if offset % 16 or nbytes % 16:
                raise ValueError("parts are multiples of 16 bytes at 16-byte aligned offsets")
            ptrs = (ctypes.c_void_p * self.world)(*[int(p) + offset for p in self.gather_hdl.buffer_ptrs])
            out = torch.empty(self.world * nbytes, dtype=torch.uint8, device=self.gather_buf.device)
            check(lib().vq_peer_gather(ptrs, self.world, nbytes, out.data_ptr(), _stream()), "vq_peer_gather")
            outs.append(out)
        return outs

    def reduce_scatter_rows(self, partial: torch.Tensor) -> torch.Tensor:
        """``partial``: ``reduce_slot(shape)`` already written.  Returns this rank's rows of the sum over ranks."""
        from ._native import check, lib
        from .ops import _stream

        rows = partial.shape[0]
        if rows % self.world:
            raise ValueError(f"{rows} token rows do not split over {self.world} ranks")
        chunk = partial.numel() // self.world
        out = torch.empty((rows // self.world, *partial.shape[1:]), dtype=torch.float32, device=partial.device)
        self.reduce_hdl.barrier(channel=0)
        check(lib().vq_peer_reduce_rows(self._reduce_ptrs, self.world, self.rank, chunk, out.data_ptr(), _stream()),
              "vq_peer_reduce_rows")
        return out


def shard_fp8_layer(params, shape, rank: int, world: int):
    """The slices of one decoder layer's weights that ``rank`` of ``world`` holds: q/k/v by whole heads
    (rows), gate/up by rows, o and down by the matching input columns.  Returns ``(weights, heads)``
    with ``heads = (query heads, kv heads)`` on this rank."""
    if shape.kv_heads % world or shape.heads % world or shape.intermediate % (32 * world):
        raise ValueError(f"{shape.heads}/{shape.kv_heads} heads and {shape.intermediate} hidden units do not split "
                         f"over {world} ranks in whole heads and whole 32-row runs")
    d = shape.head_dim
    hq, hkv = shape.heads // world, shape.kv_heads // world
    lo_q, lo_kv = rank * hq * d, rank * hkv * d
    lo_i, hi_i = shard_bounds(shape.intermediate, rank, world, 32)
    w = {"q": params["q"][lo_q:lo_q + hq * d], "k": params["k"][lo_kv:lo_kv + hkv * d],
         "v": params["v"][lo_kv:lo_kv + hkv * d], "o": params["o"][:, lo_q:lo_q + hq * d],
         "gate": params["gate"][lo_i:hi_i], "up": params["up"][lo_i:hi_i], "down": params["down"][:, lo_i:hi_i]}
    return {k: v.contiguous() for k, v in w.items()}, (hq, hkv)


class Fp8DecoderLayerTP:
    """``workloads.Fp8DecoderLayer`` over the ranks of a process group.

    Activations between the blocks are sharded by token rows (``[T / world, hidden]``); q/k/v and
    gate/up are column-parallel (whole attention heads per rank: 4 query + 1 KV head at 8 ranks),
    o_proj and down_proj row-parallel:

        RMSNorm + FP8 cast on the rank's rows -> all-gather of the FP8 codes (1 byte per element)
        -> merged QKV GEMM (this rank's heads) -> RoPE + casts -> fused attention over its heads
        -> o_proj on its input columns, float32 partial sums -> reduce-scatter over token rows
        -> round, scale, add the residual rows -> RMSNorm + FP8 cast -> all-gather of the codes
        -> gate/up GEMM with the SwiGLU epilogue (its hidden units) -> down_proj partial sums
        -> reduce-scatter -> round, scale, add the residual rows.

    Per-tensor scales are those of the unsharded layer, so every FP8 code equals the single-GPU
    one; the row-parallel sums differ from it in float32 summation order only.  The collectives are
    NCCL's (``torch.distributed``); remote data always lands in this GPU's memory before a kernel
    reads it.  ``collective_seconds`` accumulates CUDA-event time around them when ``timed`` is set.
    """

    def __init__(self, params, scales, shape, group=None, graph_rounding=True, exchange=None):
        from . import fp8 as FP8

        self.FP8, self.shape, self.group, self.scales = FP8, shape, group, scales
        self.exchange = exchange          # a PeerExchange: pulls over peer memory instead of NCCL collectives
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.ra = bool(graph_rounding)
        w, (self.hq, self.hkv) = shard_fp8_layer(params, shape, self.rank, self.world)
        s = scales
        self.ln1, self.ln2 = params["ln1"], params["ln2"]
        w8 = {n: FP8.quantize_fp8(w[n], s["w_" + n]) for n in w}
        alpha = {n: (s[src] * s["w_" + n]).reshape(()) for n, src in
                 (("q", "h"), ("k", "h"), ("v", "h"), ("o", "ctx"), ("gate", "h2"), ("up", "h2"), ("down", "act"))}
        self.w8_qkv = torch.cat([w8["q"], w8["k"], w8["v"]], 0)
        self.alpha_qkv = torch.cat([alpha[n].float().expand(w8[n].shape[0]) for n in ("q", "k", "v")]).contiguous()
        self.w8_swiglu = FP8.interleave_gate_up(w8["gate"], w8["up"])
        rows = w8["gate"].shape[0]
        self.alpha_swiglu = FP8.interleave_gate_up(alpha["gate"].float().expand(rows).contiguous(),
                                                   alpha["up"].float().expand(rows).contiguous())
        self.w8_o, self.w8_down = w8["o"], w8["down"]
        self.alpha_o, self.alpha_down = alpha["o"], alpha["down"]
        self.alpha_qk = (s["q"] * s["k"]).reshape(())
        self.alpha_pv = (s["p"] * s["v"]).reshape(())
        self._rope = None
        self.timed = False
        self.collective_events = []

    # kernels of this package per forward: 2 norm+cast, the q/k/v casts (one launch), attention, 4 GEMMs
    LAUNCHES = 8
    COLLECTIVES = 4

    def _collective(self, fn, t):
        if not self.timed:
            return fn(t, self.group)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = fn(t, self.group)
        stop.record()
        self.collective_events.append((start, stop))
        return out

    def collective_seconds(self):
        """Device time spent inside the collectives since ``timed`` was set (synchronises)."""
        torch.cuda.synchronize()
        total = sum(a.elapsed_time(b) for a, b in self.collective_events) * 1e-3
        self.collective_events = []
        return total

    def _gather(self, x_rows, ln, scale):
        """RMSNorm + FP8 cast of this rank's rows, then every rank's codes."""
        FP8, sh = self.FP8, self.shape
        if self.exchange is None:
            return self._collective(all_gather_rows, FP8.rmsnorm_quantize_fp8(x_rows, ln, sh.eps, scale))
        mine = FP8.rmsnorm_quantize_fp8(x_rows, ln, sh.eps, scale, out=self.exchange.gather_slot(x_rows.numel()))
        return self._collective(lambda t, group: self.exchange.all_gather_rows(t), mine)

    def _partial_out(self, rows, cols):
        """Where a row-parallel GEMM writes its float32 partial sums: memory the peers can read, or a new tensor."""
        return None if self.exchange is None else self.exchange.reduce_slot((rows, cols))

    def _finish_row_parallel(self, partial, alpha, residual_rows):
        """Reduce-scatter the float32 partial sums over token rows, then what the single-GPU epilogue
        does: round the sum (the matmul's rounding), scale (the dequantize), add the residual rows."""
        if self.exchange is None:
            total = self._collective(reduce_scatter_rows, partial)
        else:
            total = self._collective(lambda t, group: self.exchange.reduce_scatter_rows(t), partial)
        y = total.to(torch.bfloat16) * alpha if self.ra else (total * alpha.float()).to(torch.bfloat16)
        return residual_rows + y

    def forward(self, x_rows):
        """``x_rows``: this rank's ``[T / world, hidden]`` rows.  Returns its rows of the layer output."""
        import math

        from .workloads import rope_tables

        FP8, sh, s = self.FP8, self.shape, self.scales
        T = x_rows.shape[0] * self.world
        if self._rope is None or self._rope[0].shape[0] != T:
            self._rope = rope_tables(T, sh, x_rows.device)
        cos, sin = self._rope
        d, hq, hkv = sh.head_dim, self.hq, self.hkv
        h8 = self._gather(x_rows, self.ln1, s["h"])
        qkv = FP8.fp8_gemm(h8, self.w8_qkv, alpha_cols=self.alpha_qkv, round_acc=self.ra)
        q = qkv[:, :hq * d].unflatten(1, (hq, d))
        k = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
        v = qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d))
        q8, k8, vt8 = FP8.qkv_post_fp8(q, k, v, cos, sin, s["q"], s["k"], s["v"])
        q8 = q8.view(hkv, (hq // hkv) * T, d)
        ctx8 = FP8.attention_fp8(q8, k8, vt8, self.alpha_qk, 1.0 / math.sqrt(d), s["p"], self.alpha_pv, s["ctx"],
                                 round_acc=self.ra)                                   # [T, hq * d]
        partial = FP8.fp8_gemm(ctx8, self.w8_o, out_dtype=torch.float32,
                               out=self._partial_out(T, sh.hidden))                   # [T, hidden], this rank's K
        x1 = self._finish_row_parallel(partial, self.alpha_o, x_rows)
        h28 = self._gather(x1, self.ln2, s["h2"])
        act8 = FP8.fp8_gemm(h28, self.w8_swiglu, alpha_cols=self.alpha_swiglu, gated_scale=s["act"],
                            round_acc=self.ra)                                        # [T, intermediate / world]
        partial = FP8.fp8_gemm(act8, self.w8_down, out_dtype=torch.float32, out=self._partial_out(T, sh.hidden))
        return self._finish_row_parallel(partial, self.alpha_down, x1)

    __call__ = forward


# ---------------------------------------------------------------------------
# NVFP4 decoder layer, tensor-parallel
# ---------------------------------------------------------------------------
def _slice_packed_nvfp4(codes, scales, n, k, rows=None, cols=None):
    """Rows ``[r0, r1)`` (multiples of 128) or contraction columns ``[c0, c1)`` (multiples of 64) of a packed
    NVFP4 matrix ``[n, k]``: codes ``[n, k / 2]`` and 512-byte scale tiles ``[n / 128, k / 64]``."""
    tiles = scales.reshape(-1).view(n // 128, k // 64, 512)
    if rows is not None:
        r0, r1 = rows
        if r0 % 128 or r1 % 128:
            raise ValueError("row shards of a packed NVFP4 matrix are whole 128-row scale tiles")
        return codes[r0:r1].contiguous(), tiles[r0 // 128:r1 // 128].contiguous().reshape(-1)
    c0, c1 = cols
    if c0 % 64 or c1 % 64:
        raise ValueError("column shards of a packed NVFP4 matrix are whole 64-element scale tiles")
    return codes[:, c0 // 2:c1 // 2].contiguous(), tiles[:, c0 // 64:c1 // 64].contiguous().reshape(-1)


class Nvfp4DecoderLayerTP:
    """``workloads.Nvfp4DecoderLayer`` over the ranks of a process group (north_star's column / row split).

    Activations between the blocks are sharded by token rows.  q/k/v and gate/up are column-parallel
    (whole heads / whole 128-row scale tiles per rank), o_proj and down_proj row-parallel:

        RMSNorm on the rank's rows -> amax all-reduce (one scalar: the global scale, hence every code, equals the
        single-GPU one) -> NVFP4 cast of its rows -> all-gather of packed codes and scale tiles (0.56 byte per
        element) -> merged QKV GEMM (its heads) -> RoPE -> fused bfloat16 attention over its heads
        -> amax all-reduce of the K-sharded context -> cast -> o_proj on its input columns, float32 partial
        products -> reduce-scatter over token rows -> round, add the residual rows; the MLP likewise.

    Weights are quantized unsharded (global scale from the whole weight) and then sliced, so every weight code
    equals the single-GPU one; the row-parallel sums differ in float32 summation order only.
    """

    LAUNCHES = 15
    COLLECTIVES = 10

    def __init__(self, params, shape, group=None, exchange=None):
        from . import nvfp4 as NV

        self.NV, self.shape, self.group = NV, shape, group
        self.exchange = exchange          # a PeerExchange: row exchanges pull over peer memory instead of NCCL
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        w, d = self.world, shape.head_dim
        if shape.kv_heads % w or shape.heads % w or shape.intermediate % (128 * w) or (shape.kv_heads // w * d) % 128:
            raise ValueError("heads and hidden units must split over the ranks in whole heads and whole 128-row tiles")
        self.hq, self.hkv = shape.heads // w, shape.kv_heads // w
        hq, hkv, r = self.hq, self.hkv, self.rank
        inter = shape.intermediate // w
        self.ln1, self.ln2 = params["ln1"], params["ln2"]
        hidden = shape.hidden

        def packed(name):
            codes, scales, t = NV.quantize_nvfp4(params[name])
            return codes, scales, t, params[name].shape[0], params[name].shape[1]

        def rows_of(name, r0, r1):
            codes, scales, t, n, k = packed(name)
            c, s = _slice_packed_nvfp4(codes, scales, n, k, rows=(r0, r1))
            return c, s, t

        def cols_of(name, c0, c1):
            codes, scales, t, n, k = packed(name)
            c, s = _slice_packed_nvfp4(codes, scales, n, k, cols=(c0, c1))
            return NV.PackedNVFP4(c, s), t

        def merged(parts):
            codes = torch.cat([c for c, _, _ in parts], 0)
            scales = torch.cat([s for _, s, _ in parts])
            tw = torch.cat([t.reshape(1).expand(c.shape[0]) for c, _, t in parts]).contiguous()
            return NV.PackedNVFP4(codes, scales), tw

        self.w_qkv, self.tw_qkv = merged([rows_of("q", r * hq * d, (r + 1) * hq * d),
                                          rows_of("k", r * hkv * d, (r + 1) * hkv * d),
                                          rows_of("v", r * hkv * d, (r + 1) * hkv * d)])
        self.w_gu, self.tw_gu = merged([rows_of("gate", r * inter, (r + 1) * inter),
                                        rows_of("up", r * inter, (r + 1) * inter)])
        self.w_o, self.t_o = cols_of("o", r * hq * d, (r + 1) * hq * d)
        self.w_down, self.t_down = cols_of("down", r * inter, (r + 1) * inter)
        self.hidden, self.inter = hidden, inter
        self._rope = None
        self.timed = False
        self.collective_events = []

    _collective = Fp8DecoderLayerTP._collective
    collective_seconds = Fp8DecoderLayerTP.collective_seconds

    def _global_scale(self, x, amax=None):
        """NVFP4's per-tensor scale of a tensor sharded over the group: the amax (computed here unless the
        producer already has it) is all-reduced first."""
        from . import ops as O
        from .nvfp4 import E4M3_MAX, FP4_MAX

        if amax is None:
            amax = O.tensor_amax(x)
        if self.world > 1 and self.exchange is not None:
            amax = self._collective(lambda t, group: self.exchange.all_reduce_max(t), amax)
        elif self.world > 1:
            def reduce_max(t, group):
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                return t
            amax = self._collective(reduce_max, amax)
        return O.global_scale_of_amax(amax, x.dtype, FP4_MAX, E4M3_MAX)

    def _gathered_cast(self, x_rows):
        """This rank's rows cast to NVFP4 with the whole tensor's global scale, then every rank's rows gathered."""
        NV = self.NV
        t = self._global_scale(x_rows)
        mine = NV.cast_nvfp4(x_rows, t)
        rows, k = x_rows.shape
        if rows % 128:
            raise ValueError("a rank's token rows must be whole 128-row scale tiles")
        if self.world == 1:
            return mine, t
        if self.exchange is not None:
            cb, sb = mine.codes.numel(), mine.scales.numel()
            slot = self.exchange.gather_slot(cb + sb)
            slot[:cb].copy_(mine.codes.reshape(-1))
            slot[cb:].copy_(mine.scales.reshape(-1))
            codes, tiles = self._collective(lambda parts, group: self.exchange.all_gather_parts(parts),
                                            [(0, cb), (cb, sb)])
            return NV.PackedNVFP4(codes.view(self.world * rows, k // 2), tiles), t
        codes = self._collective(all_gather_rows, mine.codes)
        tiles = self._collective(all_gather_rows, mine.scales.reshape(-1).view(rows // 128, -1))
        return NV.PackedNVFP4(codes, tiles.reshape(-1)), t

    def _row_parallel(self, x_cols, weight, t_w, residual_rows, amax=None):
        """``x_cols``: all token rows, this rank's slice of the contraction: float32 partial products are
        reduce-scattered over token rows, rounded once and added to the residual rows."""
        NV = self.NV
        t = self._global_scale(x_cols, amax)
        peer = self.exchange is not None and self.world > 1
        out = self.exchange.reduce_slot((x_cols.shape[0], weight.codes.shape[0])) if peer else None
        partial = NV.nvfp4_gemm(NV.cast_nvfp4(x_cols, t), weight, (t * t_w).float(), None, torch.float32, out=out)
        if self.world == 1:
            total = partial
        elif peer:
            total = self._collective(lambda p, group: self.exchange.reduce_scatter_rows(p), partial)
        else:
            total = self._collective(reduce_scatter_rows, partial)
        return residual_rows + total.to(torch.bfloat16)

    def forward(self, x_rows):
        """``x_rows``: this rank's ``[T / world, hidden]`` rows.  Returns its rows of the layer output."""
        import torch.nn.functional as F

        from . import fp8 as F8
        from .workloads import rope_tables

        NV, sh = self.NV, self.shape
        T = x_rows.shape[0] * self.world
        if self._rope is None or self._rope[0].shape[0] != T:
            self._rope = rope_tables(T, sh, x_rows.device)
        cos, sin = self._rope
        d, hq, hkv = sh.head_dim, self.hq, self.hkv
        act, t = self._gathered_cast(F.rms_norm(x_rows, (sh.hidden,), self.ln1, sh.eps))
        qkv = NV.nvfp4_gemm(act, self.w_qkv, None, None, torch.bfloat16, alpha_cols=(t * self.tw_qkv).float())
        ctx = F8.attention_bf16_heads(F8.rope_heads_bf16(qkv[:, :hq * d].unflatten(1, (hq, d)), cos, sin),
                                      F8.rope_heads_bf16(qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d)), cos, sin),
                                      qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d)).permute(1, 2, 0).contiguous())
        x1 = self._row_parallel(ctx, self.w_o, self.t_o, x_rows)
        act, t = self._gathered_cast(F.rms_norm(x1, (sh.hidden,), self.ln2, sh.eps))
        gu = NV.nvfp4_gemm(act, self.w_gu, None, None, torch.bfloat16, alpha_cols=(t * self.tw_gu).float())
        act, amax = NV.silu_mul_amax(gu[:, :self.inter], gu[:, self.inter:])
        return self._row_parallel(act, self.w_down, self.t_down, x1, amax)

    __call__ = forward
