"""Shared driver of the tensor-parallel tests: one SwiGLU MLP, sharded over the ranks of a
process group, against the unsharded computation."""

import os
import types

import torch
import torch.distributed as dist

from oracle import gemm as OG
from oracle import quantizers as OQ
from oracle import tables as OT


def oracle_ops():
    return types.SimpleNamespace(quantize_mx=OQ.quantize_mx, linear_mx=OG.linear_mx)


def problem(scheme, device="cpu"):
    import voyager_b200

    P = voyager_b200.parallel
    g = torch.Generator().manual_seed(21)
    T, H, I = 64, 128, 256
    x = torch.randn(T, H, generator=g).bfloat16().to(device)
    gate = (torch.randn(I, H, generator=g) * 0.05).bfloat16().to(device)
    up = (torch.randn(I, H, generator=g) * 0.05).bfloat16().to(device)
    down = (torch.randn(H, I, generator=g) * 0.05).bfloat16().to(device)
    if scheme == "mxint8":
        spec = P.MXSpec(qmap=OT.quantization_map("int8").to(device), block_size=16, quant_max=127.0, power_of_two=True)
    elif scheme == "nvfp4":
        spec = P.MXSpec(qmap=OT.quantization_map("fp4_e2m1").to(device), block_size=16, quant_max=6.0,
                        scale_qmap=OT.quantization_map("fp8_e4m3").to(device), global_scale_max=448.0)
    else:
        raise ValueError(scheme)
    return x, gate, up, down, spec


def run_rank(rank, world, backend, scheme, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if backend == "nccl":
        torch.cuda.set_device(rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        import voyager_b200

        P = voyager_b200.parallel
        device = f"cuda:{rank}" if backend == "nccl" else "cpu"
        ops = None if backend == "nccl" else oracle_ops()
        x, gate, up, down, spec = problem(scheme, device)
        mlp = P.TensorParallelMLP(gate, up, down, spec, spec, ops=ops)
        full = mlp(x, scatter_output=False)
        part = mlp(x, scatter_output=True)
        gathered = P.all_gather_rows(part)
        # token-sharded input: codes and scales are gathered instead of values
        lo, hi = P.shard_bounds(x.shape[0], rank, world)
        col = P.column_parallel_linear(x[lo:hi], *mlp.shards["gate"][:2], spec, spec, gather_input=True,
                                       ops=ops) if spec.global_scale_max is None else None
        col_ref = P.column_parallel_linear(x, *mlp.shards["gate"][:2], spec, spec, ops=ops) \
            if spec.global_scale_max is None else None
        if rank == 0:
            results["full"] = full.cpu()
            results["gathered"] = gathered.cpu()
            if col is not None:
                results["col_equal"] = bool(torch.equal(col.cpu(), col_ref.cpu()))
    finally:
        dist.destroy_process_group()


def single_process_reference(scheme):
    """The unsharded MLP on the CPU oracle."""
    import voyager_b200

    P = voyager_b200.parallel
    x, gate, up, down, spec = problem(scheme)
    mlp = P.TensorParallelMLP(gate, up, down, spec, spec, ops=oracle_ops())
    return mlp(x)


def fp8_layer_problem(seed=3):
    import voyager_b200

    W = voyager_b200.workloads
    shape = W.LlamaShape(hidden=512, heads=8, kv_heads=4, head_dim=128, intermediate=1024, vocab=1024)
    tokens = 256
    params = W.make_layer_params(seed, shape)
    x = W.make_hidden_states(seed + 1, tokens, shape)
    scales = W.calibrate_fp8_scales(x, params, shape)
    return shape, tokens, params, x, scales


def run_rank_fp8_layer(rank, world, port, results, peer=False):
    """The tensor- and sequence-parallel FP8 decoder layer on ``world`` GPUs; rank 0 gathers the output rows.
    ``peer``: the exchanges pull over peer memory (``PeerExchange``) instead of calling NCCL."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        import voyager_b200

        P = voyager_b200.parallel
        dev = f"cuda:{rank}"
        shape, tokens, params, x, scales = fp8_layer_problem()
        exchange = P.PeerExchange(tokens // world * shape.hidden, tokens * shape.hidden, dev) if peer else None
        layer = P.Fp8DecoderLayerTP({k: v.to(dev) for k, v in params.items()}, {k: v.to(dev) for k, v in scales.items()},
                                    shape, exchange=exchange)
        lo, hi = P.shard_bounds(tokens, rank, world)
        rows = layer(x[lo:hi].to(dev))
        if peer:                       # twice more: the buffers are reused across steps
            rows = layer(x[lo:hi].to(dev))
            rows = layer(x[lo:hi].to(dev))
        out = P.all_gather_rows(rows)
        voyager_b200.ops.gemm_status()
        assert voyager_b200.fp8.attention_status() == 0
        if rank == 0:
            results["out"] = out.cpu()
    finally:
        dist.destroy_process_group()


def nvfp4_layer_problem(seed=7):
    import voyager_b200

    W = voyager_b200.workloads
    shape = W.LlamaShape(hidden=512, heads=8, kv_heads=4, head_dim=128, intermediate=1024, vocab=1024)
    tokens = 256
    return shape, tokens, W.make_layer_params(seed, shape), W.make_hidden_states(seed + 1, tokens, shape)


def run_rank_nvfp4_layer(rank, world, port, results, peer=False):
    """The tensor-parallel NVFP4 decoder layer on ``world`` GPUs; rank 0 gathers the output rows."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        import voyager_b200

        P = voyager_b200.parallel
        dev = f"cuda:{rank}"
        shape, tokens, params, x = nvfp4_layer_problem()
        exchange = None
        if peer:
            per_rank = tokens // world * shape.hidden
            exchange = P.PeerExchange(per_rank // 2 + per_rank // 16, tokens * shape.hidden, dev)
        layer = P.Nvfp4DecoderLayerTP({k: v.to(dev) for k, v in params.items()}, shape, exchange=exchange)
        lo, hi = P.shard_bounds(tokens, rank, world)
        rows = layer(x[lo:hi].to(dev))
        if peer:
            rows = layer(x[lo:hi].to(dev))      # the buffers are reused across steps
        out = P.all_gather_rows(rows)
        voyager_b200.ops.gemm_status()
        assert voyager_b200.fp8.attention_status() == 0
        if rank == 0:
            results["out"] = out.cpu()
    finally:
        dist.destroy_process_group()


def gptq_problems(device="cpu"):
    g = torch.Generator().manual_seed(5)
    problems = []
    for out_f, in_f in ((64, 256), (32, 128), (96, 256), (32, 128), (64, 128)):
        x = torch.randn(1024, in_f, generator=g)
        problems.append(dict(weight=(torch.randn(out_f, in_f, generator=g) * 0.02).bfloat16().to(device),
                             hessian=(x.T @ x).to(device), tokens=1024))
    return problems


def run_rank_gptq(rank, world, port, results):
    """Layer-parallel GPTQ with the device solve on every rank's own GPU, results exchanged over NCCL."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        import voyager_b200

        dev = f"cuda:{rank}"
        G, P = voyager_b200.gptq, voyager_b200.parallel
        fq = G.grid_of(OT.quantization_map("int4").to(dev), OT.quantization_map("fp8_e5m3").to(dev), 7.0, 32)
        solved = []

        def solve(p):
            solved.append(tuple(p["weight"].shape))
            return G.compensate_weight(p["weight"].float(), p["hessian"].clone(), p["tokens"], fq, 0.01, act_order=False)

        out = P.gptq_layer_parallel(gptq_problems(dev), solve)
        torch.cuda.synchronize()
        results[rank] = (len(solved), [o.cpu() for o in out])
    finally:
        dist.destroy_process_group()
