"""Tensor-parallel sharding logic on CPU: two gloo ranks, the oracle's operators injected
for the kernels.  The sharded MLP must reproduce the unsharded one (codes are identical by
construction; only the fp32 summation of the row-parallel partials is reordered)."""

import pytest
import torch
import torch.multiprocessing as mp

import tp_common


@pytest.mark.parametrize("scheme", ["mxint8", "nvfp4"])
def test_two_rank_mlp_matches_unsharded(scheme):
    want = tp_common.single_process_reference(scheme)
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(tp_common.run_rank, args=(2, "gloo", scheme, 29611 if scheme == "mxint8" else 29612, results), nprocs=2,
             join=True)
    full, gathered = results["full"], results["gathered"]
    assert full.shape == want.shape and full.dtype == want.dtype
    err = float((full.float() - want.float()).abs().max() / want.float().abs().max())
    assert err <= 1e-2, err
    # reduce-scatter + all-gather of the rows equals the all-reduced result
    assert torch.equal(gathered, full)
    if scheme == "mxint8":
        assert results["col_equal"] is True


def test_shard_bounds_respect_blocks():
    import voyager_b200

    P = voyager_b200.parallel
    assert P.shard_bounds(14336, 3, 8, 64) == (5376, 7168)
    with pytest.raises(ValueError):
        P.shard_bounds(4096 + 16, 0, 8, 64)
    codes, scale = torch.arange(32.0).reshape(4, 8), torch.arange(8.0).reshape(4, 2)
    c, s = P.shard_weight(codes, scale, "row", 1, 2, 4)
    assert c.shape == (4, 4) and s.shape == (4, 1) and float(s[0, 0]) == 1.0
    c, s = P.shard_weight(codes, scale, "column", 1, 2, 4)
    assert c.shape == (2, 8) and s.shape == (2, 2)


def test_lpt_schedule_balances_llama_linears():
    import voyager_b200

    P = voyager_b200.parallel
    shapes = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (14336, 4096), (4096, 14336)] * 32
    costs = [P.gptq_cost(262144, o, k) for o, k in shapes]
    plan = P.lpt_schedule(costs, 8)
    assert sorted(i for part in plan for i in part) == list(range(len(shapes)))
    loads = [sum(costs[i] for i in part) for part in plan]
    assert max(loads) <= 1.02 * (sum(costs) / 8)          # within 2 % of a perfect split
    assert P.lpt_schedule(costs, 8) == plan               # deterministic: every rank derives the same table


def _gptq_rank(rank, world, port, results, weight_dtype=torch.float32):
    import os

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import voyager_b200
    from oracle import gptq as OG
    from oracle import tables as OT

    g = torch.Generator().manual_seed(5)
    problems = []
    for out_f, in_f in ((16, 128), (8, 64), (24, 128), (8, 64), (16, 64)):
        x = torch.randn(256, in_f, generator=g)
        problems.append(dict(weight=(torch.randn(out_f, in_f, generator=g) * 0.02).to(weight_dtype), hessian=x.T @ x,
                             tokens=256))
    calls = []

    def solve(p):
        calls.append(tuple(p["weight"].shape))
        fq = type("FQ", (), dict(block_size=32, ch_axis=-1, qmap=OT.quantization_map("int4"),
                                 scale_qmap=OT.quantization_map("fp8_e5m3"), quant_max=7.0))
        # the solve works in float32 whatever the weight's dtype, as the reference's does
        return OG.compensate_weight(p["weight"].float(), p["hessian"].clone(), p["tokens"], fq.qmap, fq.scale_qmap,
                                    fq.quant_max, fq.block_size, 0.01, False, True, False)

    out = voyager_b200.parallel.gptq_layer_parallel(problems, solve)
    results[rank] = (len(calls), [o.clone() for o in out])
    dist.destroy_process_group()


def test_gptq_layer_parallel_two_ranks():
    from oracle import gptq as OG
    from oracle import tables as OT

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_gptq_rank, args=(2, 29613, results), nprocs=2, join=True)
    (n0, out0), (n1, out1) = results[0], results[1]
    assert n0 + n1 == 5 and n0 >= 2 and n1 >= 2          # the work was split, nobody solved everything
    for a, b in zip(out0, out1):
        assert torch.equal(a, b)                          # every rank ends with every compensated weight
    g = torch.Generator().manual_seed(5)
    x = torch.randn(256, 128, generator=g)
    w = torch.randn(16, 128, generator=g) * 0.02
    want = OG.compensate_weight(w, x.T @ x, 256, OT.quantization_map("int4"), OT.quantization_map("fp8_e5m3"), 7.0, 32,
                                0.01, False, True, False)
    assert torch.equal(out0[0], want)


def test_gptq_layer_parallel_bfloat16_weights():
    """The solve returns float32 while the model's weights are bfloat16: owner and receivers must still agree on
    what crosses the wire, and every rank ends with the weights in the model's dtype."""
    from oracle import gptq as OG
    from oracle import tables as OT

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_gptq_rank, args=(2, 29617, results, torch.bfloat16), nprocs=2, join=True)
    (n0, out0), (n1, out1) = results[0], results[1]
    assert n0 + n1 == 5
    for a, b in zip(out0, out1):
        assert a.dtype == torch.bfloat16 and torch.equal(a, b)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(256, 128, generator=g)
    w = (torch.randn(16, 128, generator=g) * 0.02).bfloat16()
    want = OG.compensate_weight(w.float(), x.T @ x, 256, OT.quantization_map("int4"), OT.quantization_map("fp8_e5m3"),
                                7.0, 32, 0.01, False, True, False)
    assert torch.equal(out0[0], want.bfloat16())


def test_fp8_layer_shards_tile_the_layer():
    """Every weight element of a decoder layer belongs to exactly one rank's slice, heads stay whole, and the
    gate/up slices keep whole 32-row runs (the SwiGLU epilogue's interleave)."""
    import voyager_b200

    W, P = voyager_b200.workloads, voyager_b200.parallel
    shape = W.LlamaShape(hidden=256, heads=8, kv_heads=4, head_dim=32, intermediate=512, vocab=64)
    params = W.make_layer_params(1, shape)
    for world in (1, 2, 4):
        shards = [P.shard_fp8_layer(params, shape, r, world) for r in range(world)]
        assert all(h == (8 // world, 4 // world) for _, h in shards)
        for name in ("q", "k", "v", "gate", "up"):
            assert torch.equal(torch.cat([s[name] for s, _ in shards], 0), params[name])
        for name in ("o", "down"):
            assert torch.equal(torch.cat([s[name] for s, _ in shards], 1), params[name])
        assert all(s["gate"].shape[0] % 32 == 0 for s, _ in shards)
    with pytest.raises(ValueError):
        P.shard_fp8_layer(params, shape, 0, 8)          # more ranks than KV heads
