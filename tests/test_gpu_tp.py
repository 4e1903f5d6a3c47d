"""Tensor-parallel MLP on two GPUs over NCCL (skipped with fewer than two devices)."""

import pytest
import torch
import torch.multiprocessing as mp

import tp_common

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("scheme", ["mxint8", "nvfp4"])
def test_two_gpu_mlp_matches_unsharded(scheme):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    want = tp_common.single_process_reference(scheme)
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(tp_common.run_rank, args=(2, "nccl", scheme, 29621 if scheme == "mxint8" else 29622, results), nprocs=2,
             join=True)
    full, gathered = results["full"], results["gathered"]
    err = float((full.float() - want.float()).abs().max() / want.float().abs().max())
    assert err <= 1e-2, err
    assert torch.equal(gathered, full)


def test_two_gpu_fp8_decoder_layer_matches_one_gpu_and_the_oracle():
    """Column-parallel QKV and gate/up, head-parallel attention, row-parallel o_proj and down_proj with
    reduce-scattered float32 partial sums, activations sharded by token rows in between."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import voyager_b200
    from oracle import layers as OL

    W = voyager_b200.workloads
    shape, tokens, params, x, scales = tp_common.fp8_layer_problem()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(tp_common.run_rank_fp8_layer, args=(2, 29625, results), nprocs=2, join=True)
    got = results["out"]
    single = W.Fp8DecoderLayer({k: v.cuda() for k, v in params.items()}, {k: v.cuda() for k, v in scales.items()},
                               shape)(x.cuda()).cpu()
    # the same codes everywhere; the row-parallel sums differ in float32 summation order only
    err = (got.float() - single.float()).abs()
    assert float(err.max()) <= 2e-2 * float(single.float().abs().max())
    assert float((err > 0).float().mean()) < 0.05
    want = OL.fp8_decoder_layer(x, params, scales, shape, W.rope_tables(tokens, shape, "cpu"),
                                W.causal_mask(tokens, "cpu"))
    assert float((got.float() - want.float()).abs().max()) <= 2e-2 * float(want.float().abs().max())


def test_two_gpu_fp8_decoder_layer_over_peer_memory_equals_the_nccl_layer():
    """The same layer with its all-gathers and reduce-scatters as pulls over peer memory: the gathered codes are
    the same bytes and the float32 partial sums are added in rank order, as NCCL's two-rank reduction does."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    manager = mp.Manager()
    nccl, peer = manager.dict(), manager.dict()
    mp.spawn(tp_common.run_rank_fp8_layer, args=(2, 29631, nccl), nprocs=2, join=True)
    mp.spawn(tp_common.run_rank_fp8_layer, args=(2, 29633, peer, True), nprocs=2, join=True)
    a, b = nccl["out"].float(), peer["out"].float()
    assert float((a - b).abs().max()) <= 2e-2 * float(a.abs().max())
    assert float((a != b).float().mean()) < 0.02


def test_two_gpu_nvfp4_decoder_layer():
    """The NVFP4 layer sharded over two GPUs (packed codes and scale tiles gathered, amax all-reduced, float32
    partial products reduce-scattered) against the same layer on one GPU and against the CPU oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import voyager_b200
    from oracle import layers as OL

    W = voyager_b200.workloads
    shape, tokens, params, x = tp_common.nvfp4_layer_problem()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(tp_common.run_rank_nvfp4_layer, args=(2, 29629, results), nprocs=2, join=True)
    got = results["out"].float()
    single = W.Nvfp4DecoderLayer({k: v.cuda() for k, v in params.items()}, shape)(x.cuda()).float().cpu()
    # every weight code and global scale equals the single-GPU one; float32 summation order differs in the
    # row-parallel linears, and a 4-bit code that flips downstream moves a value by up to a third
    err = (got - single).abs()
    assert float(err.max()) <= 6e-2 * float(single.abs().max())
    assert float(err.pow(2).mean().sqrt() / single.pow(2).mean().sqrt()) <= 1e-2
    want = OL.nvfp4_decoder_layer(x, params, shape, W.rope_tables(tokens, shape, "cpu"), W.causal_mask(tokens, "cpu")).float()
    err = (got - want).abs()
    assert float(err.max()) <= 6e-2 * float(want.abs().max())
    assert float(err.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) <= 2e-2


def test_two_gpu_nvfp4_decoder_layer_over_peer_memory_equals_the_nccl_layer():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    manager = mp.Manager()
    nccl, peer = manager.dict(), manager.dict()
    mp.spawn(tp_common.run_rank_nvfp4_layer, args=(2, 29635, nccl), nprocs=2, join=True)
    mp.spawn(tp_common.run_rank_nvfp4_layer, args=(2, 29637, peer, True), nprocs=2, join=True)
    a, b = nccl["out"].float(), peer["out"].float()
    # the same gathered bytes; two-rank float32 sums in rank order either way
    assert float((a - b).abs().max()) <= 6e-2 * float(a.abs().max())
    assert float((a - b).pow(2).mean().sqrt() / a.pow(2).mean().sqrt()) <= 5e-3


def test_nvfp4_tensor_parallel_layer_on_one_rank_is_the_layer():
    """World size 1 (no process group): the sharding code paths with whole tensors give the single-GPU layer."""
    import voyager_b200

    W, P = voyager_b200.workloads, voyager_b200.parallel
    shape, tokens, params, x = tp_common.nvfp4_layer_problem()
    dev = {k: v.cuda() for k, v in params.items()}
    got = P.Nvfp4DecoderLayerTP(dev, shape)(x.cuda())
    want = W.Nvfp4DecoderLayer(dev, shape)(x.cuda())
    voyager_b200.ops.gemm_status()
    assert torch.equal(got, want)


def test_two_gpu_layer_parallel_gptq_with_the_device_solve():
    """Five GPTQ problems dealt to two GPUs by cost, each solved by the CUDA sweep on its owner, the
    compensated weights broadcast over NCCL (bfloat16 model weights, float32 on the wire)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import gptq as OG
    from oracle import tables as OT

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(tp_common.run_rank_gptq, args=(2, 29627, results), nprocs=2, join=True)
    (n0, out0), (n1, out1) = results[0], results[1]
    assert n0 + n1 == 5 and n0 >= 2 and n1 >= 2
    for a, b in zip(out0, out1):
        assert a.dtype == torch.bfloat16 and torch.equal(a, b)
    for got, p in zip(out0, tp_common.gptq_problems()):
        want = OG.compensate_weight(p["weight"].float(), p["hessian"], p["tokens"], OT.quantization_map("int4"),
                                    OT.quantization_map("fp8_e5m3"), 7.0, 32, 0.01, False, True, False)
        assert float((got.float() == want.bfloat16().float()).float().mean()) >= 0.99
