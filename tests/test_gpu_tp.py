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
