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
