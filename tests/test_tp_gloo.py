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
