"""RMSNorm's backward: the oracle against vectors from the reference's own CPU code, and the
CUDA operator against both."""

import os

import numpy as np
import pytest
import torch

from oracle import training as oracle_training

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "rmsnorm_backward.npz")
CASES = ["one_grad", "two_grads_residual", "three_grads_residual", "three_grads"]


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16) if a.dtype == np.int16 else torch.from_numpy(a.copy())


def _load(name):
    z = np.load(GOLDEN)
    get = lambda key: _bf16(z[f"{name}/{key}"])
    grads = [get(f"grad{i}") for i in range(3) if f"{name}/grad{i}" in z]
    residual = get("residual") if f"{name}/residual" in z else None
    return grads, get("x"), get("rsqrt"), get("weight"), residual, get("dx"), get("dw")


@pytest.mark.parametrize("name", CASES)
def test_oracle_reproduces_the_reference_vectors(name):
    grads, x, rsqrt, weight, residual, dx, dw = _load(name)
    got_dx, got_dw = oracle_training.rmsnorm_backward(grads, x, rsqrt, weight, residual)
    assert torch.equal(got_dx.view(torch.int16), dx.view(torch.int16))
    assert torch.equal(got_dw.view(torch.int16), dw.view(torch.int16))


def _close(got, want, exact_fraction):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    # only the two sums add in another order: a value moves by a bfloat16 step at most now and then
    assert float(err.max()) <= 1e-2 * float(want.abs().max())
    assert float((err == 0).float().mean()) >= exact_fraction


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_kernel_matches_the_reference_vectors(name):
    import voyager_b200 as vb
    grads, x, rsqrt, weight, residual, dx, dw = _load(name)
    cuda = lambda t: None if t is None else t.cuda()
    got_dx, got_dw = vb.training.rmsnorm_backward([g.cuda() for g in grads], x.cuda(), rsqrt.cuda(), weight.cuda(),
                                                  cuda(residual))
    _close(got_dx, dx, 0.98)
    _close(got_dw, dw, 0.8)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,count,with_residual", [(2048, 4096, 3, True), (300, 1024, 1, False),
                                                          (77, 8192, 2, True), (5, 8, 1, False)])
def test_kernel_matches_the_oracle(rows, cols, count, with_residual):
    import voyager_b200 as vb
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * 1.5).bfloat16()
    weight = (1.0 + 0.2 * torch.randn(cols, generator=g)).bfloat16()
    grads = [(torch.randn(rows, cols, generator=g) * 0.05).bfloat16() for _ in range(count)]
    residual = (torch.randn(rows, cols, generator=g) * 0.05).bfloat16() if with_residual else None
    rsqrt = torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    want_dx, want_dw = oracle_training.rmsnorm_backward(grads, x, rsqrt, weight, residual)
    got_dx, got_dw = torch.ops.voyager_gpu.rmsnorm_backward([t.cuda() for t in grads], x.cuda(), rsqrt.cuda(),
                                                            weight.cuda(), None if residual is None else residual.cuda())
    _close(got_dx, want_dx, 0.98)
    _close(got_dw, want_dw, 0.5)


@pytest.mark.gpu
def test_kernel_refuses_what_it_cannot_run():
    import voyager_b200 as vb
    x = torch.randn(4, 12).bfloat16().cuda()                      # 12 columns: not a multiple of 8
    r = torch.ones(4, 1).cuda()
    with pytest.raises(NotImplementedError):
        vb.training.rmsnorm_backward([x], x, r, torch.ones(12).bfloat16().cuda(), None)
