"""Generate ``rmsnorm_backward.npz``: inputs and outputs of the reference's ``rmsnorm_backward``
(``src/voyager_compiler/backend/gpu/rmsnorm.py:190-238``) run on CPU, where it takes its
decomposed-backward path.  Run in the build container, in a process of its own:

    VOYAGER_REFERENCE_ROOT=<checkout> python tests/golden/make_rmsnorm_backward.py
"""

import importlib.util
import os
import sys
import types

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import reference_shim as rs  # noqa: E402

CASES = [  # name, rows shape, cols, gradients, residual
    ("one_grad", (6,), 64, 1, False),
    ("two_grads_residual", (2, 5), 128, 2, True),
    ("three_grads_residual", (9,), 256, 3, True),
    ("three_grads", (3, 4), 72, 3, False),
]


def load_reference():
    rs._install_shims()
    root = os.path.join(rs._SRC, "voyager_compiler", "backend")
    for name, path in (("voyager_compiler.backend", root), ("voyager_compiler.backend.gpu", os.path.join(root, "gpu"))):
        module = types.ModuleType(name)
        module.__path__ = [path]
        sys.modules[name] = module
    spec = importlib.util.spec_from_file_location("voyager_compiler.backend.gpu.rmsnorm",
                                                  os.path.join(root, "gpu", "rmsnorm.py"))
    module = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = module
    spec.loader.exec_module(module)
    return module


def bits(t):
    return t.contiguous().view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def main():
    ref = load_reference()
    out = {}
    for index, (name, lead, cols, count, with_residual) in enumerate(CASES):
        g = torch.Generator().manual_seed(1000 + index)
        shape = (*lead, cols)
        x = (torch.randn(shape, generator=g) * 1.5).bfloat16()
        weight = (1.0 + 0.2 * torch.randn(cols, generator=g)).bfloat16()
        grads = [(torch.randn(shape, generator=g) * 0.05).bfloat16() for _ in range(count)]
        residual = (torch.randn(shape, generator=g) * 0.05).bfloat16() if with_residual else None
        rsqrt = torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)
        dx, dw = ref.rmsnorm_backward(grads, x, rsqrt, weight, residual)
        out[f"{name}/x"] = bits(x)
        out[f"{name}/weight"] = bits(weight)
        out[f"{name}/rsqrt"] = rsqrt.numpy()
        for i, grad in enumerate(grads):
            out[f"{name}/grad{i}"] = bits(grad)
        if residual is not None:
            out[f"{name}/residual"] = bits(residual)
        out[f"{name}/dx"] = bits(dx)
        out[f"{name}/dw"] = bits(dw)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rmsnorm_backward.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, len(out), "arrays")


if __name__ == "__main__":
    main()
