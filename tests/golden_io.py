"""Load the committed golden fixtures (see tests/golden/make_golden.py)."""

import json
import os

import numpy as np
import torch

import cases as C

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

_tables = None
_cases = None


def golden_tables():
    global _tables
    if _tables is None:
        with np.load(os.path.join(HERE, "tables.npz")) as z:
            _tables = {k: C.from_numpy(z[k], "bf16") for k in z.files}
    return _tables


def golden_cases(table):
    """``{name: (op, args, kwargs, expected_outputs)}`` with stored inputs
    substituted for the regenerated ones."""
    global _cases
    with np.load(os.path.join(HERE, "cases.npz")) as z:
        meta = json.loads(bytes(z["__meta__"]).decode())
        out = {}
        for name, op, args, kwargs in C.build_cases(table):
            m = meta[name]
            assert m["op"] == op
            for i, tag in enumerate(m["in"]):
                key = f"{name}/in{i}"
                if tag is not None and key in z.files:
                    stored = C.from_numpy(z[key], tag)
                    assert stored.shape == args[i].shape, (name, i)
                    args[i] = stored
            expected = [C.from_numpy(z[f"{name}/out{i}"], tag) for i, tag in enumerate(m["out"])]
            out[name] = (op, args, kwargs, expected)
    return out


def bits_equal(a, b):
    """Exact equality of two tensors' bit patterns (NaN payloads included;
    any NaN equals any NaN)."""
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.is_floating_point():
        both_nan = torch.isnan(a) & torch.isnan(b)
        if a.dtype == torch.bfloat16 or a.dtype == torch.float16:
            ia, ib = a.contiguous().view(torch.int16), b.contiguous().view(torch.int16)
        elif a.dtype == torch.float32:
            ia, ib = a.contiguous().view(torch.int32), b.contiguous().view(torch.int32)
        else:
            ia, ib = a.contiguous().view(torch.int64), b.contiguous().view(torch.int64)
        return bool(((ia == ib) | both_nan).all())
    return bool(torch.equal(a, b))


def describe_mismatch(a, b, limit=5):
    if a.shape != b.shape or a.dtype != b.dtype:
        return f"shape/dtype {tuple(a.shape)} {a.dtype} vs {tuple(b.shape)} {b.dtype}"
    af, bf = a.double().flatten(), b.double().flatten()
    bad = ~((af == bf) | (torch.isnan(af) & torch.isnan(bf)))
    idx = bad.nonzero().flatten()[:limit].tolist()
    return f"{int(bad.sum())} of {af.numel()} differ; first: " + ", ".join(
        f"[{i}] got {af[i].item()!r} want {bf[i].item()!r}" for i in idx)
