"""Generate the golden fixtures from the reference's own CPU code.

Run where a checkout of the reference is available, naming it in the environment::

    VOYAGER_REFERENCE_ROOT=<checkout> python tests/golden/make_golden.py

Writes, next to this script:

* ``tables.npz``  -- the reference's 65 536-entry lookup table for every dtype
  in ``TABLE_DTYPES`` (bfloat16 bit patterns as uint16);
* ``cases.npz``   -- for every case of ``cases.build_cases`` the inputs and the
  reference's outputs.

The reference is imported through ``reference_shim`` (no reference file is
edited or copied).  The test-suite then checks the oracle and the CUDA
kernels against these files, so nothing at test time needs the checkout.
"""

import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import cases as C  # noqa: E402
import reference_shim  # noqa: E402

TABLE_DTYPES = [
    "int8", "int6", "int4", "int3", "int2", "uint8", "uint4", "uint2", "int16",
    "fp8_e4m3", "fp8_e5m2", "fp8_e5m3", "fp8_e8m0", "fp8_e4m3_ieee", "fp6_e3m2", "fp6_e2m3",
    "fp4_e2m1", "fp4_e3m0", "fp16_e5m10",
    "posit8_0", "posit8_1", "posit8_2", "posit6_1", "posit4_1", "posit16_1",
    "lut4_to_int6", "lut4", "lut3_to_int6", "lut4_to_fp8_e4m3", "lut2",
]


class ReferenceImpl:
    """The reference's functions under the names ``cases.run_case`` uses."""

    def __init__(self):
        ref = reference_shim.load()
        q = ref.quantized
        self.fq = ref.fake_quantize
        self.gptq = ref.gptq
        for name in ("vmap", "quantize", "dequantize", "calculate_mx_qparam", "quantize_mx", "dequantize_mx",
                     "quantize_affine", "linear_mx", "matmul_mx", "sdpa_mx", "hadamard_rotate",
                     "quantize_mx_transpose", "filter_outlier", "quantize_mx_outlier", "slice_csr_tensor", "spmm_csr"):
            setattr(self, name, getattr(q, name))
        import importlib

        fake_quant_ops = importlib.import_module("voyager_compiler.quantization.ops")
        for name in ("fake_quant", "group_wise_affine_fake_quant", "mx_fake_quant", "hadamard_amax"):
            setattr(self, name, getattr(fake_quant_ops, name))
        self.calculate_global_scale = self.fq.calculate_global_scale
        self.hadamard_matrix = self.fq.hadamard_matrix
        self.dense_linear = torch.nn.functional.linear

    def table(self, name):
        return self.fq.get_quantization_map(name)

    def amax_observer(self, sequence, dtype, quant_max, history_len, ch_axis, power_2_scale):
        """Feed ``sequence[i]`` through one FusedAmaxObsFakeQuantize; outputs and scales after each call."""
        Q = self.fq.QScheme
        scheme = Q.PER_TENSOR_SYMMETRIC if ch_axis is None else Q.PER_CHANNEL_SYMMETRIC
        module = self.fq.FusedAmaxObsFakeQuantize(dtype, scheme, quant_max, history_len, ch_axis, power_2_scale)
        outs, scales = [], []
        for x in sequence:
            outs.append(module(x))
            scales.append(module.scale.clone())
        return torch.stack(outs), torch.stack(scales)

    def compensate_weight(self, w, h, tokens, qmap, scale_qmap, qmax, bs, damping, act_order, within_block, shrink):
        fake_quant = types.SimpleNamespace(block_size=bs, ch_axis=-1, qmap=qmap, scale_qmap=scale_qmap,
                                           quant_max=qmax)
        return self.gptq.compensate_weight(w, h, tokens, fake_quant, damping, act_order, within_block, shrink)


def main():
    torch.manual_seed(0)
    impl = ReferenceImpl()

    tables = {}
    for name in TABLE_DTYPES:
        tables[name] = C.to_numpy(impl.table(name))[0]
    np.savez_compressed(os.path.join(HERE, "tables.npz"), **tables)

    arrays, meta = {}, {}
    for name, op, args, kwargs in C.build_cases(impl.table):
        outs = C.run_case(impl, op, args, kwargs)
        tags = []
        for i, t in enumerate(outs):
            arrays[f"{name}/out{i}"], tag = C.to_numpy(t)
            tags.append(tag)
        in_tags = []
        for i, a in enumerate(args):
            # Lookup tables are rebuilt from their dtype name, not stored per case.
            if isinstance(a, torch.Tensor) and not (a.dim() == 1 and a.numel() == 65536):
                arrays[f"{name}/in{i}"], tag = C.to_numpy(a)
                in_tags.append(tag)
            else:
                in_tags.append(None)
        meta[name] = {"op": op, "out": tags, "in": in_tags}
        print(f"{name:36s} {op:22s} -> {[tuple(t.shape) for t in outs]}")
    arrays["__meta__"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "cases.npz"), **arrays)
    for f in ("tables.npz", "cases.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
