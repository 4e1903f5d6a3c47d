"""One decode step of one MXNF4 decoder layer over a KIVI cache (the unit of bench workload c3), run three
times: the command the launch list under ``profiles/`` was taken from.

    python voyager-compiler-2_b200/profile_c3_layer.py
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import bench
    import voyager_b200 as vb

    W, P = vb.workloads, vb.packed
    dev = torch.device("cuda")
    shape = W.LLAMA_8B
    t = W.nf4_tables(dev)
    weights, cache = bench.C3.layer_state(700, shape, t, dev, bench.C3.batch, bench.C3.cached, bench.C3.recent)
    packed = {n: P.pack_lut4_weight(*weights[n], t["levels"], 64, check=False) for n in ("qkv", "o", "gate_up", "down")}
    packed["ln1"], packed["ln2"] = weights["ln1"], weights["ln2"]
    scale = torch.tensor(8.0 / 448.0, dtype=torch.bfloat16, device=dev)
    layer = W.Mxnf4DecodeLayer(packed, t, cache, scale, shape)
    x = W.make_hidden_states(800, bench.C3.batch, shape, dev)
    cos, sin = W.rope_tables(bench.C3.cached, shape, dev)
    rope = (cos[-1].contiguous(), sin[-1].contiguous())
    for _ in range(3):
        y = layer(x, rope)
    torch.cuda.synchronize()
    print("ok", float(y.float().abs().max()))


if __name__ == "__main__":
    main()
