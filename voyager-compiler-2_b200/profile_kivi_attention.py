"""The decode-step attention over a packed KIVI cache, alone: batch 16, 8 KV heads x 4 query heads, 3968 cached
+ 128 recent positions (the shape of bench workload c3), three launches.  The command the ncu summary under
``profiles/`` was taken from.

    python voyager-compiler-2_b200/profile_kivi_attention.py
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import voyager_b200 as vb

    dev = "cuda"
    B, hkv, G, Tm, R, d = 16, 8, 4, 3968, 128, 128
    g = torch.Generator(device=dev).manual_seed(0)
    uint2, e4m3 = vb.get_quantization_map("uint2").to(dev), vb.get_quantization_map("fp8_e4m3").to(dev)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev).bfloat16()
    keys = vb.kivi.quantize_cache(rnd(B, hkv, Tm, d), uint2, -2, 64, 2, e4m3)
    values = vb.kivi.quantize_cache(rnd(B, hkv, Tm, d), uint2, -1, 64, 2, e4m3)
    q, k_res, v_res = rnd(B, hkv, G, d), rnd(B, hkv, R, d), rnd(B, hkv, R, d)
    for _ in range(3):
        y = vb.kivi.decode_attention(q, keys, values, k_res, v_res)
    torch.cuda.synchronize()
    print("ok", float(y.float().abs().max()))


if __name__ == "__main__":
    main()
