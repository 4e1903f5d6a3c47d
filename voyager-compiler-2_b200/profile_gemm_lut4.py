"""The decode-step linear on a packed lookup-format weight, alone: 16 rows against a Llama-3.1-8B lm_head
(128256 x 4096, 279 MB packed), three launches.  The command the ncu summary under ``profiles/`` was taken from.

    python voyager-compiler-2_b200/profile_gemm_lut4.py
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import voyager_b200 as vb

    P = vb.packed
    dev = "cuda"
    levels = torch.tensor([-31, -22, -16, -12, -9, -6, -3, 0, 2, 5, 8, 10, 14, 17, 22, 31], dtype=torch.bfloat16, device=dev)
    m, n, k = 16, 128256, 4096
    g = torch.Generator(device=dev).manual_seed(0)
    codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=g)
    scale = (torch.rand(n, k // 64, device=dev, generator=g) * 0.01 + 0.001).bfloat16()
    weight = P.PackedLUT4Weight(codes, scale, levels, 64)
    x = torch.randint(0, 16, (m, k), device=dev, generator=g).bfloat16()
    sx = (torch.rand(m, k // 64, device=dev, generator=g) * 0.1 + 0.01).bfloat16()
    for _ in range(3):
        y = P.linear_lut4(x, weight, input_scale=sx, input_code=levels)
    torch.cuda.synchronize()
    print("ok", float(y.float().abs().max()))


if __name__ == "__main__":
    main()
