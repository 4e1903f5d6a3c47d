"""The fused causal attention on bfloat16 operands, alone: 32 query heads over 8 KV heads, 2048 tokens, head_dim 128
(a quarter of workload c4m's sequence, so that a profiler's replays stay short), three launches.  The command
the ncu summary under ``profiles/`` was taken from.

    python voyager-compiler-2_b200/profile_attention_bf16.py
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import voyager_b200 as vb

    T = 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(T, 32, 128, generator=g, device="cuda").bfloat16()
    k = torch.randn(T, 8, 128, generator=g, device="cuda").bfloat16()
    v = torch.randn(T, 8, 128, generator=g, device="cuda").bfloat16()
    for _ in range(3):
        y = vb.fp8.attention_bf16(q, k, v)
    torch.cuda.synchronize()
    assert vb.fp8.attention_status() == 0
    print("ok", float(y.float().abs().max()))


if __name__ == "__main__":
    main()
