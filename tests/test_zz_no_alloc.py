"""The allocation-free GPTQ block step against the two-call path.

``vq_gptq_block_step_static`` exists for hosts that cannot allocate device memory
while they run (a runtime confined to a pre-planned arena, a plugin in a process
that forbids cudaMalloc after start-up): it keeps the per-column errors in an
array inside the library instead of a caller's buffer.  Here it is called
straight through the C ABI on two consecutive blocks of one weight -- the second
call reuses the array with the first call's contents still in it -- and both the
grid values and the compensated remainder must equal, bit for bit, what
``vq_gptq_block`` + ``vq_gptq_update`` produce with an ordinary buffer.  Sizes
beyond the built-in array must be refused with a clear message.

The file sorts last so that a run stopping at the first failure has already run
every other test; it also passes when run alone in a fresh process.
"""

import math

import pytest
import torch

from oracle import gptq as OG
from oracle import tables as OT

pytestmark = pytest.mark.gpu


def test_static_block_step_matches_buffered_path_twice():
    import voyager_b200

    N, R = voyager_b200._native, voyager_b200.rounding
    lib = N.lib()
    g = torch.Generator().manual_seed(11)
    rows, K, bs, tokens = 300, 192, 64, 1024
    x = 0.7 * torch.randn(tokens, K, generator=g) + 0.3 * (
        torch.randn(tokens, 8, generator=g) @ torch.randn(8, K, generator=g)) / math.sqrt(8)
    w = torch.randn(rows, K, generator=g) * 0.02
    U = OG.hessian_inverse_chol((x.T @ x).clone(), tokens, 0.01).cuda().contiguous()
    qmap = R.table_round(OT.quantization_map("lut4_to_int6").cuda())
    smap = R.table_round(OT.quantization_map("fp8_e5m3").cuda())
    stream = torch.cuda.current_stream().cuda_stream

    work_a, work_b = w.cuda().clone(), w.cuda().clone()
    out_a, out_b = torch.zeros_like(work_a), torch.zeros_like(work_b)
    deltas = torch.empty(rows, bs, dtype=torch.float32, device="cuda")
    for start in (0, bs):  # two calls in a row; the second finds the first call's errors in the array
        N.check(lib.vq_gptq_block(work_a.data_ptr(), out_a.data_ptr(), deltas.data_ptr(), U.data_ptr(), None, rows, K,
                                  start, bs, 0, 0.0, 31.0, 0, smap.ref, qmap.ref, stream), "vq_gptq_block")
        N.check(lib.vq_gptq_update(work_a.data_ptr(), deltas.data_ptr(), U.data_ptr(), rows, K, start, bs, stream),
                "vq_gptq_update")
        N.check(lib.vq_gptq_block_step_static(work_b.data_ptr(), out_b.data_ptr(), U.data_ptr(), None, rows, K, start,
                                              bs, 0, 0.0, 31.0, 0, smap.ref, qmap.ref, stream),
                "vq_gptq_block_step_static")
        torch.cuda.synchronize()
        assert torch.equal(out_a.view(torch.int32), out_b.view(torch.int32)), f"grid values differ at block {start}"
        assert torch.equal(work_a.view(torch.int32), work_b.view(torch.int32)), f"remainder differs at block {start}"
    assert float(out_b[:, : 2 * bs].abs().max()) > 0  # the step really wrote grid values

    # a request larger than the built-in array is refused, and says why
    rc = lib.vq_gptq_block_step_static(work_b.data_ptr(), out_b.data_ptr(), U.data_ptr(), None, 1 << 20, K, 0, bs, 0,
                                       0.0, 31.0, 0, smap.ref, qmap.ref, stream)
    assert rc == -1
    assert b"exceeds the built-in buffer" in lib.vq_last_error()
