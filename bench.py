"""Benchmark of the quantized hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c2s|c1|c4|q1|r1]

One "step" is one pass of the hot path over one batch of synthetic input.

Workload ``c2`` (default; the configuration the headline metric is quoted on): one FP8 E4M3 per-tensor
quantized Llama-3.1-8B-shaped decoder layer, prefill of 1 x 2048 tokens,
random-init weights ~N(0,0.02); all seven linears run as FP8 casts + FP8 tensor-core
GEMMs, the causal attention as one fused FP8 kernel (``c2s``: as separate kernels), bf16 elsewhere.

Workload ``c1`` (the reference's own CPU-runnable case): X [2048,4096] bf16 ~N(0,1) with
0.1 % of entries x20, W [4096,4096] ~N(0,0.02); both are quantized to int8
microscaling (block 16 along K, power-of-two scales) and multiplied to
Y [2048,4096] bf16 -- ``quantize_mx`` x2 + ``linear_mx``.

Each step is replayed from a CUDA graph captured once per input set.  With
N > 1 (launched under torchrun, one rank per GPU) every rank processes its own
batches: the path shards by token rows with no exchange, so scaling is weak and
``value`` is the sum over ranks.  The timed region is K steps bracketed by a
barrier and a device synchronize; time is taken with CUDA events and the
maximum over ranks.  Successive steps use different input sets and the
tensors touched per step exceed the 126 MB L2 several times over, so no step
finds its inputs cached.

``--impl reference`` times the CPU oracle (a port of the reference's CPU
operators) on the host cores for the same workload, on a bounded sample.
"""

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# ncu-measured DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum, bytes per
# launch) of each workload's dominant kernel, from the captures summarised under
# profiles/; None until one has been taken.
NCU_TRAFFIC_BYTES = {"c1": 53.5e6, "c2": 145.2e6, "r1": 390.3e6}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while a region runs."""

    def __init__(self, index):
        self.index = index
        self.sm, self.max_sm, self.reasons = [], None, set()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _open(self):
        import pynvml as nv

        nv.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        index = self.index
        if visible:
            try:
                index = int(visible.split(",")[self.index])
            except ValueError:
                pass
        self._nv, self._handle = nv, nv.nvmlDeviceGetHandleByIndex(index)
        self.max_sm = nv.nvmlDeviceGetMaxClockInfo(self._handle, nv.NVML_CLOCK_SM)

    def _run(self):
        nv, h = self._nv, self._handle
        names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        try:
            while not self._stop.is_set():
                self.sm.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                self._stop.wait(0.004)
        except Exception as exc:  # NVML went away: report what we have
            self.error = repr(exc)

    def __enter__(self):
        try:
            self._open()          # NVML is up before the timed region starts, so short regions are sampled too
            self._thread.start()
        except Exception as exc:
            self.error = repr(exc)
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=10)

    def summary(self):
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.max_sm, "reasons": [], "samples": 0,
                    "note": getattr(self, "error", "no samples")}
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.max_sm, "reasons": sorted(self.reasons),
                "samples": len(sm)}


def time_region(fn, steps, barrier, finish=None):
    """Device time of ``steps`` calls of ``fn``.  ``finish()`` runs before the stop event is recorded
    (it makes the timing stream wait for work that ``fn`` queued on other streams)."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(steps):
        fn(i)
    if finish is not None:
        finish()
    stop.record()
    barrier()
    return start.elapsed_time(stop) * 1e-3


class HostPipeline:
    """End-to-end steps with host buffers: every step copies its input from pinned host memory,
    replays its graph and copies its result back to pinned host memory.  The three run on three
    streams chained by events, so the copy-in of step i+1 and the copy-out of step i-1 overlap the
    compute of step i (PCIe is full duplex); each step still waits for its own input and its result
    still reaches the host inside the timed region."""

    def __init__(self, device_inputs, host_inputs, graphs):
        self.dev_in, self.host_in, self.graphs = device_inputs, host_inputs, graphs
        self.host_out = [torch.empty(g[1].shape, dtype=g[1].dtype).pin_memory() for g in graphs]
        self.h2d, self.d2h = torch.cuda.Stream(), torch.cuda.Stream()
        n = len(graphs)
        self.in_ready = [torch.cuda.Event() for _ in range(n)]
        self.computed = [torch.cuda.Event() for _ in range(n)]
        self.out_copied = [torch.cuda.Event() for _ in range(n)]
        self.used = [False] * n

    def step(self, i):
        j = i % len(self.graphs)
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.h2d):
            if self.used[j]:
                self.h2d.wait_event(self.computed[j])      # the set's previous step has consumed its input
            else:
                self.h2d.wait_stream(main)
            self.dev_in[j].copy_(self.host_in[j], non_blocking=True)
            self.in_ready[j].record(self.h2d)
        main.wait_event(self.in_ready[j])
        if self.used[j]:
            main.wait_event(self.out_copied[j])            # the graph's output buffer has been read out
        self.graphs[j][0].replay()
        self.computed[j].record(main)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(self.computed[j])
            self.host_out[j].copy_(self.graphs[j][1], non_blocking=True)
            self.out_copied[j].record(self.d2h)
        self.used[j] = True

    def finish(self):
        torch.cuda.current_stream().wait_stream(self.d2h)


def capture(fn):
    """Capture ``fn()`` into a CUDA graph (after a warm-up call on a side stream);
    returns (graph, outputs)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fn()
    return graph, out


# ---------------------------------------------------------------------------
# workload c1: MXINT8 quantized linear
# ---------------------------------------------------------------------------
class C1:
    name = "c1"
    description = ("c1: MXINT8 (int8, bs=16, power-of-two scales) quantize_mx x2 + linear_mx, "
                   "X[2048,4096] W[4096,4096] per GPU")
    tokens = 2048
    K, N, BLOCK, QMAX = 4096, 4096, 16, 127.0
    launches_per_step = 5  # quantize_mx x2, operand read-back x2, tensor-core GEMM
    n_sets = 6
    dtype = "bf16"
    cpu_sample = "full c1 steps"
    cpu_tokens = 2048

    @staticmethod
    def inputs(seed, device="cpu"):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(C1.tokens, C1.K, generator=g)
        x = torch.where(torch.rand(C1.tokens, C1.K, generator=g) < 0.001, x * 20, x).bfloat16()
        w = (torch.randn(C1.N, C1.K, generator=g) * 0.02).bfloat16()
        return x.to(device), w.to(device)

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        self.Q = torch.ops.quantized_ops
        self.table = voyager_b200.get_quantization_map("int8", dev)
        self.sets = [self.inputs(1000 * rank + i, dev) for i in range(self.n_sets)]
        self.h2d_bytes = self.tokens * self.K * 2
        self.d2h_bytes = self.tokens * self.N * 2
        for x, w in self.sets[:2]:
            self._run(x, w)
        self.graphs = [capture(lambda x=x, w=w: self._run(x, w)) for x, w in self.sets]
        self.pipeline = HostPipeline([s[0] for s in self.sets], [s[0].cpu().pin_memory() for s in self.sets],
                                     self.graphs)

    def _run(self, x, w):
        Q = self.Q
        sx, cx = Q.quantize_mx(x, self.table, [-1], self.BLOCK, self.QMAX, True)
        sw, cw = Q.quantize_mx(w, self.table, [-1], self.BLOCK, self.QMAX, True)
        return Q.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=self.BLOCK)

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def roofline(self, peaks, reps):
        ops, Q = self.vb.ops, self.Q
        pairs = []
        for x, w in self.sets:
            sx, cx = Q.quantize_mx(x, self.table, [-1], self.BLOCK, self.QMAX, True)
            sw, cw = Q.quantize_mx(w, self.table, [-1], self.BLOCK, self.QMAX, True)
            pairs.append((ops._decode_and_scale(cx, sx, None, self.BLOCK), ops._decode_and_scale(cw, sw, None, self.BLOCK)))
        for a, b in pairs[:3]:
            ops.gemm_tn(a, b)
        secs = time_region(lambda i: ops.gemm_tn(*pairs[i % len(pairs)]), reps, torch.cuda.synchronize) / reps
        flops = 2.0 * self.tokens * self.N * self.K
        achieved = flops / secs / 1e12
        return secs, {"kernel": "gemm_tn_kernel (tcgen05 kind::f16 bf16, 2048x4096x4096)", "bound": "tensor",
                      "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                      "frac": achieved / peaks["bf16_tflops"],
                      "peak_source": f"{peaks['source']} bf16 cuBLAS burst", "traffic": NCU_TRAFFIC_BYTES["c1"]}

    @staticmethod
    def cpu_setup():
        from oracle import tables as OT

        x, w = C1.inputs(0)
        return x, w, OT.quantization_map("int8")

    @staticmethod
    def cpu_step(state):
        from oracle import gemm as OG
        from oracle import quantizers as OQ

        x, w, table = state
        sx, cx = OQ.quantize_mx(x, table, [-1], C1.BLOCK, C1.QMAX, True)
        sw, cw = OQ.quantize_mx(w, table, [-1], C1.BLOCK, C1.QMAX, True)
        return OG.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=C1.BLOCK)


# ---------------------------------------------------------------------------
# workload c2: FP8 per-tensor Llama-3.1-8B-shaped decoder layer, prefill 2048
# ---------------------------------------------------------------------------
class C2:
    name = "c2"
    description = ("c2: FP8 E4M3 per-tensor quantized Llama-3.1-8B-shaped decoder layer (hidden 4096, 32q/8kv heads "
                   "x128, SwiGLU 14336), prefill 1x2048 tokens per GPU, 7 linears as FP8 tensor-core GEMMs, causal "
                   "attention (QK^T, softmax, PV) as one fused FP8 tensor-core kernel")
    fuse_attention = True
    tokens = 2048
    n_sets = 4
    dtype = "fp8_e4m3 (fp32 accumulate), bf16 elsewhere"
    cpu_tokens = 256
    cpu_sample = "decoder-layer forwards of a 256-token prefill (1/8 of the GPU step's tokens)"

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        W = voyager_b200.workloads
        self.shape = W.LLAMA_8B
        params = W.make_layer_params(7 + rank, self.shape, dev)
        self.x = [W.make_hidden_states(100 * rank + i, self.tokens, self.shape, dev) for i in range(self.n_sets)]
        scales = W.calibrate_fp8_scales(self.x[0], params, self.shape)
        self.layer = W.Fp8DecoderLayer(params, scales, self.shape, fuse_attention=self.fuse_attention)
        del params
        self.launches_per_step = self.layer.LAUNCHES
        self.h2d_bytes = self.tokens * self.shape.hidden * 2
        self.d2h_bytes = self.tokens * self.shape.hidden * 2
        self.layer(self.x[0])
        self.graphs = [capture(lambda x=x: self.layer(x)) for x in self.x]
        self.pipeline = HostPipeline(self.x, [x.cpu().pin_memory() for x in self.x], self.graphs)

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def roofline(self, peaks, reps):
        # the dominant kernel is the FP8 GEMM; its largest launch is the merged gate/up projection
        # [2048,4096] x [2*14336,4096]^T with one scale per output column and the SwiGLU epilogue
        FP8 = self.vb.fp8
        sh, s = self.shape, self.layer.scales
        acts = [FP8.quantize_fp8(torch.nn.functional.rms_norm(x, (sh.hidden,)), s["h2"]) for x in self.x]
        w, cols = self.layer.w8_swiglu, self.layer.alpha_swiglu
        for a in acts[:3]:
            FP8.fp8_gemm(a, w, alpha_cols=cols, gated_scale=s["act"])
        secs = time_region(lambda i: FP8.fp8_gemm(acts[i % len(acts)], w, alpha_cols=cols, gated_scale=s["act"]), reps,
                           torch.cuda.synchronize) / reps
        flops = 2.0 * self.tokens * 2 * sh.intermediate * sh.hidden
        achieved = flops / secs / 1e12
        peak = 2.0 * peaks["bf16_tflops"]
        return secs, {"kernel": "gemm_tn_pair_kernel (tcgen05 kind::f8f6f4 e4m3, cta_group::2, 2048x28672x4096 merged gate/up projection, SwiGLU + FP8 cast epilogue)",
                      "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                      "peak_source": f"2 x {peaks['source']} bf16 cuBLAS burst (no FP8 peak was measured)",
                      "traffic": NCU_TRAFFIC_BYTES["c2"]}

    @staticmethod
    def cpu_setup():
        import voyager_b200  # host-side workload definitions only; no kernel runs on this path

        W = voyager_b200.workloads
        shape = W.LLAMA_8B
        params = W.make_layer_params(7, shape)
        x = W.make_hidden_states(100, C2.cpu_tokens, shape)
        scales = W.calibrate_fp8_scales(x, params, shape)
        return x, params, scales, shape, W.rope_tables(C2.cpu_tokens, shape, "cpu"), W.causal_mask(C2.cpu_tokens, "cpu")

    @staticmethod
    def cpu_step(state):
        from oracle import layers as OL

        return OL.fp8_decoder_layer(*state)


# ---------------------------------------------------------------------------
# workload q1: the MX quantizer alone on an activation larger than L2 (HBM roofline)
# ---------------------------------------------------------------------------

class C2Separate(C2):
    """The same layer with the attention run as separate kernels (QK^T GEMM, softmax + cast, PV GEMM, cast)."""
    name = "c2s"
    description = C2.description.replace("as one fused FP8 tensor-core kernel",
                                         "as separate kernels: FP8 GEMM, softmax + cast, FP8 GEMM, cast")
    fuse_attention = False


class Q1:
    name = "q1"
    description = ("q1: quantize_mx (int8, bs=16, power-of-two scales) of a [16384,4096] bfloat16 activation per GPU: "
                   "the C1 quantizer at 8x C1's rows, so that the kernel is HBM-bound rather than launch-bound")
    tokens = 16384
    K, BLOCK, QMAX = 4096, 16, 127.0
    launches_per_step = 1
    n_sets = 3
    dtype = "bf16"
    cpu_tokens = 2048
    cpu_sample = "quantize_mx calls on 2048 of the step's 16384 rows"

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        self.Q = torch.ops.quantized_ops
        self.table = voyager_b200.get_quantization_map("int8", dev)
        g = torch.Generator().manual_seed(77 + rank)
        self.x = [torch.randn(self.tokens, self.K, generator=g).bfloat16().to(dev) for _ in range(self.n_sets)]
        self.h2d_bytes = self.tokens * self.K * 2
        self.d2h_bytes = self.tokens * self.K * 2
        self._run(self.x[0])
        self.graphs = [capture(lambda x=x: self._run(x)) for x in self.x]
        self.pipeline = HostPipeline(self.x, [x.cpu().pin_memory() for x in self.x], self.graphs)

    def _run(self, x):
        return self.Q.quantize_mx(x, self.table, [-1], self.BLOCK, self.QMAX, True)[1]

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def roofline(self, peaks, reps):
        # the step's graphs hold this one kernel: replaying them times it without host launch gaps
        secs = time_region(self.step, reps, torch.cuda.synchronize) / reps
        nbytes = self.tokens * self.K * (2 + 2 + 2 / self.BLOCK)      # input + codes + one scale per block
        achieved = nbytes / secs / 1e9
        return secs, {"kernel": "mx_flat_bf16_kernel (quantize_mx int8, block 16, power-of-two scales, 16384x4096)",
                      "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                      "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth",
                      "traffic": None}

    @staticmethod
    def cpu_setup():
        from oracle import tables as OT

        g = torch.Generator().manual_seed(77)
        return torch.randn(Q1.cpu_tokens, Q1.K, generator=g).bfloat16(), OT.quantization_map("int8")

    @staticmethod
    def cpu_step(state):
        from oracle import quantizers as OQ

        x, table = state
        return OQ.quantize_mx(x, table, [-1], Q1.BLOCK, Q1.QMAX, True)


# ---------------------------------------------------------------------------
# workload r1: RMSNorm's backward of a training step (three gradients summed, residual added)
# ---------------------------------------------------------------------------
class R1:
    name = "r1"
    description = ("r1: voyager_gpu::rmsnorm_backward of [8192,4096] bfloat16 rows per GPU, three gradients summed "
                   "into dy and the input gradient added to the residual stream's")
    tokens = 8192
    K = 4096
    launches_per_step = 2
    n_sets = 2
    dtype = "bf16 (float32 sums)"
    cpu_tokens = 1024
    cpu_sample = "rmsnorm_backward calls on 1024 of the step's 8192 rows"

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        g = torch.Generator().manual_seed(91 + rank)
        make = lambda scale: (torch.randn(self.tokens, self.K, generator=g) * scale).bfloat16().to(dev)
        self.x = [make(1.5) for _ in range(self.n_sets)]
        self.grads = [[make(0.05) for _ in range(3)] for _ in range(self.n_sets)]
        self.residual = [make(0.05) for _ in range(self.n_sets)]
        self.rsqrt = [torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) for x in self.x]
        self.weight = (1.0 + 0.2 * torch.randn(self.K, generator=g)).bfloat16().to(dev)
        self.h2d_bytes = self.tokens * self.K * 2
        self.d2h_bytes = self.tokens * self.K * 2
        self._run(0)
        self.graphs = [capture(lambda i=i: self._run(i)) for i in range(self.n_sets)]
        # the host supplies the norm's input and takes the input gradient back
        self.pipeline = HostPipeline(self.x, [x.cpu().pin_memory() for x in self.x], self.graphs)

    def _run(self, i):
        return self.vb.training.rmsnorm_backward(self.grads[i], self.x[i], self.rsqrt[i], self.weight, self.residual[i])[0]

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def roofline(self, peaks, reps):
        secs = time_region(self.step, reps, torch.cuda.synchronize) / reps
        nbytes = self.tokens * self.K * 2 * (3 + 1 + 1 + 1)       # three gradients, x, residual in; dx out
        achieved = nbytes / secs / 1e9
        return secs, {"kernel": "rmsnorm_backward_kernel<2, 3, true> + rmsnorm_dw_sum_kernel (8192x4096)",
                      "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                      "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth",
                      "traffic": NCU_TRAFFIC_BYTES["r1"]}

    @staticmethod
    def cpu_setup():
        g = torch.Generator().manual_seed(91)
        make = lambda scale: (torch.randn(R1.cpu_tokens, R1.K, generator=g) * scale).bfloat16()
        x = make(1.5)
        return ([make(0.05) for _ in range(3)], x, torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5),
                (1.0 + 0.2 * torch.randn(R1.K, generator=g)).bfloat16(), make(0.05))

    @staticmethod
    def cpu_step(state):
        from oracle import training as OTR

        return OTR.rmsnorm_backward(*state)


# ---------------------------------------------------------------------------
# workload c4: one NVFP4 linear (fused cast to packed e2m1 + e4m3 block scales, block-scaled GEMM)
# ---------------------------------------------------------------------------
class C4:
    name = "c4"
    description = ("c4: NVFP4 (e2m1, bs=16, e4m3 block scales, bf16 global scale) linear of a Llama-3.1-8B-shaped "
                   "up projection: cast X[2048,4096] per step, packed W[14336,4096] resident, "
                   "kind::mxf4nvf4 block-scaled tensor-core GEMM")
    tokens = 2048
    K, N = 4096, 14336
    launches_per_step = 3   # amax of the activation, cast, GEMM
    n_sets = 4
    dtype = "fp4_e2m1 x fp8_e4m3 block scales (fp32 accumulate)"
    cpu_tokens = 256
    cpu_sample = "quantize_mx + linear_mx on 256 of the step's 2048 tokens (weight quantized once outside)"

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        NV = voyager_b200.nvfp4
        g = torch.Generator().manual_seed(40 + rank)
        w = (torch.randn(self.N, self.K, generator=g) * 0.02).bfloat16().to(dev)
        self.w_codes, self.w_scales, self.tw = NV.quantize_nvfp4(w)
        del w
        self.x = [torch.randn(self.tokens, self.K, generator=g).bfloat16().to(dev) for _ in range(self.n_sets)]
        self.one = torch.ones((), device=dev)
        self.h2d_bytes = self.tokens * self.K * 2
        self.d2h_bytes = self.tokens * self.N * 2
        self._run(self.x[0])
        self.graphs = [capture(lambda x=x: self._run(x)) for x in self.x]
        self.pipeline = HostPipeline(self.x, [x.cpu().pin_memory() for x in self.x], self.graphs)

    def _run(self, x):
        NV = self.vb.nvfp4
        codes, scales, t = NV.quantize_nvfp4(x)
        return NV.nvfp4_linear(codes, scales, self.w_codes, self.w_scales, (t * self.tw).float(), self.one, None)

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def roofline(self, peaks, reps):
        NV = self.vb.nvfp4
        packed = [NV.quantize_nvfp4(x) for x in self.x]
        alpha = [(t * self.tw).float() for _, _, t in packed]

        def gemm(i):
            codes, scales, _ = packed[i % len(packed)]
            return NV.nvfp4_linear(codes, scales, self.w_codes, self.w_scales, alpha[i % len(packed)], self.one, None)

        for i in range(3):
            gemm(i)
        secs = time_region(gemm, reps, torch.cuda.synchronize) / reps
        achieved = 2.0 * self.tokens * self.N * self.K / secs / 1e12
        peak = 4.0 * peaks["bf16_tflops"]
        return secs, {"kernel": "gemm_nvfp4_kernel (tcgen05 kind::mxf4nvf4.block_scale, 2048x14336x4096)",
                      "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                      "peak_source": f"4 x {peaks['source']} bf16 cuBLAS burst (no FP4 peak was measured)",
                      "traffic": None}

    @staticmethod
    def cpu_setup():
        from oracle import quantizers as OQ
        from oracle import tables as OT

        g = torch.Generator().manual_seed(40)
        w = (torch.randn(C4.N, C4.K, generator=g) * 0.02).bfloat16()
        x = torch.randn(C4.cpu_tokens, C4.K, generator=g).bfloat16()
        e2m1, e4m3 = OT.quantization_map("fp4_e2m1"), OT.quantization_map("fp8_e4m3")
        tw = OQ.calculate_global_scale(w, 6.0, 448.0)
        sw, cw = OQ.quantize_mx(w, e2m1, [-1], 16, 6.0, False, e4m3, None, None, tw)
        return x, cw, sw, tw, e2m1, e4m3

    @staticmethod
    def cpu_step(state):
        from oracle import gemm as OG
        from oracle import quantizers as OQ

        x, cw, sw, tw, e2m1, e4m3 = state
        t = OQ.calculate_global_scale(x, 6.0, 448.0)
        sx, cx = OQ.quantize_mx(x, e2m1, [-1], 16, 6.0, False, e4m3, None, None, t)
        return OG.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=16, alpha=t * tw)


WORKLOADS = {"c1": C1, "c2": C2, "c2s": C2Separate, "c4": C4, "q1": Q1, "r1": R1}


def time_cpu_baseline(workload, reps):
    """The CPU port of the reference operators on the host cores."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    state = workload.cpu_setup()
    workload.cpu_step(state)
    t0 = time.perf_counter()
    for _ in range(reps):
        workload.cpu_step(state)
    dt = (time.perf_counter() - t0) / reps
    return workload.cpu_tokens / dt, dt, cores


def run_reference(args, rank):
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    reps = max(1, min(args.steps, 5))
    value, dt, cores = time_cpu_baseline(wl, reps)
    sample = f"{reps} {wl.cpu_sample} after 1 warm-up"
    print(json.dumps({
        "impl": "reference", "metric": "tok/s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": reps,
        "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic", "config": {"workload": wl.description, "cpu_sample": sample},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    wl = WORKLOADS[args.workload](dev, rank)
    warmup = max(args.warmup, 3)
    for i in range(warmup):
        wl.step(i)
    wl.vb.ops.gemm_status()

    barrier()   # NCCL communicators come up here, not inside the sampled region
    with ClockSampler(local_rank) as clocks:
        elapsed = time_region(wl.step, args.steps, barrier)
    wl.vb.ops.gemm_status()

    for i in range(3):
        wl.e2e_step(i)
    e2e_elapsed = time_region(wl.e2e_step, args.steps, barrier, wl.pipeline.finish)

    peaks = measured_peaks()
    kernel_s, roof = wl.roofline(peaks, max(12, min(args.steps, 50)))

    times = torch.tensor([elapsed, e2e_elapsed], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed, e2e_elapsed = times.tolist()

    if rank == 0:
        tokens_total = wl.tokens * args.steps * world
        line = {
            "metric": "tok/s", "value": tokens_total / elapsed, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": wl.description,
                       "l2": f"{wl.n_sets} rotating input sets; tensors touched per step exceed the 126 MB L2",
                       "launch": "CUDA graph replay per step",
                       "e2e": "pinned host input copied in, graph replayed, result copied out to pinned host memory "
                              "every step; copies on their own streams overlap neighbouring steps' compute"},
            "e2e": {"value": tokens_total / e2e_elapsed, "unit": "tok/s", "h2d_bytes_per_step": wl.h2d_bytes,
                    "d2h_bytes_per_step": wl.d2h_bytes},
            "gpu_launches": wl.launches_per_step * args.steps,
            "roofline": roof,
            "clocks": clocks.summary(),
        }
        if world == 1:
            value, dt, cores = time_cpu_baseline(WORKLOADS[args.workload], 3)
            line["cpu_baseline"] = {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": f"3 {wl.cpu_sample} after 1 warm-up"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
