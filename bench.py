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

Beside the timed region the line carries: ``self_check`` (the GPU path run on the
CPU leg's own inputs and compared with the CPU leg's output, plus workload-specific
comparisons; a failed check makes the process exit non-zero), ``gpu_reference``
(library kernels -- ``torch._scaled_mm``, cuBLAS ``torch.matmul``, ``F.scaled_mm`` --
timed on the workload's GEMM shapes in the same process: a baseline, never the product
path), and, for the default workload, ``secondary``: the quantizer (``q1``), the MXINT8
linear (``c1``) and the NVFP4 linear (``c4``) measured after the main region.
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


# Library FP8 / FP4 GEMM throughput measured in this process (``gpu_reference``); the roofline peak
# of the FP8 / FP4 kernels when present, else a multiple of the measured bf16 figure.
MEASURED_LIBRARY = {}


def fp8_peak(peaks):
    if MEASURED_LIBRARY.get("fp8"):
        return MEASURED_LIBRARY["fp8"], "best torch._scaled_mm FP8 GEMM over this layer's shapes, measured in this run"
    return 2.0 * peaks["bf16_tflops"], f"2 x {peaks['source']} bf16 cuBLAS burst (no FP8 library GEMM could be timed)"


def fp4_peak(peaks):
    if MEASURED_LIBRARY.get("fp4"):
        return MEASURED_LIBRARY["fp4"], "torch scaled_mm NVFP4 GEMM on this shape, measured in this run"
    return 4.0 * peaks["bf16_tflops"], f"4 x {peaks['source']} bf16 cuBLAS burst (no FP4 library GEMM could be timed)"


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


def max_rel(got, want):
    """Largest absolute difference over the largest magnitude of ``want`` (both moved to the CPU)."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def time_library(fn, n_sets, reps=40):
    """Seconds per call of a library kernel, rotating over ``n_sets`` operand sets (beyond L2 together)."""
    for i in range(3):
        fn(i % n_sets)
    return time_region(lambda i: fn(i % n_sets), reps, torch.cuda.synchronize) / reps


def fp8_library_gemms(shapes, ours, n_sets=3):
    """``torch._scaled_mm`` (cuBLASLt FP8, one float32 scale per operand, bfloat16 out) and this
    package's FP8 GEMM on the same ``[M, N, K]`` shapes and the same packed operands."""
    rows = []
    one = torch.ones((), device="cuda")
    for m, n, k in shapes:
        a = [torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn) for _ in range(n_sets)]
        b = [torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn) for _ in range(n_sets)]
        row = {"mnk": [m, n, k]}
        try:
            t = time_library(lambda i: torch._scaled_mm(a[i], b[i].t(), scale_a=one, scale_b=one,
                                                        out_dtype=torch.bfloat16), n_sets)
            row["library_tflops"] = 2.0 * m * n * k / t / 1e12
        except Exception as exc:  # the library has no kernel for this shape or build
            row["library_tflops"] = None
            row["library_error"] = repr(exc)[:160]
        au, bu = [x.view(torch.uint8) for x in a], [x.view(torch.uint8) for x in b]
        t = time_library(lambda i: ours(au[i], bu[i], one), n_sets)
        row["ours_tflops"] = 2.0 * m * n * k / t / 1e12
        rows.append(row)
        del a, b, au, bu
    best = max([r["library_tflops"] for r in rows if r.get("library_tflops")] or [None], key=lambda v: v or 0)
    return {"library": "torch._scaled_mm (cuBLASLt FP8 e4m3, tensor-wise scales, bf16 out), same process",
            "shapes": rows, "best_library_tflops": best}


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
        return secs, {"kernel": "gemm_tn_pair_kernel (tcgen05 kind::f16 bf16, cta_group::2, 2048x4096x4096)", "bound": "tensor",
                      "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                      "frac": achieved / peaks["bf16_tflops"],
                      "peak_source": f"{peaks['source']} bf16 cuBLAS burst", "traffic": NCU_TRAFFIC_BYTES["c1"]}

    def gpu_reference(self):
        """cuBLAS bf16 (``torch.matmul``) on the C1 GEMM shape beside this package's bf16 GEMM."""
        m, n, k, sets = self.tokens, self.N, self.K, 6
        a = [torch.randn(m, k, device="cuda").bfloat16() for _ in range(sets)]
        b = [torch.randn(n, k, device="cuda").bfloat16() for _ in range(sets)]
        lib = time_library(lambda i: torch.matmul(a[i], b[i].t()), sets)
        ours = time_library(lambda i: self.vb.ops.gemm_tn(a[i], b[i]), sets)
        fl = 2.0 * m * n * k / 1e12
        return {"library": "torch.matmul bf16 (cuBLAS), same process", "shapes": [
            {"mnk": [m, n, k], "library_tflops": fl / lib, "ours_tflops": fl / ours}], "best_library_tflops": fl / lib}

    def gpu_check(self, state, cpu_out):
        x, w, _ = state
        return {"linear_mx_vs_cpu_oracle": (max_rel(self._run(x.cuda(), w.cuda()), cpu_out), 1e-2)}

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
    cpu_tokens = 2048
    cpu_sample = "decoder-layer forwards of the same 2048-token prefill"
    GEMM_SHAPES = [(2048, 6144, 4096), (2048, 4096, 4096), (2048, 28672, 4096), (2048, 4096, 14336)]

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        W = voyager_b200.workloads
        self.shape = W.LLAMA_8B
        params = W.make_layer_params(7 + rank, self.shape, dev)
        self.x = [W.make_hidden_states(1000 * rank + 100 + i, self.tokens, self.shape, dev) for i in range(self.n_sets)]
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
        peak, source = fp8_peak(peaks)
        return secs, {"kernel": "gemm_tn_pair_kernel (tcgen05 kind::f8f6f4 e4m3, cta_group::2, 2048x28672x4096 merged gate/up projection, SwiGLU + FP8 cast epilogue)",
                      "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                      "peak_source": source, "traffic": NCU_TRAFFIC_BYTES["c2"]}

    def gpu_reference(self):
        """``torch._scaled_mm`` on the layer's four GEMM shapes beside this package's FP8 GEMM."""
        return fp8_library_gemms(self.GEMM_SHAPES, lambda a, b, one: self.vb.fp8.fp8_gemm(a, b, one))

    def self_check(self):
        """One graph replay against the same layer run kernel by kernel with torch producers."""
        self.graphs[0][0].replay()
        fused = self.graphs[0][1].clone()
        # torch's rsqrt / exp producers differ from the fused kernels' in the last bit on a few elements; the FP8
        # re-quantizations downstream turn that into the same few-percent tail as against the CPU oracle
        return {"graph_replay_vs_unfused_kernels": (max_rel(fused, self.layer.forward_unfused(self.x[0])), 6e-2)}

    def gpu_check(self, state, cpu_out):
        """The CPU leg's layer (its weights, scales and input) on the GPU kernels against the CPU leg's output."""
        x, params, scales, shape, _, _ = state
        W = self.vb.workloads
        layer = W.Fp8DecoderLayer({k: v.cuda() for k, v in params.items()}, {k: v.cuda() for k, v in scales.items()},
                                  shape, fuse_attention=self.fuse_attention)
        got = layer(x.cuda()).double().cpu()
        want = cpu_out.double()
        rms = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
        # kernel by kernel the layer reproduces the converted graph to summation order (tests/); end to end that
        # noise passes five FP8 re-quantizations, each flipped code moving a value by up to 1/8
        return {"layer_vs_cpu_oracle_max": (max_rel(got, want), 6e-2), "layer_vs_cpu_oracle_rms": (rms, 2e-2)}

    @staticmethod
    def cpu_setup():
        import voyager_b200  # host-side workload definitions only; no kernel runs on this path

        W = voyager_b200.workloads
        shape = W.LLAMA_8B
        params = W.make_layer_params(7, shape)
        x = W.make_hidden_states(100, C2.cpu_tokens, shape)   # rank 0's first input set
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

    def gpu_check(self, state, cpu_out):
        """Codes and scales are compared bit for bit: the figure is the fraction of differing values."""
        x, _ = state
        scale, codes = self.Q.quantize_mx(x.cuda(), self.table, [-1], self.BLOCK, self.QMAX, True)
        want_scale, want_codes = cpu_out
        bad = (codes.cpu().view(torch.int16) != want_codes.view(torch.int16)).float().mean() + \
            (scale.cpu().view(torch.int16) != want_scale.view(torch.int16)).float().mean()
        return {"codes_and_scales_differing_from_cpu_oracle": (float(bad), 0.0)}

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

    def gpu_check(self, state, cpu_out):
        grads, x, rsqrt, weight, residual = state
        dx, dw = self.vb.training.rmsnorm_backward([t.cuda() for t in grads], x.cuda(), rsqrt.cuda(), weight.cuda(),
                                                   residual.cuda())
        return {"dx_vs_cpu_oracle": (max_rel(dx, cpu_out[0]), 2e-2), "dw_vs_cpu_oracle": (max_rel(dw, cpu_out[1]), 2e-2)}

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
        peak, source = fp4_peak(peaks)
        return secs, {"kernel": "gemm_nvfp4_kernel (tcgen05 kind::mxf4nvf4.block_scale, 2048x14336x4096)",
                      "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                      "peak_source": source, "traffic": None}

    def gpu_reference(self):
        """The library's block-scaled NVFP4 GEMM (``torch.nn.functional.scaled_mm``, the call the reference's
        ``nvfp4_linear`` makes) on this shape and these packed operands, beside this package's kernel."""
        import torch.nn.functional as F

        NV = self.vb.nvfp4
        packed = [NV.quantize_nvfp4(x) for x in self.x]
        alpha = [(t * self.tw).float() for _, _, t in packed]
        fl = 2.0 * self.tokens * self.N * self.K / 1e12
        ours = time_library(lambda i: NV.nvfp4_linear(packed[i][0], packed[i][1], self.w_codes, self.w_scales,
                                                      alpha[i], self.one, None), len(packed))
        row = {"mnk": [self.tokens, self.N, self.K], "ours_tflops": fl / ours, "library_tflops": None}
        try:
            from torch.nn.functional import ScalingType, SwizzleType

            b4 = self.w_codes.view(torch.float4_e2m1fn_x2).t()
            sb = self.w_scales.reshape(-1).view(torch.float8_e4m3fn)
            block, tensor = ScalingType.BlockWise1x16, ScalingType.TensorWise
            swz, none = SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE

            def lib(i):
                codes, scales, _ = packed[i]
                return F.scaled_mm(codes.view(torch.float4_e2m1fn_x2), b4,
                                   [scales.reshape(-1).view(torch.float8_e4m3fn), alpha[i]], [block, tensor],
                                   [sb, self.one], [block, tensor], swizzle_a=[swz, none], swizzle_b=[swz, none],
                                   output_dtype=torch.bfloat16)

            row["library_vs_ours_max_rel"] = max_rel(lib(0), NV.nvfp4_linear(packed[0][0], packed[0][1], self.w_codes,
                                                                             self.w_scales, alpha[0], self.one, None))
            row["library_tflops"] = fl / time_library(lib, len(packed))
        except Exception as exc:  # this torch build has no block-scaled FP4 GEMM
            row["library_error"] = repr(exc)[:160]
        return {"library": "torch.nn.functional.scaled_mm NVFP4 (BlockWise1x16 e4m3 scales + tensor-wise alpha), same process",
                "shapes": [row], "best_library_tflops": row["library_tflops"]}

    def gpu_check(self, state, cpu_out):
        x = state[0]
        return {"nvfp4_linear_vs_cpu_oracle": (max_rel(self._run_with(x.cuda(), state), cpu_out), 1e-2)}

    def _run_with(self, x, state):
        """The CPU leg's weight (its codes, scales and global scale) packed for the GPU kernel."""
        NV = self.vb.nvfp4
        _, cw, sw, tw, _, _ = state
        w = NV.pack_nvfp4(cw.cuda(), sw.cuda())
        codes, scales, t = NV.quantize_nvfp4(x)
        return NV.nvfp4_linear(codes, scales, w.codes, w.scales, (t * tw.cuda()).float(), self.one, None)

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


# ---------------------------------------------------------------------------
# workload c4m: NVFP4 prefill of a full 32-layer Llama-3.1-8B-shaped model, 1 x 8192 tokens
# ---------------------------------------------------------------------------
class C4Model:
    name = "c4m"
    description = ("c4m: NVFP4 (e2m1, bs=16, e4m3 block scales, bf16 global scale on activations and weights) prefill of a "
                   "full 32-layer Llama-3.1-8B-shaped model, 1 x 8192 tokens per GPU: 7 linears per layer as fused casts "
                   "+ kind::mxf4nvf4 block-scaled tensor-core GEMMs (q/k/v and gate/up merged), the graph's bf16 causal attention "
                   "as one tcgen05 kernel with its roundings, bf16 RMSNorm / RoPE / SwiGLU as torch operators, final norm + "
                   "NVFP4 lm_head on the last position")
    tokens = 8192
    layers = 32
    n_sets = 2
    dtype = "fp4_e2m1 x fp8_e4m3 block scales (fp32 accumulate), bf16 elsewhere"
    cpu_tokens = 64           # 2048 tokens through one of 32 layers
    cpu_rows = 2048
    cpu_sample = ("forwards of ONE decoder layer on 2048 tokens, a quarter of the prefill (the model is 32 such layers: "
                  "tok/s = 2048 / (32 x layer time); the eager attention of 8192 tokens needs 13 GB of host scores)")

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        W = voyager_b200.workloads
        self.shape = W.LLAMA_8B
        self.model = W.Nvfp4Model(self.layers, self.shape, dev, seed=50 + 100 * rank)
        self.x = [W.make_hidden_states(300 + 10 * rank + i, self.tokens, self.shape, dev) for i in range(self.n_sets)]
        self.launches_per_step = self.model.LAUNCHES
        self.h2d_bytes = self.tokens * self.shape.hidden * 2
        self.d2h_bytes = self.shape.vocab * 2
        self.model(self.x[0])
        self.graphs = [capture(lambda x=x: self.model(x)) for x in self.x]
        self.pipeline = HostPipeline(self.x, [x.cpu().pin_memory() for x in self.x], self.graphs)

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def roofline(self, peaks, reps):
        """The dominant kernel: the NVFP4 GEMM of the merged gate/up projection, 8192 x 28672 x 4096."""
        NV = self.vb.nvfp4
        layer = self.model.layers[0]
        acts = [torch.randn(self.tokens, self.shape.hidden, device="cuda").bfloat16() for _ in range(2)]
        packed = [NV.quantize_nvfp4(a) for a in acts]
        wc, ws, tw = layer.merged["gate_up"]
        cols = [(t * tw).float() for _, _, t in packed]
        run = lambda i: NV.nvfp4_gemm(NV.PackedNVFP4(packed[i % 2][0], packed[i % 2][1]), NV.PackedNVFP4(wc, ws), None, None,
                                      torch.bfloat16, alpha_cols=cols[i % 2])
        for i in range(3):
            run(i)
        reps = min(reps, 50)
        secs = time_region(run, reps, torch.cuda.synchronize) / reps
        n = wc.shape[0]
        achieved = 2.0 * self.tokens * n * self.shape.hidden / secs / 1e12
        peak, source = fp4_peak(peaks)
        return secs, {"kernel": f"gemm_nvfp4 (tcgen05 kind::mxf4nvf4.block_scale, 8192x{n}x4096 merged gate/up projection)",
                      "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                      "peak_source": source, "traffic": None}

    def gpu_reference(self):
        """``torch.nn.functional.scaled_mm`` NVFP4 on the model's four GEMM shapes beside this package's kernel."""
        import torch.nn.functional as F
        from torch.nn.functional import ScalingType, SwizzleType

        NV = self.vb.nvfp4
        one = torch.ones((), device="cuda")
        rows = []
        block, tensor = ScalingType.BlockWise1x16, ScalingType.TensorWise
        swz, none = SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE
        for m, n, k in [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336)]:
            a = NV.quantize_nvfp4(torch.randn(m, k, device="cuda").bfloat16())
            b = NV.quantize_nvfp4((torch.randn(n, k, device="cuda") * 0.02).bfloat16())
            alpha = (a[2] * b[2]).float()
            fl = 2.0 * m * n * k / 1e12
            row = {"mnk": [m, n, k], "library_tflops": None,
                   "ours_tflops": fl / time_library(lambda i: NV.nvfp4_linear(a[0], a[1], b[0], b[1], alpha, one, None), 1, 20)}
            try:
                lib = lambda i: F.scaled_mm(a[0].view(torch.float4_e2m1fn_x2), b[0].view(torch.float4_e2m1fn_x2).t(),
                                            [a[1].reshape(-1).view(torch.float8_e4m3fn), alpha], [block, tensor],
                                            [b[1].reshape(-1).view(torch.float8_e4m3fn), one], [block, tensor],
                                            swizzle_a=[swz, none], swizzle_b=[swz, none], output_dtype=torch.bfloat16)
                row["library_tflops"] = fl / time_library(lib, 1, 20)
            except Exception as exc:  # this torch build has no block-scaled FP4 GEMM
                row["library_error"] = repr(exc)[:160]
            rows.append(row)
        best = max([r["library_tflops"] for r in rows if r["library_tflops"]] or [None], key=lambda v: v or 0)
        return {"library": "torch.nn.functional.scaled_mm NVFP4 (BlockWise1x16 e4m3 scales + tensor-wise alpha), same process",
                "shapes": rows, "best_library_tflops": best}

    def gpu_check(self, state, cpu_out):
        """The CPU leg's layer (its weights and input) on the GPU kernels against the CPU leg's output."""
        x, params, shape, _, _ = state
        W = self.vb.workloads
        layer = W.Nvfp4DecoderLayer({k: v.cuda() for k, v in params.items()}, shape)
        got, want = layer(x.cuda()).double().cpu(), cpu_out.double()
        rms = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
        # 4-bit re-quantization after every block amplifies summation-order noise (a moved code changes a value by
        # up to a third), and the GPU attention is a fused bfloat16 kernel where the graph's is eager
        return {"layer_vs_cpu_oracle_max": (max_rel(got, want), 1e-1), "layer_vs_cpu_oracle_rms": (rms, 3e-2)}

    @staticmethod
    def cpu_setup():
        import voyager_b200  # host-side workload definitions only; no kernel runs on this path

        W = voyager_b200.workloads
        shape = W.LLAMA_8B
        params = W.make_layer_params(50, shape)
        x = W.make_hidden_states(300, C4Model.cpu_rows, shape)
        return x, params, shape, W.rope_tables(C4Model.cpu_rows, shape, "cpu"), W.causal_mask(C4Model.cpu_rows, "cpu")

    @staticmethod
    def cpu_step(state):
        from oracle import layers as OL

        return OL.nvfp4_decoder_layer(*state)


# ---------------------------------------------------------------------------
# workload c3: MXNF4 decode step over a KIVI cache, full 32-layer model
# ---------------------------------------------------------------------------
class C3:
    name = "c3"
    batch, cached, recent, layers = 16, 4096, 128, 32
    description = ("c3: MXNF4 decode step of a full 32-layer Llama-3.1-8B-shaped model, batch 16 (one new token per "
                   "sequence), 4096 positions cached: weights lut4_to_int6 (NF4 levels) bs=64 with fp8_e5m3 scales, stored "
                   "packed (0.53 B/parameter) and read by the weight-streaming linear; activations quantize_mx'd the same "
                   "way every step; residual adds through a per-tensor fp8_e4m3 cast; KV cache KIVI 2-bit (keys per channel, "
                   "values per token, groups of 64, packed) with the newest 128 positions in bf16; RoPE + append, the attention "
                   "straight from the 2-bit codes and the residual casts as one kernel each; final norm + lm_head")
    tokens = 16
    n_sets = 2
    dtype = "bf16 operands decoded from 4-bit codes x e5m3 block scales (fp32 accumulate)"
    cpu_tokens = 16 / 32
    cpu_sample = ("decode steps of ONE decoder layer, batch 16, 4096 cached positions (the model is 32 such layers: "
                  "tok/s = 16 / (32 x layer time); lm_head not included)")

    @staticmethod
    def layer_state(seed, shape, tables, device, batch, cached, recent):
        """Weights (index codes + block scales), the KIVI cache and the recent window of one layer, drawn from
        N(0, 0.02) weights and N(0, 1) keys / values through the real quantizers."""
        import voyager_b200

        Q = torch.ops.quantized_ops
        g = torch.Generator(device=device).manual_seed(seed)
        d, hq, hkv, h, inter = shape.head_dim, shape.heads, shape.kv_heads, shape.hidden, shape.intermediate
        rows = {"qkv": ((hq + 2 * hkv) * d, h), "o": (h, hq * d), "gate_up": (2 * inter, h), "down": (h, inter)}
        weights = {}
        for name, (n, k) in rows.items():
            w = (torch.randn(n, k, generator=g, device=device) * 0.02).bfloat16()
            s, c = Q.quantize_mx(w, tables["index"], [-1], 64, 31.0, False, tables["e5m3"], tables["mid"])
            weights[name] = (c, s)
        weights["ln1"] = torch.ones(h, dtype=torch.bfloat16, device=device)
        weights["ln2"] = torch.ones(h, dtype=torch.bfloat16, device=device)
        main = cached - recent
        kv = lambda t: torch.randn(batch, hkv, t, d, generator=g, device=device).bfloat16()
        K = voyager_b200.kivi
        cache = {"k": K.quantize_cache(kv(main), tables["uint2"], -2, 64, 2, tables["e4m3"]),
                 "v": K.quantize_cache(kv(main), tables["uint2"], -1, 64, 2, tables["e4m3"]),
                 "k_res": kv(recent), "v_res": kv(recent)}
        return weights, cache

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        W, P = voyager_b200.workloads, voyager_b200.packed
        self.shape = W.LLAMA_8B
        self.tables = W.nf4_tables(dev)
        t = self.tables
        self.scale = torch.tensor(8.0 / 448.0, dtype=torch.bfloat16, device=dev)          # residual stream within +-8
        self.model = []
        self.weight_bytes = self.cache_bytes = 0
        for i in range(self.layers):
            weights, cache = self.layer_state(700 + 100 * rank + i, self.shape, t, dev, self.batch, self.cached, self.recent)
            packed = {n: P.pack_lut4_weight(*weights[n], t["levels"], 64, check=False)
                      for n in ("qkv", "o", "gate_up", "down")}
            packed["ln1"], packed["ln2"] = weights["ln1"], weights["ln2"]
            del weights
            self.model.append(W.Mxnf4DecodeLayer(packed, t, cache, self.scale, self.shape))
            self.weight_bytes += sum(v.nbytes for k, v in packed.items() if k not in ("ln1", "ln2"))
            self.cache_bytes += cache["k"].nbytes + cache["v"].nbytes + 2 * cache["k_res"].numel() * 2
        g = torch.Generator(device=dev).manual_seed(699 + rank)
        head = (torch.randn(self.shape.vocab, self.shape.hidden, generator=g, device=dev) * 0.02).bfloat16()
        s, c = torch.ops.quantized_ops.quantize_mx(head, t["index"], [-1], 64, 31.0, False, t["e5m3"], t["mid"])
        self.head = P.pack_lut4_weight(c, s, t["levels"], 64, check=False)
        del head, s, c
        self.weight_bytes += self.head.nbytes
        self.norm = torch.ones(self.shape.hidden, dtype=torch.bfloat16, device=dev)
        cos, sin = W.rope_tables(self.cached, self.shape, dev)
        self.rope = (cos[-1].contiguous(), sin[-1].contiguous())
        self.x = [W.make_hidden_states(800 + 10 * rank + i, self.batch, self.shape, dev) for i in range(self.n_sets)]
        self.launches_per_step = self.layers * W.Mxnf4DecodeLayer.LAUNCHES + 2
        self.h2d_bytes = self.batch * self.shape.hidden * 2
        self.d2h_bytes = self.batch * self.shape.vocab * 2
        self._run(self.x[0])
        self.graphs = [capture(lambda x=x: self._run(x)) for x in self.x]
        self.pipeline = HostPipeline(self.x, [x.cpu().pin_memory() for x in self.x], self.graphs)

    def _run(self, x):
        P, t = self.vb.packed, self.tables
        for layer in self.model:
            x = layer(x, self.rope)
        h = torch.nn.functional.rms_norm(x, (self.shape.hidden,), self.norm, self.shape.eps)
        s, c = torch.ops.quantized_ops.quantize_mx(h, t["index"], [-1], 64, 31.0, False, t["e5m3"], t["mid"])
        return P.linear_lut4(c, self.head, input_scale=s, input_code=t["levels"])

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def roofline(self, peaks, reps):
        """The step against the bytes it must read: packed weights + packed cache (what an HBM-bound decode step
        costs at best), and the weight-streaming kernel alone on the merged gate/up projection."""
        P, t = self.vb.packed, self.tables
        ws = [layer.w["gate_up"] for layer in self.model[:8]]                      # 8 x 62 MB: beyond L2
        x = torch.randint(0, 16, (self.batch, self.shape.hidden), device="cuda").bfloat16()
        sx = torch.full((self.batch, self.shape.hidden // 64), 0.05, dtype=torch.bfloat16, device="cuda")
        run = lambda i: P.linear_lut4(x, ws[i % len(ws)], input_scale=sx, input_code=t["levels"])
        for i in range(3):
            run(i)
        secs = time_region(run, reps, torch.cuda.synchronize) / reps
        achieved = ws[0].nbytes / secs / 1e9
        step_secs = time_region(self.step, 10, torch.cuda.synchronize) / 10
        return secs, {"kernel": "gemm_lut4_kernel (packed 4-bit codes + block scales -> bf16 mma.sync, 16 x 28672 x 4096 merged gate/up)",
                      "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                      "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth", "traffic": None,
                      "whole_step": {"algorithmic_bytes": self.weight_bytes + self.cache_bytes,
                                     "weight_bytes": self.weight_bytes, "cache_bytes": self.cache_bytes,
                                     "achieved_gbs": (self.weight_bytes + self.cache_bytes) / step_secs / 1e9,
                                     "frac": (self.weight_bytes + self.cache_bytes) / step_secs / 1e9 / peaks["hbm_gbs"]}}

    def gpu_check(self, state, cpu_out):
        """The CPU leg's layer (its weights, cache and input) on the GPU kernels against the CPU leg's output."""
        x, weights, tables, cache, rope, scale, shape = state
        W, P, K = self.vb.workloads, self.vb.packed, self.vb.kivi
        t = self.tables
        packed = {n: P.pack_lut4_weight(weights[n][0].cuda(), weights[n][1].cuda(), t["levels"], 64)
                  for n in ("qkv", "o", "gate_up", "down")}
        packed["ln1"], packed["ln2"] = weights["ln1"].cuda(), weights["ln2"].cuda()
        dev_cache = {}
        for name, axis in (("k", -2), ("v", -1)):
            codes, sc, zp = cache[name]
            dev_cache[name] = K.PackedCache(K.pack_codes(codes.cuda(), 2), sc.cuda(), zp.cuda(), tuple(codes.shape),
                                            [axis], 64, 2)
        dev_cache["k_res"], dev_cache["v_res"] = cache["k_res"].cuda().clone(), cache["v_res"].cuda().clone()
        layer = W.Mxnf4DecodeLayer(packed, t, dev_cache, scale.cuda(), shape)
        got = layer(x.cuda(), (rope[0].cuda(), rope[1].cuda())).double().cpu()
        want = cpu_out.double()
        rms = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
        # 4-bit activation casts after every block amplify summation-order noise (a moved code changes a value by a third)
        return {"layer_vs_cpu_oracle_max": (max_rel(got, want), 1e-1), "layer_vs_cpu_oracle_rms": (rms, 3e-2)}

    @staticmethod
    def cpu_setup():
        import voyager_b200  # host-side definitions only
        from oracle import quantizers as OQ
        from oracle import tables as OT

        W = voyager_b200.workloads
        shape = W.LLAMA_8B
        nf4 = OT.quantization_map("lut4_to_int6")
        levels = torch.unique(nf4)
        tables = {"levels": levels, "index": torch.searchsorted(levels, nf4).to(torch.int64),
                  "mid": (levels[:-1] + levels[1:]) / 2, "e5m3": OT.quantization_map("fp8_e5m3"),
                  "e4m3": OT.quantization_map("fp8_e4m3"), "uint2": OT.quantization_map("uint2")}
        g = torch.Generator().manual_seed(700)
        d, hq, hkv, h, inter = shape.head_dim, shape.heads, shape.kv_heads, shape.hidden, shape.intermediate
        weights = {}
        for name, (n, k) in {"qkv": ((hq + 2 * hkv) * d, h), "o": (h, hq * d), "gate_up": (2 * inter, h),
                             "down": (h, inter)}.items():
            w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
            s, c = OQ.quantize_mx(w, tables["index"], [-1], 64, 31.0, False, tables["e5m3"], tables["mid"])
            weights[name] = (c, s)
        weights["ln1"] = torch.ones(h, dtype=torch.bfloat16)
        weights["ln2"] = torch.ones(h, dtype=torch.bfloat16)
        main = C3.cached - C3.recent
        kv = lambda t: torch.randn(C3.batch, hkv, t, d, generator=g).bfloat16()
        cache = {}
        for name, axis in (("k", -2), ("v", -1)):
            sc, zp, codes = OQ.quantize_affine(kv(main), tables["uint2"], [axis], 64, 0.0, 3.0, tables["e4m3"])
            cache[name] = (codes, sc, zp)
        cache["k_res"], cache["v_res"] = kv(C3.recent), kv(C3.recent)
        x = W.make_hidden_states(800, C3.batch, shape)
        cos, sin = W.rope_tables(C3.cached, shape, "cpu")
        return x, weights, tables, cache, (cos[-1], sin[-1]), torch.tensor(8.0 / 448.0, dtype=torch.bfloat16), shape

    @staticmethod
    def cpu_step(state):
        from oracle import layers as OL

        x, weights, tables, cache, rope, scale, shape = state
        return OL.mxnf4_decode_layer(x, weights, tables, cache, rope, scale, shape)


# ---------------------------------------------------------------------------
# workload c5: GPTQ of one decoder layer's seven linears at the real calibration size
# ---------------------------------------------------------------------------
class C5:
    name = "c5"
    LINEARS = (("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096), ("gate", 14336, 4096),
               ("up", 14336, 4096), ("down", 4096, 14336))
    calibration = 128 * 2048
    chunk = 16384
    description = ("c5: GPTQ 4-bit asymmetric group-wise quantization (group 128, damp 0.01, act-order off) of ONE "
                   "Llama-3.1-8B-shaped decoder layer's 7 linears per step (the model is 32 such layers, 224 linears), "
                   "calibration 128 x 2048 = 262144 tokens per linear, N(0,1) mixed with a rank-64 component: per linear "
                   "the Hessian X^T X on the tensor cores streamed in 16384-row chunks, damped Cholesky inverse "
                   "(torch.linalg on the device), blocked column sweep + trailing updates (CUDA kernels). tok/s = "
                   "calibration tokens / (32 x the layer's time)")
    tokens = calibration // 32
    n_sets = 1
    launches_per_step = None
    dtype = "fp32 solve, bf16 tensor-core Hessian (fp32 accumulate)"
    cpu_sample = ("GPTQ solves of ONE 4096x4096 linear with 16384 calibration rows; scaled to the layer's seven linears at "
                  "262144 rows by the cost model T K^2 + K^3 + N K^2 (factor 206.6)")
    cpu_tokens = (128 * 2048 // 32) / 206.6

    @staticmethod
    def calibration_rows(seed, rows, k, device):
        g = torch.Generator(device=device).manual_seed(seed)
        base = torch.randn(rows, k, generator=g, device=device)
        low = torch.randn(rows, 64, generator=g, device=device) @ torch.randn(64, k, generator=g, device=device)
        return (0.7 * base + 0.3 * low / 8).bfloat16()

    def __init__(self, dev, rank):
        import voyager_b200

        self.vb = voyager_b200
        self.qmap = voyager_b200.get_quantization_map("uint4", dev)
        g = torch.Generator(device=dev).manual_seed(60 + rank)
        sizes = [n * k for _, n, k in self.LINEARS]
        self.flat_in = (torch.randn(sum(sizes), generator=g, device=dev) * 0.02).bfloat16()
        self.flat_out = torch.empty_like(self.flat_in)
        self.offsets = [0]
        for sz in sizes:
            self.offsets.append(self.offsets[-1] + sz)
        # calibration activations per input width, resident in HBM (2.1 GB and 7.5 GB), drawn in slices
        self.x = {}
        for k in (4096, 14336):
            self.x[k] = torch.cat([self.calibration_rows(600 + k + i, self.chunk, k, dev)
                                   for i in range(self.calibration // self.chunk)])
        self.h2d_bytes = self.flat_in.numel() * 2
        self.d2h_bytes = self.flat_out.numel() * 2
        self.parts = {"hessian": 0.0, "cholesky": 0.0, "sweep": 0.0}
        self.events = []
        self.launches = 0
        self._run()
        self.launches_per_step = self.launches
        step = EagerStep(self._run, self.flat_out)
        step.replay = self._run          # the step writes its output buffer itself
        self.graphs = [(step, self.flat_out)]
        self.pipeline = HostPipeline([self.flat_in], [self.flat_in.cpu().pin_memory()], self.graphs)

    def _mark(self, name):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.events.append((name, e))

    def _run(self):
        G = self.vb.gptq
        self.launches = 0
        for i, (name, n, k) in enumerate(self.LINEARS):
            w = self.flat_in[self.offsets[i]:self.offsets[i + 1]].view(n, k)
            self._mark("start")
            h = None
            for chunk in self.x[k].split(self.chunk):
                h = G.accumulate_hessian(h, chunk)
                self.launches += 1
            self._mark("hessian")
            hinv = G.hessian_inverse_chol(h, self.calibration, 0.01)
            del h
            self._mark("cholesky")
            out = G.sweep(w, hinv, 128, self.qmap, affine_range=(0.0, 15.0))
            self.launches += 2 * (k // 128) - 1
            self.flat_out[self.offsets[i]:self.offsets[i + 1]].view(n, k).copy_(out)
            self._mark("sweep")
        return self.flat_out

    def parts_ms(self, steps):
        """Device time per step spent in the three phases, from the events recorded during the steps."""
        torch.cuda.synchronize()
        total = {"hessian": 0.0, "cholesky": 0.0, "sweep": 0.0}
        for (_, a), (name, b) in zip(self.events, self.events[1:]):
            if name != "start":
                total[name] += a.elapsed_time(b)
        self.events = []
        return {k: v / steps for k, v in total.items()}

    def step(self, i):
        self._run()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def roofline(self, peaks, reps):
        """The dominant kernel: the Hessian GEMM X^T X of the down projection, 14336 x 14336 x 16384 per chunk."""
        ops = self.vb.ops
        xt = self.x[14336][:self.chunk].T.contiguous()
        for _ in range(2):
            ops.gemm_tn(xt, xt, out_dtype=torch.float32)
        reps = min(reps, 20)
        secs = time_region(lambda i: ops.gemm_tn(xt, xt, out_dtype=torch.float32), reps, torch.cuda.synchronize) / reps
        achieved = 2.0 * 14336 * 14336 * self.chunk / secs / 1e12
        return secs, {"kernel": "gemm_tn_pair_kernel (tcgen05 kind::f16 bf16, cta_group::2, 14336x14336x16384 Hessian chunk, fp32 out)",
                      "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                      "frac": achieved / peaks["bf16_tflops"], "peak_source": f"{peaks['source']} bf16 cuBLAS burst",
                      "traffic": None}

    def gpu_check(self, state, cpu_out):
        """The CPU leg's problem solved on the device: the reconstruction error tr(D H D^T) of the two solutions
        (the figure is the relative excess of the device's; LAPACK and the device factorisation are not bit-identical)."""
        w, h, tokens = state
        G = self.vb.gptq
        got = G.compensate_weight_affine(w.cuda(), h.cuda().clone(), tokens, self.qmap, 0.0, 15.0, 128, 0.01).cpu()

        def loss(q):
            d = (q - w).double()
            return float(((d @ h.double()) * d).sum())

        # a group's scale and zero point are continuous (they follow the compensated values), so equal codes give
        # values that agree to rounding, not bit for bit: count values that moved by more than a quarter of a step
        step = float(w.abs().max()) * 2.0 / 15.0
        moved = float(((got - cpu_out).abs() > 0.25 * step).float().mean())
        return {"reconstruction_error_excess_over_cpu_oracle": (max(loss(got) / loss(cpu_out) - 1.0, 0.0), 2e-2),
                "grid_values_a_quarter_step_from_cpu_oracle": (moved, 5e-2)}

    @staticmethod
    def cpu_setup():
        tokens = 16384
        x = C5.calibration_rows(604096, tokens, 4096, "cpu").float()
        g = torch.Generator().manual_seed(61)
        w = (torch.randn(4096, 4096, generator=g) * 0.02).bfloat16().float()
        return w, x.T @ x, tokens

    @staticmethod
    def cpu_step(state):
        from oracle import gptq as OGP
        from oracle import tables as OT

        w, h, tokens = state
        hinv = OGP.hessian_inverse_chol(h.clone(), tokens, 0.01)
        return OGP.sweep_affine(w, hinv, OT.quantization_map("uint4"), 0.0, 15.0, 128)


class EagerStep:
    """Stands in for a captured graph when a step cannot be captured: ``replay()`` runs it again into the
    same output buffer."""

    def __init__(self, fn, out):
        self.fn, self.out = fn, out

    def replay(self):
        self.out.copy_(self.fn())


class C2TP:
    """Workload c2 over N GPUs as ONE tensor-parallel layer (strong scaling): the same 2048-token prefill,
    q/k/v and gate/up column-parallel, attention head-parallel, o_proj / down_proj row-parallel with float32
    partial sums reduce-scattered over NCCL, activations sharded by token rows between the blocks."""
    name = "c2"
    tokens = 2048
    n_sets = 4
    dtype = C2.dtype
    cpu_tokens = C2.cpu_tokens
    cpu_sample = C2.cpu_sample

    def __init__(self, dev, rank, world):
        import torch.distributed as dist

        import voyager_b200

        self.vb = voyager_b200
        W, P = voyager_b200.workloads, voyager_b200.parallel
        self.shape = W.LLAMA_8B
        self.description = C2.description.replace("per GPU", f"split over {world} GPUs (tensor parallel: column-parallel "
                                                  "QKV and gate/up, head-parallel attention, row-parallel o_proj and "
                                                  "down_proj, NCCL all-gather of FP8 codes and reduce-scatter of float32 "
                                                  "partial sums)")
        params = W.make_layer_params(7, self.shape, dev)                 # every rank holds the slices it needs
        full = [W.make_hidden_states(100 + i, self.tokens, self.shape, dev) for i in range(self.n_sets)]
        scales = W.calibrate_fp8_scales(full[0], params, self.shape)
        for name in sorted(scales):                                       # one set of scales on every rank
            dist.broadcast(scales[name], src=0)
        # the four exchanges of a layer as pulls over peer memory (NVLink) where the GPUs can map one another's
        # memory, else NCCL's collectives
        self.exchange_kind = "nccl"
        exchange = None
        if EXCHANGE == "peer":
            try:
                exchange = P.PeerExchange(self.tokens // world * self.shape.hidden, self.tokens * self.shape.hidden, dev)
                self.exchange_kind = "peer memory (symmetric buffers, cross-rank barrier, vq_peer_gather / vq_peer_reduce_rows)"
            except Exception as exc:  # no peer access on this box
                self.exchange_kind = f"nccl (peer memory unavailable: {type(exc).__name__})"
        self.layer = P.Fp8DecoderLayerTP(params, scales, self.shape, exchange=exchange)
        del params
        lo, hi = P.shard_bounds(self.tokens, rank, world)
        self.x = [x[lo:hi].contiguous() for x in full]
        del full
        self.launches_per_step = self.layer.LAUNCHES
        self.h2d_bytes = (hi - lo) * self.shape.hidden * 2
        self.d2h_bytes = (hi - lo) * self.shape.hidden * 2
        for x in self.x[:2]:
            self.layer(x)
        torch.cuda.synchronize()
        self.launch = "CUDA graph replay per step (collectives captured)"
        try:
            self.graphs = [capture(lambda x=x: self.layer(x)) for x in self.x]
        except Exception as exc:  # the collectives could not be captured on this build: launch every kernel
            torch.cuda.synchronize()
            self.launch = f"eager launches per step (graph capture refused: {type(exc).__name__})"
            self.graphs = [(EagerStep(lambda x=x: self.layer(x), self.layer(x)),) for x in self.x]
            self.graphs = [(g[0], g[0].out) for g in self.graphs]
        self.pipeline = HostPipeline(self.x, [x.cpu().pin_memory() for x in self.x], self.graphs)

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def self_check(self):
        """This rank's output rows from one graph replay against the same rows of the unsharded layer run on
        this GPU alone (same weights, scales and input)."""
        W = self.vb.workloads
        self.graphs[0][0].replay()
        rows = self.graphs[0][1].clone()
        params = W.make_layer_params(7, self.shape, rows.device)
        single = W.Fp8DecoderLayer(params, self.layer.scales, self.shape)
        del params
        full = single(W.make_hidden_states(100, self.tokens, self.shape, rows.device))
        n = rows.shape[0]
        lo = self.layer.rank * n
        return {"tensor_parallel_rows_vs_one_gpu_layer": (max_rel(rows, full[lo:lo + n]), 6e-2)}

    def collective_share(self, steps):
        """Share of an (uncaptured) step's device time spent inside the four collectives, from CUDA events
        around them; a collective's span includes waiting for the slowest rank."""
        for i in range(3):
            self.layer(self.x[i % self.n_sets])
        self.layer.timed = True
        self.layer.collective_events = []
        elapsed = time_region(lambda i: self.layer(self.x[i % self.n_sets]), steps, torch.cuda.synchronize)
        inside = self.layer.collective_seconds()
        self.layer.timed = False
        return {"share": inside / elapsed, "collective_ms_per_step": inside / steps * 1e3,
                "eager_ms_per_step": elapsed / steps * 1e3, "collectives_per_step": self.layer.COLLECTIVES,
                "exchange": self.exchange_kind,
                "what": "2 x all-gather of FP8 codes [T, 4096] bytes, 2 x reduce-scatter of float32 [T, 4096] partial sums"}

    def roofline(self, peaks, reps):
        """This rank's slice of the gate/up GEMM with the SwiGLU epilogue: [2048, 4096] x [2 * 14336 / N, 4096]^T."""
        FP8 = self.vb.fp8
        sh, s, L = self.shape, self.layer.scales, self.layer
        full = [torch.randn(self.tokens, sh.hidden, device="cuda").bfloat16() for _ in range(3)]
        acts = [FP8.quantize_fp8(torch.nn.functional.rms_norm(x, (sh.hidden,)), s["h2"]) for x in full]
        run = lambda i: FP8.fp8_gemm(acts[i % len(acts)], L.w8_swiglu, alpha_cols=L.alpha_swiglu, gated_scale=s["act"],
                                     round_acc=True)
        for i in range(3):
            run(i)
        secs = time_region(run, reps, torch.cuda.synchronize) / reps
        n = L.w8_swiglu.shape[0]
        achieved = 2.0 * self.tokens * n * sh.hidden / secs / 1e12
        peak, source = fp8_peak(peaks)
        return secs, {"kernel": f"gemm_tn_pair_kernel (tcgen05 kind::f8f6f4 e4m3, cta_group::2, 2048x{n}x4096: this rank's "
                                "columns of the merged gate/up projection, SwiGLU + FP8 cast epilogue)",
                      "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                      "peak_source": source, "traffic": None}


WORKLOADS = {"c1": C1, "c2": C2, "c2s": C2Separate, "c4": C4, "c3": C3, "c4m": C4Model, "c5": C5, "q1": Q1, "r1": R1}


def time_cpu_baseline(workload, reps):
    """The CPU port of the reference operators on the host cores.  Returns
    ``(tok/s, seconds per step, threads, setup state, last output)``."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    state = workload.cpu_setup()
    out = workload.cpu_step(state)          # warm-up: tables built, pages touched
    t0 = time.perf_counter()
    for _ in range(reps):
        out = workload.cpu_step(state)
    dt = (time.perf_counter() - t0) / reps
    return workload.cpu_tokens / dt, dt, cores, state, out


def run_reference(args, rank):
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    reps = max(1, min(args.steps, 3))
    value, dt, cores, _, _ = time_cpu_baseline(wl, reps)
    sample = f"{reps} {wl.cpu_sample} after 1 warm-up"
    print(json.dumps({
        "impl": "reference", "metric": "tok/s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": reps,
        "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic", "config": {"workload": wl.description, "cpu_sample": sample},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def timed_roofline(wl, peaks, reps, device_index):
    """The dominant kernel alone over ``reps`` launches, with the SM clock sampled meanwhile."""
    with ClockSampler(device_index) as clocks:
        secs, roof = wl.roofline(peaks, reps)
    mhz = clocks.summary()["sm_mhz"]
    roof.update({"launches_timed": reps, "us_per_launch": secs * 1e6, "sm_mhz_median": mhz,
                 "us_x_mhz": None if mhz is None else secs * 1e6 * mhz})
    return roof


def library_leg(wl, kind=None):
    """``wl.gpu_reference()`` if the workload has one; its best figure becomes the measured FP8 / FP4 peak."""
    if not hasattr(wl, "gpu_reference"):
        return None
    ref = wl.gpu_reference()
    if kind and ref.get("best_library_tflops"):
        MEASURED_LIBRARY[kind] = ref["best_library_tflops"]
    return ref


LIBRARY_KIND = {"c2": "fp8", "c2s": "fp8", "c4": "fp4", "c4m": "fp4"}


class C4TP:
    """Workload c4m over N GPUs, tensor-parallel (strong scaling): the same 8192-token prefill of 32 NVFP4
    decoder layers, q/k/v and gate/up column-parallel, attention head-parallel, o_proj / down_proj row-parallel
    with float32 partial products reduce-scattered over NCCL, activations sharded by token rows between the
    blocks and gathered as packed NVFP4 codes + scale tiles; final norm + lm_head on the rank that holds the last
    position."""
    name = "c4m"
    tokens = C4Model.tokens
    layers = C4Model.layers
    n_sets = 2
    dtype = C4Model.dtype
    cpu_tokens = C4Model.cpu_tokens
    cpu_sample = C4Model.cpu_sample

    def __init__(self, dev, rank, world):
        import voyager_b200

        self.vb = voyager_b200
        W, P, NV = voyager_b200.workloads, voyager_b200.parallel, voyager_b200.nvfp4
        self.shape, self.rank, self.world = W.LLAMA_8B, rank, world
        self.description = C4Model.description.replace("1 x 8192 tokens per GPU", f"1 x 8192 tokens split over {world} GPUs "
                                                       "(tensor parallel: column-parallel QKV and gate/up, head-parallel "
                                                       "attention, row-parallel o_proj and down_proj; NCCL all-gather of "
                                                       "packed NVFP4 codes + scale tiles, amax all-reduce, reduce-scatter "
                                                       "of float32 partial products)")
        self.exchange_kind = "nccl"
        exchange = None
        if EXCHANGE == "peer":
            try:
                per_rank = self.tokens // world * self.shape.hidden
                exchange = P.PeerExchange(per_rank // 2 + per_rank // 16, self.tokens * self.shape.hidden, dev)
                self.exchange_kind = "peer memory (symmetric buffers, cross-rank barrier, vq_peer_gather / vq_peer_reduce_rows / vq_peer_max)"
            except Exception as exc:
                self.exchange_kind = f"nccl (peer memory unavailable: {type(exc).__name__})"
        self.model = []
        for i in range(self.layers):                 # the same seeds on every rank: each quantizes, then keeps its slices
            params = W.make_layer_params_on_device(50 + i, self.shape, dev)
            self.model.append(P.Nvfp4DecoderLayerTP(params, self.shape, exchange=exchange))
            del params
        self.last = rank == world - 1
        if self.last:
            g = torch.Generator(device=dev).manual_seed(50 + self.layers)
            head = (torch.randn(self.shape.vocab, self.shape.hidden, generator=g, device=dev) * 0.02).bfloat16()
            self.head = NV.quantize_nvfp4(head)
            del head
            self.norm = torch.ones(self.shape.hidden, dtype=torch.bfloat16, device=dev)
            self.one = torch.ones((), device=dev)
        full = [W.make_hidden_states(300 + i, self.tokens, self.shape, dev) for i in range(self.n_sets)]
        lo, hi = P.shard_bounds(self.tokens, rank, world)
        self.lo, self.hi = lo, hi
        self.x = [x[lo:hi].contiguous() for x in full]
        del full
        self.launches_per_step = self.layers * P.Nvfp4DecoderLayerTP.LAUNCHES + (3 if self.last else 0)
        self.h2d_bytes = (hi - lo) * self.shape.hidden * 2
        self.d2h_bytes = (hi - lo) * self.shape.hidden * 2
        self.forward(self.x[0])
        torch.cuda.synchronize()
        self.launch = "CUDA graph replay per step (collectives captured)"
        try:
            self.graphs = [capture(lambda x=x: self.forward(x)) for x in self.x]
        except Exception as exc:  # the collectives could not be captured on this build: launch every kernel
            torch.cuda.synchronize()
            self.launch = f"eager launches per step (graph capture refused: {type(exc).__name__})"
            self.graphs = [(EagerStep(lambda x=x: self.forward(x), self.forward(x)),) for x in self.x]
            self.graphs = [(g[0], g[0].out) for g in self.graphs]
        self.pipeline = HostPipeline(self.x, [x.cpu().pin_memory() for x in self.x], self.graphs)

    def forward(self, rows):
        import torch.nn.functional as F

        for layer in self.model:
            rows = layer(rows)
        if self.last:
            NV = self.vb.nvfp4
            h = F.rms_norm(rows[-1:], (self.shape.hidden,), self.norm, self.shape.eps)
            codes, scales, t = NV.quantize_nvfp4(h)
            self.logits = NV.nvfp4_linear(codes, scales, self.head[0], self.head[1], (t * self.head[2]).float(), self.one, None)
        return rows

    def step(self, i):
        self.graphs[i % self.n_sets][0].replay()

    def e2e_step(self, i):
        self.pipeline.step(i)

    def self_check(self):
        """This rank's rows out of the FIRST tensor-parallel layer against the same rows of the unsharded layer run
        on this GPU alone (same weights and input; the full model's 32 layers compound 4-bit code flips)."""
        W = self.vb.workloads
        rows = self.model[0](self.x[0])
        params = W.make_layer_params_on_device(50, self.shape, rows.device)
        single = W.Nvfp4DecoderLayer(params, self.shape)
        del params
        full = single(W.make_hidden_states(300, self.tokens, self.shape, rows.device))
        want = full[self.lo:self.hi].float()
        rms = float((rows.float() - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
        return {"tensor_parallel_rows_vs_one_gpu_layer_max": (max_rel(rows, full[self.lo:self.hi]), 1e-1),
                "tensor_parallel_rows_vs_one_gpu_layer_rms": (rms, 2e-2)}

    def collective_share(self, steps):
        """Share of an (uncaptured) step's device time spent inside the collectives, from CUDA events around them;
        a collective's span includes waiting for the slowest rank."""
        steps = min(steps, 3)
        self.forward(self.x[0])
        for layer in self.model:
            layer.timed = True
            layer.collective_events = []
        elapsed = time_region(lambda i: self.forward(self.x[i % self.n_sets]), steps, torch.cuda.synchronize)
        inside = sum(layer.collective_seconds() for layer in self.model)
        for layer in self.model:
            layer.timed = False
        per_layer = self.vb.parallel.Nvfp4DecoderLayerTP.COLLECTIVES
        return {"share": inside / elapsed, "collective_ms_per_step": inside / steps * 1e3,
                "eager_ms_per_step": elapsed / steps * 1e3, "collectives_per_step": per_layer * self.layers,
                "exchange": self.exchange_kind,
                "what": "per layer: 4 x all-reduce(max) of one amax, 2 x (all-gather of packed codes [T, 2048] bytes + "
                        "scale tiles), 2 x reduce-scatter of float32 [T, 4096] partial products"}

    def roofline(self, peaks, reps):
        """This rank's rows of the merged gate/up NVFP4 GEMM: [8192, 4096] x [2 * 14336 / N, 4096]^T."""
        NV = self.vb.nvfp4
        layer = self.model[0]
        acts = [torch.randn(self.tokens, self.shape.hidden, device="cuda").bfloat16() for _ in range(2)]
        packed = [NV.quantize_nvfp4(a) for a in acts]
        cols = [(t * layer.tw_gu).float() for _, _, t in packed]
        run = lambda i: NV.nvfp4_gemm(NV.PackedNVFP4(packed[i % 2][0], packed[i % 2][1]), layer.w_gu, None, None,
                                      torch.bfloat16, alpha_cols=cols[i % 2])
        for i in range(3):
            run(i)
        reps = min(reps, 50)
        secs = time_region(run, reps, torch.cuda.synchronize) / reps
        n = layer.w_gu.codes.shape[0]
        achieved = 2.0 * self.tokens * n * self.shape.hidden / secs / 1e12
        peak, source = fp4_peak(peaks)
        return secs, {"kernel": f"gemm_nvfp4 (tcgen05 kind::mxf4nvf4.block_scale, 8192x{n}x4096: this rank's columns of the "
                                "merged gate/up projection)",
                      "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                      "peak_source": source, "traffic": None}


TENSOR_PARALLEL = {"c2": C2TP, "c4m": C4TP}
EXCHANGE = "peer"      # --exchange: how a tensor-parallel layer moves token rows between ranks


def run_secondary(name, dev, rank, peaks, steps, device_index):
    """A further workload measured after the main region: device-timed throughput, its dominant kernel's
    roofline and its library baseline."""
    wl = WORKLOADS[name](dev, rank)
    for i in range(3):
        wl.step(i)
    elapsed = time_region(wl.step, steps, torch.cuda.synchronize)
    ref = library_leg(wl, LIBRARY_KIND.get(name))
    entry = {"workload": wl.description, "name": name, "metric": "tok/s", "value": wl.tokens * steps / elapsed,
             "ms_per_step": elapsed / steps * 1e3, "steps": steps, "dtype": wl.dtype,
             "gpu_launches": wl.launches_per_step * steps,
             "roofline": timed_roofline(wl, peaks, 200, device_index)}
    if ref is not None:
        entry["gpu_reference"] = ref
    wl.vb.ops.gemm_status()
    del wl
    torch.cuda.empty_cache()
    return entry


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL's own log settings (NCCL_DEBUG and friends) are left as the caller's environment has them
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tensor_parallel = world > 1 and args.workload in TENSOR_PARALLEL and not args.replicas
    wl = TENSOR_PARALLEL[args.workload](dev, rank, world) if tensor_parallel else WORKLOADS[args.workload](dev, rank)
    warmup = max(args.warmup, 3)
    for i in range(warmup):
        wl.step(i)
    wl.vb.ops.gemm_status()

    barrier()   # NCCL communicators come up here, not inside the sampled region
    if hasattr(wl, "parts_ms"):
        wl.parts_ms(1)                      # drop the warm-up's events
    with ClockSampler(local_rank) as clocks:
        elapsed = time_region(wl.step, args.steps, barrier)
    phases = wl.parts_ms(args.steps) if hasattr(wl, "parts_ms") else None
    wl.vb.ops.gemm_status()

    for i in range(3):
        wl.e2e_step(i)
    e2e_elapsed = time_region(wl.e2e_step, args.steps, barrier, wl.pipeline.finish)

    peaks = measured_peaks()
    reference = library_leg(wl, LIBRARY_KIND.get(args.workload)) if rank == 0 else None
    roof = timed_roofline(wl, peaks, 200, local_rank)
    collectives = wl.collective_share(min(args.steps, 50)) if tensor_parallel else None
    replicas_elapsed = 0.0
    # a tensor-parallel self-check runs collectives: every rank takes part, rank 0 reports
    checks = dict(wl.self_check()) if hasattr(wl, "self_check") and (rank == 0 or tensor_parallel) else {}
    if tensor_parallel:
        # the same workload as N independent replicas (one full batch per GPU, no exchange)
        del wl.graphs, wl.pipeline
        if hasattr(wl, "model"):
            del wl.model
        torch.cuda.empty_cache()
        rep = WORKLOADS[args.workload](dev, rank)
        for i in range(3):
            rep.step(i)
        replicas_elapsed = time_region(rep.step, args.steps, barrier)
        del rep
        torch.cuda.empty_cache()

    times = torch.tensor([elapsed, e2e_elapsed, replicas_elapsed], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed, e2e_elapsed, replicas_elapsed = times.tolist()

    failed = False
    if rank == 0:
        tokens_total = wl.tokens * args.steps * (1 if tensor_parallel else world)
        line = {
            "metric": "tok/s", "value": tokens_total / elapsed, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong" if tensor_parallel else "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": wl.description,
                       "parallelism": f"tp{world}" if tensor_parallel else (f"{world} replicas" if world > 1 else "1 GPU"),
                       "l2": f"{wl.n_sets} rotating input sets; tensors touched per step exceed the 126 MB L2",
                       "launch": getattr(wl, "launch", "CUDA graph replay per step"),
                       "e2e": "pinned host input copied in, graph replayed, result copied out to pinned host memory "
                              "every step; copies on their own streams overlap neighbouring steps' compute"},
            "e2e": {"value": tokens_total / e2e_elapsed, "unit": "tok/s", "h2d_bytes_per_step": wl.h2d_bytes,
                    "d2h_bytes_per_step": wl.d2h_bytes},
            "gpu_launches": wl.launches_per_step * args.steps,
            "roofline": roof,
            "clocks": clocks.summary(),
        }
        if reference is not None:
            line["gpu_reference"] = reference
        if hasattr(wl, "parts_ms"):
            line["phases_ms_per_step"] = phases
        if tensor_parallel:
            line["collectives"] = collectives
            line["replicas"] = {"value": wl.tokens * args.steps * world / replicas_elapsed, "unit": "tok/s",
                                "scaling": "weak", "ms_per_step": replicas_elapsed / args.steps * 1e3,
                                "what": f"the same workload as independent replicas, one {wl.tokens}-token batch per GPU, no exchange"}
        if world == 1:
            reps = 2 if wl.cpu_tokens >= 2048 and args.workload.startswith("c2") else 3
            value, dt, cores, state, cpu_out = time_cpu_baseline(WORKLOADS[args.workload], reps)
            line["cpu_baseline"] = {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": f"{reps} {wl.cpu_sample} after 1 warm-up"}
            checks.update(wl.gpu_check(state, cpu_out))
            del state, cpu_out
        line["self_check"] = {"max_rel": max((v for v, _ in checks.values()), default=None),
                              "ok": all(v <= tol for v, tol in checks.values()),
                              "checks": {k: {"value": v, "tolerance": tol} for k, (v, tol) in checks.items()}}
        failed = not line["self_check"]["ok"]
        wl.vb.ops.gemm_status()
        if world == 1 and args.workload == "c2" and not args.no_secondary:
            del wl
            torch.cuda.empty_cache()
            # every other BASELINE configuration, so that the default run's line carries them all (their CPU legs
            # and self-checks run when they are the --workload)
            line["secondary"] = [run_secondary(name, dev, rank, peaks, steps, local_rank)
                                 for name, steps in (("q1", 50), ("c1", 50), ("c4", 50), ("c3", 10), ("c4m", 3), ("c5", 2))]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if failed:
        raise SystemExit("self_check failed: the benchmarked path disagrees with its reference beyond the tolerance")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--replicas", action="store_true",
                    help="with N > 1 GPUs run N independent replicas instead of one tensor-parallel layer")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="tensor-parallel token-row exchanges: pulls over peer memory (default, NCCL if the GPUs cannot "
                         "map one another's memory) or NCCL collectives")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the q1 / c1 / c4 measurements that follow the default workload's line")
    args = ap.parse_args()
    global EXCHANGE
    EXCHANGE = args.exchange
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
