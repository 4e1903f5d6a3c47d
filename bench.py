"""Benchmark of the quantized hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1]

One "step" is one pass of the hot path over one batch of synthetic input.
Workload ``c1`` (BASELINE.json configs[0]): X [2048,4096] bf16 ~N(0,1) with
0.1 % of entries x20, W [4096,4096] ~N(0,0.02); both are quantized to int8
microscaling (block 16 along K, power-of-two scales) and multiplied to
Y [2048,4096] bf16 -- ``quantize_mx`` x2 + ``linear_mx``.

With N > 1 (launched under torchrun, one rank per GPU) every rank processes its
own batches: the path shards by rows with no exchange, so scaling is weak and
``value`` is the sum over ranks.  The timed region is K steps bracketed by a
barrier and a device synchronize; time is taken with CUDA events and the
maximum over ranks.  Successive steps use different input sets whose combined
size exceeds the 126 MB L2, so no step finds its inputs cached.

``--impl reference`` times the CPU oracle (a port of the reference's CPU
operators) on the host cores for the same workload.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# ncu-measured DRAM traffic (bytes per launch) of the dominant kernel, from the
# capture summarised under profiles/; None until one has been taken.
NCU_TRAFFIC_BYTES = {"c1": None}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(names, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# workload c1: MXINT8 quantized linear
# ---------------------------------------------------------------------------
C1 = dict(tokens=2048, k=4096, n=4096, block=16, qmax=127.0)


def c1_inputs(seed, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(C1["tokens"], C1["k"], generator=g)
    x = torch.where(torch.rand(C1["tokens"], C1["k"], generator=g) < 0.001, x * 20, x).bfloat16()
    w = (torch.randn(C1["n"], C1["k"], generator=g) * 0.02).bfloat16()
    return x.to(device), w.to(device)


def c1_step_gpu(Q, x, w, table):
    sx, cx = Q.quantize_mx(x, table, [-1], C1["block"], C1["qmax"], True)
    sw, cw = Q.quantize_mx(w, table, [-1], C1["block"], C1["qmax"], True)
    return Q.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=C1["block"])


C1_LAUNCHES_PER_STEP = 5  # quantize_mx x2, operand read-back x2, tensor-core GEMM


def c1_step_cpu(x, w, table):
    from oracle import gemm as OG
    from oracle import quantizers as OQ

    sx, cx = OQ.quantize_mx(x, table, [-1], C1["block"], C1["qmax"], True)
    sw, cw = OQ.quantize_mx(w, table, [-1], C1["block"], C1["qmax"], True)
    return OG.linear_mx(cx, cw, None, input_scale=sx, weight_scale=sw, block_size=C1["block"])


def time_cpu_baseline(reps):
    """The CPU port of the reference operators on the host cores: ``reps`` full
    c1 steps after one warm-up."""
    from oracle import tables as OT

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, w = c1_inputs(0)
    table = OT.quantization_map("int8")
    c1_step_cpu(x, w, table)
    t0 = time.perf_counter()
    for _ in range(reps):
        c1_step_cpu(x, w, table)
    dt = (time.perf_counter() - t0) / reps
    return dt, cores


def run_reference(args, rank):
    if rank != 0:
        return
    reps = max(1, args.steps)
    for _ in range(max(0, args.warmup - 1)):
        pass
    dt, cores = time_cpu_baseline(reps)
    value = C1["tokens"] / dt
    line = {
        "impl": "reference", "metric": "tok/s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": reps, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "c1: MXINT8 (int8, bs=16, pot) quantize_mx x2 + linear_mx, X[2048,4096] W[4096,4096]"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": f"{reps} full c1 steps after 1 warm-up"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import voyager_b200

    Q = torch.ops.quantized_ops
    table = voyager_b200.get_quantization_map("int8", dev)
    n_sets = 6  # ~120 MB of tensors touched per step -> 6 sets exceed L2 several times over
    sets = [c1_inputs(1000 * rank + i, dev) for i in range(n_sets)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        c1_step_gpu(Q, *sets[i % n_sets], table)
    voyager_b200.ops.gemm_status()

    # ---- device-resident timing (the `value`) ----
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        start.record()
        for i in range(args.steps):
            c1_step_gpu(Q, *sets[i % n_sets], table)
        stop.record()
        barrier()
    elapsed = start.elapsed_time(stop) * 1e-3
    voyager_b200.ops.gemm_status()

    # ---- end to end through the operator API with host buffers ----
    host_x = [s[0].cpu().pin_memory() for s in sets]
    weights = [s[1] for s in sets]
    host_y = torch.empty(C1["tokens"], C1["n"], dtype=torch.bfloat16).pin_memory()
    for i in range(3):
        y = c1_step_gpu(Q, host_x[i].to(dev, non_blocking=True), weights[i], table)
        host_y.copy_(y, non_blocking=True)
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for i in range(args.steps):
        xd = host_x[i % n_sets].to(dev, non_blocking=True)
        y = c1_step_gpu(Q, xd, weights[i % n_sets], table)
        host_y.copy_(y, non_blocking=True)
    e_stop.record()
    barrier()
    e2e_elapsed = e_start.elapsed_time(e_stop) * 1e-3

    # ---- the dominant kernel alone (roofline) ----
    ops = voyager_b200.ops

    def dequantized_pair(x, w):
        sx, cx = Q.quantize_mx(x, table, [-1], C1["block"], C1["qmax"], True)
        sw, cw = Q.quantize_mx(w, table, [-1], C1["block"], C1["qmax"], True)
        return (ops._decode_and_scale(cx, sx, None, C1["block"]), ops._decode_and_scale(cw, sw, None, C1["block"]))

    deq = [dequantized_pair(*s) for s in sets]
    for a, b in deq[:3]:
        ops.gemm_tn(a, b)
    torch.cuda.synchronize()
    g_start, g_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(args.steps, 12)
    g_start.record()
    for i in range(reps):
        ops.gemm_tn(*deq[i % n_sets])
    g_stop.record()
    torch.cuda.synchronize()
    gemm_s = g_start.elapsed_time(g_stop) * 1e-3 / reps
    flops = 2.0 * C1["tokens"] * C1["n"] * C1["k"]

    times = torch.tensor([elapsed, e2e_elapsed, gemm_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed, e2e_elapsed, gemm_s = times.tolist()

    if rank == 0:
        peaks = measured_peaks()
        tokens_total = C1["tokens"] * args.steps * world
        cpu_dt, cores = time_cpu_baseline(5) if world == 1 else (None, None)
        achieved = flops / gemm_s / 1e12
        line = {
            "metric": "tok/s", "value": tokens_total / elapsed, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": elapsed / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "c1: MXINT8 (int8, bs=16, pot) quantize_mx x2 + linear_mx, "
                                   "X[2048,4096] W[4096,4096] per GPU",
                       "l2": f"{n_sets} rotating input sets (~120 MB touched per step) exceed the 126 MB L2"},
            "e2e": {"value": tokens_total / e2e_elapsed, "unit": "tok/s",
                    "h2d_bytes_per_step": C1["tokens"] * C1["k"] * 2, "d2h_bytes_per_step": C1["tokens"] * C1["n"] * 2},
            "gpu_launches": C1_LAUNCHES_PER_STEP * args.steps,
            "roofline": {"kernel": "gemm_tn_kernel (tcgen05 bf16, 2048x4096x4096)", "bound": "tensor",
                         "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (burst)",
                         "traffic": NCU_TRAFFIC_BYTES["c1"]},
            "clocks": clocks.summary(),
        }
        if cpu_dt is not None:
            line["cpu_baseline"] = {"value": C1["tokens"] / cpu_dt, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": "5 full c1 steps after 1 warm-up"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=["c1"])
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
