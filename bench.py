"""Benchmark of the decode-GEMV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload auto|c1|stack]

Metric: weight-stream throughput (algorithmic weight bytes / time, TB/s), the reference's headline for this path.

Workloads
  c1     (N = 1 default) FP8 E4M3 W8A16, K = 8192, N = 28672, a step = one call at each M in {1, 2, 4, 8, 16}, every
         call on its own copy of the weights (5 x 235 MB in rotation, so nothing is served from the 126 MB L2). The
         timed region replays a CUDA graph of the step (the reference's own method for its published numbers).
  stack  (N > 1 default) the 70B-shaped NVFP4 projection stack: 80 layers x {qkv, o, gate_up, down}, output columns
         sharded over the ranks, every GEMV with the all-gather of its [M][N/P] outputs in its epilogue (peer stores over
         NVLink; `--gather nccl` runs an NCCL all-gather after every GEMV instead); a step = one pass
         over the stack at each M in {1, 8, 16}, each pass one CUDA-graph replay. Total work is fixed ("strong").

The line printed by rank 0 carries: `value` (device-timed, inputs resident in HBM), `e2e` (the same step through the
public torch ops with the activations copied from pinned host memory and the outputs copied back inside the timed
region, uploads and downloads on their own streams beside the other calls of the step; the weights are the model and
stay resident), `roofline` for the kernel that takes the most time with
per-M detail, `cpu_baseline` (the reference tests' dequantize-then-matmul on the host cores, a bounded sample) and the
SM clocks sampled while the GPU worked. `--impl reference` times that CPU path alone.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

C1 = {"fmt": "fp8", "N": 28672, "K": 8192, "Ms": (1, 2, 4, 8, 16)}
STACK_MS = (1, 8, 16)
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the c1 kernels, from the ncu captures summarised in
# profiles/gemv_fp8_m1_28672x8192.md and profiles/gemv_fp8_m16_28672x8192.md (algorithmic bytes: 234,995,712).
NCU_TRAFFIC_C1 = {1: 240_238_592, 16: 239_695_360}
METRIC = "decode_gemv_weight_stream"
UNIT = "TB/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, read through NVML every 20 ms while a region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.reasons.update(k for k, bit in names.items() if mask & bit)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def time_region(fn, reps, barrier=None):
    """Device time of `reps` calls of fn in ms (CUDA events on the current stream, synchronised on both sides)."""
    if barrier:
        barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b)


# ----- CPU arm: the reference tests' dequantize-then-matmul on the host cores -----------------------------------------

def cpu_reference_sample(rows=2048, reps=1):
    """One bounded sample of workload c1 on the host: `rows` output channels of the FP8 matrix, dequantised to FP32
    and multiplied in FP32 at each M of the configuration. Returns (seconds per pass, weight bytes per pass)."""
    from oracle import decode_gemv_oracle as oc
    from oracle import workloads as wl
    codes, scale = wl.cfg_fp8(rows, C1["K"], seed=1)
    xs = [wl.activations(m, C1["K"], seed=8) for m in C1["Ms"]]
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        for x in xs:
            oc.gemv_fp32(x, oc.dequant_fp32("fp8", (codes, scale)))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, len(C1["Ms"]) * wl.weight_bytes("fp8", rows, C1["K"])


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    rows = 2048
    for _ in range(max(args.warmup, 1)):
        cpu_reference_sample(rows)
    times = []
    for _ in range(args.steps):
        dt, nbytes = cpu_reference_sample(rows)
        times.append(dt)
    sec = sum(times) / len(times)
    value = nbytes / sec / 1e12
    cores = torch.get_num_threads()
    sample = f"{rows} of {C1['N']} output channels of workload c1, M in {list(C1['Ms'])}, torch CPU FP32"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "c1: FP8 E4M3 W8A16 GEMV K=8192 N=28672 M in {1,2,4,8,16} (CPU arm: bounded sample)"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----- workload c1 on one GPU --------------------------------------------------------------------------------------

def run_c1(args, dev):
    import crit_kernels_b200
    from oracle import workloads as wl
    from crit_kernels_b200 import cabi
    k = crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)
    cabi.load().dg_set_static_weights(1)     # the weights are resident and never rewritten between calls
    n, kk, ms = C1["N"], C1["K"], C1["Ms"]
    g = torch.Generator(device=dev).manual_seed(1234)
    copies = []
    for _ in range(len(ms)):
        codes = (torch.randn(n, kk, device=dev, generator=g) * 0.02).to(torch.float8_e4m3fn).view(torch.uint8)
        scale = (torch.rand(n, device=dev, generator=g) * 1.5 + 0.5) / 64
        copies.append((codes, scale))
    xs_host = [wl.activations(m, kk, seed=8 + m).pin_memory() for m in ms]
    xs = [x.to(dev) for x in xs_host]
    outs = [torch.empty(m, n, dtype=torch.bfloat16, device=dev) for m in ms]
    outs_host = [torch.empty(m, n, dtype=torch.bfloat16).pin_memory() for m in ms]
    wbytes = wl.weight_bytes("fp8", n, kk)

    def step():
        for i in range(len(ms)):
            k.gemv_fp8(xs[i], copies[i][0], copies[i][1], outs[i])

    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    # a small call first and last: the largest upload and the largest download then run beside other calls
    e2e_order = sorted(range(len(ms)), key=lambda i: (ms[i] == min(ms), -ms[i]))
    e2e_order = e2e_order[-2:-1] + e2e_order[:-2] + e2e_order[-1:] if len(ms) > 2 else e2e_order

    def step_e2e_body():
        # what a serving loop does per decode step: activations up from pinned host memory, the GEMV through the
        # public op, results down to pinned host memory (the weights are the model and stay resident). Uploads and
        # downloads run on their own streams, each call waits for its own activations only and each download for
        # its own call only; the step ends when every download has landed.
        main = torch.cuda.current_stream()
        up.wait_stream(main)
        down.wait_stream(main)
        ready = []
        with torch.cuda.stream(up):
            for i in e2e_order:
                xs[i].copy_(xs_host[i], non_blocking=True)
                ready.append(torch.cuda.Event())
                ready[-1].record(up)
        for j, i in enumerate(e2e_order):
            main.wait_event(ready[j])
            k.gemv_fp8(xs[i], copies[i][0], copies[i][1], outs[i])
            done = torch.cuda.Event()
            done.record(main)
            down.wait_event(done)
            with torch.cuda.stream(down):
                outs_host[i].copy_(outs[i], non_blocking=True)
        main.wait_stream(up)
        main.wait_stream(down)

    def graph_of(fn):
        """fn captured once in a CUDA graph (the calls allocate nothing and never wait for the device)."""
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g

    with ClockSampler(dev.index or 0) as clocks:
        step_graph = graph_of(step)
        for _ in range(args.warmup):
            step_graph.replay()
        ms_total = time_region(step_graph.replay, args.steps)
        # per-M kernel times: a graph of ten calls at that M, rotating over the weight copies
        per_m = []
        for i, m in enumerate(ms):
            def ten(i=i):
                for c in range(10):
                    w = copies[c % len(copies)]
                    k.gemv_fp8(xs[i], w[0], w[1], outs[i])
            g = graph_of(ten)
            for _ in range(3):
                g.replay()
            reps = max(5, args.steps // 10)
            per_m.append(time_region(g.replay, reps) / (10 * reps))
        e2e_graph = graph_of(step_e2e_body)      # the copies are captured with the calls: one replay + one wait per step
        for _ in range(3):
            e2e_graph.replay()
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_graph.replay()
            torch.cuda.synchronize()             # the host reads the results every step
        e2e_s = (time.perf_counter() - t0) / args.steps
        for i in range(len(ms)):                 # what came down is what the calls wrote
            if not torch.equal(outs_host[i], outs[i].cpu()):
                raise RuntimeError(f"end-to-end step: downloaded results of M={ms[i]} differ from the device's")
    return {"ms_per_step": ms_total / args.steps, "bytes_per_step": wbytes * len(ms), "per_m_ms": per_m,
            "wbytes": wbytes, "clocks": clocks.summary(), "e2e_s": e2e_s,
            "h2d": sum(x.numel() * 2 for x in xs_host), "d2h": sum(o.numel() * 2 for o in outs_host),
            "launches": args.steps * len(ms)}


# ----- workload stack on N GPUs ------------------------------------------------------------------------------------

def run_stack(args, dev, rank, world, ms=STACK_MS, layers=None):
    import torch.distributed as dist
    import crit_kernels_b200
    from crit_kernels_b200 import stack as stk
    from oracle import workloads as wl
    layers = layers or wl.STACK_LAYERS
    model = stk.ShardedStack.random(layers, wl.STACK_ROLES, rank, world, dev, seed=99, gather=args.gather)
    runs = {m: model.capture(m) for m in ms}
    barrier = (lambda: dist.barrier()) if world > 1 else None

    def step():
        for m in ms:
            runs[m].replay()

    with ClockSampler(dev.index or 0) as clocks:
        for _ in range(args.warmup):
            step()
        ms_total = time_region(step, args.steps, barrier)
        per_m = []
        for m in ms:
            reps = max(3, args.steps)
            per_m.append(time_region(runs[m].replay, reps, barrier) / reps)
        # end to end: activations from pinned host memory, the last projection's gathered output back
        for _ in range(2):
            for m in ms:
                runs[m].replay_e2e()
        if barrier:
            barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            for m in ms:
                runs[m].replay_e2e()
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) / args.steps
    t = torch.tensor([ms_total / args.steps, e2e_s * 1e3] + per_m, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    t = t.tolist()
    full_bytes = layers * sum(wl.weight_bytes("nvfp4", n, k) for _, k, n in wl.STACK_ROLES)
    return {"ms_per_step": t[0], "e2e_s": t[1] / 1e3, "per_m_ms": t[2:], "bytes_per_step": full_bytes * len(ms),
            "pass_bytes": full_bytes, "clocks": clocks.summary(),
            "h2d": sum(runs[m].h2d_bytes for m in ms), "d2h": sum(runs[m].d2h_bytes for m in ms),
            "launches": args.steps * sum(runs[m].kernel_launches for m in ms), "gather": model.gather_kind}


def run_case(args):
    """`--case fmt:M:N:K`: seeded inputs in the benchmark distributions, --warmup + --steps calls, device time."""
    import crit_kernels_b200
    from oracle import workloads as wl
    fmt, m, n, kk = args.case.split(":")
    m, n, kk = int(m), int(n), int(kk)
    dev = torch.device("cuda", 0)
    k = crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)
    host = {"nvfp4": lambda: wl.cfg_nvfp4(n, kk), "fp8": lambda: wl.cfg_fp8(n, kk), "mxfp8": lambda: wl.cfg_mxfp8(n, kk),
            "bf16": lambda: (wl.cfg_bf16(n, kk),)}[fmt]()
    t = tuple(a.to(dev) for a in host)
    x = wl.activations(m, kk).to(dev)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    call = {"nvfp4": lambda: k.gemv(x, t[0], t[1], t[2], out), "fp8": lambda: k.gemv_fp8(x, t[0], t[1], out),
            "mxfp8": lambda: k.gemv_fp8(x, t[0], t[1], out), "bf16": lambda: k.gemv_bf16(x, t[0], out)}[fmt]
    for _ in range(args.warmup):
        call()
    ms = time_region(call, args.steps) / args.steps
    nbytes = wl.weight_bytes(fmt, n, kk)
    print(json.dumps({"case": args.case, "us": ms * 1e3, "GBps": nbytes / ms / 1e6, "weight_bytes": nbytes}), flush=True)


def leave_distributed():
    """End of a multi-rank run. destroy_process_group blocks while a CUDA graph that captured the group's collectives
    is alive (seen on this torch/NCCL build), so the graphs are released first; a timer ends the process anyway
    should the teardown still not return (the printed line and exit code 0 are what the caller needs)."""
    import gc
    import torch.distributed as dist
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    guard = threading.Timer(30.0, lambda: os._exit(0))
    guard.daemon = True
    guard.start()
    dist.destroy_process_group()
    guard.cancel()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "c1", "stack"])
    ap.add_argument("--layers", type=int, default=None, help="stack depth (default 80)")
    ap.add_argument("--gather", default="fused", choices=["fused", "fused-overlap", "nccl"],
                    help="stack workload on N > 1 GPUs: all-gather fused into the GEMV epilogue, or NCCL per GEMV")
    ap.add_argument("--case", default=None, metavar="FMT:M:N:K",
                    help="run `--steps` calls of one GEMV (fmt in bf16, fp8, mxfp8, nvfp4) and exit: the small case "
                         "profilers capture")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return
    if args.case:
        run_case(args)
        return
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the GEMVs have no CPU path")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    workload = args.workload if args.workload != "auto" else ("c1" if world == 1 else "stack")
    hbm_gbs, peak_kind = measured_peaks()
    fma_per_clk = 148 * 128

    if workload == "c1":
        r = run_c1(args, dev)
        ms, n, kk = C1["Ms"], C1["N"], C1["K"]
        sm_mhz = r["clocks"]["sm_mhz"] or 1965.0
        detail = []
        for m, t_ms in zip(ms, r["per_m_ms"]):
            gbs = r["wbytes"] / (t_ms * 1e-3) / 1e9
            fma_rate = m * n * kk / (t_ms * 1e-3)
            detail.append({"M": m, "us": t_ms * 1e3, "GBps": gbs, "frac_hbm": gbs / hbm_gbs,
                           "frac_fp32_fma": fma_rate / (fma_per_clk * sm_mhz * 1e6)})
        top = max(range(len(ms)), key=lambda i: r["per_m_ms"][i])
        roofline = {"bound": "hbm", "kernel": f"gemv_kernel<FP8, M={ms[top]}, bf16>",
                    "achieved": detail[top]["GBps"], "peak": hbm_gbs, "unit": "GB/s",
                    "frac": detail[top]["frac_hbm"], "traffic": NCU_TRAFFIC_C1.get(ms[top]), "peak_kind": peak_kind,
                    "frac_fp32_fma_ceiling": detail[top]["frac_fp32_fma"], "per_m": detail}
        config = {"workload": "c1: FP8 E4M3 W8A16 GEMV K=8192 N=28672, one call at each M in {1,2,4,8,16} per step",
                  "l2": "each call streams its own 235 MB copy of the weights (5 copies in rotation, 126 MB L2)",
                  "parallelism": "1 GPU", "launch": "CUDA graph of the step; programmatic dependent launch with static "
                                                    "weights (dg_set_static_weights(1))"}
        scaling = "weak"
    else:
        r = run_stack(args, dev, rank, world, layers=args.layers)
        detail = []
        for m, t_ms in zip(STACK_MS, r["per_m_ms"]):
            gbs = r["pass_bytes"] / (t_ms * 1e-3) / 1e9
            detail.append({"M": m, "ms_per_pass": t_ms, "GBps_all_gpus": gbs, "frac_hbm": gbs / (hbm_gbs * world)})
        top = max(range(len(STACK_MS)), key=lambda i: r["per_m_ms"][i])
        roofline = {"bound": "hbm", "kernel": f"gemv_kernel<NVFP4, M={STACK_MS[top]}, bf16> (+ all-gather)",
                    "achieved": detail[top]["GBps_all_gpus"] / world, "peak": hbm_gbs, "unit": "GB/s",
                    "frac": detail[top]["frac_hbm"], "traffic": None, "peak_kind": peak_kind, "per_m": detail}
        config = {"workload": f"stack: NVFP4 W4A16, {args.layers or 80} layers x (qkv 8192->10240, o 8192->8192, "
                              "gate_up 8192->57344, down 28672->8192), one pass at each M in {1,8,16} per step",
                  "l2": f"every projection has its own weights ({r['pass_bytes'] / world / 1e9:.1f} GB per GPU)",
                  "parallelism": f"output columns sharded over {world} GPU(s); gather: {r['gather']}"}
        scaling = "strong"

    if rank != 0:
        if world > 1:
            leave_distributed()
        return
    value = r["bytes_per_step"] / (r["ms_per_step"] * 1e-3) / 1e12
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config, "clocks": r["clocks"],
            "e2e": {"value": r["bytes_per_step"] / r["e2e_s"] / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
            "gpu_launches": r["launches"], "roofline": roofline}
    if world == 1:
        sec, nbytes = cpu_reference_sample(2048, reps=3)
        line["cpu_baseline"] = {"value": nbytes / sec / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
                                "kind": "port",
                                "sample": "2048 of 28672 output channels of workload c1 at each M in {1,2,4,8,16}: "
                                          "FP32 dequantise + FP32 matmul with torch on the host"}
    print(json.dumps(line), flush=True)
    if world > 1:
        leave_distributed()


if __name__ == "__main__":
    main()
