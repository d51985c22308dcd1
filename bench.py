"""Benchmark of the decode-GEMV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--gather fused|fused-overlap|nccl]

Metric: weight-stream throughput (algorithmic weight bytes / time, TB/s), the reference's headline for this path.

Workload (the same at every N, so that the 1 -> 8 GPU curve is one workload): the 70B-shaped NVFP4 projection stack,
80 layers x {qkv 8192->10240, o 8192->8192, gate_up 8192->57344, down 28672->8192}, 38.5 GB of weights, output columns
sharded over the N ranks. A step = one pass over the stack at each M in {1, 8, 16}; a pass is one CUDA-graph replay per
rank; on N > 1 GPUs every GEMV ends with the all-gather of its outputs (fused into the kernel: peer stores over NVLink;
`--gather nccl` runs an NCCL all-gather after every GEMV instead). Total work is fixed as N grows ("strong").

The line rank 0 prints carries
  value         device-timed (CUDA events, barrier + synchronize on both sides, max over ranks), inputs resident in HBM
  e2e           the same step driven from host buffers: activations copied up from pinned memory and every role's
                gathered output copied back inside the timed region
  roofline      for the kernel with the largest share of the step (NVFP4, M = 16, gate_up), timed live; per_m = the
                passes; per_config (N = 1) = the single-GPU configurations C0-C3 (NVFP4 4096^2, FP8 28672x8192, MXFP8
                13824x5120, BF16 8192^2): median / min / max of 7 trials of graph replays over rotating weight copies,
                against the HBM peak and the FP32-FMA ceiling, each checked against the CPU oracle on sampled rows, with
                the reference's own sm_100a kernel timed beside it where that comparator was built (gpu_reference_us)
  parity        after the timed region: N > 1: every rank recomputes the last layer's four projections from the whole
                matrices on its own GPU and compares them bit for bit with what the sharded pass gathered; N = 1: the
                same outputs against the CPU oracle on sampled rows, row i bit-identical across M, replays identical
  cpu_baseline  (N = 1) the reference tests' dequantize-then-matmul on the host cores, on a bounded sample
`--impl reference` times that CPU path alone on a bounded sample of the same workload (rank 0 only).
"""
from __future__ import annotations

import argparse
import ctypes
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

STACK_MS = (1, 8, 16)
METRIC = "decode_gemv_weight_stream"
UNIT = "TB/s"
FMA_PER_CLK = 148 * 128
# single-GPU configurations: id, format, N, K, row counts timed here (the tests sweep every M)
CONFIGS = (("C0", "nvfp4", 4096, 4096, (1,)),
           ("C1", "fp8", 28672, 8192, (1, 2, 4, 8, 16)),
           ("C2", "mxfp8", 13824, 5120, (1, 4, 16)),
           ("C3", "bf16", 8192, 8192, (1, 2, 4, 8, 16)))
TRIALS = 7
TRIAL_MS = 50.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def ncu_traffic(key):
    """dram bytes per launch of a kernel from the tracked ncu summary (profiles/ncu_traffic.json), or None."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            entry = json.load(f).get(key)
        return entry and entry.get("dram_bytes")
    except OSError:
        return None


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


def trials_of(fn, per_call=1, barrier=None, reduce_max=None):
    """Median / min / max over TRIALS trials of the device time of one fn(), each trial at least TRIAL_MS long.
    per_call: GEMV calls inside one fn(). Returns microseconds per call."""
    once = time_region(fn, 1, barrier)
    if reduce_max:
        once = reduce_max(once)      # every rank must make the same number of calls: they hold collectives
    reps = max(1, int(TRIAL_MS / max(once, 1e-3)) + 1)
    times = []
    for _ in range(TRIALS):
        t = time_region(fn, reps, barrier) / reps
        if reduce_max:
            t = reduce_max(t)
        times.append(t * 1e3 / per_call)
    return {"us": statistics.median(times), "us_min": min(times), "us_max": max(times), "trials": TRIALS,
            "ms_per_trial": reps * once}


def graph_of(fn, dev):
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


def stack_config(world, layers, gather):
    """The `config` both arms print for the same N."""
    return {"workload": f"stack: NVFP4 W4A16, {layers} layers x (qkv 8192->10240, o 8192->8192, gate_up 8192->57344, "
                        "down 28672->8192), one pass at each M in {1,8,16} per step",
            "l2": "every projection has its own weights (38.5 GB in total; per GPU 38.5 GB / N >> the 126 MB L2)",
            "parallelism": f"output columns sharded over {world} GPU(s)",
            "gather": "none (1 GPU)" if world == 1 else gather}


# ----- CPU arm: the reference tests' dequantize-then-matmul on the host cores -----------------------------------------

CPU_SAMPLE_DIV = 64     # the CPU arm multiplies 1 / 64 of every projection's output channels of one layer


def cpu_stack_sample(reps=1):
    """One bounded sample of the stack workload on the host: for each of a layer's four projections, N / 64 output
    channels of an NVFP4 matrix in the workload's distribution, dequantised to FP32 and multiplied in FP32 at each M
    in {1, 8, 16} (the dequantisation is part of every call, as in the reference's dequantize-then-matmul path).
    Returns (seconds per step of the sample, weight bytes the sample streams per step, description)."""
    from oracle import decode_gemv_oracle as oc
    from oracle import workloads as wl
    mats = [(wl.cfg_nvfp4(n // CPU_SAMPLE_DIV, k, seed=70 + i), k) for i, (_, k, n) in enumerate(wl.STACK_ROLES)]
    xs = {(m, k): wl.activations(m, k, seed=8 + m) for m in STACK_MS for _, k in mats}
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        for m in STACK_MS:
            for tensors, k in mats:
                oc.gemv_fp32(xs[(m, k)], oc.dequant_fp32("nvfp4", tensors))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    nbytes = len(STACK_MS) * sum(wl.weight_bytes("nvfp4", n // CPU_SAMPLE_DIV, k) for _, k, n in wl.STACK_ROLES)
    what = (f"1/{CPU_SAMPLE_DIV} of the output channels of each of one layer's four projections at each M in "
            f"{list(STACK_MS)}: FP32 dequantise + FP32 matmul with torch on the host")
    return best, nbytes, what


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)     # torch.distributed.run exports OMP_NUM_THREADS=1
    for _ in range(max(args.warmup, 1)):
        cpu_stack_sample()
    times = []
    for _ in range(args.steps):
        dt, nbytes, what = cpu_stack_sample()
        times.append(dt)
    sec = sum(times) / len(times)
    value = nbytes / sec / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": stack_config(args.gpus, args.layers or 80, args.gather),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": what},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----- the stack on N GPUs ---------------------------------------------------------------------------------------------

def stack_parity(model, runs, dev, rank, world):
    """Untimed gate after the timed region (see the module docstring). Returns the `parity` object; raises on a
    mismatch."""
    from crit_kernels_b200 import stack as stk
    from oracle import decode_gemv_oracle as oc
    roles = model.roles
    layer = model.layers - 1
    checked, oracle_rows = 0, 0
    first_rows = {}
    for m in STACK_MS:
        run = runs[m]
        run.replay()
        torch.cuda.synchronize()
        got = {role: t.clone() for role, t in run.outputs().items()}
        run.replay()
        torch.cuda.synchronize()
        for role, t in run.outputs().items():
            if not torch.equal(t.view(torch.int16), got[role].view(torch.int16)):
                raise RuntimeError(f"parity: M={m} {role}: two replays differ")
        for idx, (role, k, n) in enumerate(roles):
            codes, scales, inverse = stk.ShardedStack.full_matrix(model.seed, layer, idx, roles[idx], dev)
            if world > 1:
                want = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
                model.kernel.gemv(run.x[role], codes, scales, inverse, want)
                torch.cuda.synchronize()
                if not torch.equal(want.view(torch.int16), got[role].view(torch.int16)):
                    raise RuntimeError(f"parity: M={m} {role}: the gathered output differs from the single-GPU output")
            else:
                rows = torch.arange(0, n, max(1, n // 48))[:48]
                sub = (codes[rows].cpu(), scales[rows].cpu(), inverse[rows].cpu())
                exact = oc.gemv_exact(run.x[role].cpu(), oc.values_of("nvfp4", sub))
                err = oc.max_rel_error(got[role][:, rows].cpu(), exact)
                if not err <= 1e-2:
                    raise RuntimeError(f"parity: M={m} {role}: max relative error {err} against the oracle")
                oracle_rows += len(rows)
            row0 = got[role][0].view(torch.int16)
            if role in first_rows and not torch.equal(first_rows[role], row0):
                raise RuntimeError(f"parity: {role}: row 0 differs between M={m} and M={STACK_MS[0]}")
            first_rows.setdefault(role, row0)
            checked += 1
            del codes, scales, inverse
    out = {"checked": True, "ranks": world, "projections": checked, "bit_equal": True,
           "row_invariant_across_m": True, "replays_identical": True}
    if world == 1:
        out["oracle_rows"] = oracle_rows
        out["oracle_tolerance"] = "max relative error <= 1e-2 of the FP64 product, BF16 outputs"
    else:
        out["against"] = "the whole matrices multiplied on each rank's own GPU (last layer, 4 projections x 3 M)"
    return out


def run_stack(args, dev, rank, world):
    import torch.distributed as dist
    from crit_kernels_b200 import cabi
    from crit_kernels_b200 import stack as stk
    from oracle import workloads as wl
    layers = args.layers or wl.STACK_LAYERS
    model = stk.ShardedStack.random(layers, wl.STACK_ROLES, rank, world, dev, seed=99, gather=args.gather)
    runs = {m: model.capture(m) for m in STACK_MS}
    barrier = (lambda: dist.barrier()) if world > 1 else None

    def reduce_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def step():
        for m in STACK_MS:
            runs[m].replay()

    with ClockSampler(dev.index or 0) as clocks:
        for _ in range(args.warmup):
            step()
        ms_step = reduce_max(time_region(step, args.steps, barrier) / args.steps)
        per_m = [trials_of(runs[m].replay, 1, barrier, reduce_max) for m in STACK_MS]
        # the kernel with the largest share: NVFP4 M = 16 on gate_up (with its all-gather on N > 1), timed alone over
        # the layers' distinct weights
        m_top = STACK_MS[-1]
        top = runs[m_top]
        gate = [p for p in model.projections if p.role == "gate_up"]

        def gate_ups():
            for p in gate[:16]:
                if top.fused:
                    top._gemv_allgather(p)
                else:
                    model.kernel.gemv(top.x[p.role], p.codes, p.scales, p.inverse, top.shard[p.role])
        cabi.load().dg_set_static_weights(1)
        g_top = graph_of(gate_ups, dev)
        cabi.load().dg_set_static_weights(0)
        top_kernel = trials_of(g_top.replay, min(16, len(gate)), barrier, reduce_max)
        del g_top
        # the same passes with several GEMVs a launch (legal only because the stack's GEMVs are independent; reported
        # beside the default, never instead of it): a layer's four, and the whole pass
        batched = []
        if args.gather == "fused":
            for per_launch in (4, len(model.projections)):
                variant = model.with_batch(per_launch)
                entry = {"gemvs_per_launch": per_launch, "ms_per_pass": [], "bit_equal_to_default": True}
                for m in STACK_MS:
                    vrun = variant.capture(m)
                    entry["ms_per_pass"].append(trials_of(vrun.replay, 1, barrier, reduce_max)["us"] / 1e3)
                    runs[m].replay()
                    torch.cuda.synchronize()
                    if barrier:
                        barrier()
                    for role, t in vrun.outputs().items():
                        if not torch.equal(t.view(torch.int16), runs[m].outputs()[role].view(torch.int16)):
                            entry["bit_equal_to_default"] = False
                    if barrier:
                        barrier()
                    del vrun
                if not entry["bit_equal_to_default"]:
                    raise RuntimeError(f"{per_launch} GEMVs a launch: outputs differ from the default path's")
                batched.append(entry)
        # one GPU: the down projection fed by SwiGLU of the layer's gate_up output, as two steps and fused
        fusion = None
        if world == 1:
            fusion = {"what": "each layer's down projection reads bf16(SwiGLU(gate_up sums)): 'unfused' = gate_up GEMV "
                              "(FP32 out) + SwiGLU kernel, 'fused' = SwiGLU in the gate_up GEMV's epilogue "
                              "(dg_enqueue_nvfp4_gate_up_swiglu); then the down GEMV in both",
                      "ms_per_pass": {}, "bit_equal": True}
            for m in STACK_MS:
                two, one = model.with_swiglu("unfused").capture(m), model.with_swiglu("fused").capture(m)
                fusion["ms_per_pass"][str(m)] = {"unfused": trials_of(two.replay)["us"] / 1e3,
                                                 "fused": trials_of(one.replay)["us"] / 1e3}
                torch.cuda.synchronize()
                if not torch.equal(two.outputs()["down"].view(torch.int16), one.outputs()["down"].view(torch.int16)):
                    fusion["bit_equal"] = False
                del two, one
            if not fusion["bit_equal"]:
                raise RuntimeError("SwiGLU fused into the down projection gives other bits than the two-step path")
        # end to end: activations from pinned host memory, every role's gathered output back
        for _ in range(2):
            for m in STACK_MS:
                runs[m].replay_e2e()
        if barrier:
            barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            for m in STACK_MS:
                runs[m].replay_e2e()
        torch.cuda.synchronize()
        e2e_s = reduce_max((time.perf_counter() - t0) / args.steps)
    parity = stack_parity(model, runs, dev, rank, world)
    status = cabi.load().dg_take_status()
    if status:
        raise RuntimeError(f"a bounded wait inside a kernel ran out during the run (status word {status}): the "
                           "timings above are not those of complete passes")
    full_bytes = layers * sum(wl.weight_bytes("nvfp4", n, k) for _, k, n in wl.STACK_ROLES)
    gate_bytes = wl.weight_bytes("nvfp4", 57344 // world, 8192)
    return {"ms_per_step": ms_step, "e2e_s": e2e_s, "per_m": per_m, "bytes_per_step": full_bytes * len(STACK_MS),
            "pass_bytes": full_bytes, "clocks": clocks.summary(), "top_kernel": top_kernel, "top_bytes": gate_bytes,
            "h2d": sum(runs[m].h2d_bytes for m in STACK_MS), "d2h": sum(runs[m].d2h_bytes for m in STACK_MS),
            "launches": args.steps * sum(runs[m].kernel_launches for m in STACK_MS), "gather": model.gather_kind,
            "parity": parity, "layers": layers, "model": model, "runs": runs, "batched": batched, "fusion": fusion}


# ----- single-GPU configurations C0-C3 -----------------------------------------------------------------------------

def make_copies(fmt, n, k, dev, copies):
    """`copies` matrices of one configuration in its benchmark distribution, generated on the device."""
    g = torch.Generator(device=dev).manual_seed(4321)
    out = []
    for _ in range(copies):
        if fmt == "nvfp4":
            c = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=g)
            s = torch.exp2(torch.rand(n, k // 16, device=dev, generator=g) * 6 - 4).to(torch.float8_e4m3fn)
            out.append((c, s.view(torch.uint8), torch.ones(n, device=dev)))
        elif fmt == "fp8":
            c = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.float8_e4m3fn).view(torch.uint8)
            out.append((c, (torch.rand(n, device=dev, generator=g) * 1.5 + 0.5) / 64))
        elif fmt == "mxfp8":
            w = (torch.randn(n, k, device=dev, generator=g) * 0.02).view(n, k // 32, 32)
            _, e = torch.frexp(w.abs().amax(dim=-1))
            shared = torch.where(w.abs().amax(dim=-1) > 0, e - 1 - 8, torch.zeros_like(e)).clamp(-127, 127).float()
            c = (w / torch.exp2(shared)[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
            out.append((c.view(n, k), (shared + 127).to(torch.uint8)))
        else:
            out.append(((torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16),))
    return out


def run_configs(dev, hbm_gbs, sm_mhz):
    """C0-C3 on one GPU: per (configuration, M) the time of a call (graph replays over rotating weight copies larger
    than L2 in total), the same for the reference's sm_100a kernel when oracle/_ref holds it, and an oracle check."""
    import crit_kernels_b200
    from oracle import build_ref
    from oracle import decode_gemv_oracle as oc
    from oracle import workloads as wl
    k_mod = crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)
    ref = build_ref.load()
    ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    entries = []
    for cid, fmt, n, k, ms in CONFIGS:
        nbytes = wl.weight_bytes(fmt, n, k)
        copies = max(2, min(32, int(1.0e9 // nbytes)))          # >= 256 MB of distinct weights in rotation
        while copies * nbytes < 256e6:
            copies += 1
        ws = make_copies(fmt, n, k, dev, copies)
        x16 = wl.activations(16, k, seed=8).to(dev)
        calls = max(copies, 8)
        rows = torch.arange(0, n, max(1, n // 64))[:64]
        values = oc.values_of(fmt, tuple(t[rows].cpu() if t.dim() and t.shape[0] == n else t.cpu() for t in ws[0]))
        row0 = None
        for m in ms:
            x = x16[:m].contiguous()
            out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)

            def ours(i):
                t = ws[i % copies]
                if fmt == "nvfp4":
                    k_mod.gemv(x, t[0], t[1], t[2], out)
                elif fmt == "bf16":
                    k_mod.gemv_bf16(x, t[0], out)
                else:
                    k_mod.gemv_fp8(x, t[0], t[1], out)

            def theirs(i):
                t = ws[i % copies]
                st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
                if fmt == "nvfp4":
                    rc = ref.ref_enqueue_nvfp4(ptr(x), x.stride(0), 1, ptr(t[0]), ptr(t[1]), 0, ptr(t[2]), ptr(out),
                                               out.stride(0), 1, m, n, k, st)
                elif fmt == "bf16":
                    rc = ref.ref_enqueue_bf16(ptr(x), x.stride(0), ptr(t[0]), ptr(out), out.stride(0), 1, m, n, k, st)
                else:
                    mx = fmt == "mxfp8"
                    rc = ref.ref_enqueue_fp8(ptr(x), x.stride(0), 1, ptr(t[0]), None if mx else ptr(t[1]),
                                             ptr(t[1]) if mx else None, ptr(out), out.stride(0), 1, m, n, k, st)
                if rc:
                    raise RuntimeError(f"reference kernel refused {cid} M={m}: cudaError {rc}")

            def many(fn):
                return lambda: [fn(i) for i in range(calls)]
            # oracle check and invariants on copy 0
            ours(0)
            torch.cuda.synchronize()
            first = out.clone()
            err = oc.max_rel_error(first[:, rows].cpu(), oc.gemv_exact(x.cpu(), values))
            if not err <= 1e-2:
                raise RuntimeError(f"{cid} M={m}: max relative error {err} against the oracle")
            ours(0)
            torch.cuda.synchronize()
            if not torch.equal(out.view(torch.int16), first.view(torch.int16)):
                raise RuntimeError(f"{cid} M={m}: two calls differ")
            if row0 is not None and not torch.equal(row0, first[0].view(torch.int16)):
                raise RuntimeError(f"{cid}: row 0 differs between M={m} and M={ms[0]}")
            row0 = first[0].view(torch.int16).clone()
            g = graph_of(many(ours), dev)
            t_ours = trials_of(g.replay, calls)
            del g
            entry = {"config": cid, "fmt": fmt, "N": n, "K": k, "M": m, "us": t_ours["us"], "us_min": t_ours["us_min"],
                     "us_max": t_ours["us_max"], "trials": TRIALS, "ms_per_trial": t_ours["ms_per_trial"],
                     "weight_bytes": nbytes, "copies_in_rotation": copies,
                     "GBps": nbytes / t_ours["us"] / 1e3, "frac_hbm": nbytes / t_ours["us"] / 1e3 / hbm_gbs,
                     "frac_fp32_fma": m * n * k / (t_ours["us"] * 1e-6) / (FMA_PER_CLK * sm_mhz * 1e6),
                     "oracle_max_rel_err": err, "gpu_reference_us": None, "speedup_vs_gpu_reference": None}
            if ref is not None:
                g = graph_of(many(theirs), dev)
                t_ref = trials_of(g.replay, calls)
                del g
                entry["gpu_reference_us"] = t_ref["us"]
                entry["gpu_reference_us_minmax"] = [t_ref["us_min"], t_ref["us_max"]]
                entry["speedup_vs_gpu_reference"] = t_ref["us"] / t_ours["us"]
            entries.append(entry)
        del ws
        torch.cuda.empty_cache()
    return entries


def host_cost(dev):
    """Host time of one eager (un-captured) call through the public op: what a caller that does not use CUDA graphs
    pays per GEMV. 1000 calls of a small NVFP4 GEMV, wall clock around the enqueues only."""
    import crit_kernels_b200
    from oracle import workloads as wl
    k_mod = crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)
    n, k = 1024, 4096
    c, s, i = (t.to(dev) for t in wl.cfg_nvfp4(n, k))
    x = wl.activations(1, k).to(dev)
    out = torch.empty(1, n, dtype=torch.bfloat16, device=dev)
    for _ in range(50):
        k_mod.gemv(x, c, s, i, out)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(1000):
        k_mod.gemv(x, c, s, i, out)
    dt = time.perf_counter() - t0
    torch.cuda.synchronize()
    return dt / 1000 * 1e6


def run_case(args):
    """`--case fmt:M:N:K`: seeded inputs in the benchmark distributions, --warmup + --steps calls, device time: the
    small program that profilers capture."""
    import crit_kernels_b200
    from oracle import workloads as wl
    dev = torch.device("cuda", 0)
    k = crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)
    if args.case.split(":")[0] in ("dequant", "quant_fp8", "quant_nvfp4"):
        # the streaming kernels either side of the GEMVs: `dequant:N:K` (NVFP4 -> BF16), `quant_fp8:M:K`,
        # `quant_nvfp4:M:K` (BF16 rows -> FP8 per row / NVFP4), two buffers in rotation, bytes read + written
        kind, a, b = args.case.split(":")
        a, b = int(a), int(b)
        g = torch.Generator(device=dev).manual_seed(5)
        if kind == "dequant":
            sets = []
            for _ in range(2):
                c, s_, i = (t.to(dev) for t in wl.cfg_nvfp4(a, b))
                sets.append((c, s_, i, torch.empty(a, b, dtype=torch.bfloat16, device=dev)))
            calls = [lambda t=t: k.decode(t[0], t[1], t[2], t[3]) for t in sets]
            nbytes = a * b // 2 + a * b // 16 + 4 * a + 2 * a * b
        else:
            xs = [(torch.randn(a, b, device=dev, generator=g) * 3).to(torch.bfloat16) for _ in range(2)]
            if kind == "quant_fp8":
                outs = [(torch.empty(a, b, dtype=torch.uint8, device=dev), torch.empty(a, device=dev)) for _ in xs]
                calls = [lambda x=x, o=o: k.quantize_fp8_rows(x, o[0], o[1]) for x, o in zip(xs, outs)]
                nbytes = 2 * a * b + a * b + 4 * a
            else:
                tiled = ((a + 127) // 128) * 128 * ((b // 16 + 3) // 4) * 4
                outs = [(torch.empty(a, b // 2, dtype=torch.uint8, device=dev),
                         torch.empty(tiled, dtype=torch.uint8, device=dev)) for _ in xs]
                calls = [lambda x=x, o=o: k.quantize_nvfp4(x, 300.0, o[0], o[1]) for x, o in zip(xs, outs)]
                nbytes = 2 * a * b + a * b // 2 + tiled
        both = lambda: [c() for c in calls]
        for _ in range(args.warmup):
            both()
        ms = time_region(both, args.steps) / (2 * args.steps)
        print(json.dumps({"case": args.case, "us": ms * 1e3, "GBps": nbytes / ms / 1e6, "bytes_read_and_written": nbytes}),
              flush=True)
        return
    fmt, m, n, kk = args.case.split(":")
    m, n, kk = int(m), int(n), int(kk)
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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="stack depth (default 80)")
    ap.add_argument("--gather", default="fused", choices=["fused", "fused-overlap", "nccl"],
                    help="N > 1 GPUs: all-gather fused into the GEMV epilogue (default), the same with the arrivals "
                         "collected once per pass (legal only because the stack's GEMVs are independent), or NCCL")
    ap.add_argument("--no-configs", action="store_true", help="skip the single-GPU configurations C0-C3")
    ap.add_argument("--case", default=None, metavar="FMT:M:N:K",
                    help="run `--steps` calls of one GEMV (fmt in bf16, fp8, mxfp8, nvfp4) and exit: the small case "
                         "profilers capture; also dequant:N:K, quant_fp8:M:K, quant_nvfp4:M:K")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(args.warmup, 3)
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
    hbm_gbs, peak_kind = measured_peaks()

    r = run_stack(args, dev, rank, world)
    sm_mhz = r["clocks"]["sm_mhz"] or 1965.0
    detail = []
    for m, t in zip(STACK_MS, r["per_m"]):
        gbs = r["pass_bytes"] / (t["us"] * 1e-6) / 1e9
        detail.append({"M": m, "ms_per_pass": t["us"] / 1e3, "ms_min": t["us_min"] / 1e3, "ms_max": t["us_max"] / 1e3,
                       "trials": TRIALS, "GBps_all_gpus": gbs, "frac_hbm": gbs / (hbm_gbs * world)})
    top_us = r["top_kernel"]["us"]
    top_gbs = r["top_bytes"] / top_us / 1e3
    n_top = 57344 // world
    roofline = {"bound": "hbm", "kernel": f"gemv_kernel<NVFP4, M=16, bf16> on gate_up {n_top} x 8192"
                                          + (" with its all-gather" if world > 1 else ""),
                "achieved": top_gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": top_gbs / hbm_gbs,
                "traffic": ncu_traffic(f"nvfp4:16:{n_top}:8192"), "peak_kind": peak_kind,
                "us": top_us, "us_minmax": [r["top_kernel"]["us_min"], r["top_kernel"]["us_max"]],
                "algorithmic_bytes": r["top_bytes"],
                "frac_fp32_fma_ceiling": 16 * n_top * 8192 / (top_us * 1e-6) / (FMA_PER_CLK * sm_mhz * 1e6),
                "note": "M = 16 on CUDA cores is bound by FP32 FMA issue, not HBM (16 FMAs per 4-bit weight): the FMA "
                        "floor of this call is 16 N K / (148 x 128 x clock)",
                "per_m": detail}
    model, runs = r.pop("model"), r.pop("runs")
    per_config, host_us = None, None
    if world == 1:
        runs.clear()
        del model
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        host_us = host_cost(dev)
        if not args.no_configs:
            per_config = run_configs(dev, hbm_gbs, sm_mhz)
            roofline["per_config"] = per_config
    if rank != 0:
        if world > 1:
            runs.clear()
            leave_distributed()
        return
    value = r["bytes_per_step"] / (r["ms_per_step"] * 1e-3) / 1e12
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": stack_config(world, r["layers"], args.gather), "clocks": r["clocks"],
            "e2e": {"value": r["bytes_per_step"] / r["e2e_s"] / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
            "gpu_launches": r["launches"], "roofline": roofline, "parity": r["parity"], "gather": r["gather"],
            "batched_launches": {"note": "the same passes with several GEMVs a launch (dg_enqueue_batch): legal only "
                                         "because this workload's GEMVs do not read each other's outputs; the headline "
                                         "numbers are the one-launch-per-GEMV chain", "modes": r["batched"]}}
    if host_us is not None:
        line["host_us_per_eager_call"] = host_us
    if r["fusion"] is not None:
        line["swiglu_fusion"] = r["fusion"]
    if world == 1:
        sec, nbytes, what = cpu_stack_sample(reps=2)
        line["cpu_baseline"] = {"value": nbytes / sec / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
                                "kind": "port", "sample": what}
    print(json.dumps(line), flush=True)
    if world > 1:
        runs.clear()
        leave_distributed()


if __name__ == "__main__":
    main()
