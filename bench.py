#!/usr/bin/env python
"""RMSNorm forward + VJP throughput on B200 (rows/s), with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one forward + VJP pass over the workload's rows: rmsnorm_fwd, rmsnorm_bwd (dx fused
with the dgamma partials), the fixed-order dgamma reduction and, for N > 1, the NCCL all-reduce
of the fp64 dgamma sums.  N > 1 is launched by torchrun, one rank per GPU; every rank holds the
same number of rows (weak scaling) and `value` counts the rows of all ranks.

Workload (default): x [16,2048,4096] fp32 ~ N(0,1), gamma = 1 + 0.02 N(0,1), gy ~ N(0,1),
eps 1e-5 -- 32768 rows per GPU, synthetic, seed 0.  Inputs (2 x 537 MB) and outputs are far
larger than the 126 MB L2, so no flush is needed between iterations.

Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (rows per GPU, hidden, dtype, eps)
    "rmsnorm_fwd_vjp_fp32_16x2048x4096": (16 * 2048, 4096, "float32", 1e-5),
    "rmsnorm_fwd_vjp_fp32_8x512x1024": (8 * 512, 1024, "float32", 1e-6),
    "rmsnorm_fwd_vjp_fp32_8192x4096": (8192, 4096, "float32", 1e-5),     # small case for ncu captures
    "rmsnorm_fwd_vjp_bf16_16384x8192": (16384, 8192, "bfloat16", 1e-6),  # small case for ncu captures
    "rmsnorm_fwd_vjp_bf16_65536x8192": (65536, 8192, "bfloat16", 1e-6),
    "rmsnorm_fwd_vjp_bf16_65536x1000": (65536, 1000, "bfloat16", 1e-6),
    "rmsnorm_fwd_vjp_bf16_65536x5120": (65536, 5120, "bfloat16", 1e-6),
    "rmsnorm_fwd_vjp_bf16_65536x12288": (65536, 12288, "bfloat16", 1e-6),
    # configuration 5: 524288 rows in total, split evenly over the ranks (strong scaling)
    "rmsnorm_fwd_vjp_bf16_sharded_64x8192x8192": (64 * 8192, 8192, "bfloat16", 1e-6),
}
STRONG_SCALING = {"rmsnorm_fwd_vjp_bf16_sharded_64x8192x8192"}
# configuration 4: 32 fused residual-add + RMSNorm layers, forward + VJP as one CUDA graph (C++ host layer)
STACK_WORKLOADS = {"residual_stack_fp32_32x4x4096x4096": (32, 4 * 4096, 4096, 0)}
# Next rows of the path, same bar: one forward + VJP pass per step, per-kernel CUDA events.
OP_WORKLOADS = {
    # name: (op, rows, hidden, dtype)
    "layernorm_fwd_vjp_fp32_32768x4096": ("layernorm", 32768, 4096, "float32"),
    "layernorm_fwd_vjp_bf16_65536x8192": ("layernorm", 65536, 8192, "bfloat16"),
    "softmax_fwd_vjp_fp32_32768x4096": ("softmax", 32768, 4096, "float32"),
    "softmax_fwd_vjp_bf16_65536x8192": ("softmax", 65536, 8192, "bfloat16"),
    "logsumexp_fwd_vjp_fp32_32768x4096": ("logsumexp", 32768, 4096, "float32"),
    "layernorm_fwd_vjp_fp32_8192x4096": ("layernorm", 8192, 4096, "float32"),     # small cases for ncu captures
    "softmax_fwd_vjp_fp32_8192x4096": ("softmax", 8192, 4096, "float32"),
}
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one backward launch, from the ncu
# captures summarised under profiles/ (taken on a smaller case of the same kernel and scaled by rows).
NCU_TRAFFIC = {
    "rmsnorm_fwd_vjp_fp32_16x2048x4096": {
        "bwd_dram_bytes_per_launch": 1475391488,
        "source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on the 8192 x 4096 case (profiles/rmsnorm_bwd_staged_fp32_8192x4096.md), scaled x4 by rows; writes still dirty in L2 at kernel end are not counted by the DRAM counter"},
    "rmsnorm_fwd_vjp_bf16_sharded_64x8192x8192": {
        "bwd_dram_bytes_per_launch": 24952111104,
        "source": "ncu capture on the 16384 x 8192 bf16 case (profiles/rmsnorm_bwd_staged_bf16_16384x8192.md), scaled x32 by rows (per rank at N=1)"},
}
DEFAULT_WORKLOAD = "rmsnorm_fwd_vjp_fp32_16x2048x4096"
METRIC = "rmsnorm_fwd_vjp_rows_per_s"
UNIT = "rows/s"
SPEC_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def bytes_per_row(hidden, elem):
    """Algorithmic traffic: fwd reads x, writes y, writes rstd; vjp reads x, gy, rstd, writes dx."""
    return 5 * hidden * elem + 8


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            p = [s.strip() for s in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
                power.append(float(p[3]))
            except ValueError:
                continue
            for name, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm
def _reference_build():
    """oracle/_ref (the reference's own sources over a stand-in tensor library) if it was built."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        import ref_ffi as REF

        if REF.available():
            REF.lib()
            return REF
    except Exception:
        pass
    return None


REF_KIND_NOTE = ("the reference's own op builders and autodiff engine (cgadimpl/src/{core,ops,autodiff}, compiled "
                 "unmodified into oracle/_ref) over a CPU stand-in for its absent OwnTensor library, OpenMP")
PORT_KIND_NOTE = "op-by-op fp32 restatement of the reference composition (oracle/agb_oracle.c), OpenMP"


def cpu_pass(hidden, eps, sample_rows, reps, seed=0):
    """Times the reference's CPU path (all host threads) on a bounded sample of the workload.
    Returns (rows/s, threads, seconds per pass, kind, note)."""
    REF = _reference_build()
    if REF is not None and abs(eps - 1e-5) < 1e-12:     # the reference hard-codes eps = 1e-5
        cores = REF.use_all_cores()
        REF.set_reduce_fp64(False)
        secs = min(REF.time_fwd_bwd(sample_rows, hidden, 1, 1) for _ in range(max(1, reps)))
        return sample_rows / secs, cores, secs, "reference", REF_KIND_NOTE
    import numpy as np

    import oracle_ffi as O

    O.use_all_cores()
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((sample_rows, hidden), dtype=np.float32)
    gy = rng.standard_normal((sample_rows, hidden), dtype=np.float32)
    gamma = (1 + 0.02 * rng.standard_normal(hidden)).astype(np.float32)
    O.rmsnorm_fwd_bwd(x, gamma, gy, eps, O.RED_F32)  # warm-up (page faults, thread pool)
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        O.rmsnorm_fwd_bwd(x, gamma, gy, eps, O.RED_F32)
        ts.append(time.perf_counter() - t0)
    best = min(ts)
    return sample_rows / best, O.num_threads(), best, "port", PORT_KIND_NOTE


def cpu_fused_pass(hidden, eps, sample_rows, reps, seed=0):
    """The row-fused CPU variant of the same arithmetic (one read of each input per pass), all host threads."""
    import numpy as np

    if os.path.join(ROOT, "tests") not in sys.path:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_ffi as O

    O.use_all_cores()
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((sample_rows, hidden), dtype=np.float32)
    gy = rng.standard_normal((sample_rows, hidden), dtype=np.float32)
    gamma = (1 + 0.02 * rng.standard_normal(hidden)).astype(np.float32)
    O.rmsnorm_fwd_bwd(x, gamma, gy, eps, fused=True)
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        O.rmsnorm_fwd_bwd(x, gamma, gy, eps, fused=True)
        ts.append(time.perf_counter() - t0)
    return sample_rows / min(ts), O.num_threads(), min(ts)


def run_reference_arm(args, rank, world):
    """The reference's own CPU implementation of the path on the host cores: oracle/_ref when it was
    built (the reference's unmodified graph / op / autodiff sources over a stand-in tensor library),
    else the C restatement.  cgadimpl's own build cannot run here (OwnTensor, MLIR, Nova absent).
    Each step is one forward + backward pass over a bounded sample of the workload.  Rank 0 only."""
    if rank != 0:
        return
    rows, hidden, dtype, eps = WORKLOADS[args.workload]
    sample_rows = min(rows, 4096)
    REF = _reference_build()
    if REF is not None and abs(eps - 1e-5) < 1e-12:
        cores = REF.use_all_cores()
        REF.set_reduce_fp64(False)
        secs = REF.time_fwd_bwd(sample_rows, hidden, args.steps, max(1, args.warmup))
        kind, note = "reference", REF_KIND_NOTE
    else:
        import numpy as np

        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_ffi as O

        cores = O.use_all_cores()
        rng = np.random.default_rng(0)
        x = rng.standard_normal((sample_rows, hidden), dtype=np.float32)
        gy = rng.standard_normal((sample_rows, hidden), dtype=np.float32)
        gamma = (1 + 0.02 * rng.standard_normal(hidden)).astype(np.float32)
        for _ in range(max(1, args.warmup)):
            O.rmsnorm_fwd_bwd(x, gamma, gy, eps, O.RED_F32)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            O.rmsnorm_fwd_bwd(x, gamma, gy, eps, O.RED_F32)
        secs = (time.perf_counter() - t0) / args.steps
        kind, note = "port", PORT_KIND_NOTE
    value = sample_rows / secs
    elem = 4 if dtype == "float32" else 2
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "rows_per_gpu": rows, "hidden": hidden, "eps": eps,
                   "io_dtype": dtype, "sample_rows_per_step": sample_rows},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"{sample_rows} of {rows} rows per step; {note}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "hbm_gbs": value * bytes_per_row(hidden, elem) / 1e9,
    }
    print(json.dumps(line), flush=True)


def run_stack(args, rank):
    """Configuration 4 through the C++ host layer: ag::nn::ResidualRMSNormStack captured by
    ag::CudaGraphRunner, timed by cgadimpl_b200/host/build/bench_stack.  One GPU."""
    if rank != 0:
        return
    from cgadimpl_b200.host import build as host_build

    host_build.build()
    layers, rows, hidden, bf16 = STACK_WORKLOADS[args.workload]
    exe = os.path.join(os.path.dirname(host_build.__file__), "build", "bench_stack")
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    r = subprocess.run([exe, str(layers), str(rows), str(hidden), str(args.steps), str(max(3, args.warmup)), str(bf16)],
                       capture_output=True, text=True)
    clocks = sampler.stop()
    if r.returncode != 0:
        raise SystemExit("bench_stack failed:\n" + r.stdout + r.stderr)
    d = json.loads(r.stdout.strip().splitlines()[-1])
    peak, peak_kind = measured_peak()
    print(json.dumps({
        "metric": "residual_rmsnorm_stack_row_layers_per_s", "value": d["row_layers_per_s"], "unit": "row-layers/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": d["ms_per_replay"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "layers": layers, "rows": rows, "hidden": hidden,
                   "cuda_graph_nodes": d["graph_nodes"], "saved_activation_bytes": d["saved_activation_bytes"],
                   "l2": "each layer streams 7*H*s bytes per row (1.9 GB per layer), far beyond the 126 MB L2"},
        "gpu_launches": d["launches_per_replay"] * args.steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": d["gbs"], "peak": peak, "unit": "GB/s", "frac": d["gbs"] / peak,
                     "peak_kind": f"of {peak_kind}", "bytes_per_row_layer": 7 * hidden * (2 if bf16 else 4) + 8,
                     "frac_of_spec_8TBs": d["gbs"] / SPEC_HBM_GBS, "traffic": None},
    }), flush=True)


def run_op(args, rank):
    """LayerNorm / softmax / logsumexp rows: forward + VJP per step on one GPU, each kernel timed with
    CUDA events on the launching stream; roofline per kernel from its algorithmic bytes."""
    if rank != 0:
        return
    import torch

    from cgadimpl_b200 import ops

    op, rows, hidden, dtype_name = OP_WORKLOADS[args.workload]
    dtype = getattr(torch, dtype_name)
    elem = 4 if dtype == torch.float32 else 2
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(rows, hidden, device="cuda", generator=gen) * (3.0 if op != "layernorm" else 1.0)).to(dtype)
    gy = torch.randn(rows, hidden, device="cuda", generator=gen).to(dtype)
    gyr = torch.randn(rows, device="cuda", generator=gen).to(dtype)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    orow = torch.empty(rows, device="cuda", dtype=dtype)
    B = rows * hidden * elem
    if op == "layernorm":
        _, mean, var = ops.layernorm_fwd(x, 1e-5, out=y)
        fwd, bwd = (lambda: ops.layernorm_fwd(x, 1e-5, out=y)), (lambda: ops.layernorm_bwd(x, mean, var, gy, 1e-5, dx=dx))
        fwd_bytes, bwd_bytes, names = 2 * B + 8 * rows, 3 * B + 8 * rows, ("layernorm_fwd_staged", "layernorm_bwd_staged")
    elif op == "softmax":
        fwd, bwd = (lambda: ops.softmax_row(x, out=y)), (lambda: ops.softmax_row_bwd(y, gy, dz=dx))
        fwd_bytes, bwd_bytes, names = 2 * B, 3 * B, ("softmax_fwd_staged<0>", "softmax_bwd_staged")
    else:
        fwd, bwd = (lambda: ops.logsumexp_row(x, out=orow)), (lambda: ops.logsumexp_row_bwd(x, gyr, dz=dx))
        fwd_bytes, bwd_bytes, names = B + rows * elem, 2 * B + rows * elem, ("softmax_fwd_staged<1>", "softmax_fwd_staged<2>")
    warm = max(3, args.warmup)
    for _ in range(warm):
        fwd(); bwd()
    torch.cuda.synchronize()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    time.sleep(0.3)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    l0 = ops.launch_count()
    torch.cuda.synchronize()
    for k in range(args.steps):
        ev[k][0].record(); fwd(); ev[k][1].record(); bwd(); ev[k][2].record()
    torch.cuda.synchronize()
    launches = ops.launch_count() - l0
    clocks = sampler.stop()
    ops.device_status()
    total_ms = ev[0][0].elapsed_time(ev[-1][2])
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    peak, peak_kind = measured_peak()
    fa, ba = fwd_bytes / fwd_ms / 1e6, bwd_bytes / bwd_ms / 1e6
    dom = ("bwd", names[1], ba, bwd_bytes, bwd_ms) if bwd_ms >= fwd_ms else ("fwd", names[0], fa, fwd_bytes, fwd_ms)
    print(json.dumps({
        "metric": f"{op}_fwd_vjp_rows_per_s", "value": rows * args.steps / (total_ms / 1e3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": warm, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "rows": rows, "hidden": hidden, "io_dtype": dtype_name,
                   "l2": "inputs + outputs per step exceed the 126 MB L2; no flush needed"},
        "gpu_launches": launches, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": dom[1], "achieved": dom[2], "peak": peak, "unit": "GB/s",
                     "frac": dom[2] / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                     "algorithmic_bytes_per_launch": dom[3], "avg_launch_ms": dom[4],
                     "fwd": {"kernel": names[0], "achieved": fa, "frac": fa / peak, "avg_launch_ms": fwd_ms},
                     "bwd": {"kernel": names[1], "achieved": ba, "frac": ba / peak, "avg_launch_ms": bwd_ms}},
    }), flush=True)


# --------------------------------------------------------------------------- GPU arm
def run_single_process(args):
    """--single-process --gpus N: ONE host process drives N GPUs through the C-ABI executor of
    include/agb/agb_shard.h (weak scaling, the default workload's rows on every GPU); the dgamma
    exchange is the executor's peer-sum kernel instead of an NCCL all-reduce.  Device-timed per shard
    stream, max over shards.  Kernel-only line: no e2e, no CPU leg."""
    import torch

    from cgadimpl_b200 import ops
    from cgadimpl_b200.shard_executor import ShardExecutor

    n = args.gpus
    if torch.cuda.device_count() < n:
        raise SystemExit(f"--single-process --gpus {n}: only {torch.cuda.device_count()} device(s) visible")
    rows, hidden, dtype_name, eps = WORKLOADS[args.workload]
    dtype = getattr(torch, dtype_name)
    elem = 4 if dtype == torch.float32 else 2
    xs, gys, gammas, ys, dxs, rstds, dgs = [], [], [], [], [], [], []
    for d in range(n):
        dev = torch.device("cuda", d)
        gen = torch.Generator(device=dev).manual_seed(1000 * d)
        xs.append(torch.randn(rows, hidden, device=dev, generator=gen, dtype=torch.float32).to(dtype))
        gys.append(torch.randn(rows, hidden, device=dev, generator=gen, dtype=torch.float32).to(dtype))
        ggen = torch.Generator(device=dev).manual_seed(7)
        gammas.append((1 + 0.02 * torch.randn(hidden, device=dev, generator=ggen)).to(dtype))
        ys.append(torch.empty_like(xs[-1]))
        dxs.append(torch.empty_like(xs[-1]))
        rstds.append(torch.empty(rows, dtype=torch.float32, device=dev))
        dgs.append(torch.empty(hidden, dtype=torch.float32, device=dev))
    for d in range(n):
        torch.cuda.synchronize(d)
    # --replicas: N independent one-GPU executors (no exchange between GPUs): what each GPU does alone while
    # the others are busy too -- the yardstick for what the exchange and the lock step cost
    groups = [[d] for d in range(n)] if args.replicas else [list(range(n))]
    exs = [ShardExecutor(g, hidden) for g in groups]
    try:
        for ex in exs:
            ex.set_deferred_exchange(args.deferred_exchange)
        pick = lambda seq, g: [seq[d] for d in g]
        prepared = [ex.prepare(pick(xs, g), pick(gammas, g), pick(gys, g), pick(ys, g), pick(rstds, g), pick(dxs, g),
                               pick(dgs, g)) for ex, g in zip(exs, groups)]
        stream_of = {d: ex.stream(i) for ex, g in zip(exs, groups) for i, d in enumerate(g)}

        def step():
            for ex, (io, h, dt) in zip(exs, prepared):
                ex.run_prepared(io, h, eps, dt)

        def sync():
            for ex in exs:
                ex.synchronize()

        for _ in range(args.warmup):
            step()
        sync()
        sampler = ClockSampler(0)
        sampler.start()
        time.sleep(0.3)
        t0 = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        t1 = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        launches0 = ops.launch_count()
        for d in range(n):
            t0[d].record(stream_of[d])
        for _ in range(args.steps):
            step()
        for d in range(n):
            t1[d].record(stream_of[d])
        sync()
        launches = ops.launch_count() - launches0
        per_gpu_ms = [t0[d].elapsed_time(t1[d]) / args.steps for d in range(n)]
        elapsed_ms = max(per_gpu_ms) * args.steps
        time.sleep(0.2)
        clocks = sampler.stop()
    finally:
        for ex in exs:
            ex.close()
    if not args.replicas:
        for d in dgs[1:]:
            assert torch.equal(d.cpu(), dgs[0].cpu()), "shards disagree on dgamma"
    value = rows * n * args.steps / (elapsed_ms / 1e3)
    bpr = bytes_per_row(hidden, elem)
    peak, peak_kind = measured_peak()
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "rows_per_gpu": rows, "global_rows": rows * n, "hidden": hidden,
                   "io_dtype": dtype_name, "eps": eps,
                   "parallelism": (f"{n} independent replicas, one host process, no exchange" if args.replicas else
                                   f"rows{n}, one host process (agb_shard_run_fwd_bwd, peer-sum dgamma exchange"
                                   f"{' on side streams' if args.deferred_exchange else ''})"),
                   "per_gpu_ms_per_step": per_gpu_ms,
                   "l2": "inputs+outputs per step (>= 2 GB per GPU) exceed the 126 MB L2; no flush needed"},
        "hbm_gbs": value / n * bpr / 1e9, "bytes_per_row": bpr, "gpu_launches": launches, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": value / n * bpr / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": value / n * bpr / 1e9 / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                     "kernel": "whole step per GPU (forward + backward + dgamma reduce + peer sum)"},
        "e2e": None, "cpu_baseline": None}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(STACK_WORKLOADS) + sorted(OP_WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "collective"],
                    help="N > 1: how dgamma crosses the ranks (the library's peer-load kernel, or an NCCL all-reduce)")
    ap.add_argument("--single-process", action="store_true",
                    help="drive --gpus N devices from this one process through the C-ABI shard executor")
    ap.add_argument("--deferred-exchange", action="store_true",
                    help="with --single-process: dgamma exchange on side streams (agb_shard_set_deferred_exchange)")
    ap.add_argument("--replicas", action="store_true",
                    help="with --single-process: N independent one-GPU executors, no exchange (a yardstick)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.workload in STACK_WORKLOADS:
        run_stack(args, rank)
        return
    if args.workload in OP_WORKLOADS:
        run_op(args, rank)
        return
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if args.single_process:
        if world > 1:
            raise SystemExit("--single-process is for a plain `python bench.py` launch, not torchrun")
        run_single_process(args)
        return

    import torch

    from cgadimpl_b200 import ops
    from cgadimpl_b200.executor import RowShardedRMSNorm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        # the path's only collective is an all-reduce of 8 * hidden bytes: latency-bound, and measured fastest
        # with the tree algorithm (8 GPUs: 0.460 ms per step against 0.470 ring, 0.480 NCCL's own choice)
        os.environ.setdefault("NCCL_ALGO", "Tree")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.gpus != world and rank == 0 and world > 1:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)

    rows, hidden, dtype_name, eps = WORKLOADS[args.workload]
    strong = args.workload in STRONG_SCALING
    if strong:
        from cgadimpl_b200.executor import shard_rows

        a, b = shard_rows(rows, world, rank)
        total_rows_fixed = rows
        rows = b - a
    dtype = getattr(torch, dtype_name)
    elem = 4 if dtype == torch.float32 else 2
    gen = torch.Generator(device="cuda").manual_seed(1000 * rank)
    x = torch.randn(rows, hidden, device="cuda", generator=gen, dtype=torch.float32).to(dtype)
    gy = torch.randn(rows, hidden, device="cuda", generator=gen, dtype=torch.float32).to(dtype)
    ggen = torch.Generator(device="cuda").manual_seed(7)
    gamma = (1 + 0.02 * torch.randn(hidden, device="cuda", generator=ggen)).to(dtype)
    y = torch.empty_like(x)
    dx = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device="cuda")
    dgamma = torch.empty(hidden, dtype=torch.float32, device="cuda")
    ex = RowShardedRMSNorm(hidden, dtype, eps, exchange=args.exchange)

    def step():
        ex.fwd_bwd(x, gy, gamma, y=y, rstd=rstd, dx=dx, dgamma=dgamma, wait=False)

    def sync_all():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()
    ops.device_status()

    # ---- timed region: K steps, device-timed, plus per-kernel events on the launching stream
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    # per-kernel events on every 5th step only: three event records per step cost a few microseconds of
    # stream bubbles, which is not negligible against a 0.4 ms step
    sampled = [k for k in range(args.steps) if k % 5 == 0]
    ev = {k: [torch.cuda.Event(enable_timing=True) for _ in range(3)] for k in sampled}
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prepared = ex.prepare_step(x, gy, gamma, y, rstd, dx, dgamma)   # operands validated once, bare calls per step
    launches0 = ops.launch_count()
    sync_all()
    t_start.record()
    for k in range(args.steps):
        e = ev.get(k)
        if e:
            e[0].record()
        prepared.fwd()
        if e:
            e[1].record()
        # backward on this stream; for N > 1 the exchange of the 8*H-byte fp64 sums and the final rounding
        # run on the executor's side stream and overlap the next step's kernels (sum buffers alternate)
        prepared.bwd()
        if e:
            e[2].record()
    if world > 1:
        ex.wait_dgamma()          # the timed region ends when the last dgamma is final
    t_end.record()
    sync_all()
    launches = ops.launch_count() - launches0
    elapsed_ms = t_start.elapsed_time(t_end)
    if dist is not None:
        t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    if sampler:
        time.sleep(0.2)
    clocks = sampler.stop() if sampler else None
    ops.device_status()

    fwd_ms = statistics.mean(ev[k][0].elapsed_time(ev[k][1]) for k in sampled)
    bwd_ms = statistics.mean(ev[k][1].elapsed_time(ev[k][2]) for k in sampled)
    total_rows = total_rows_fixed if strong else rows * world
    value = total_rows * args.steps / (elapsed_ms / 1e3)
    bpr = bytes_per_row(hidden, elem)
    peak, peak_kind = measured_peak()

    # dominant launch: the backward call (rmsnorm_bwd_staged followed by the ~µs dgamma reduction)
    bwd_bytes = rows * (3 * hidden * elem + 4)
    fwd_bytes = rows * (2 * hidden * elem + 4)
    achieved = bwd_bytes / (bwd_ms / 1e3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "rmsnorm_bwd_staged (+dgamma_reduce_kernel)", "achieved": achieved, "peak": peak,
        "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
        "algorithmic_bytes_per_launch": bwd_bytes, "avg_launch_ms": bwd_ms, "launches_timed": len(sampled),
        "fwd": {"kernel": "rmsnorm_fwd_staged", "achieved": fwd_bytes / (fwd_ms / 1e3) / 1e9,
                "frac": fwd_bytes / (fwd_ms / 1e3) / 1e9 / peak, "avg_launch_ms": fwd_ms,
                "algorithmic_bytes_per_launch": fwd_bytes},
        "step_gbs": value / world * bpr / 1e9,
        "step_frac_of_spec_8TBs": value / world * bpr / 1e9 / SPEC_HBM_GBS,
        "step_frac_of_peak": value / world * bpr / 1e9 / peak,
    }
    tr = NCU_TRAFFIC.get(args.workload)
    if tr:
        roofline["traffic"] = tr["bwd_dram_bytes_per_launch"]
        roofline["traffic_source"] = tr["source"]

    # ---- end to end: pinned host buffers in, host buffers out, copies inside the timed region
    e2e = None
    if not args.no_e2e:
        xh = torch.empty(rows, hidden, dtype=dtype).pin_memory()
        gyh = torch.empty(rows, hidden, dtype=dtype).pin_memory()
        xh.copy_(x)
        gyh.copy_(gy)
        gh = gamma.cpu().pin_memory()
        yh = torch.empty(rows, hidden, dtype=dtype).pin_memory()
        dxh = torch.empty(rows, hidden, dtype=dtype).pin_memory()
        dgh = torch.empty(hidden, dtype=torch.float32).pin_memory()
        for _ in range(2):
            ex.fwd_bwd_host(xh, gyh, gh, yh, dxh, dgh)
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            ex.fwd_bwd_host(xh, gyh, gh, yh, dxh, dgh)
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        # the host results must be the device results
        assert torch.equal(yh[:64].cuda(), y[:64]) and torch.equal(dxh[-64:].cuda(), dx[-64:]), "e2e mismatch"
        h2d = rows * hidden * elem * 2 + hidden * elem
        d2h = rows * hidden * elem * 2 + hidden * 4
        e2e = {"value": total_rows * args.e2e_steps / (ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": args.e2e_steps, "ms_per_step": ms / args.e2e_steps,
               "api": "cgadimpl_b200.executor.RowShardedRMSNorm.fwd_bwd_host (pinned host buffers, chunked "
                      "copy/compute overlap on three streams)"}
        del xh, gyh, yh, dxh

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_rows = min(rows, 4096)
        v, cores, secs, kind, note = cpu_pass(hidden, eps, sample_rows, reps=8)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                        "sample": f"{sample_rows} of {rows} rows, best of 8 passes ({secs*1e3:.1f} ms each); {note}"}
        # the same arithmetic as ONE pass per row over memory, so that the comparison is not flattered by the
        # reference's many passes and temporaries
        fv, fcores, fsecs = cpu_fused_pass(hidden, eps, sample_rows, reps=8)
        cpu_baseline["fused_single_pass"] = {"value": fv, "unit": UNIT, "cores": fcores,
                                             "note": f"row-fused C restatement (oracle/agb_oracle.c), best of 8 passes ({fsecs*1e3:.1f} ms each)"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "rows_per_gpu": rows, "global_rows": total_rows, "hidden": hidden,
                       "io_dtype": dtype_name, "eps": eps, "parallelism": f"rows{world}",
                       "dgamma_exchange": ex.exchange,
                       "l2": "inputs+outputs per step (>= 2 GB) exceed the 126 MB L2; no flush needed",
                       "launch": {"fwd": ops.describe_launch("fwd", rows, hidden, dtype),
                                  "bwd": ops.describe_launch("bwd", rows, hidden, dtype)}},
            "hbm_gbs": value / world * bpr / 1e9, "bytes_per_row": bpr,
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
            "e2e": e2e, "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    ex.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
