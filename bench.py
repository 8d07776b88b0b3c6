#!/usr/bin/env python
"""RMSNorm forward + VJP throughput on B200 (rows/s), with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one forward + VJP pass over the workload's rows: rmsnorm_fwd, rmsnorm_bwd (dx fused
with the dgamma partials), the fixed-order dgamma reduction and, for N > 1, the exchange of the
fp64 dgamma sums between the ranks (the library's push exchange over peer memory by default, an
NCCL all-reduce with --exchange collective).  N > 1 is launched by torchrun, one rank per GPU.

Workload (default): the row-sharded configuration -- x [64,8192,8192] bf16 ~ N(0,1) (524288 rows),
gamma = 1 + 0.02 N(0,1), gy ~ N(0,1), eps 1e-6, synthetic, seeded; the rows are split evenly over the
ranks (strong scaling), `value` counts all 524288 rows.  Inputs and outputs per step (>= 5 GB per GPU at
N = 8, 43 GB at N = 1) are far larger than the 126 MB L2, so no flush is needed between iterations.

Timing: after W warm-up steps the K-step block is timed with CUDA events, bracketed by a barrier and a
device synchronize on both sides, max over ranks; the block is repeated until about one second has been
timed and the MEDIAN block is reported (every block's time is in `timing.block_ms`).

At N = 1 the line also carries the other single-GPU configurations (`other_configs`) and the same step
through the C++ graph API (`api_path`); at N > 1 every rank's own pace with the exchange switched off
(`no_exchange`: one short block before the timed region, and as many blocks as it had right after it).

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
    # the row-sharded configuration: 524288 rows in total, split evenly over the ranks (strong scaling)
    "rmsnorm_fwd_vjp_bf16_sharded_64x8192x8192": (64 * 8192, 8192, "bfloat16", 1e-6),
}
STRONG_SCALING = {"rmsnorm_fwd_vjp_bf16_sharded_64x8192x8192"}
# input distributions: (std of x, std of gamma - 1, fraction of rows of x multiplied by 100)
DISTRIBUTIONS = {name: (3.0, 0.1, 0.01) for name in WORKLOADS if "65536x" in name}   # the odd-width bf16 configuration
DEFAULT_DISTRIBUTION = (1.0, 0.02, 0.0)
# single-GPU configurations carried in the default line at N = 1
OTHER_CONFIGS = ["rmsnorm_fwd_vjp_fp32_16x2048x4096", "rmsnorm_fwd_vjp_bf16_65536x1000", "rmsnorm_fwd_vjp_bf16_65536x5120",
                 "rmsnorm_fwd_vjp_bf16_65536x8192", "rmsnorm_fwd_vjp_bf16_65536x12288"]
OTHER_STACK = "residual_stack_fp32_32x4x4096x4096"
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
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE backward launch at the benchmarked shape:
# the table cgadimpl_b200/ncu_traffic.json holds the figures of the ncu captures summarised under profiles/
# (its "command" entry is the capture command).  No entry for a width and type -> roofline.traffic is null.
def ncu_traffic(rows, hidden, dtype_name):
    """The capture of exactly this shape, else the largest captured shape of the same width and type with
    fewer rows, scaled by the row count (the kernel streams rows: its traffic is proportional to them)."""
    try:
        with open(os.path.join(ROOT, "cgadimpl_b200", "ncu_traffic.json")) as f:
            table = json.load(f)["captures"]
    except Exception:
        return None
    exact = table.get(f"rmsnorm_bwd_{dtype_name}_{rows}x{hidden}")
    if exact:
        return exact
    best = None
    for key, entry in table.items():
        if entry.get("hidden") == hidden and entry.get("dtype") == dtype_name and entry.get("rows", 0) < rows:
            if best is None or entry["rows"] > best["rows"]:
                best = entry
    if best is None:
        return None
    scale = rows / best["rows"]
    return {"dram_bytes_per_launch": int(best["dram_bytes_per_launch"] * scale),
            "source": f"{best['source']}; scaled x{scale:g} by rows ({rows} rows here: too large to capture under ncu)"}


DEFAULT_WORKLOAD = "rmsnorm_fwd_vjp_bf16_sharded_64x8192x8192"
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
REF_EPS_NOTE = ("; fp32 on the CPU with the reference's hard-coded eps = 1e-5 (it has no bf16 path and no eps "
                "argument; the work per row is the same)")
PORT_KIND_NOTE = "op-by-op fp32 restatement of the reference composition (oracle/agb_oracle.c), OpenMP"


def cpu_sample_rows(rows, hidden):
    """A bounded sample of the workload for the CPU legs: 16 Mi elements per array (4096 rows of 4096)."""
    return max(1, min(rows, (1 << 24) // hidden))


def cpu_pass(hidden, eps, sample_rows, reps, seed=0):
    """Times the reference's CPU path (all host threads) on a bounded sample of the workload.
    Returns (rows/s, threads, seconds per pass, kind, note)."""
    REF = _reference_build()
    if REF is not None:     # the reference hard-codes eps = 1e-5 and computes in fp32; neither changes the work per row
        cores = REF.use_all_cores()
        REF.set_reduce_fp64(False)
        secs = min(REF.time_fwd_bwd(sample_rows, hidden, 1, 1) for _ in range(max(1, reps)))
        return sample_rows / secs, cores, secs, "reference", REF_KIND_NOTE + REF_EPS_NOTE
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
    sample_rows = cpu_sample_rows(rows, hidden)
    REF = _reference_build()
    if REF is not None:
        cores = REF.use_all_cores()
        REF.set_reduce_fp64(False)
        secs = REF.time_fwd_bwd(sample_rows, hidden, args.steps, max(1, args.warmup))
        kind, note = "reference", REF_KIND_NOTE + REF_EPS_NOTE
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
    strong = args.workload in STRONG_SCALING
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3,
        "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "rows_per_gpu": rows // world if strong else rows,
                   "global_rows": rows if strong else rows * world, "hidden": hidden, "io_dtype": dtype, "eps": eps,
                   "parallelism": f"rows{world}"},
        "sample_rows_per_step": sample_rows,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"{sample_rows} of {rows} rows per step; {note}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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

    for kv in args.option:
        k, v = kv.split("=")
        ops.set_option(k, int(v))
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


# --------------------------------------------------------------------------- GPU arm: helpers
def synth(rows, hidden, dtype, seed, std=1.0, outlier_frac=0.0, chunk=16384):
    """[rows, hidden] ~ N(0, std) on the current device, generated chunk by chunk in fp32 and rounded once;
    a seeded fraction of rows is multiplied by 100 before rounding (outlier rows)."""
    import torch

    out = torch.empty(rows, hidden, dtype=dtype, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(seed)
    scale = None
    if outlier_frac > 0 and rows > 0:
        scale = torch.full((rows, 1), std, device="cuda")
        k = max(1, int(round(rows * outlier_frac)))
        idx = torch.randperm(rows, generator=gen, device="cuda")[:k]
        scale[idx] = std * 100.0
    for r0 in range(0, rows, chunk):
        n = min(chunk, rows - r0)
        t = torch.randn(n, hidden, device="cuda", generator=gen)
        out[r0:r0 + n] = (t * (scale[r0:r0 + n] if scale is not None else std)).to(dtype)
    return out


def make_operands(name, rows, hidden, dtype, seed):
    import torch

    x_std, g_std, outl = DISTRIBUTIONS.get(name, DEFAULT_DISTRIBUTION)
    x = synth(rows, hidden, dtype, seed, x_std, outl)
    gy = synth(rows, hidden, dtype, seed + 1)
    ggen = torch.Generator(device="cuda").manual_seed(7)
    gamma = (1 + g_std * torch.randn(hidden, device="cuda", generator=ggen)).to(dtype)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device="cuda")
    dgamma = torch.empty(hidden, dtype=torch.float32, device="cuda")
    return x, gy, gamma, y, dx, rstd, dgamma


def time_steps(prepared, ex, steps, warmup, world, dist, target_s, sample_every=5):
    """W warm-up steps, then blocks of exactly `steps` steps, each bracketed by barrier + synchronize and
    timed with CUDA events on the launching stream (max over ranks), repeated until ~target_s seconds are
    timed.  Returns (block times in ms, mean fwd ms, mean bwd ms, kernel launches in all blocks)."""
    import torch

    from cgadimpl_b200 import ops

    def sync_all():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        prepared.fwd()
        prepared.bwd()
    if world > 1:
        ex.wait_dgamma()
    sync_all()
    ops.device_status()
    # one untimed probe block decides how many blocks make up the target
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for _ in range(min(steps, 5)):
        prepared.fwd()
        prepared.bwd()
    if world > 1:
        ex.wait_dgamma()
    p1.record()
    sync_all()
    est = p0.elapsed_time(p1) / min(steps, 5) * steps / 1e3
    nblocks = max(1, min(400, int(target_s / max(est, 1e-6) + 0.999)))
    if dist is not None:       # every rank must run the same number of blocks
        t = torch.tensor([nblocks], device="cuda", dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        nblocks = int(t.item())
    block_ms, fwd_ms, bwd_ms = [], [], []
    launches0 = ops.launch_count()
    for b in range(nblocks):
        # per-kernel events on every `sample_every`-th step only: three event records per step cost a few
        # microseconds of stream bubbles and keep dependent kernels from being placed early
        sampled = [k for k in range(steps) if k % sample_every == 0]
        ev = {k: [torch.cuda.Event(enable_timing=True) for _ in range(3)] for k in sampled}
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        t0.record()
        for k in range(steps):
            e = ev.get(k)
            if e:
                e[0].record()
            prepared.fwd()
            if e:
                e[1].record()
            prepared.bwd()
            if e:
                e[2].record()
        if world > 1:
            ex.wait_dgamma()          # the block ends when its last dgamma is final
        t1.record()
        sync_all()
        block_ms.append(t0.elapsed_time(t1))
        fwd_ms += [ev[k][0].elapsed_time(ev[k][1]) for k in sampled]
        bwd_ms += [ev[k][1].elapsed_time(ev[k][2]) for k in sampled]
    launches = ops.launch_count() - launches0
    if dist is not None:
        t = torch.tensor(block_ms, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        block_ms = [float(v) for v in t.tolist()]
    ops.device_status()
    return block_ms, statistics.mean(fwd_ms), statistics.mean(bwd_ms), launches


def check_dgamma(x, gy, gamma, rstd, dgamma, dist, rows_total, chunk=8192):
    """Outside the timed region: the exchanged dgamma against an fp64 column sum of gy * x * rstd over ALL
    ranks' rows (each rank sums its rows in fp64 with torch, the sums are added over the ranks in fp64)."""
    import torch

    rows, hidden = x.shape
    want = torch.zeros(hidden, dtype=torch.float64, device="cuda")
    for r0 in range(0, rows, chunk):
        sl = slice(r0, min(rows, r0 + chunk))
        want += (gy[sl].double() * x[sl].double() * rstd[sl].double()[:, None]).sum(0)
    if dist is not None:
        dist.all_reduce(want, op=dist.ReduceOp.SUM)
    err = (dgamma.double() - want).abs()
    # fp32-accumulated (16-bit I/O) or fp64-accumulated fp32-rounded products (fp32 I/O): the floor grows like
    # sqrt(rows) * 2^-24 * a few; typical columns are of size sqrt(rows)
    rtol = 1e-5
    atol = (4e-6 if x.element_size() == 2 else 5e-7) * float(rows_total) ** 0.5
    ok = bool((err <= atol + rtol * want.abs()).all())
    return {"ok": ok, "max_abs_err": float(err.max()), "rtol": rtol, "atol": atol,
            "dgamma_rms": float(want.pow(2).mean().sqrt()),
            "against": "fp64 column sum of gy*x*rstd over all ranks' rows (torch), outside the timed region"}


def measure_one(name, steps, warmup, target_s):
    """One single-GPU configuration for `other_configs`: allocate, time, free."""
    import torch

    from cgadimpl_b200 import ops
    from cgadimpl_b200.executor import RowShardedRMSNorm

    rows, hidden, dtype_name, eps = WORKLOADS[name]
    dtype = getattr(torch, dtype_name)
    elem = 4 if dtype == torch.float32 else 2
    x, gy, gamma, y, dx, rstd, dgamma = make_operands(name, rows, hidden, dtype, seed=11)
    ex = RowShardedRMSNorm(hidden, dtype, eps)
    prepared = ex.prepare_step(x, gy, gamma, y, rstd, dx, dgamma)
    block_ms, fwd_ms, bwd_ms, _ = time_steps(prepared, ex, steps, warmup, 1, None, target_s)
    chk = check_dgamma(x, gy, gamma, rstd, dgamma, None, rows)
    ms = statistics.median(block_ms) / steps
    peak, _ = measured_peak()
    gbs = rows * bytes_per_row(hidden, elem) / (ms / 1e3) / 1e9
    out = {"workload": name, "rows": rows, "hidden": hidden, "io_dtype": dtype_name, "eps": eps, "ms_per_step": ms,
           "rows_per_s": rows / (ms / 1e3), "step_gbs": gbs, "frac": gbs / peak, "frac_of_spec_8TBs": gbs / SPEC_HBM_GBS,
           "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
           "fwd_frac": rows * (2 * hidden * elem + 4) / (fwd_ms / 1e3) / 1e9 / peak,
           "bwd_frac": rows * (3 * hidden * elem + 4) / (bwd_ms / 1e3) / 1e9 / peak,
           "blocks": len(block_ms), "fastest_block_ms_per_step": min(block_ms) / steps,
           "slowest_block_ms_per_step": max(block_ms) / steps,
           "dgamma_check_ok": chk["ok"],
           "launch": {"fwd": ops.describe_launch("fwd", rows, hidden, dtype), "bwd": ops.describe_launch("bwd", rows, hidden, dtype)}}
    ex.close()
    del x, gy, gamma, y, dx, rstd, dgamma, prepared
    torch.cuda.empty_cache()
    return out


def measure_stack(steps, warmup):
    """The 32-layer residual stack as one CUDA graph, through the C++ host layer (bench_stack)."""
    from cgadimpl_b200.host import build as host_build

    host_build.build()
    layers, rows, hidden, bf16 = STACK_WORKLOADS[OTHER_STACK]
    exe = os.path.join(os.path.dirname(host_build.__file__), "build", "bench_stack")
    # 60 replays of ~10 ms: long enough to settle under the power cap; the first five are reported beside them
    r = subprocess.run([exe, str(layers), str(rows), str(hidden), str(max(steps, 60)), str(max(3, warmup)), str(bf16)],
                       capture_output=True, text=True)
    if r.returncode != 0:
        return {"workload": OTHER_STACK, "error": (r.stdout + r.stderr)[-400:]}
    d = json.loads(r.stdout.strip().splitlines()[-1])
    peak, _ = measured_peak()
    return {"workload": OTHER_STACK, "layers": layers, "rows": rows, "hidden": hidden, "io_dtype": "float32",
            "ms_per_step": d["ms_per_replay"], "first_replays_ms_per_step": d.get("first_replays_ms"),
            "replays": d["iters"], "row_layers_per_s": d["row_layers_per_s"], "step_gbs": d["gbs"],
            "frac": d["gbs"] / peak, "frac_of_spec_8TBs": d["gbs"] / SPEC_HBM_GBS, "cuda_graph_nodes": d["graph_nodes"],
            "api": "ag::nn::ResidualRMSNormStack captured by ag::CudaGraphRunner (C++ host layer)"}


def measure_api(steps, warmup):
    """The path a cgadimpl user calls -- ag::rmsnorm + ag::backward through the C++ graph API -- on the fp32
    Llama-7B-width configuration, eager and as one CUDA graph (cgadimpl_b200/host/build/bench_api)."""
    from cgadimpl_b200.host import build as host_build

    host_build.build()
    rows, hidden, _, _ = WORKLOADS["rmsnorm_fwd_vjp_fp32_16x2048x4096"]
    exe = os.path.join(os.path.dirname(host_build.__file__), "build", "bench_api")
    # 1500 steps of ~0.4 ms per mode: long enough to settle under the power cap; the first twenty are reported too
    r = subprocess.run([exe, str(rows), str(hidden), str(max(steps, 1500)), str(max(3, warmup)), "0"], capture_output=True, text=True)
    if r.returncode != 0:
        return {"error": (r.stdout + r.stderr)[-400:]}
    d = json.loads(r.stdout.strip().splitlines()[-1])
    peak, _ = measured_peak()
    return {"workload": "rmsnorm_fwd_vjp_fp32_16x2048x4096", "api": "ag::rmsnorm + ag::zero_grad + ag::backward (C++ host layer)",
            "steps": d["iters"], "eager_ms_per_step": d["eager_ms_per_step"],
            "eager_first_steps_ms_per_step": d.get("eager_first_steps_ms"), "eager_frac": d["eager_gbs"] / peak,
            "graph_ms_per_step": d["graph_ms_per_step"], "graph_frac": d["graph_gbs"] / peak,
            "cuda_graph_nodes": d["graph_nodes"], "launches_per_step": d["launches_per_step"],
            "composed": {"api": "ag::mul(ag::rms(x), gamma) + ag::zero_grad + ag::backward: the reference's own op-by-op "
                                "composition of the layer (eps 1e-5) on this library's kernels, eager",
                         "ms_per_step": d.get("composed_ms_per_step"), "launches_per_step": d.get("composed_launches_per_step")}}


def no_exchange_pace(x, gy, gamma, y, dx, rstd, eps, steps, dist, rank, world, blocks=1):
    """N > 1: what each GPU does on its shard with NO exchange while all ranks are busy at the same time
    (ms per step, per rank; the median of `blocks` blocks of `steps` steps).  Taken briefly before the timed
    region (a GPU that has not yet met its power cap) and after it for as many blocks as the timed region had
    (the settled pace: under the 1 kW cap the SM clock sinks within a second and these kernels slow down by
    several per cent), so that the cost of coupling the ranks can be told from what each GPU does alone."""
    import torch

    from cgadimpl_b200 import ops

    ws = ops.bwd_workspace(x)
    scratch_dg = torch.empty(x.shape[-1], dtype=torch.float32, device="cuda")

    def local_step():
        ops.rmsnorm_fwd(x, gamma, eps, out=y, rstd=rstd)
        ops.rmsnorm_bwd(x, gamma, rstd, gy, dx=dx, dgamma=scratch_dg, workspace=ws)

    for _ in range(3):
        local_step()
    dist.barrier()
    torch.cuda.synchronize()
    per_block = []
    for _ in range(blocks):
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for _ in range(steps):
            local_step()
        q1.record()
        torch.cuda.synchronize()
        per_block.append(q0.elapsed_time(q1) / steps)
    every = torch.zeros(world, device="cuda", dtype=torch.float64)   # a SUM all-reduce of a one-hot table: it
    every[rank] = statistics.median(per_block)                       # exists for every algorithm NCCL may be pinned to
    dist.all_reduce(every, op=dist.ReduceOp.SUM)
    return [round(float(v), 4) for v in every.tolist()]


def copy_probe(dist, nbytes=1 << 30):
    """Host <-> device copy rate of this rank's GPU with every rank copying at the same time (pinned memory,
    one direction at a time, then both): what bounds the end-to-end figure.  GB/s, min over ranks."""
    import torch

    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h2 = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    d2 = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    def both():
        with torch.cuda.stream(s1):
            d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s2):
            h2.copy_(d2, non_blocking=True)

    res = {"h2d_gbs": nbytes / timed(lambda: d.copy_(h, non_blocking=True)) / 1e9,
           "d2h_gbs": nbytes / timed(lambda: h2.copy_(d2, non_blocking=True)) / 1e9,
           "both_each_gbs": nbytes / timed(both) / 1e9}
    if dist is not None:
        t = torch.tensor([res["h2d_gbs"], res["d2h_gbs"], res["both_each_gbs"]], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        res = dict(zip(("h2d_gbs", "d2h_gbs", "both_each_gbs"), (float(v) for v in t.tolist())))
    res["note"] = "per rank, all ranks copying at once, 1 GiB pinned buffers; min over ranks"
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(STACK_WORKLOADS) + sorted(OP_WORKLOADS))
    ap.add_argument("--target-seconds", type=float, default=1.0, help="repeat the K-step block until this much is timed")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-rows", type=int, default=65536, help="rows per rank and step of the end-to-end leg (a sample of the shard when it is larger)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--option", action="append", default=[], metavar="KEY=VALUE", help="agb_set_option before anything runs")
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
    from cgadimpl_b200.executor import RowShardedRMSNorm, shard_rows

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    for kv in args.option:
        k, v = kv.split("=")
        ops.set_option(k, int(v))
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
    total_rows = rows if strong else rows * world
    if strong:
        a, b = shard_rows(rows, world, rank)
        rows = b - a
    dtype = getattr(torch, dtype_name)
    elem = 4 if dtype == torch.float32 else 2
    x, gy, gamma, y, dx, rstd, dgamma = make_operands(args.workload, rows, hidden, dtype, seed=1000 * rank)
    ex = RowShardedRMSNorm(hidden, dtype, eps, exchange=args.exchange)
    prepared = ex.prepare_step(x, gy, gamma, y, rstd, dx, dgamma)   # operands validated once, bare calls per step

    pace_before = no_exchange_pace(x, gy, gamma, y, dx, rstd, eps, args.steps * 3, dist, rank, world) if world > 1 else None

    # ---- timed region
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    block_ms, fwd_ms, bwd_ms, launches = time_steps(prepared, ex, args.steps, args.warmup, world, dist, args.target_seconds)
    if sampler:
        time.sleep(0.2)
    clocks = sampler.stop() if sampler else None
    block = statistics.median(block_ms)
    ms_per_step = block / args.steps
    value = total_rows / (ms_per_step / 1e3)
    bpr = bytes_per_row(hidden, elem)
    peak, peak_kind = measured_peak()
    if clocks and clocks.get("sm_mhz"):
        clocks["ms_per_step_x_sm_mhz"] = ms_per_step * clocks["sm_mhz"]

    # ---- N > 1: the ranks' own pace without any exchange, again after the timed region
    no_exchange = None
    if world > 1:
        after = no_exchange_pace(x, gy, gamma, y, dx, rstd, eps, args.steps, dist, rank, world, blocks=len(block_ms))
        no_exchange = {"per_rank_ms_per_step_before": pace_before, "per_rank_ms_per_step_after": after,
                       "slowest_ms": max(after), "slowest_before_ms": max(pace_before),
                       "blocks_after": len(block_ms),
                       "note": "forward + VJP on each rank's shard without any exchange, all ranks running at once; "
                               "before: one short block ahead of the timed region (GPU not yet at its power cap); "
                               "after: as many blocks as the timed region, right after it (the settled pace)"}
        ex.fwd_bwd(x, gy, gamma, y=y, rstd=rstd, dx=dx, dgamma=dgamma, wait=True)   # dgamma of the real path again

    # ---- the exchanged dgamma is the column sum over all ranks' rows (outside the timed region)
    dgamma_check = check_dgamma(x, gy, gamma, rstd, dgamma, dist, total_rows)
    if not dgamma_check["ok"]:
        raise SystemExit(f"rank {rank}: dgamma check failed: {dgamma_check}")

    # dominant launch: the backward call (rmsnorm_bwd followed by the few-microsecond dgamma reduction)
    bwd_bytes = rows * (3 * hidden * elem + 4)
    fwd_bytes = rows * (2 * hidden * elem + 4)
    achieved = bwd_bytes / (bwd_ms / 1e3) / 1e9
    step_gbs = value / world * bpr / 1e9
    roofline = {
        "bound": "hbm", "kernel": "rmsnorm_bwd (+dgamma_reduce_kernel)", "achieved": achieved, "peak": peak,
        "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
        "algorithmic_bytes_per_launch": bwd_bytes, "avg_launch_ms": bwd_ms,
        "fwd": {"kernel": "rmsnorm_fwd", "achieved": fwd_bytes / (fwd_ms / 1e3) / 1e9,
                "frac": fwd_bytes / (fwd_ms / 1e3) / 1e9 / peak, "avg_launch_ms": fwd_ms,
                "algorithmic_bytes_per_launch": fwd_bytes},
        "step_gbs": step_gbs, "step_frac_of_spec_8TBs": step_gbs / SPEC_HBM_GBS, "step_frac_of_peak": step_gbs / peak,
    }
    tr = ncu_traffic(rows, hidden, dtype_name)
    if tr:
        roofline["traffic"] = tr["dram_bytes_per_launch"]
        roofline["traffic_source"] = tr["source"]

    # ---- end to end: pinned host buffers in, host buffers out, copies inside the timed region
    e2e = None
    if not args.no_e2e:
        er = min(rows, args.e2e_rows)
        xh = torch.empty(er, hidden, dtype=dtype).pin_memory()
        gyh = torch.empty(er, hidden, dtype=dtype).pin_memory()
        xh.copy_(x[:er])
        gyh.copy_(gy[:er])
        gh = gamma.cpu().pin_memory()
        yh = torch.empty(er, hidden, dtype=dtype).pin_memory()
        dxh = torch.empty(er, hidden, dtype=dtype).pin_memory()
        dgh = torch.empty(hidden, dtype=torch.float32).pin_memory()

        def sync_all():
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()

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
        assert torch.equal(yh[:64].cuda(), y[:64]) and torch.equal(dxh[er - 64:].cuda(), dx[er - 64:er]), "e2e mismatch"
        e2e_rows_all = er * world if not strong else min(total_rows, er * world)
        h2d = er * hidden * elem * 2 + hidden * elem
        d2h = er * hidden * elem * 2 + hidden * 4
        e2e = {"value": e2e_rows_all * args.e2e_steps / (ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": args.e2e_steps, "ms_per_step": ms / args.e2e_steps,
               "rows_per_rank_and_step": er,
               "sample": (f"{er} of this rank's {rows} rows per step" if er < rows else "the rank's whole shard per step")
                         + "; bytes are per rank",
               "api": ("agb_host_pipe_fwd_bwd (C ABI, include/agb/agb_host.h) through RowShardedRMSNorm.fwd_bwd_host"
                       if world == 1 else "cgadimpl_b200.executor.RowShardedRMSNorm.fwd_bwd_host") +
                      ": pinned host buffers, chunked copy/compute overlap on three streams"}
        del xh, gyh, yh, dxh
        e2e["copy_probe"] = copy_probe(dist)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_rows = cpu_sample_rows(rows, hidden)
        v, cores, secs, kind, note = cpu_pass(hidden, eps, sample_rows, reps=8)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                        "sample": f"{sample_rows} of {rows} rows, best of 8 passes ({secs*1e3:.1f} ms each); {note}"}
        # the same arithmetic as ONE pass per row over memory, so that the comparison is not flattered by the
        # reference's many passes and temporaries
        fv, fcores, fsecs = cpu_fused_pass(hidden, eps, sample_rows, reps=8)
        cpu_baseline["fused_single_pass"] = {"value": fv, "unit": UNIT, "cores": fcores,
                                             "note": f"row-fused C restatement (oracle/agb_oracle.c), best of 8 passes ({fsecs*1e3:.1f} ms each)"}

    other = api_path = None
    if rank == 0 and world == 1 and not args.no_other_configs and args.workload == DEFAULT_WORKLOAD:
        del x, gy, y, dx, prepared          # make room: the other configurations bring their own operands
        torch.cuda.empty_cache()
        other = []
        # Each side configuration gets a short pause first: the main workload has just held the GPU at its
        # 1 kW cap for tens of seconds, and a configuration's own half second of timed work should show ITS
        # sustained pace, not the heat of the one before it (the pause is reported; clocks are not touched).
        pause_s = 3.0
        for name in OTHER_CONFIGS:
            time.sleep(pause_s)
            try:
                o = measure_one(name, args.steps, args.warmup, min(0.5, args.target_seconds))
                o["pause_before_s"] = pause_s
                other.append(o)
            except Exception as e:  # noqa: BLE001 -- one failing side configuration must not lose the line
                other.append({"workload": name, "error": repr(e)[:300]})
        time.sleep(pause_s)
        other.append(measure_stack(args.steps, args.warmup))
        time.sleep(pause_s)
        api_path = measure_api(args.steps, args.warmup)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "rows_per_gpu": rows, "global_rows": total_rows, "hidden": hidden,
                       "io_dtype": dtype_name, "eps": eps, "parallelism": f"rows{world}",
                       "dgamma_exchange": ex.exchange,
                       "arithmetic": "fp32 accumulation (16-bit I/O)" if elem == 2 else "reference rounding points, fp64 reductions",
                       "l2": "inputs+outputs per step (>= 5 GB per GPU) exceed the 126 MB L2; no flush needed",
                       "launch": {"fwd": ops.describe_launch("fwd", rows, hidden, dtype),
                                  "bwd": ops.describe_launch("bwd", rows, hidden, dtype)}},
            "timing": {"statistic": "median over blocks of exactly `steps` steps; each block barrier + synchronize "
                                    "bracketed, CUDA events, max over ranks",
                       "blocks": len(block_ms), "block_ms": [round(b, 4) for b in block_ms],
                       "block_ms_min": min(block_ms), "block_ms_max": max(block_ms),
                       "timed_seconds": sum(block_ms) / 1e3},
            "hbm_gbs": step_gbs, "bytes_per_row": bpr,
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "dgamma_check": dgamma_check,
            "no_exchange": no_exchange,
            "e2e": e2e, "cpu_baseline": cpu_baseline, "other_configs": other, "api_path": api_path,
        }
        print(json.dumps(line), flush=True)
    ex.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
