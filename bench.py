"""Benchmark of the sparse-attention hot path (24 heads x 33272 tokens, 30 % video-KV density).

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One step = one attention layer over one batch of synthetic input: column
statistics -> INT8 Q/K + FP8 V carriers -> block router -> block-sparse
attention (-> all-gather of the head-sharded output when N > 1).  Workload:
B1, 24 heads x 128, 512 text + 32760 video tokens, 30 % video-KV density,
bf16 inputs drawn from a seeded CPU generator (see
h3_optimizations_b200/workloads.py).  Heads are sharded over the N ranks, the
total work is fixed ("strong" scaling).

Rank 0 prints ONE JSON line.  `value` is effective TOPS: algorithmic
attention operations of the whole layer (4*128 per query-row x key-row pair on
the listed tiles) divided by the device time of the full step, inputs resident
in HBM.  `e2e` is the same quantity through the backend with host buffers
(pinned H2D of Q/K/V and D2H of the output inside the timed region).
`--impl reference` times the reference's own torch path (its router + its
FP32 sparse attention, run from the sources staged under oracle/_ref) on the
host cores instead, with every core the process may use.

Other workloads: `--config config2` puts the chunked ConvRot INT8 QKV projection
(hidden 3072, 4096-token chunks, carriers written by the GEMM epilogue) in front
of the attention, head-sharded at N > 1 (each rank holds the weight rows of its
heads, the activations are replicated); `--config config3` is the 76112-token
sequence, `--budget` a fixed density and `--schedule` the 30-step sampler
schedule (2 early and 2 late steps at 50 %, 26 at 30 %) with per-step times.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from h3_optimizations_b200 import workloads  # noqa: E402

VIDEO_BUDGET = 0.3
HEAD_DIM = 128
NOMINAL_INT8_TOPS = 4500.0
METRIC = "sparse_attn_effective_tops"
UNIT = "TOPS"


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("native", "reference"), default="native")
    parser.add_argument("--config", choices=("config1", "config2", "config3", "config4"), default="config1",
                        help="config1 is the headline workload; config2 adds the chunked QKV projection in front; "
                             "config3 is the 76112-token sequence; config4 is the mixed-modality block with batch 2, "
                             "out_proj and the chunked FP8 MLP behind the attention")
    parser.add_argument("--schedule", action="store_true",
                        help="run the 30-step sampler schedule (budgets 0.5, 0.5, 0.3 x 26, 0.5, 0.5) instead of one budget")
    parser.add_argument("--exchange", choices=("auto", "peer", "nccl"), default="auto",
                        help="N > 1: how the head-sharded output is reassembled")
    parser.add_argument("--budget", type=float, default=VIDEO_BUDGET)
    parser.add_argument("--heads", type=int, default=0,
                        help="run a head subset of the workload (profiling captures); 0 = all heads")
    parser.add_argument("--skip-cpu-baseline", action="store_true")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--no-graph", action="store_true",
                        help="time the eager step only; by default the step (with its peer-store exchange at N > 1) is "
                             "also captured into a CUDA graph (backend.capture) and `value` is the replayed step, with "
                             "the eager figure beside it; the NCCL exchange is never captured")
    return parser.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def attention_ops(spec, route, geo, heads):
    """Algorithmic operations of the layer for `heads` heads: 2*D for QK^T plus
    2*D for PV per (query row, key row) pair on the visited tiles."""
    sequence = spec.sequence
    q_rows = [min(128, sequence - t * 128) for t in range(geo.q_tiles)]
    tail_rows = sequence - (geo.kv_tiles - 1) * 64
    pairs = 0
    for tq in range(geo.q_tiles):
        routed = route is not None and geo.pure_video_q_start <= tq < geo.pure_video_q_stop
        if not routed:
            pairs += heads * q_rows[tq] * sequence
    if route is not None:
        has_tail = (route[0] == geo.kv_tiles - 1).any(dim=-1).to(torch.int64).cpu()  # (H, pure_q)
        keys = route.shape[-1] * 64 - (64 - tail_rows) * has_tail
        rows = torch.tensor(q_rows[geo.pure_video_q_start:geo.pure_video_q_stop], dtype=torch.int64)
        pairs += int((keys * rows[None, :]).sum())
    return 4 * HEAD_DIM * pairs


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU during the timed region.

    The sampling runs in a child process (NVML handle opened once, three
    read-only queries every 5 ms, each a few microseconds): a thread inside this
    process competes with the launching thread for the interpreter lock and
    stretched a 2.2 ms multi-GPU step to 4 ms, and `nvidia-smi -lms` re-reads
    its whole field list every period.  `nvidia-smi -lms 100` remains the
    fallback when the NVML bindings are missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    CHILD = r"""
import sys, time
import pynvml as nv
nv.nvmlInit()
h = nv.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
print("max", nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM), flush=True)
while True:
    print("%.6f %d %.1f %d" % (time.time(), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                               nv.nvmlDeviceGetPowerUsage(h) / 1000.0, reasons(h)), flush=True)
    time.sleep(0.005)
"""
    REASON_BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.file = None
        self.mode = None
        self.t_begin = None

    def start(self):
        """Spawn the sampler (call before the warm-up: the child needs a moment to import)."""
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".log", delete=False)
        try:
            import pynvml  # noqa: F401  (only to know whether the child can use it)

            self.proc = subprocess.Popen([sys.executable, "-c", self.CHILD, str(self.index)], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
            self.mode = "nvml"
            deadline = time.time() + 10.0  # the child is sampling once its first lines are in the file
            while time.time() < deadline and self.proc.poll() is None and os.path.getsize(self.file.name) < 64:
                time.sleep(0.02)
            return
        except Exception:
            pass
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
            self.mode = "smi"
        except Exception:
            self.proc = None

    def mark_begin(self):
        self.t_begin = time.time()

    def stop(self):
        t_end = time.time()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "no sampler available"}
        if self.mode == "smi":
            time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        lines = self.file.read().splitlines()
        self.file.close()
        os.unlink(self.file.name)
        sm, power, reasons, sm_max = [], [], set(), None
        if self.mode == "nvml":
            for line in lines:
                parts = line.split()
                if len(parts) == 2 and parts[0] == "max":
                    sm_max = float(parts[1])
                    continue
                if len(parts) != 4:
                    continue
                stamp = float(parts[0])
                if self.t_begin is not None and not (self.t_begin <= stamp <= t_end):
                    continue
                sm.append(float(parts[1])); power.append(float(parts[2]))
                mask = int(parts[3])
                reasons.update(name for name, bit in self.REASON_BITS.items() if mask & bit)
            source = "NVML queries every 5 ms from a child process, samples inside the timed region"
        else:
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            maxima = []
            for line in lines:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0])); maxima.append(float(parts[1])); power.append(float(parts[2]))
                except ValueError:
                    continue
                reasons.update(name for name, value in zip(names, parts[3:7]) if value.lower() == "active")
            sm_max = max(maxima) if maxima else None
            source = "nvidia-smi -lms 100"
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": sm_max, "reasons": [], "note": "no samples inside the timed region"}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": sm_max, "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons), "source": source}


def host_threads():
    """Every core this process may run on.  torch.distributed.run exports
    OMP_NUM_THREADS=1, so the count is set explicitly rather than inherited."""
    try:
        count = len(os.sched_getaffinity(0))
    except AttributeError:
        count = os.cpu_count() or 1
    torch.set_num_threads(max(1, count))
    return torch.get_num_threads()


def cpu_reference_sample(spec, budget, steps=1, warmup=0, heads=4, keep=False):
    """The reference's own torch path on the host cores, on a bounded sample:
    the first `heads` heads of the workload, `SparseTileRouter.build_lut`
    (attention/sparse/router.py:248) + `sparse_float_reference`
    (benchmarks/bench_sparse_backends.py:302-326) over every query tile, FP32,
    run from the unmodified sources staged under oracle/_ref.  Without the
    staged copy the CPU restatement of the same two functions runs instead
    (kind "port").  Returns a dict: tops, seconds, sample, cores, kind and, with
    `keep`, the FP32 output and the packed route of the sample."""
    from oracle import h3_oracle as oracle
    from oracle import ref_bridge

    threads = host_threads()
    q, k, v = workloads.structured_qkv(spec, seed=0, heads=range(heads))
    q, k, v = q.float(), k.float(), v.float()
    start, stop = spec.video_range
    geo = oracle.geometry(spec.sequence, start, stop)
    use_ref = ref_bridge.available() and stop == spec.sequence
    ref_layout = ref_bridge.layout(spec.sequence, spec.segments, spec.video_range, spec.video_shape, spec.audio_t)
    router = ref_bridge.router_module().SparseTileRouter(q_tile=128, kv_tile=64) if use_ref else None
    subset = list(range(geo.q_tiles))
    times = []
    out = None
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        if use_ref:
            lut, valid, _ = router.build_lut(q, k, ref_layout, budget)
            out = ref_bridge.sparse_float_reference(q, k, v, lut, valid)
        else:
            _, _, _, route = oracle.build_route(q, k, spec.sequence, start, budget, stop)
            out = oracle.sparse_float_reference(q, k, v, geo, route, q_tile_subset=subset)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    _, _, _, route = oracle.build_route(q, k, spec.sequence, start, budget, stop)
    ops = attention_ops(spec, route, geo, heads)
    sec = statistics.mean(times)
    desc = ("heads 0-%d of %s (%d of %d heads): %s router + FP32 sparse attention over all %d query tiles, "
            "throughput = the sample's algorithmic ops / its time"
            % (heads - 1, spec.name, heads, spec.heads,
               "the reference's own (oracle/_ref)" if use_ref else "restated (oracle port)", geo.q_tiles))
    result = {"tops": ops / sec / 1e12, "seconds": sec, "sample": desc, "cores": threads,
              "kind": "reference" if use_ref else "port"}
    if keep:
        result["out"], result["route"] = out, route
    return result



WARM_SECONDS = 0.3


def warm_up(step, count, world):
    """`count` untimed steps, then more until every rank has kept its GPU busy for
    WARM_SECONDS: a GPU that sat idle while the smaller runs of a scaling series
    used its neighbours starts at idle clocks, and the max over ranks would time
    its ramp instead of the kernels.  Every rank runs the same number of steps
    (the exchange inside a step is collective), agreed on through one all-reduce."""
    import torch
    import torch.distributed as dist

    count = max(1, count)
    begin = time.perf_counter()
    for i in range(count):
        result = step(i)
    torch.cuda.synchronize()
    per_step = max((time.perf_counter() - begin) / count, 1e-5)
    extra = int(max(0.0, WARM_SECONDS - (time.perf_counter() - begin)) / per_step)
    if world > 1:
        agreed = torch.tensor([extra], dtype=torch.int64, device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
        extra = int(agreed.item())
    for i in range(min(extra, 2000)):
        result = step(count + i)
    return result


class quiet_host:
    """Timed regions run with the cyclic garbage collector off (collected once
    before): at 8 GPUs a step lasts under a millisecond while the host needs a
    good part of that to queue it, so a collector pause of a few milliseconds
    would show up as device idle time."""

    def __enter__(self):
        import gc

        gc.collect()
        gc.disable()
        return self

    def __exit__(self, *exc):
        import gc

        gc.enable()
        return False


class Stdout:
    """stdout carries exactly one JSON line.  Libraries that log to file
    descriptor 1 (NCCL with NCCL_DEBUG=INFO does) are sent to stderr instead, so
    their output stays visible without being mixed into the result."""

    def __init__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def emit(self, line):
        sys.stdout.flush()
        os.write(self.saved, (json.dumps(line) + "\n").encode())


def run_reference(args, spec, stdout):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ref = cpu_reference_sample(spec, args.budget, steps=max(1, args.steps), warmup=args.warmup, heads=2)
    line = {
        "impl": "reference", "metric": METRIC, "value": ref["tops"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ref["seconds"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(spec, args.budget), "sample": ref["sample"]},
        "cpu_baseline": {"value": ref["tops"], "unit": UNIT, "cores": ref["cores"], "kind": ref["kind"],
                         "sample": ref["sample"]},
        "e2e": {"value": ref["tops"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    stdout.emit(line)


def workload_name(spec, budget):
    return ("%s: B1 H%d D128, %d tokens (%s), video-KV density %.0f%%, tiles 128x64, INT8 Q/K + FP8-E4M3 V"
            % (spec.name, spec.heads, spec.sequence,
               " + ".join("%d %s" % (b - a, kind) for a, b, kind in spec.segments), budget * 100))


# DRAM traffic of one sparse_attn_tc_kernel launch per head of the 33272-token,
# 30 % workload: dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture
# summarised in profiles/sparse_attn_tc_kernel_config1_4heads.md (4 heads), divided
# by 4; the traffic grows in proportion to the heads of a launch.
ATTN_DRAM_BYTES_PER_HEAD = (51.9e6 + 6.9e6) / 4


def init_ranks(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d does not match WORLD_SIZE %d (launch with torch.distributed.run)" % (args.gpus, world))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # plain peer stores only: the symmetric allocation needs no NVLink multicast binding
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=device)
    return world, rank, local_rank, device


def int8_gemm_peak(device, size=8192, repeats=10):
    """INT8 GEMM rate of this box through cuBLASLt (`torch._int_mm`, 8192^3),
    best of `repeats`: the measured counterpart of the nominal 4.5 POP/s."""
    try:
        a = torch.randint(-127, 128, (size, size), dtype=torch.int8, device=device)
        b = torch.randint(-127, 128, (size, size), dtype=torch.int8, device=device)
        torch._int_mm(a, b)
        torch.cuda.synchronize(device)
        best = float("inf")
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize(device)
            best = min(best, e0.elapsed_time(e1))
        return {"tops": 2.0 * size ** 3 / (best * 1e-3) / 1e12, "how": "torch._int_mm (cuBLASLt) %d^3, best of %d" % (size, repeats)}
    except Exception as exc:  # the measurement is reported, never required
        return {"tops": None, "how": "unavailable: %s" % str(exc).splitlines()[0][:80]}


def tensor_roofline(kernel, achieved_tops, peaks, peak_source, region_seconds, traffic):
    burst = 2.0 * float(peaks["bf16_tflops"])
    sustained = 2.0 * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    long_region = region_seconds >= 1.0
    peak = sustained if long_region else burst
    return {
        "bound": "tensor", "kernel": kernel, "achieved": achieved_tops, "peak": peak, "unit": "TOP/s",
        "frac": achieved_tops / peak,
        "peak_source": "2 x %s of MEASURED_PEAKS.json (%s): INT8/FP8 tensor rate is twice BF16; the timed region "
                       "lasts %.2f s" % ("bf16_tflops_sustained" if long_region else "bf16_tflops (burst)", peak_source,
                                         region_seconds),
        "frac_of_burst": achieved_tops / burst, "frac_of_sustained": achieved_tops / sustained,
        "frac_of_nominal_4500": achieved_tops / NOMINAL_INT8_TOPS, "traffic": traffic,
    }


def projection_summary(spec, device, steps=3):
    """The chunked QKV projection of the same layer on one GPU, timed briefly so that
    the default benchmark line also carries the projection's figures: hidden 3072 ->
    3 x 24 x 128, 4096-token chunks, carriers from the GEMM epilogue."""
    from types import SimpleNamespace

    from h3_optimizations_b200 import ChunkedSparseQKVProjector, ops

    hidden = 3072
    x, w, w_scale = workloads.projection_inputs(spec.sequence, hidden=hidden, heads=spec.heads, seed=0)
    x, w, w_scale = x.to(device), w.to(device), w_scale.to(device)
    module = SimpleNamespace(heads=spec.heads, head_dim=HEAD_DIM, qkv_weight_int8=w, qkv_weight_scale=w_scale)
    projector = ChunkedSparseQKVProjector()

    def timed(fn):
        for _ in range(2): fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps): fn()
        e1.record(); torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / steps

    project_ms = timed(lambda: projector.project(module, x, None, layer_index=0, transformer_options={}))
    chunks = [(a, min(a + 4096, spec.sequence)) for a in range(0, spec.sequence, 4096)]
    x_i8, x_scale = ops.convrot_quant_rows(x)
    shape = (1, spec.heads, spec.sequence, HEAD_DIM)
    q8 = torch.empty(shape, dtype=torch.int8, device=device)
    qs = torch.empty((1, spec.heads, (spec.sequence + 127) // 128), device=device)
    qsum = torch.empty((1, spec.heads, (spec.sequence + 127) // 128, HEAD_DIM), device=device)
    ksum = torch.empty((1, spec.heads, (spec.sequence + 63) // 64, HEAD_DIM), device=device)
    v_stage = torch.empty(shape, dtype=torch.bfloat16, device=device)
    k_stage = torch.empty_like(v_stage)
    stats = ops.column_stats_scratch(spec.heads, device)

    def gemm():
        for a, b in chunks:
            ops.qkv_gemm_chunk_carriers(x_i8[a:b], x_scale[a:b], w, w_scale, heads=spec.heads, row_start=a, q_int8=q8,
                                        q_scale=qs, q_summary=qsum, k_summary=ksum, v_stage=v_stage, stats=stats,
                                        k_stage=k_stage)

    gemm_ms = timed(gemm)
    gemm_ops = 2.0 * spec.sequence * hidden * 3 * spec.heads * HEAD_DIM
    peaks, _ = measured_peaks()
    tops = gemm_ops / (gemm_ms * 1e-3) / 1e12
    return {"workload": "x (%d,%d) bf16 -> ConvRot INT8 QKV projection (W %dx%d int8), 4096-token chunks, carriers from the "
                        "GEMM epilogue" % (spec.sequence, hidden, 3 * spec.heads * HEAD_DIM, hidden),
            "projection_ms": project_ms, "qkv_gemm_all_chunks_ms": gemm_ms, "qkv_gemm_ops": gemm_ops,
            "qkv_gemm_tops": tops, "frac_of_burst": tops / (2.0 * float(peaks["bf16_tflops"])),
            "frac_of_nominal_4500": tops / NOMINAL_INT8_TOPS, "gpu_launches_per_projection": len(chunks) * 2 + 4}


def run_attention(args, spec, stdout):
    """The headline workload (and the 76112-token one): carriers -> router ->
    attention (-> exchange) on N GPUs through the backend objects."""
    import torch.distributed as dist

    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig, runtime_options
    from h3_optimizations_b200.sharding import HeadShardedBackend, head_partition

    world, rank, local_rank, device = init_ranks(args)
    h0, h1 = head_partition(spec.heads, world, rank)
    q_host, k_host, v_host = (t.pin_memory() for t in workloads.structured_qkv(spec, seed=0, heads=range(h0, h1)))
    q, k, v = (t.to(device, non_blocking=True) for t in (q_host, k_host, v_host))
    if args.schedule:
        config = HybridSparseConfig(video_budget=args.budget, early_steps=2, early_kv=0.5, late_steps=2, late_kv=0.5)
        positions = list(range(30))
    else:
        config = HybridSparseConfig(video_budget=args.budget)
        positions = [5]
    options = [runtime_options(spec.layout(), step_index=p, total_steps=30) for p in positions]
    backend = B200SparseBackend(config)
    sharded = HeadShardedBackend(backend, spec.heads, exchange=args.exchange) if world > 1 else None
    owner = sharded if sharded is not None else backend

    records = []  # (position, start, prepared, kernel_done, end) events of the timed steps

    def step(position=0, record=False):
        opts = options[position]
        if record:
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            e[0].record()
        prepared = owner.prepare(q, k, v, layer_index=0, transformer_options=opts)
        if record:
            e[1].record()
        if sharded is not None:
            out = sharded.execute(prepared, kernel_done=e[2] if record else None)
        else:
            out = backend.execute(prepared)
            if record:
                e[2].record()
        if record:
            e[3].record()
            records.append((position, e))
        return out, prepared.sparse

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the fused scatter must reproduce what an NCCL all-gather of the local outputs gives ----
    exchange = "none"
    if sharded is not None:
        prepared = sharded.prepare(q, k, v, layer_index=0, transformer_options=options[0])
        if not sharded.check_exchange(prepared):
            raise SystemExit("rank %d: the reassembled output differs from the NCCL all-gather" % rank)
        exchange = sharded.exchange_note
        del prepared

    # ---- device-resident timing ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _, sparse = warm_up(lambda i: step(i % len(positions)), args.warmup, world)
    fence()
    sampler.mark_begin()
    t_begin = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    out = None
    sparse_by_position = {}
    calls = args.steps * len(positions)
    with quiet_host():
        t_begin.record()
        for i in range(calls):
            out, sparse = step(i % len(positions), record=True)
            sparse_by_position.setdefault(i % len(positions), sparse)
        t_end.record()
        fence()
    region_seconds = time.perf_counter() - wall0

    # ---- the same step replayed from a CUDA graph (backend.capture) ----
    # One layer call is the same ten kernels every sampler step: captured once, a replay costs the host
    # one launch, so a rank whose Python thread is late no longer holds up the barrier of the others.
    launch, graph_ms = "eager: prepare() + execute() per step", None
    if not args.no_graph and not args.schedule and (world == 1 or args.exchange != "nccl"):
        captured, failure = None, None
        try:
            captured = owner.capture(q, k, v, layer_index=0, transformer_options=options[0])
        except Exception as exc:  # the eager figure stands
            failure = "%s: %s" % (type(exc).__name__, str(exc).splitlines()[0][:160] if str(exc) else "")
        agreed = torch.tensor([0 if captured is None else 1], dtype=torch.int32, device=device)
        if world > 1:
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 1:
            for _ in range(3):
                replayed = captured.replay()
            fence()
            same = bool(torch.equal(replayed[:, (h0 if world > 1 else 0):(h1 if world > 1 else spec.heads)],
                                    out[:, (h0 if world > 1 else 0):(h1 if world > 1 else spec.heads)]))
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            wall0 = time.perf_counter()
            with quiet_host():
                g0.record()
                for _ in range(calls):
                    captured.replay()
                g1.record()
                fence()
            region_seconds = max(region_seconds, time.perf_counter() - wall0)
            backend.check_status()
            ms = torch.tensor([g0.elapsed_time(g1) / calls, 1.0 if same else 0.0], dtype=torch.float64, device=device)
            if world > 1:
                worst = ms.clone(); dist.all_reduce(worst, op=dist.ReduceOp.MAX)
                least = ms.clone(); dist.all_reduce(least, op=dist.ReduceOp.MIN)
                ms = torch.stack([worst[0], least[1]])
            if float(ms[1]) == 1.0:
                graph_ms = float(ms[0])
                launch = "CUDA graph replay of prepare + attention%s (backend.capture), one launch per step" % (
                    " + exchange" if world > 1 else "")
            else:
                launch = "eager (the replayed step did not reproduce the eager output; its time is discarded)"
        elif failure is not None:
            launch = "eager (capture failed: %s)" % failure
        else:
            launch = "eager (capture failed on another rank)"
    clocks = sampler.stop() if rank == 0 else None
    device_ms = t_begin.elapsed_time(t_end) / calls
    prep_ms = statistics.mean(e[0].elapsed_time(e[1]) for _, e in records)
    attn_ms = statistics.mean(e[1].elapsed_time(e[2]) for _, e in records)
    exch_ms = statistics.mean(e[2].elapsed_time(e[3]) for _, e in records)

    ops_by_position = {p: float(attention_ops(spec, sp.route.indices, sp.route.geometry, h1 - h0))
                       for p, sp in sparse_by_position.items()}
    local_ops = statistics.mean(ops_by_position[p] for p, _ in records)
    attn_ops_rate = statistics.mean(ops_by_position[p] / (e[1].elapsed_time(e[2]) * 1e-3) for p, e in records) / 1e12
    totals = torch.tensor([local_ops, device_ms, attn_ms, prep_ms, exch_ms], dtype=torch.float64, device=device)
    per_rank = None
    if world > 1:
        every = [torch.zeros_like(totals) for _ in range(world)]
        dist.all_gather(every, totals)
        per_rank = [{"prepare": round(float(t[3]), 4), "attention": round(float(t[2]), 4),
                     "exchange tail": round(float(t[4]), 4)} for t in every]
        summed = totals.clone(); dist.all_reduce(summed, op=dist.ReduceOp.SUM)
        maxed = totals.clone(); dist.all_reduce(maxed, op=dist.ReduceOp.MAX)
        total_ops, device_ms, attn_ms, prep_ms, exch_ms = (float(summed[0]), float(maxed[1]), float(maxed[2]),
                                                            float(maxed[3]), float(maxed[4]))
    else:
        total_ops = local_ops
    schedule = None
    if args.schedule:
        per_position = torch.tensor([statistics.mean(e[0].elapsed_time(e[3]) for p, e in records if p == pos)
                                     for pos in positions], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(per_position, op=dist.ReduceOp.MAX)
        from h3_optimizations_b200 import resolve_video_budget
        schedule = [{"step": pos, "budget": resolve_video_budget(config, pos, 30, 0), "ms": float(per_position[i])}
                    for i, pos in enumerate(positions)]

    # ---- end to end with host buffers ----
    e2e = None
    if not args.skip_e2e:
        out_host = torch.empty((1, h1 - h0, spec.sequence, HEAD_DIM), dtype=torch.bfloat16).pin_memory()
        e2e_calls = max(1, args.steps)

        def e2e_step(i):
            # the host entry of the backend: H2D of head chunk c+1, kernels of chunk c and D2H of chunk
            # c-1 overlap on three streams; every rank moves its own heads over its own PCIe link
            owner.forward_host(q_host, k_host, v_host, out_host, layer_index=0,
                               transformer_options=options[i % len(positions)])
        for i in range(max(1, min(args.warmup, 2))):
            e2e_step(i)
        fence()
        b0 = torch.cuda.Event(enable_timing=True); b1 = torch.cuda.Event(enable_timing=True)
        with quiet_host():
            b0.record()
            for i in range(e2e_calls):
                e2e_step(i)
            b1.record()
            fence()
        e2e_ms = torch.tensor([b0.elapsed_time(b1) / e2e_calls], dtype=torch.float64, device=device)
        moved = torch.tensor([3.0 * q_host.numel() * q_host.element_size(),
                              float(out_host.numel() * out_host.element_size())], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(moved, op=dist.ReduceOp.SUM)
        e2e_ops = total_ops if not args.schedule else float(
            statistics.mean(ops_by_position[i % len(positions)] for i in range(e2e_calls))) * (total_ops / local_ops)
        e2e = {"value": e2e_ops / (float(e2e_ms[0]) * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": float(e2e_ms[0]),
               "api": "%s.forward_host: pinned host Q/K/V of the rank's heads in, its output slice back to the host, "
                      "head chunks pipelined over three streams%s"
                      % ("HeadShardedBackend" if world > 1 else "B200SparseBackend",
                         "; every rank uses its own PCIe link, nothing crosses GPUs" if world > 1 else ""),
               "h2d_bytes_per_step": int(moved[0]), "d2h_bytes_per_step": int(moved[1])}

    if rank == 0:
        peaks, peak_source = measured_peaks()
        heads_local = h1 - h0
        carrier_bytes = heads_local * spec.sequence * HEAD_DIM * (3 * 2 + 3 * 1) + heads_local * spec.sequence * HEAD_DIM * 2 * 2
        traffic = ATTN_DRAM_BYTES_PER_HEAD * heads_local if (spec.sequence == 33272 and abs(args.budget - 0.3) < 1e-9
                                                              and not args.schedule) else None
        step_ms = graph_ms if graph_ms is not None else device_ms
        line = {
            "metric": METRIC, "value": total_ops / (step_ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 QK^T / fp8-e4m3 PV, fp32 softmax",
            "data": "synthetic",
            "launch": launch, "eager_ms_per_step": device_ms,
            "config": {
                "workload": workload_name(spec, args.budget) + (" [30-step schedule 0.5,0.5,0.3x26,0.5,0.5]" if args.schedule else ""),
                "heads_per_gpu": heads_local, "parallelism": "head-sharded x%d" % world, "exchange": exchange,
                "l2_policy": "no flush: a step streams %.0f MB of bf16 Q/K/V, %.0f MB of carriers (written, then read) and "
                             "the %.0f MB gathered output through this GPU's 126 MB L2"
                             % (heads_local * spec.sequence * HEAD_DIM * 2 * 3 / 1e6,
                                heads_local * spec.sequence * HEAD_DIM * 3 / 1e6,
                                spec.heads * spec.sequence * HEAD_DIM * 2 / 1e6),
                "p_terms": 2, "algorithmic_ops": total_ops, "route_len": sparse.route.route_len,
                "layer_calls_per_step": len(positions),
            },
            "stages_ms": {"prepare (stats+quant+route)": prep_ms, "attention": attn_ms, "exchange tail": exch_ms},
            "stages_from": "CUDA events around the stages of the eager steps (eager_ms_per_step is their step time)",
            "stages_ms_per_rank": per_rank,
            "prepare_hbm": {"bytes": carrier_bytes, "gbs": carrier_bytes / (prep_ms * 1e-3) / 1e9,
                            "frac_of_measured_copy": carrier_bytes / (prep_ms * 1e-3) / 1e9 / float(peaks["hbm_gbs"])},
            "roofline": tensor_roofline("sparse_attn_tc_kernel", attn_ops_rate, peaks, peak_source, region_seconds, traffic),
            "int8_peak_measured": int8_gemm_peak(device),
            "clocks": clocks,
            "gpu_launches": calls * 7,
        }
        if traffic is not None:
            line["roofline"]["traffic_source"] = ("dram__bytes_read.sum + dram__bytes_write.sum of a 4-head ncu capture "
                                                  "(profiles/), scaled to the %d heads of one launch" % heads_local)
        if schedule is not None:
            line["schedule_ms"] = schedule
        if world == 1 and spec.sequence == 33272 and not args.heads and not args.schedule and not args.skip_e2e:
            line["qkv_projection"] = projection_summary(spec, device)
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.skip_cpu_baseline:
            sample_heads = min(8, spec.heads)
            ref = cpu_reference_sample(spec, args.budget, heads=sample_heads, keep=not args.schedule)
            line["cpu_baseline"] = {"value": ref["tops"], "unit": UNIT, "cores": ref["cores"], "kind": ref["kind"],
                                    "sample": ref["sample"], "seconds": ref["seconds"]}
            if "out" in ref and out is not None:
                # the reference's FP32 attention on the same block mask against this backend's output
                got = out[:, :sample_heads].float().cpu()
                want = ref["out"]
                a, b = got.double().flatten(), want.double().flatten()
                route_gpu = sparse.route.indices[:, :sample_heads].cpu()
                line["fp32_sdpa_same_mask"] = {
                    "heads": sample_heads,
                    "cosine": float((a @ b) / (a.norm() * b.norm())),
                    "rel_max_abs": float((a - b).abs().max() / b.abs().max()),
                    "rel_rmse": float((a - b).norm() / b.norm()),
                    "mask_rows_differing": int((route_gpu != ref["route"]).any(dim=-1).sum()),
                    "note": "reported, not gated: INT8 Q/K + FP8 V carriers against FP32 attention",
                }
        stdout.emit(line)
    if world > 1:
        dist.destroy_process_group()


def run_config2(args, spec, stdout):
    """Chunked ConvRot INT8 QKV projection (hidden 3072 -> 3 x H x 128,
    4096-token chunks, carriers from the GEMM epilogue) + router + attention.
    N > 1: each rank holds the weight rows of its heads and the whole x."""
    import torch.distributed as dist
    from types import SimpleNamespace

    from h3_optimizations_b200 import B200SparseBackend, ChunkedSparseQKVProjector, HybridSparseConfig, ops, runtime_options
    from h3_optimizations_b200.sharding import HeadShardedBackend, head_partition, shard_qkv_weight

    world, rank, local_rank, device = init_ranks(args)
    h0, h1 = head_partition(spec.heads, world, rank)
    heads_local = h1 - h0
    hidden = 3072
    x, w, w_scale = workloads.projection_inputs(spec.sequence, hidden=hidden, heads=spec.heads, seed=0)
    w, w_scale = shard_qkv_weight(w, w_scale, spec.heads, h0, h1)
    x, w, w_scale = x.to(device), w.to(device), w_scale.to(device)
    module = SimpleNamespace(heads=heads_local, head_dim=HEAD_DIM, qkv_weight_int8=w, qkv_weight_scale=w_scale)
    projector = ChunkedSparseQKVProjector()
    backend = B200SparseBackend(HybridSparseConfig(video_budget=args.budget))
    sharded = HeadShardedBackend(backend, spec.heads, exchange=args.exchange) if world > 1 else None
    owner = sharded if sharded is not None else backend
    options = runtime_options(spec.layout(), step_index=5, total_steps=30)

    marks = []

    def step(record=False):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if record else None
        if record: e[0].record()
        projected = projector.project(module, x, None, layer_index=0, transformer_options=options)
        if record: e[1].record()
        prepared = owner.prepare_projected(projected, layer_index=0, transformer_options=options)
        if record: e[2].record()
        out = owner.execute(prepared)
        if record:
            e[3].record(); marks.append(e)
        return out, prepared.sparse

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    exchange = "none"
    if sharded is not None:
        projected = projector.project(module, x, None, layer_index=0, transformer_options=options)
        prepared = sharded.prepare_projected(projected, layer_index=0, transformer_options=options)
        if not sharded.check_exchange(prepared):
            raise SystemExit("rank %d: the reassembled output differs from the NCCL all-gather" % rank)
        exchange = sharded.exchange_note
        del projected, prepared
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _, sparse = warm_up(lambda i: step(), args.warmup, world)
    fence()
    sampler.mark_begin()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    with quiet_host():
        t0.record()
        for _ in range(args.steps):
            _, sparse = step(record=True)
        t1.record(); fence()
    region_seconds = time.perf_counter() - wall0
    clocks = sampler.stop() if rank == 0 else None
    step_ms = t0.elapsed_time(t1) / args.steps
    proj_ms = statistics.mean(m[0].elapsed_time(m[1]) for m in marks)
    route_ms = statistics.mean(m[1].elapsed_time(m[2]) for m in marks)
    attn_ms = statistics.mean(m[2].elapsed_time(m[3]) for m in marks)

    # the GEMM of every chunk alone: carrier epilogue, and plain bf16 staging for comparison
    chunks = [(a, min(a + 4096, spec.sequence)) for a in range(0, spec.sequence, 4096)]
    x_i8, x_scale = ops.convrot_quant_rows(x)
    shape = (1, heads_local, spec.sequence, HEAD_DIM)
    q8 = torch.empty(shape, dtype=torch.int8, device=device)
    qs = torch.empty((1, heads_local, (spec.sequence + 127) // 128), device=device)
    qsum = torch.empty((1, heads_local, (spec.sequence + 127) // 128, HEAD_DIM), device=device)
    ksum = torch.empty((1, heads_local, (spec.sequence + 63) // 64, HEAD_DIM), device=device)
    v_stage = torch.empty(shape, dtype=torch.bfloat16, device=device)
    k_stage = torch.empty_like(v_stage)
    staging = torch.empty((3 * heads_local, spec.sequence, HEAD_DIM), dtype=torch.bfloat16, device=device)
    stats = ops.column_stats_scratch(heads_local, device)

    def gemm_carriers():
        for a, b in chunks:
            ops.qkv_gemm_chunk_carriers(x_i8[a:b], x_scale[a:b], w, w_scale, heads=heads_local, row_start=a, q_int8=q8,
                                        q_scale=qs, q_summary=qsum, k_summary=ksum, v_stage=v_stage, stats=stats,
                                        k_stage=k_stage)

    def gemm_plain():
        for a, b in chunks:
            ops.qkv_gemm_chunk(x_i8[a:b], x_scale[a:b], w, w_scale, staging, row_start=a)

    def timed(fn):
        for _ in range(3): fn()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps): fn()
        g1.record(); torch.cuda.synchronize()
        return g0.elapsed_time(g1) / args.steps

    gemm_ms = timed(gemm_carriers)
    plain_ms = timed(gemm_plain)
    rot_ms = timed(lambda: ops.convrot_quant_rows(x, x_i8, x_scale))

    geo = sparse.route.geometry
    local = torch.tensor([float(attention_ops(spec, sparse.route.indices, geo, heads_local)),
                          2.0 * spec.sequence * hidden * 3 * heads_local * HEAD_DIM], dtype=torch.float64, device=device)
    worst = torch.tensor([step_ms, proj_ms, route_ms, attn_ms, gemm_ms, plain_ms, rot_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(local, op=dist.ReduceOp.SUM)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    attn_ops, gemm_ops = float(local[0]), float(local[1])
    step_ms, proj_ms, route_ms, attn_ms, gemm_ms, plain_ms, rot_ms = (float(t) for t in worst)
    if rank == 0:
        peaks, peak_source = measured_peaks()
        gemm_tops = gemm_ops / world / (gemm_ms * 1e-3) / 1e12  # per GPU
        rot_bytes = spec.sequence * hidden * 3 + spec.sequence * 4
        line = {
            "metric": METRIC, "value": (attn_ops + gemm_ops) / (step_ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 GEMM + int8 QK^T / fp8-e4m3 PV", "data": "synthetic",
            "config": {"workload": "config2: x (%d,%d) bf16 -> ConvRot INT8 QKV projection (W %dx%d int8, 4096-token chunks, "
                                   "carriers from the GEMM epilogue) -> %s"
                                   % (spec.sequence, hidden, 3 * spec.heads * HEAD_DIM, hidden, workload_name(spec, args.budget)),
                       "heads_per_gpu": heads_local, "exchange": exchange,
                       "parallelism": "head-sharded x%d: weight rows {q,k,v} x local heads per rank, x replicated" % world,
                       "algorithmic_ops": {"attention": attn_ops, "qkv_gemm": gemm_ops},
                       "l2_policy": "activations + staging (>600 MB) exceed the 126 MB L2; no flush"},
            "stages_ms": {"projection (rotate + gemm with carrier epilogue + K/V second phase)": proj_ms, "router": route_ms,
                          "attention (+ exchange)": attn_ms, "qkv_gemm with carrier epilogue, all chunks": gemm_ms,
                          "qkv_gemm with plain bf16 epilogue, all chunks": plain_ms, "convrot, all chunks": rot_ms},
            "roofline": tensor_roofline("qkv_gemm_kernel<carriers>", gemm_tops, peaks, peak_source, region_seconds, None),
            "int8_peak_measured": int8_gemm_peak(device),
            "convrot_hbm": {"bytes": rot_bytes, "gbs": rot_bytes / (rot_ms * 1e-3) / 1e9,
                            "frac_of_measured_copy": rot_bytes / (rot_ms * 1e-3) / 1e9 / float(peaks["hbm_gbs"])},
            "clocks": clocks, "gpu_launches": args.steps * (len(chunks) * 2 + 7),
        }
        stdout.emit(line)
    if world > 1:
        dist.destroy_process_group()


def run_config4(args, spec, stdout):
    """Mixed-modality DiT block, batch 2: text + reference + audio + video
    tokens, only video x video tiles sparse; attention, then out_proj (bf16) and
    the chunked FP8-E4M3 MLP 3072 -> 12288 (GELU-tanh) -> 3072 in 4096-token
    chunks.  Batch elements and heads are both independent units on the attention
    path, so the 2 x 24 (batch, head) pairs are sharded over the ranks like 48
    heads; behind the exchange every rank runs out_proj and the MLP on its share
    of the 2 x 35832 token rows."""
    import torch.distributed as dist

    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig, ops, runtime_options
    from h3_optimizations_b200.mlp import ChunkedFP8MLP
    from h3_optimizations_b200.sharding import HeadShardedBackend, head_partition

    world, rank, local_rank, device = init_ranks(args)
    batch, hidden, ffn = 2, 3072, 12288
    units = batch * spec.heads
    u0, u1 = head_partition(units, world, rank)
    pieces = []
    for unit in range(u0, u1):  # unit = batch element * heads + head; every batch element has its own seed
        b, head = divmod(unit, spec.heads)
        pieces.append(workloads.structured_qkv(spec, seed=b, heads=[head]))
    q, k, v = (torch.cat([p[i] for p in pieces], dim=1).to(device) for i in range(3))
    gen = torch.Generator().manual_seed(7)
    w_out = (torch.randn((hidden, spec.heads * HEAD_DIM), generator=gen) * 0.02).to(torch.bfloat16).to(device)
    mlp = ChunkedFP8MLP(torch.randn((ffn, hidden), generator=gen) * 0.02, torch.zeros(ffn),
                        torch.randn((hidden, ffn), generator=gen) * 0.02, torch.zeros(hidden)).to(device)
    backend = B200SparseBackend(HybridSparseConfig(video_budget=args.budget))
    sharded = HeadShardedBackend(backend, units, exchange=args.exchange) if world > 1 else None
    owner = sharded if sharded is not None else backend
    options = runtime_options(spec.layout(), step_index=5, total_steps=30)
    total_rows = batch * spec.sequence
    r0, r1 = head_partition(total_rows, world, rank)  # this rank's token rows of the (batch * S, hidden) activations
    marks = []

    def step(record=False):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if record else None
        if record: e[0].record()
        prepared = owner.prepare(q, k, v, layer_index=0, transformer_options=options)
        if record: e[1].record()
        out = owner.execute(prepared)                                        # (1, units, S, 128) on every rank
        if record: e[2].record()
        # (batch, heads, S, 128) -> token-major rows (batch * S, heads * 128) of this rank's share
        by_token = out.view(batch, spec.heads, spec.sequence, HEAD_DIM).permute(0, 2, 1, 3)   # (batch, S, heads, 128)
        parts = []
        for b in range(batch):
            s0, s1 = max(r0 - b * spec.sequence, 0), min(r1 - b * spec.sequence, spec.sequence)
            if s0 < s1:
                parts.append(by_token[b, s0:s1].reshape(s1 - s0, spec.heads * HEAD_DIM))
        rows = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        rows = rows if rows.is_contiguous() else rows.contiguous()
        y = ops.dense_gemm(rows, w_out)
        if record: e[3].record()
        z = mlp(y)
        if record:
            e[4].record(); marks.append(e)
        return z, prepared.sparse

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _, sparse = warm_up(lambda i: step(), args.warmup, world)
    fence()
    sampler.mark_begin()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    with quiet_host():
        t0.record()
        for _ in range(args.steps):
            _, sparse = step(record=True)
        t1.record(); fence()
    region_seconds = time.perf_counter() - wall0
    clocks = sampler.stop() if rank == 0 else None
    stage = [statistics.mean(m[i].elapsed_time(m[i + 1]) for m in marks) for i in range(4)]
    worst = torch.tensor([t0.elapsed_time(t1) / args.steps] + stage, dtype=torch.float64, device=device)
    local = torch.tensor([float(attention_ops(spec, sparse.route.indices, sparse.route.geometry, u1 - u0)),
                          2.0 * (r1 - r0) * hidden * spec.heads * HEAD_DIM, 4.0 * (r1 - r0) * hidden * ffn],
                         dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(local, op=dist.ReduceOp.SUM)
    if rank == 0:
        peaks, peak_source = measured_peaks()
        step_ms, prep_ms, attn_ms, proj_ms, mlp_ms = (float(t) for t in worst)
        attn_ops, proj_ops, mlp_ops = (float(t) for t in local)
        mlp_tops = mlp_ops / world / (mlp_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": (attn_ops + proj_ops + mlp_ops) / (step_ms * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 QK^T / fp8-e4m3 PV; bf16 out_proj; fp8-e4m3 MLP", "data": "synthetic",
            "config": {"workload": "config4: B2 H%d D128, %d tokens per batch element (%s), video x video tiles sparse at %.0f%%, "
                                   "then out_proj %d->%d (bf16) and FP8-E4M3 MLP %d->%d (GELU-tanh)->%d in 4096-token chunks"
                                   % (spec.heads, spec.sequence, " + ".join("%d %s" % (b - a, kind) for a, b, kind in spec.segments),
                                      args.budget * 100, spec.heads * HEAD_DIM, hidden, hidden, ffn, hidden),
                       "parallelism": "%d (batch, head) units and %d token rows sharded x%d" % (units, total_rows, world),
                       "exchange": sharded.exchange_note if sharded is not None else "none",
                       "algorithmic_ops": {"attention": attn_ops, "out_proj": proj_ops, "mlp": mlp_ops},
                       "l2_policy": "Q,K,V (%.0f MB per GPU) exceed the 126 MB L2; no flush"
                                    % ((u1 - u0) * spec.sequence * HEAD_DIM * 2 * 3 / 1e6)},
            "stages_ms": {"prepare": prep_ms, "attention (+ exchange)": attn_ms, "out_proj": proj_ms, "fp8 mlp": mlp_ms},
            "roofline": tensor_roofline("qkv_gemm_kernel<dense> (FP8 MLP: two GEMMs + two row quantisers)", mlp_tops, peaks,
                                        peak_source, region_seconds, None),
            "clocks": clocks,
            "gpu_launches": args.steps * (7 + 1 + 4 * ((r1 - r0 + 4095) // 4096)),
        }
        stdout.emit(line)
    if world > 1:
        dist.destroy_process_group()


def pin_rank_cores():
    """Multi-rank runs: give every rank its own share of the host cores before any
    thread is started.  At a step of under a millisecond a rank whose launching
    thread is moved or preempted for 50 us leaves its GPU idle, and the barrier at
    the end of the step makes every other rank wait for it.  Off unless
    H3S_BENCH_PIN=1."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1 or os.environ.get("H3S_BENCH_PIN", "0") != "1" or not hasattr(os, "sched_setaffinity"):
        return None
    allowed = sorted(os.sched_getaffinity(0))
    share = len(allowed) // world
    if share < 1:
        return None
    local = int(os.environ.get("LOCAL_RANK", "0"))
    mine = allowed[local * share:(local + 1) * share]
    try:
        os.sched_setaffinity(0, mine)
    except OSError:
        return None
    return mine


def main():
    args = parse_args()
    if args.impl != "reference":
        pin_rank_cores()
    stdout = Stdout()
    spec = {"config1": workloads.CONFIG1, "config2": workloads.CONFIG1, "config3": workloads.CONFIG3,
            "config4": workloads.CONFIG4}[args.config]
    if args.heads:
        import dataclasses

        spec = dataclasses.replace(spec, heads=args.heads, name="%s[%d heads]" % (spec.name, args.heads))
    if args.impl == "reference":
        run_reference(args, spec, stdout)
    elif args.config == "config2":
        run_config2(args, spec, stdout)
    elif args.config == "config4":
        run_config4(args, spec, stdout)
    else:
        run_attention(args, spec, stdout)


if __name__ == "__main__":
    main()
