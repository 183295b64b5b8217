"""Benchmark of the sparse-attention hot path (BASELINE config 1).

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
`--impl reference` times the CPU restatement of the reference's torch path
(router + float sparse attention) on the host cores instead.
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
    parser.add_argument("--config", choices=("config1", "config2", "config3"), default="config1",
                        help="config1 is the headline workload; config2 adds the chunked QKV projection in front; "
                             "config3 is the 76112-token sequence")
    parser.add_argument("--budget", type=float, default=VIDEO_BUDGET)
    parser.add_argument("--single-term-p", action="store_true",
                        help="carry P as one E4M3 term (faster, outside the parity gate on Gaussian V)")
    parser.add_argument("--heads", type=int, default=0,
                        help="run a head subset of the workload (profiling captures); 0 = all heads")
    parser.add_argument("--skip-cpu-baseline", action="store_true")
    parser.add_argument("--skip-e2e", action="store_true")
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


def cpu_reference_sample(spec, budget, steps=1, warmup=0, heads=4):
    """The reference's own torch path on the host cores, on a bounded sample:
    the first `heads` heads of the workload, `SparseTileRouter.build_lut`
    (attention/sparse/router.py:248) + `sparse_float_reference`
    (benchmarks/bench_sparse_backends.py:302-326) over every query tile, FP32,
    run from the unmodified sources staged under oracle/_ref.  Without the
    staged copy the CPU restatement of the same two functions runs instead
    (kind "port").  Returns (TOPS, seconds per step, description, threads, kind)."""
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
    ops = 0
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        if use_ref:
            lut, valid, _ = router.build_lut(q, k, ref_layout, budget)
            ref_bridge.sparse_float_reference(q, k, v, lut, valid)
        else:
            _, _, _, route = oracle.build_route(q, k, spec.sequence, start, budget, stop)
            oracle.sparse_float_reference(q, k, v, geo, route, q_tile_subset=subset)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
        if it == 0:
            _, _, _, route = oracle.build_route(q, k, spec.sequence, start, budget, stop)
            ops = attention_ops(spec, route, geo, heads)
    sec = statistics.mean(times)
    desc = ("heads 0-%d of %s (%d of %d heads): %s router + FP32 sparse attention over all %d query tiles, "
            "throughput = the sample's algorithmic ops / its time"
            % (heads - 1, spec.name, heads, spec.heads,
               "the reference's own (oracle/_ref)" if use_ref else "restated (oracle port)", geo.q_tiles))
    return ops / sec / 1e12, sec, desc, threads, "reference" if use_ref else "port"


def run_reference(args, spec):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tops, sec, desc, threads, kind = cpu_reference_sample(spec, args.budget, steps=max(1, args.steps),
                                                          warmup=args.warmup, heads=2)
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(spec, args.budget), "sample": desc},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": threads, "kind": kind, "sample": desc},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_name(spec, budget):
    return ("%s: B1 H%d D128, %d tokens (%s), video-KV density %.0f%%, tiles 128x64, INT8 Q/K + FP8-E4M3 V"
            % (spec.name, spec.heads, spec.sequence,
               " + ".join("%d %s" % (b - a, kind) for a, b, kind in spec.segments), budget * 100))


def run_config2(args, spec):
    """BASELINE config 2 on one GPU: chunked ConvRot INT8 QKV projection
    (hidden 3072 -> 3 x H x 128, 4096-token chunks) feeding the carriers, then
    the router and the attention kernel as in config 1.  Reports the stage times
    and the GEMM's own tensor roofline; `value` counts attention + GEMM ops."""
    from types import SimpleNamespace

    from h3_optimizations_b200 import B200SparseBackend, ChunkedSparseQKVProjector, HybridSparseConfig, ops, runtime_options

    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    hidden = 3072
    x, w, w_scale = workloads.projection_inputs(spec.sequence, hidden=hidden, heads=spec.heads, seed=0)
    x, w, w_scale = x.to(device), w.to(device), w_scale.to(device)
    module = SimpleNamespace(heads=spec.heads, head_dim=HEAD_DIM, qkv_weight_int8=w, qkv_weight_scale=w_scale)
    projector = ChunkedSparseQKVProjector()
    backend = B200SparseBackend(HybridSparseConfig(video_budget=args.budget))
    options = runtime_options(spec.layout(), step_index=5, total_steps=30)

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    marks = []

    def step(record=False):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if record else None
        if record: e[0].record()
        projected = projector.project(module, x, None, layer_index=0, transformer_options=options)
        if record: e[1].record()
        prepared = backend.prepare_projected(projected, layer_index=0, transformer_options=options)
        if record: e[2].record()
        out = backend.execute(prepared)
        if record:
            e[3].record(); marks.append(e)
        return out, prepared.sparse

    sampler = ClockSampler(0); sampler.start()
    for _ in range(args.warmup):
        _, sparse = step()
    torch.cuda.synchronize()
    sampler.mark_begin()
    t0, t1 = events(); t0.record()
    for _ in range(args.steps):
        _, sparse = step(record=True)
    t1.record(); torch.cuda.synchronize()
    clocks = sampler.stop()
    step_ms = t0.elapsed_time(t1) / args.steps
    proj_ms = statistics.mean(m[0].elapsed_time(m[1]) for m in marks)
    route_ms = statistics.mean(m[1].elapsed_time(m[2]) for m in marks)
    attn_ms = statistics.mean(m[2].elapsed_time(m[3]) for m in marks)

    # the GEMM alone, every chunk of the sequence, into a throw-away staging buffer
    staging = torch.empty((3 * spec.heads, spec.sequence, HEAD_DIM), dtype=torch.bfloat16, device=device)
    x_i8, x_scale = ops.convrot_quant_rows(x)
    chunks = [(a, min(a + 4096, spec.sequence)) for a in range(0, spec.sequence, 4096)]
    def gemm_all():
        for a, b in chunks:
            ops.qkv_gemm_chunk(x_i8[a:b], x_scale[a:b], w, w_scale, staging, row_start=a)
    for _ in range(3): gemm_all()
    g0, g1 = events(); g0.record()
    for _ in range(args.steps): gemm_all()
    g1.record(); torch.cuda.synchronize()
    gemm_ms = g0.elapsed_time(g1) / args.steps
    # the same GEMM with the per-head RMS norm and split-half rotation in its epilogue
    gen = torch.Generator().manual_seed(1)
    q_norm = (torch.rand(HEAD_DIM, generator=gen) + 0.5).to(device)
    k_norm = (torch.rand(HEAD_DIM, generator=gen) + 0.5).to(device)
    angles = torch.arange(spec.sequence * 48, dtype=torch.float32).reshape(spec.sequence, 48) * (1.0 / 8192.0)
    rope = torch.stack((torch.cos(angles), -torch.sin(angles), torch.sin(angles), torch.cos(angles)), dim=-1)
    rope = rope.reshape(1, spec.sequence, 1, 48, 2, 2).to(torch.bfloat16).to(device)
    def gemm_norm_rope_all(table):
        for a, b in chunks:
            ops.qkv_gemm_chunk(x_i8[a:b], x_scale[a:b], w, w_scale, staging, row_start=a, q_norm=q_norm,
                               k_norm=k_norm, epsilon=1e-6, rope=table)
    epilogue_ms = {}
    for label, table in (("norm", None), ("norm + rope", rope)):
        for _ in range(3): gemm_norm_rope_all(table)
        n0, n1 = events(); n0.record()
        for _ in range(args.steps): gemm_norm_rope_all(table)
        n1.record(); torch.cuda.synchronize()
        epilogue_ms[label] = n0.elapsed_time(n1) / args.steps
    c0, c1 = events(); c0.record()
    for _ in range(args.steps): ops.convrot_quant_rows(x, x_i8, x_scale)
    c1.record(); torch.cuda.synchronize()
    rot_ms = c0.elapsed_time(c1) / args.steps

    geo = sparse.route.geometry
    attn_ops = float(attention_ops(spec, sparse.route.indices, geo, spec.heads))
    gemm_ops = 2.0 * spec.sequence * hidden * 3 * spec.heads * HEAD_DIM
    peaks, peak_source = measured_peaks()
    int8_peak = 2.0 * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    gemm_tops = gemm_ops / (gemm_ms * 1e-3) / 1e12
    rot_bytes = spec.sequence * hidden * 3 + spec.sequence * 4
    line = {
        "metric": METRIC, "value": (attn_ops + gemm_ops) / (step_ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 GEMM + int8 QK^T / fp8-e4m3 PV", "data": "synthetic",
        "config": {"workload": "config2: x (%d,%d) bf16 -> ConvRot INT8 QKV projection (W %dx%d int8, 4096-token chunks) -> %s"
                               % (spec.sequence, hidden, 3 * spec.heads * HEAD_DIM, hidden, workload_name(spec, args.budget)),
                   "algorithmic_ops": {"attention": attn_ops, "qkv_gemm": gemm_ops},
                   "l2_policy": "activations + staging (>800 MB) exceed the 126 MB L2; no flush"},
        "stages_ms": {"projection (rotate+gemm+carriers)": proj_ms, "router": route_ms, "attention": attn_ms,
                      "qkv_gemm alone": gemm_ms, "qkv_gemm with RMS norm epilogue": epilogue_ms["norm"],
                      "qkv_gemm with RMS norm + RoPE epilogue": epilogue_ms["norm + rope"],
                      "convrot alone": rot_ms},
        "roofline": {"bound": "tensor", "kernel": "qkv_gemm_kernel", "achieved": gemm_tops, "peak": int8_peak,
                     "unit": "TOP/s", "frac": gemm_tops / int8_peak, "frac_of_nominal_4500": gemm_tops / NOMINAL_INT8_TOPS,
                     "peak_source": "2 x bf16_tflops_sustained of MEASURED_PEAKS.json (%s)" % peak_source, "traffic": None},
        "convrot_hbm": {"bytes": rot_bytes, "gbs": rot_bytes / (rot_ms * 1e-3) / 1e9,
                        "frac_of_measured_copy": rot_bytes / (rot_ms * 1e-3) / 1e9 / float(peaks["hbm_gbs"])},
        "clocks": clocks, "gpu_launches": args.steps * (len(chunks) * 3 + 6),
    }
    print(json.dumps(line))


def main():
    args = parse_args()
    spec = {"config1": workloads.CONFIG1, "config2": workloads.CONFIG1, "config3": workloads.CONFIG3}[args.config]
    if args.heads:
        import dataclasses

        spec = dataclasses.replace(spec, heads=args.heads, name="%s[%d heads]" % (spec.name, args.heads))
    if args.impl == "reference":
        run_reference(args, spec)
        return
    if args.config == "config2":
        if args.gpus != 1:
            raise SystemExit("config2 is a single-GPU stage benchmark here; use --gpus 1")
        run_config2(args, spec)
        return

    import torch.distributed as dist

    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig, ops, runtime_options
    from h3_optimizations_b200.sharding import SymmetricHeadOutput, gather_heads, head_partition

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
        # stdout carries exactly one JSON line: keep NCCL's version banner out of it
        if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "INFO", "TRACE"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)

    h0, h1 = head_partition(spec.heads, world, rank)
    q_host, k_host, v_host = (t.pin_memory() for t in workloads.structured_qkv(spec, seed=0, heads=range(h0, h1)))
    q, k, v = (t.to(device, non_blocking=True) for t in (q_host, k_host, v_host))
    backend = B200SparseBackend(HybridSparseConfig(video_budget=args.budget))
    options = runtime_options(spec.layout(), step_index=5, total_steps=30)
    full_out, symmetric, peer_ptrs, exchange = None, None, None, "none"
    if world > 1:
        try:
            if os.environ.get("H3S_BENCH_NCCL_GATHER"):
                raise RuntimeError("NCCL gather requested")
            symmetric = SymmetricHeadOutput(spec.heads, spec.sequence, torch.bfloat16, device)
            full_out, peer_ptrs = symmetric.tensor, symmetric.peer_slice_ptrs()
            exchange = "attention epilogue stores every tile into all peers' buffers (P2P over NVLink) + barrier"
        except Exception as exc:  # symmetric memory unavailable: plain NCCL all-gather after the kernel
            symmetric = None
            failure = exc
        agreed = torch.tensor([1 if symmetric is not None else 0], dtype=torch.int32, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:  # all ranks take the same path
            exc = failure if symmetric is None else RuntimeError("a peer could not set up symmetric memory")
            symmetric, peer_ptrs = None, None
            full_out = torch.empty((1, spec.heads, spec.sequence, HEAD_DIM), dtype=torch.bfloat16, device=device)
            exchange = "NCCL all-gather after the kernel (%s)" % str(exc).splitlines()[0][:80]

    attn_events = []
    prep_events = []

    def step(qd, kd, vd, record=False):
        if record:
            e0 = torch.cuda.Event(enable_timing=True); e0.record()
        prepared = backend.prepare(qd, kd, vd, layer_index=0, transformer_options=options)
        sparse = prepared.sparse
        geo = sparse.route.geometry
        if record:
            e1 = torch.cuda.Event(enable_timing=True); e1.record()
        if world > 1:
            local = full_out[:, h0:h1]
            out = ops.sparse_attention(
                sparse.q_int8, sparse.k_int8, sparse.v_carrier, sparse.q_scale, sparse.k_scale, sparse.v_scale,
                sparse.route.indices, q_start=geo.pure_video_q_start, q_stop=geo.pure_video_q_stop, out=local,
                single_term_p=args.single_term_p, peer_out_ptrs=peer_ptrs)
        else:
            out = ops.sparse_attention(
                sparse.q_int8, sparse.k_int8, sparse.v_carrier, sparse.q_scale, sparse.k_scale, sparse.v_scale,
                sparse.route.indices, q_start=geo.pure_video_q_start, q_stop=geo.pure_video_q_stop,
                out_dtype=torch.bfloat16, single_term_p=args.single_term_p)
        if record:
            e2 = torch.cuda.Event(enable_timing=True); e2.record()
            prep_events.append((e0, e1)); attn_events.append((e1, e2))
        if world > 1:
            if symmetric is not None:
                symmetric.barrier()
                out = full_out
            else:
                out = gather_heads(out, spec.heads, out=full_out)
        return out, sparse

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the fused scatter must reproduce what an NCCL all-gather of the local outputs gives ----
    if symmetric is not None:
        step(q, k, v)
        torch.cuda.synchronize()
        reference = gather_heads(full_out[:, h0:h1].clone(), spec.heads)
        torch.cuda.synchronize()
        if not torch.equal(reference, full_out):
            raise SystemExit("rank %d: peer-scattered output differs from the NCCL all-gather" % rank)
        dist.barrier()

    # ---- device-resident timing ----
    sparse = None
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        _, sparse = step(q, k, v)
    fence()
    sampler.mark_begin()
    t_begin = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for _ in range(args.steps):
        _, sparse = step(q, k, v, record=True)
    t_end.record()
    fence()
    clocks = sampler.stop() if rank == 0 else None
    device_ms = t_begin.elapsed_time(t_end) / args.steps
    attn_ms = statistics.mean(a.elapsed_time(b) for a, b in attn_events)
    prep_ms = statistics.mean(a.elapsed_time(b) for a, b in prep_events)

    geo = sparse.route.geometry
    local_ops = attention_ops(spec, sparse.route.indices, geo, h1 - h0)
    totals = torch.tensor([float(local_ops), device_ms, attn_ms, prep_ms], dtype=torch.float64, device=device)
    if world > 1:
        summed = totals.clone(); dist.all_reduce(summed, op=dist.ReduceOp.SUM)
        maxed = totals.clone(); dist.all_reduce(maxed, op=dist.ReduceOp.MAX)
        total_ops, device_ms, attn_ms, prep_ms = float(summed[0]), float(maxed[1]), float(maxed[2]), float(maxed[3])
    else:
        total_ops = float(local_ops)

    # ---- end to end with host buffers ----
    e2e = None
    if not args.skip_e2e:
        # N > 1: the gathered layer output reaches the host once, from rank 0; the other ranks
        # read back the heads they computed
        full_back = world > 1 and rank == 0
        out_host = torch.empty((1, spec.heads if full_back else h1 - h0, spec.sequence, HEAD_DIM),
                               dtype=torch.bfloat16).pin_memory()
        def e2e_step():
            if world == 1:
                # the backend's host entry: H2D of head chunk c+1, kernels of chunk c and D2H of
                # chunk c-1 overlap on three streams
                backend.forward_host(q_host, k_host, v_host, out_host, layer_index=0, transformer_options=options)
                return
            qd, kd, vd = (t.to(device, non_blocking=True) for t in (q_host, k_host, v_host))
            out, _ = step(qd, kd, vd)
            out_host.copy_(out if full_back else out[:, h0:h1], non_blocking=True)
        for _ in range(max(1, min(args.warmup, 2))):
            e2e_step()
        fence()
        b0 = torch.cuda.Event(enable_timing=True); b1 = torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(args.steps):
            e2e_step()
        b1.record()
        fence()
        e2e_ms = torch.tensor([b0.elapsed_time(b1) / args.steps], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
        moved = torch.tensor([3.0 * q_host.numel() * q_host.element_size(),
                              float(out_host.numel() * out_host.element_size())], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(moved, op=dist.ReduceOp.SUM)
        e2e = {"value": total_ops / (float(e2e_ms[0]) * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": float(e2e_ms[0]),
               "api": "B200SparseBackend.forward_host (pinned host Q/K/V in, host output back, head chunks pipelined)"
                      if world == 1 else "pinned host Q/K/V of the local heads -> prepare + attention + exchange -> host (rank 0: whole output, others: their heads)",
               "h2d_bytes_per_step": int(moved[0]), "d2h_bytes_per_step": int(moved[1])}

    if rank == 0:
        peaks, peak_source = measured_peaks()
        int8_peak = 2.0 * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
        attn_tops = (total_ops / world) / (attn_ms * 1e-3) / 1e12  # per GPU, per launch
        carrier_bytes = (h1 - h0) * spec.sequence * HEAD_DIM * (3 * 2 + 3 * 1) + (h1 - h0) * spec.sequence * HEAD_DIM * 2 * 2
        line = {
            "metric": METRIC, "value": total_ops / (device_ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": device_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 QK^T / fp8-e4m3 PV, fp32 softmax",
            "data": "synthetic",
            "config": {
                "workload": workload_name(spec, args.budget),
                "heads_per_gpu": h1 - h0, "parallelism": "head-sharded x%d" % world, "exchange": exchange,
                "l2_policy": "inputs (Q,K,V bf16 = %.0f MB per GPU) exceed the 126 MB L2; no flush"
                             % ((h1 - h0) * spec.sequence * HEAD_DIM * 2 * 3 / 1e6),
                "p_terms": 1 if args.single_term_p else 2,
                "algorithmic_ops": total_ops, "route_len": sparse.route.route_len,
            },
            "stages_ms": {"prepare (stats+quant+route)": prep_ms, "attention": attn_ms},
            "prepare_hbm": {"bytes": carrier_bytes, "gbs": carrier_bytes / (prep_ms * 1e-3) / 1e9,
                            "frac_of_measured_copy": carrier_bytes / (prep_ms * 1e-3) / 1e9 / float(peaks["hbm_gbs"])},
            "roofline": {
                "bound": "tensor", "kernel": "sparse_attn_tc_kernel", "achieved": attn_tops,
                "peak": int8_peak, "unit": "TOP/s", "frac": attn_tops / int8_peak,
                "peak_source": "2 x bf16_tflops_sustained of MEASURED_PEAKS.json (%s); INT8/FP8 tensor rate is twice BF16"
                               % peak_source,
                "frac_of_nominal_4500": attn_tops / NOMINAL_INT8_TOPS, "traffic": None,
            },
            "clocks": clocks,
            "gpu_launches": args.steps * 7,
        }
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.skip_cpu_baseline:
            tops, sec, desc, threads, kind = cpu_reference_sample(spec, args.budget, heads=8)
            line["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": threads, "kind": kind,
                                    "sample": desc, "seconds": sec}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
