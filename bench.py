"""Benchmark of the B200 execution target on the reference's headline configurations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A "step" is one pass of a compiled program over one batch of synthetic input.  The default
workload is the fused multi-reduction row program (softmax then layer-norm over
f32[row=32768, col=4096], the HBM-bound configuration the headline GB/s figure is quoted on);
`--workload mismatch|matmul|attention|mlp` selects the other benchmark programs.

Prints ONE JSON line (rank 0).  `value` is whole-job throughput with inputs resident in HBM,
timed with CUDA events on the launching stream, max over ranks; `e2e` is the same metric through
the drop-in host-buffer call (`Session.invoke`: pinned host -> device copies, kernels and the
device -> host read inside the timed region); `roofline` gives achieved algorithmic GB/s or
TFLOP/s against the measured peak; `cpu_baseline` is the CPU restatement of the reference's
`runCpu` arithmetic timed on this host (rank 0, N=1, bounded sample).

With N > 1 (launched by torchrun, one rank per GPU) the program is sharded along its batch-like
named axis with no exchange: every rank runs the full per-GPU workload on its own shard of an
N-times larger global problem (weak scaling).  `--impl reference` times the CPU restatement on
all host threads instead (rank 0 only).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append((time.perf_counter(), parts))

    def count_since(self, t0):
        return sum(1 for t, _ in self.samples if t >= t0)

    def stop(self, t0, t1, how):
        """Summarises the samples that arrived between t0 and t1 (perf_counter times under load)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "sampled": "nvidia-smi unavailable"}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, reasons, sm_max = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, s in self.samples:
            if t < t0 or t > t1:
                continue
            try:
                mhz.append(float(s[0]))
                sm_max = float(s[1])
            except ValueError:
                continue
            for name, flag in zip(names, s[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": sm_max, "reasons": sorted(reasons),
                "samples": len(mhz), "sampled": how}


WORKLOADS = {
    # name: (metric, unit, bound, quantity-per-step key, scale)
    "softmax_layernorm": ("fused_reduce_hbm_gbs", "GB/s", "hbm"),
    "mismatch": ("fused_reduce_gpairs_per_s", "Gpair/s", "hbm"),
    # not one of the five benchmark configurations: the mismatch program's valueAndGrad + vmap
    "refine": ("value_and_slope_gpairs_per_s", "Gpair/s", "hbm"),
    "matmul": ("matmul_tflops", "TFLOP/s", "tensor"),
    "attention": ("attention_tflops", "TFLOP/s", "tensor"),
    "mlp": ("mlp_tflops", "TFLOP/s", "tensor"),
}


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) taken from the ncu captures
# summarised under profiles/, scaled to the default size where the traffic grows with the units
# processed: bytes per row (softmax_layernorm: 26 988 B per 4096-column row; the writes of the last
# ~100 MB are still in L2 when the kernel ends, so this is below the 32 768 B the row moves) and
# bytes per launch (mismatch: the two point vectors, the guesses and the result).  The tensor-core
# kernels re-read operands through L2 in a size-dependent way, so no scaled figure is given.
NCU_TRAFFIC = {
    "softmax_layernorm": lambda cfg: 26988.0 * dict(cfg.specs[0].dims)["row"],
    "mismatch": lambda cfg: 4.0 * (2 * dict(cfg.specs[1].dims)["point"] + 2 * dict(cfg.specs[0].dims)["guess"]) * 0.957,
}


# inputs that stay the same from step to step in the workload's usual use (parameter indices)
RESIDENT_INPUTS = {"matmul": [1], "mlp": [1, 2, 3, 4, 5]}


def _size_args(name, cfg):
    """(label, extent) pairs that rebuild a config of the same size with another seed"""
    dims = {n: e for s in cfg.specs for n, e in s.dims}
    order = {"mismatch": ["guess", "point"], "refine": ["guess", "point"], "softmax_layernorm": ["row", "col"], "matmul": ["m", "n", "k"],
             "attention": ["batch", "head", "seq", "dim"], "mlp": ["token", "d", "h"]}[name]
    return [(n, dims[n]) for n in order]


def units_per_step(name, work):
    if name == "softmax_layernorm":
        return work["bytes"] / 1e9
    if name in ("mismatch", "refine"):
        return work["pairs"] / 1e9
    return work["flops"] / 1e12


def make_config(name, args, seed_offset=0):
    from accy_b200 import configs
    if seed_offset:
        base = {"mismatch": 0, "refine": 0, "softmax_layernorm": 1, "matmul": 2, "attention": 3, "mlp": 4}[name]
        sizes = make_config(name, args)
        return configs.BASELINE[name](*[e for _, e in _size_args(name, sizes)], seed=base + 1000 * seed_offset)
    if args.small:
        # profiling sizes: the same kernels, inputs still larger than L2 where the kernel is HBM-bound
        small = {"softmax_layernorm": lambda: configs.softmax_layernorm(8192, 4096),
                 "mismatch": lambda: configs.mismatch(1024, 65536),
                 "refine": lambda: configs.refine(1024, 65536),
                 "matmul": lambda: configs.matmul(4096, 4096, 4096),
                 "attention": lambda: configs.attention(1, 16, 4096, 128),
                 "mlp": lambda: configs.mlp(4096, 4096, 4096)}
        return small[name]()
    return configs.BASELINE[name]()


# ---------------------------------------------------------------------------------------------
# CPU legs (the only places that execute oracle/)
# ---------------------------------------------------------------------------------------------
def cpu_sample(name, cfg, inputs, threads, budget_s=15.0):
    """Times the CPU restatement on a bounded sample of the workload; returns (units/s, cores, text)."""
    import ctypes
    from oracle import oracle
    lib = oracle.lib()
    lib.oracle_set_threads(threads)
    c_size = ctypes.c_size_t

    def ptr(a):
        return a.ctypes.data_as(ctypes.c_void_p)

    if name == "mismatch":
        f, t, s = inputs
        total = f.shape[0]
        out = np.zeros(total, np.float32)

        def run(n):
            lib.oracle_mismatch_f32(ptr(f), ptr(t), ptr(s), ptr(out), c_size(total), c_size(t.shape[0]), c_size(0), c_size(n))
        unit_of = lambda n: n * t.shape[0] / 1e9  # noqa: E731
        label = "guesses"
    elif name == "refine":
        f, t, s = inputs
        total = f.shape[0]
        out, slope = np.zeros(total, np.float32), np.zeros(total, np.float32)

        def run(n):
            lib.oracle_mismatch_slope_f32(ptr(f), ptr(t), ptr(s), ptr(out), ptr(slope), c_size(total), c_size(t.shape[0]),
                                          c_size(0), c_size(n))
        unit_of = lambda n: n * t.shape[0] / 1e9  # noqa: E731
        label = "guesses"
    elif name == "softmax_layernorm":
        x = inputs[0]
        total, cols = x.shape
        out = np.zeros_like(x)

        def run(n):
            lib.oracle_softmax_layernorm_f32(ptr(x), ptr(out), c_size(total), c_size(cols), ctypes.c_float(1e-5), c_size(0), c_size(n))
        unit_of = lambda n: 8.0 * n * cols / 1e9  # noqa: E731
        label = "rows"
    elif name == "matmul":
        a, b = inputs
        total, k = a.shape
        n_cols = b.shape[1]
        out = np.zeros((min(total, 64), n_cols), np.float32)

        def run(n):
            lib.oracle_matmul_bf16(ptr(a), ptr(b), ptr(out), c_size(total), c_size(k), c_size(n_cols), c_size(0), c_size(n))
        unit_of = lambda n: 2.0 * n * k * n_cols / 1e12  # noqa: E731
        total = min(total, 64)
        label = "rows of C"
    elif name == "attention":
        q, k, v = inputs
        b_, h_, s_, d_ = q.shape
        total = 1
        out = np.zeros((1, s_, d_), np.float32)
        scratch = np.zeros(max(1, threads) * s_, np.float32)
        causal_pairs = s_ * (s_ + 1) / 2.0

        def run(n):
            lib.oracle_attention_bf16(ptr(q), ptr(k), ptr(v), ptr(out), c_size(b_ * h_), c_size(s_), c_size(s_), c_size(d_),
                                      ctypes.c_float(float(1.0 / np.sqrt(d_))), ctypes.c_int(1), c_size(0), c_size(n), ptr(scratch))
        unit_of = lambda n: 4.0 * d_ * causal_pairs * n / 1e12  # noqa: E731
        label = "heads"
    else:
        x, w1, b1, w2, b2, g = inputs
        tokens, d = x.shape
        h = w1.shape[1]
        total = min(tokens, 64)
        out = np.zeros((total, d), np.float32)
        hidden = np.zeros((total, h), np.float32)

        def run(n):
            lib.oracle_mlp_bf16(ptr(x), ptr(w1), ptr(b1), ptr(w2), ptr(b2), ptr(g), ptr(out), ptr(hidden), c_size(tokens),
                                c_size(d), c_size(h), ctypes.c_float(1e-6), c_size(0), c_size(n))
        unit_of = lambda n: 4.0 * n * d * h / 1e12  # noqa: E731
        label = "tokens"
    # grow the sample until it takes a measurable time, bounded by the budget
    n = max(1, min(total, threads))
    t0 = time.perf_counter()
    run(n)
    dt = time.perf_counter() - t0
    while dt < min(budget_s, 10.0) / 4 and n < total:
        n = min(total, max(n + 1, int(n * min(8.0, (budget_s / 2) / max(dt, 1e-4)))))
        t0 = time.perf_counter()
        run(n)
        dt = time.perf_counter() - t0
    return unit_of(n) / dt, threads, "%d of the workload's %s, %.1f s" % (n, label, dt), unit_of(n), dt


def reference_arm(args, name, cfg):
    """The reference's CPU implementation of the path (its restatement) on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    # every host core this process may use (torchrun sets OMP_NUM_THREADS=1, so the OpenMP default is not it)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.lib()
    inputs = cfg.make_inputs()
    metric, unit, _ = WORKLOADS[name]
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_sample(name, cfg, inputs, threads, budget_s=2.0)
    total_units, total_time, sample = 0.0, 0.0, ""
    for _ in range(args.steps):
        _, _, sample, units, dt = cpu_sample(name, cfg, inputs, threads, budget_s=8.0)
        total_units += units
        total_time += dt
    value = total_units / total_time
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_time / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic",
            "config": {"workload": name, "note": "CPU restatement of runCpu arithmetic, bounded sample per step"},
            "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="softmax_layernorm", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--small", action="store_true", help="reduced sizes (profiling captures only; not a bench value)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--strong", action="store_true",
                    help="with --gpus N > 1: cut the one-GPU problem into N pieces (strong scaling) instead of running "
                         "an N times larger problem (weak scaling, the default)")
    ap.add_argument("--tpr", type=int, default=0, help="schedule override: threads per row (experiments)")
    ap.add_argument("--vpt", type=int, default=0, help="schedule override: vectors per thread (experiments)")
    ap.add_argument("--attn-poly", type=int, default=0, help="attention_poly override (experiments)")
    ap.add_argument("--min-blocks", type=int, default=0, help="schedule override: resident CTAs per SM (experiments)")
    args = ap.parse_args()
    name = args.workload
    cfg = make_config(name, args)
    if args.impl == "reference":
        reference_arm(args, name, cfg)
        return

    import torch
    import torch.distributed as dist
    from accy_b200 import tensor

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 target has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    metric, unit, bound = WORKLOADS[name]
    peaks = load_peaks()

    # every rank holds one full per-GPU workload: its shard of a world-times larger global problem
    # along cfg.shard_axis (different seed per rank = different rows of the global input)
    if world > 1:
        # The global problem is `world` times larger along the shard axis; the shard planner cuts the
        # recorded global program into one piece per rank (no exchange), and every rank generates
        # its own block of the global input (a different seed per rank).
        from accy_b200 import configs, shard
        sizes = dict(_size_args(name, cfg))
        if args.strong:
            # strong scaling: the one-GPU problem itself is cut into `world` pieces
            if sizes[cfg.shard_axis] % world:
                raise SystemExit("--strong: axis %s of extent %d does not divide over %d ranks" % (cfg.shard_axis, sizes[cfg.shard_axis], world))
            global_cfg = cfg
        else:
            sizes[cfg.shard_axis] *= world
            global_cfg = configs.BASELINE[name](*[sizes[n] for n, _ in _size_args(name, cfg)])
        plan = shard.ShardPlan(global_cfg.program(), cfg.shard_axis, world)
        assert not plan.partial_sum
        if args.strong:
            sizes[cfg.shard_axis] //= world
            base = {"mismatch": 0, "refine": 0, "softmax_layernorm": 1, "matmul": 2, "attention": 3, "mlp": 4}[name]
            cfg = configs.BASELINE[name](*[sizes[n] for n, _ in _size_args(name, cfg)], seed=base + 1000 * rank)
        else:
            cfg = make_config(name, args, seed_offset=rank)
        program = plan.piece
    else:
        program = cfg.program()
    inputs = cfg.make_inputs()
    session = tensor.Session(device=local, threads_per_row=args.tpr, vectors_per_thread=args.vpt,
                             row_min_blocks=args.min_blocks, attention_poly=args.attn_poly)
    compiled = session.compile(program)
    work = compiled.work()
    d_in = [torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda() for a in inputs]
    out_desc = compiled.output_descriptors()
    d_out = [torch.empty(d.byte_size, dtype=torch.uint8, device="cuda") for d in out_desc]
    in_ptrs = [t.data_ptr() for t in d_in]
    out_ptrs = [t.data_ptr() for t in d_out]
    stream = torch.cuda.Stream()   # an explicit stream: its handle goes through the C ABI
    torch.cuda.set_stream(stream)
    io_bytes = sum(t.numel() * t.element_size() for t in d_in) + sum(t.numel() for t in d_out)
    flush = None
    if io_bytes < 256 * 1024 * 1024:
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")

    def step():
        session.invoke_device(compiled, in_ptrs, out_ptrs, stream.cuda_stream)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()   # nvidia-smi needs a few hundred ms before its first sample
    load_t0 = time.perf_counter()
    for _ in range(max(args.warmup, 3)):
        if flush is not None:
            flush.zero_()
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    torch.cuda.synchronize()
    load_t0 = time.perf_counter()   # clock samples count from here: the GPU is under load until load_t1
    wall0 = time.perf_counter()
    for i in range(args.steps):
        if flush is not None:
            flush.zero_()
        starts[i].record(stream)
        step()
        ends[i].record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    if world > 1:
        dist.barrier()
    clocks = None
    if rank == 0:
        # The timed region is often shorter than one nvidia-smi period.  When it holds no sample,
        # the same step keeps running right after it until a few samples exist, and those are
        # reported (the GPU never idles in between, so they show the clocks of the timed region).
        load_t1 = time.perf_counter()
        how = "during warm-up and timed steps"
        if sampler.proc and sampler.count_since(load_t0) < 3:
            how = "same step repeated right after the timed steps"
            deadline = time.perf_counter() + 2.5
            while sampler.count_since(load_t0) < 4 and time.perf_counter() < deadline:
                for _ in range(8):
                    step()
                torch.cuda.synchronize()
            load_t1 = time.perf_counter()
        clocks = sampler.stop(load_t0, load_t1, how)
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    total_ms = float(sum(step_ms))
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    units = units_per_step(name, cfg.work)
    value = world * units * args.steps / (total_ms / 1e3)

    # end to end through the drop-in host-buffer call, pinned host memory, copies inside the timing
    e2e = None
    if not args.no_e2e:
        h_in = [torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).pin_memory() for a in inputs]
        h_out = [torch.empty(d.byte_size, dtype=torch.uint8).pin_memory() for d in out_desc]
        e2e_steps = max(2, min(args.steps, 5))
        session.invoke(compiled, h_in, h_out)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            session.invoke(compiled, h_in, h_out)
        e2e_s = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        e2e = {"value": world * units * e2e_steps / e2e_s, "unit": unit,
               "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in h_in)),
               "d2h_bytes_per_step": int(sum(t.numel() for t in h_out)), "ms_per_step": 1e3 * e2e_s / e2e_steps}
        # the same call with the operands that do not change from step to step (weights, the
        # right-hand matrix) kept on the device by set_resident: only the activations travel
        weights = RESIDENT_INPUTS.get(name, [])
        if weights:
            for i in weights:
                session.set_resident(compiled, i, h_in[i])
            step_in = [None if i in weights else t for i, t in enumerate(h_in)]
            session.invoke(compiled, step_in, h_out)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                session.invoke(compiled, step_in, h_out)
            res_s = time.perf_counter() - t0
            if world > 1:
                t = torch.tensor([res_s], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                res_s = float(t.item())
            e2e["resident_weights"] = {"value": world * units * e2e_steps / res_s, "unit": unit, "inputs_kept_on_device": weights,
                                       "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for i, t in enumerate(h_in) if i not in weights)),
                                       "ms_per_step": 1e3 * res_s / e2e_steps}
            for i in weights:
                session.set_resident(compiled, i, None)

    if rank == 0:
        avg_ms = float(np.mean(step_ms))
        if bound == "hbm":
            achieved = cfg.work["bytes"] / 1e9 / (avg_ms / 1e3)
            peak, peak_unit = peaks["hbm_gbs"], "GB/s"
        else:
            achieved = cfg.work["flops"] / 1e12 / (avg_ms / 1e3)
            peak, peak_unit = peaks["bf16_tflops"], "TFLOP/s"
        roofline = {"bound": bound, "achieved": achieved, "peak": peak, "unit": peak_unit, "frac": achieved / peak,
                    "traffic": NCU_TRAFFIC[name](cfg) if name in NCU_TRAFFIC else None,
                    "peak_source": peaks["source"], "peak_sustained": peaks["bf16_tflops_sustained"] if bound == "tensor" else None,
                    "kernel_ms": avg_ms,
                    "launches_per_step": work["launches"]}
        if name == "refine":
            roofline["note"] = "not HBM-bound by construction: FP32-bound (a sine, a cosine and nine more operations per pair)"
            roofline["pairs_per_s"] = cfg.work["pairs"] / (avg_ms / 1e3)
        if name == "mismatch":
            # 0.59 MB of traffic for 5.4e8 (guess, point) pairs: the HBM fraction is reported because the
            # contract asks for it, the kernel is bound by FP32 arithmetic (ncu: FMA pipe 68 % busy,
            # 12.85 instructions per pair; profiles/row_kernel_mismatch.md)
            roofline["note"] = "not HBM-bound by construction: FP32-bound, FMA pipe 68 % busy under ncu"
            roofline["pairs_per_s"] = cfg.work["pairs"] / (avg_ms / 1e3)
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            v, cores, sample, _, _ = cpu_sample(name, cfg, inputs, 1, budget_s=15.0)
            cpu = {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample}
        line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
                "scaling": "strong" if (args.strong and world > 1) else "weak", "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic",
                "config": {"workload": name, "specs": [repr(t) for t in program.input_types],
                           "shard_axis": cfg.shard_axis, "parallelism": "shard%d" % world,
                           "l2": "flushed between steps" if flush is not None else "inputs larger than L2",
                           "small": bool(args.small), "plan": compiled.plan_summary().strip().split("\n")},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": work["launches"] * args.steps,
                "clocks": clocks, "wall_ms_per_step": 1e3 * wall / args.steps,
                "ms_min": float(min(step_ms)), "ms_median": float(np.median(step_ms))}
        print(json.dumps(line))
    session.deinit()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
