"""Benchmark of the B200 execution target on the reference's headline configurations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference] [--weak]

A "step" is one pass of a compiled program over one batch of synthetic input.  The headline
workload is the fused multi-reduction row program (softmax then layer-norm over
f32[row=32768, col=4096], the HBM-bound configuration the GB/s figure is quoted on).  Without
`--workload`, a one-GPU run also times the other four benchmark programs at their full sizes
(mismatch, matmul, attention, mlp) and reports them under `workloads`; `--workload NAME` times
that program alone as the headline.

Prints ONE JSON line (rank 0).  `value` is whole-job throughput with inputs resident in HBM,
timed with CUDA events on the launching stream, max over ranks; `e2e` is the same metric through
the drop-in host-buffer call (`Session.invoke`: pinned host -> device copies, kernels and the
device -> host read inside the timed region); `roofline` gives achieved algorithmic GB/s, TFLOP/s
or Gpair/s against the measured peak; `cpu_baseline` is the CPU restatement of the reference's
`runCpu` arithmetic timed on this host (rank 0, N=1, bounded sample).  Every timed program is also
spot-checked against the CPU oracle on sampled rows, outside the timed region (`parity`).

With N > 1 (launched by torchrun, one rank per GPU) the one-GPU problem is cut into N pieces along
its batch-like named axis with no exchange between the pieces (strong scaling; `value` is the
global problem's throughput).  `--weak` instead gives every rank a full one-GPU problem (an N
times larger global problem).  `--impl reference` times the CPU restatement on all host threads
(rank 0 only) and loads neither the package nor its native library.
"""
import argparse
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402


def load_synthetic():
    """accy_b200/synthetic.py by file path: plain numpy, so the CPU-only reference arm gets the
    benchmark's inputs and specs without importing the package (which maps the native library)."""
    spec = importlib.util.spec_from_file_location("accy_b200_synthetic", os.path.join(ROOT, "accy_b200", "synthetic.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


synthetic = load_synthetic()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi for the whole run; windows of it are
    summarised per timed region."""

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

    def window(self, t0, t1, how):
        """Summarises the samples that arrived between t0 and t1 (perf_counter times under load)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "sampled": "nvidia-smi unavailable"}
        mhz, reasons, sm_max = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, s in list(self.samples):
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

    def stop(self):
        if not self.proc:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()


WORKLOADS = {
    # name: (metric, unit, bound)
    "softmax_layernorm": ("fused_reduce_hbm_gbs", "GB/s", "hbm"),
    "mismatch": ("fused_reduce_gpairs_per_s", "Gpair/s", "fp32"),
    # not one of the five benchmark configurations: the mismatch program's valueAndGrad + vmap
    "refine": ("value_and_slope_gpairs_per_s", "Gpair/s", "fp32"),
    "matmul": ("matmul_tflops", "TFLOP/s", "tensor"),
    "attention": ("attention_tflops", "TFLOP/s", "tensor"),
    "mlp": ("mlp_tflops", "TFLOP/s", "tensor"),
}
SECONDARY = ["mismatch", "matmul", "attention", "mlp"]   # reported under `workloads` beside the headline

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from ncu captures of these
# kernels at the reduced profiling sizes, scaled to the timed size where the traffic grows with the
# units processed: bytes per row for softmax_layernorm (26 988 B per 4096-column row; the writes of
# the last ~100 MB are still in L2 when the kernel ends, so this is below the 32 768 B the row
# moves) and bytes per launch for mismatch (the two point vectors, the guesses and the result).
# The tensor-core kernels re-read operands through L2 in a size-dependent way: no scaled figure.
NCU_TRAFFIC = {
    "softmax_layernorm": lambda sizes: 26988.0 * dict(sizes)["row"] * (dict(sizes)["col"] / 4096.0),
    "mismatch": lambda sizes: 4.0 * (2 * dict(sizes)["point"] + 2 * dict(sizes)["guess"]) * 0.957,
}

# FP32 operations the row kernel executes per (guess, point) pair, counted from its source.
# mismatch: the packed sine is 19 (eight fused multiply-adds counted twice and three single
# operations) next to the program's multiply, subtract, multiply and add; the recorded program
# counts 5.  refine: the joint sine / cosine is 25 (eleven fused multiply-adds and three single
# operations) next to eight recorded operations.
EXECUTED_FLOP_PER_PAIR = {"mismatch": 23.0, "refine": 33.0}

# inputs that stay the same from step to step in the workload's usual use (parameter indices)
RESIDENT_INPUTS = {"matmul": [1], "mlp": [1, 2, 3, 4, 5]}

SMALL_SIZES = {
    # profiling sizes: the same kernels and schedules as the full sizes, inputs still larger than L2
    # where the kernel is HBM-bound, and whole rounds of work where a persistent kernel hands out
    # tiles (matmul: 37 x 8 tiles of 256 x 256 = 4 per CTA pair; attention: 37 heads x 16 query
    # pairs = 4 work items per CTA)
    "softmax_layernorm": (8192, 4096), "mismatch": (4096, 65536), "refine": (4096, 65536),
    "matmul": (9472, 2048, 4096), "attention": (1, 37, 4096, 128), "mlp": (4096, 4096, 4096),
}
SHARD_AXIS = {"mismatch": "guess", "refine": "guess", "softmax_layernorm": "row", "matmul": "m", "attention": "batch", "mlp": "token"}


def sizes_for(name, small):
    return synthetic.sizes_of(name, *SMALL_SIZES[name]) if small else synthetic.sizes_of(name)


def units_per_step(name, work):
    if name == "softmax_layernorm":
        return work["bytes"] / 1e9
    if name in ("mismatch", "refine"):
        return work["pairs"] / 1e9
    return work["flops"] / 1e12


def config_record(name, sizes, world, scaling, small, l2=None):
    """The part of `config` both arms print the same way (the global problem)."""
    record = {"workload": name, "specs": [synthetic.spec_text(s) for s in synthetic.specs(name, sizes)],
              "shard_axis": SHARD_AXIS[name], "parallelism": "shard%d" % world, "scaling": scaling, "small": bool(small),
              "distributions": "N(0, s): s is the standard deviation; numpy PCG64 streams"}
    if l2 is not None:
        record["l2"] = l2
    return record


# ---------------------------------------------------------------------------------------------
# CPU legs (the only places that execute oracle/)
# ---------------------------------------------------------------------------------------------
def cpu_sample(name, inputs, threads, budget_s=15.0):
    """Times the CPU restatement on a bounded sample of the workload; returns (units/s, cores, text, units, s)."""
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
        total = min(total, 256)
        out = np.zeros((total, n_cols), np.float32)

        def run(n):
            lib.oracle_matmul_bf16(ptr(a), ptr(b), ptr(out), c_size(a.shape[0]), c_size(k), c_size(n_cols), c_size(0), c_size(n))
        unit_of = lambda n: 2.0 * n * k * n_cols / 1e12  # noqa: E731
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


def reference_arm(args, name):
    """The reference's CPU implementation of the path (its restatement) on all host threads.  The
    reference's own `runCpu` launch is single-threaded (deps/lib/compiler/gpu/src/cpu.zig:425-449):
    the one-core figure is printed beside the all-threads one."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    # every host core this process may use (torchrun sets OMP_NUM_THREADS=1, so the OpenMP default is not it)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.lib()
    sizes = sizes_for(name, args.small)
    inputs = synthetic.inputs(name, sizes)
    metric, unit, _ = WORKLOADS[name]
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_sample(name, inputs, threads, budget_s=2.0)
    total_units, total_time, sample = 0.0, 0.0, ""
    for _ in range(args.steps):
        _, _, sample, units, dt = cpu_sample(name, inputs, threads, budget_s=8.0)
        total_units += units
        total_time += dt
    value = total_units / total_time
    one, _, one_sample, _, _ = cpu_sample(name, inputs, 1, budget_s=8.0)
    world = max(1, args.gpus)
    config = config_record(name, sizes, world, "strong" if (world > 1 and not args.weak) else "weak", args.small)
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_time / args.steps,
            "higher_is_better": True, "scaling": config["scaling"], "vs_baseline": None,
            "dtype": synthetic.DTYPES[name], "data": "synthetic", "config": config,
            "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample,
                             "single_core": {"value": one, "unit": unit, "cores": 1, "sample": one_sample,
                                             "note": "the reference's runCpu launch is single-threaded"}},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "note": "CPU restatement of runCpu arithmetic, bounded sample of this workload per step"}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# oracle spot checks of a timed program's output (outside every timed region)
# ---------------------------------------------------------------------------------------------
def spot_check(name, inputs, outputs):
    """Compares sampled rows of the GPU result with the CPU oracle.  Returns the `parity` record."""
    import ctypes
    from oracle import oracle

    def ptr(a):
        return a.ctypes.data_as(ctypes.c_void_p)

    def widen(bits):
        return synthetic.bf16_bits_to_f32(bits)

    def bf16_err(got, want):
        want = np.asarray(want, np.float64).reshape(-1)
        got = np.asarray(got, np.float64).reshape(-1)
        rms = max(float(np.sqrt(np.mean(want * want))), 1e-30)
        return float(np.max(np.abs(got - want) / (np.abs(want) + rms)))

    def f32_err(got, want, floor_frac):
        want = np.asarray(want, np.float64).reshape(-1)
        got = np.asarray(got, np.float64).reshape(-1)
        floor = max(float(np.abs(want).max()) * floor_frac, 1e-30)
        return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))

    rng = np.random.default_rng(2024)
    c_size = ctypes.c_size_t
    if name in ("mismatch", "refine"):
        f, t, s = inputs
        picks = np.unique(np.concatenate([[0, f.shape[0] - 1], rng.integers(0, f.shape[0], 14)]))
        sub = np.ascontiguousarray(f[picks])
        ref = np.zeros(len(picks), np.float32)
        exact = np.zeros(len(picks), np.float64)
        oracle.lib().oracle_mismatch_f32(ptr(sub), ptr(t), ptr(s), ptr(ref), c_size(len(picks)), c_size(t.shape[0]), c_size(0), c_size(len(picks)))
        oracle.lib().oracle_mismatch_f64(ptr(sub), ptr(t), ptr(s), ptr(exact), c_size(len(picks)), c_size(t.shape[0]))
        got = outputs[0].view(np.float32)[picks]
        err, ref_err = f32_err(got, exact, 1e-6), f32_err(ref, exact, 1e-6)
        return {"checked": "%d guesses against the f64 and reference-order f32 oracle" % len(picks), "max_err": err,
                "oracle_err": ref_err, "tol": 1e-5, "ok": bool(err < 1e-5 + ref_err)}
    if name == "softmax_layernorm":
        x = inputs[0]
        rows, cols = x.shape
        picks = np.unique(np.concatenate([[0, rows - 1], rng.integers(0, rows, 14)]))
        sub = np.ascontiguousarray(x[picks])
        ref = np.zeros_like(sub)
        oracle.lib().oracle_softmax_layernorm_f32(ptr(sub), ptr(ref), c_size(len(picks)), c_size(cols), ctypes.c_float(1e-5),
                                                  c_size(0), c_size(len(picks)))
        x64 = sub.astype(np.float64)
        e = np.exp(x64 - x64.max(axis=1, keepdims=True))
        y = e / e.sum(axis=1, keepdims=True)
        c = y - y.mean(axis=1, keepdims=True)
        exact = c / np.sqrt((c * c).mean(axis=1, keepdims=True) + 1e-5)
        got = outputs[0].view(np.float32).reshape(rows, cols)[picks]
        err, ref_err = f32_err(got, exact, 1e-3), f32_err(ref, exact, 1e-3)
        return {"checked": "%d rows against the f64 and reference-order f32 oracle" % len(picks), "max_err": err,
                "oracle_err": ref_err, "tol": 1e-5, "ok": bool(err < 1e-5 + ref_err)}
    if name == "matmul":
        a, b = inputs
        m, n = a.shape[0], b.shape[1]
        picks = np.unique(np.concatenate([[0, m - 1], rng.integers(0, m, 14)]))
        want = widen(synthetic.f32_to_bf16_bits(oracle.matmul_rows(a, b, picks)))
        got = widen(outputs[0].view(np.uint16).reshape(m, n)[picks])
        err = bf16_err(got, want)
        return {"checked": "%d rows of C, all columns, against the k-serial f32 oracle" % len(picks), "max_err": err,
                "tol": 2e-2, "ok": bool(err < 2e-2)}
    if name == "attention":
        q, k, v = inputs
        seq, dim = q.shape[-2:]
        heads_total = int(np.prod(q.shape[:-2]))
        heads = np.array([0, heads_total - 1] * 4, np.uint64)
        queries = np.concatenate([[0, seq - 1], rng.integers(0, seq, 6)]).astype(np.uint64)
        want = oracle.attention_rows(q.reshape(heads_total, seq, dim), k.reshape(heads_total, seq, dim),
                                     v.reshape(heads_total, seq, dim), heads, queries, 1.0 / np.sqrt(float(dim)), causal=True)
        got = widen(outputs[0].view(np.uint16).reshape(heads_total, seq, dim)[heads.astype(np.int64), queries.astype(np.int64)])
        err = bf16_err(got, want)
        return {"checked": "8 query rows of the first and the last head against the f32 SDPA oracle", "max_err": err,
                "tol": 2e-2, "ok": bool(err < 2e-2)}
    x = inputs[0]
    picks = np.unique(np.concatenate([[0, x.shape[0] - 1], rng.integers(0, x.shape[0], 2)]))
    want = oracle.mlp_rows(*inputs, rows=picks)
    got = widen(outputs[0].view(np.uint16).reshape(x.shape[0], -1)[picks])
    err = bf16_err(got, want)
    return {"checked": "%d tokens against the f32 oracle" % len(picks), "max_err": err, "tol": 2e-2, "ok": bool(err < 2e-2)}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class Runner:
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the B200 target has no CPU fallback")
        torch.cuda.set_device(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.stream = torch.cuda.Stream()   # an explicit stream: its handle goes through the C ABI
        torch.cuda.set_stream(self.stream)
        self.peaks = load_peaks()
        self.sampler = ClockSampler(self.local)
        if self.rank == 0:
            self.sampler.start()   # nvidia-smi needs a few hundred ms before its first sample
        self.flush = None
        self.launches = 0
        self.fp32 = None

    def max_over_ranks(self, value):
        if self.world == 1:
            return value
        t = self.torch.tensor([value], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def fp32_ceilings(self):
        """The measured FP32 ceilings of this GPU (register-only micro-kernels of the library)."""
        if self.fp32 is None:
            import ctypes
            from accy_b200._native import lib
            pairs, flops = ctypes.c_double(), ctypes.c_double()
            error = ctypes.create_string_buffer(256)
            status = lib.accy_b200_probe_fp32_rates(ctypes.c_void_p(self.stream.cuda_stream), ctypes.byref(pairs),
                                                    ctypes.byref(flops), error, 256)
            if status != 0:
                raise SystemExit("fp32 probe failed: %s" % error.value.decode(errors="replace"))
            self.fp32 = {"sinf_plus_4_flop_gpairs": pairs.value / 1e9, "packed_fma_tflops": flops.value / 1e12}
        return self.fp32

    def run(self, name, scaling, steps, warmup, with_e2e, with_cpu):
        """Times one workload.  Returns (record for rank 0, None elsewhere)."""
        torch, dist, args, world, rank = self.torch, self.dist, self.args, self.world, self.rank
        from accy_b200 import configs, shard, tensor
        metric, unit, bound = WORKLOADS[name]
        sizes = sizes_for(name, args.small)          # the one-GPU problem
        extents = [e for _, e in sizes]
        axis = SHARD_AXIS[name]
        global_sizes = list(sizes)
        if world > 1 and scaling == "weak":
            global_sizes = [(n, e * world if n == axis else e) for n, e in sizes]
        if world > 1:
            at = [n for n, _ in sizes].index(axis)
            if global_sizes[at][1] % world:
                raise SystemExit("axis %s of extent %d does not divide over %d ranks" % (axis, global_sizes[at][1], world))
            # the shard planner cuts the recorded global program into one piece per rank (no exchange);
            # every rank generates its own block of the global input (its own seed)
            global_cfg = configs.BASELINE[name](*[e for _, e in global_sizes])
            plan = shard.ShardPlan(global_cfg.program(), axis, world)
            assert not plan.partial_sum
            piece = list(extents)
            piece[at] = global_sizes[at][1] // world
            cfg = configs.BASELINE[name](*piece, seed=synthetic.SEEDS[name] + 1000 * rank)
            program = plan.piece
        else:
            cfg = configs.BASELINE[name](*extents)
            program = cfg.program()
        inputs = cfg.make_inputs()
        session = tensor.Session(device=self.local)
        compiled = session.compile(program)
        work = compiled.work()
        d_in = [torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda() for a in inputs]
        out_desc = compiled.output_descriptors()
        d_out = [torch.empty(d.byte_size, dtype=torch.uint8, device="cuda") for d in out_desc]
        stream = self.stream
        io_bytes = sum(t.numel() * t.element_size() for t in d_in) + sum(t.numel() for t in d_out)
        # No step may find its data in L2 (126 MB).  A step that moves 256 MiB or more cannot; smaller
        # ones rotate through copies of their buffers that together hold 2.5 times L2; the smallest
        # (the inputs of mismatch: 0.6 MB, reused thousands of times inside one launch anyway) have a
        # 256 MiB buffer written between steps instead, which needs one pair of events per step.
        flush, n_sets = None, 1
        if io_bytes < 16 * 1024 * 1024:
            if self.flush is None:
                self.flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
            flush = self.flush
            l2_rule = "flushed between steps"
        elif io_bytes < 256 * 1024 * 1024:
            n_sets = int(np.ceil(2.5 * 126e6 / io_bytes))
            l2_rule = "%d buffer sets in rotation, larger than L2 together" % n_sets
        else:
            l2_rule = "inputs larger than L2"
        in_sets = [d_in] + [[t.clone() for t in d_in] for _ in range(n_sets - 1)]
        out_sets = [d_out] + [[torch.empty_like(t) for t in d_out] for _ in range(n_sets - 1)]
        in_ptrs = [[t.data_ptr() for t in ts] for ts in in_sets]
        out_ptrs = [[t.data_ptr() for t in ts] for ts in out_sets]

        def step(i=0):
            session.invoke_device(compiled, in_ptrs[i % n_sets], out_ptrs[i % n_sets], stream.cuda_stream)

        warmup = max(warmup, 3)
        for i in range(warmup):
            if flush is not None:
                flush.zero_()
            step(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        load_t0 = time.perf_counter()   # clock samples count from here: the GPU is under load until load_t1
        wall0 = time.perf_counter()
        if flush is not None:
            for i in range(steps):
                flush.zero_()
                starts[i].record(stream)
                step(i)
                ends[i].record(stream)
        else:
            # the timed region: the steps back to back between one pair of events
            first.record(stream)
            for i in range(steps):
                step(i)
            last.record(stream)
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall0
        if world > 1:
            dist.barrier()
        if flush is None:
            # once more with a pair of events around every step, for the spread (min, median) only
            for i in range(steps):
                starts[i].record(stream)
                step(i)
                ends[i].record(stream)
            torch.cuda.synchronize()
        self.launches += work["launches"] * steps
        clocks = None
        if rank == 0:
            # The timed region is often shorter than one nvidia-smi period.  When it holds no sample,
            # the same step keeps running right after it until a few samples exist, and those are
            # reported (the GPU never idles in between, so they show the clocks of the timed region).
            load_t1 = time.perf_counter()
            how = "during the timed steps"
            if self.sampler.proc and self.sampler.count_since(load_t0) < 3:
                how = "same step repeated right after the timed steps"
                deadline = time.perf_counter() + 2.5
                while self.sampler.count_since(load_t0) < 4 and time.perf_counter() < deadline:
                    for _ in range(8):
                        step()
                    torch.cuda.synchronize()
                load_t1 = time.perf_counter()
            clocks = self.sampler.window(load_t0, load_t1, how)
        step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        total_ms = self.max_over_ranks(float(sum(step_ms)) if flush is not None else first.elapsed_time(last))
        global_work = synthetic.work(name, global_sizes)
        units = units_per_step(name, global_work)       # of the whole job
        local_work = cfg.work
        value = units * steps / (total_ms / 1e3)

        # oracle spot check of this rank's result (rank 0 reports its own piece)
        parity = None
        if rank == 0 and not args.no_parity:
            torch.cuda.synchronize()
            parity = spot_check(name, inputs, [t.cpu().numpy() for t in d_out])

        # end to end through the drop-in host-buffer call, pinned host memory, copies inside the timing
        e2e = None
        if with_e2e:
            h_in = [torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).pin_memory() for a in inputs]
            h_out = [torch.empty(d.byte_size, dtype=torch.uint8).pin_memory() for d in out_desc]
            e2e_steps = max(2, min(steps, 5))
            session.invoke(compiled, h_in, h_out)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                session.invoke(compiled, h_in, h_out)
            e2e_s = self.max_over_ranks(time.perf_counter() - t0)
            e2e = {"value": units * e2e_steps / e2e_s, "unit": unit,
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
                res_s = self.max_over_ranks(time.perf_counter() - t0)
                e2e["resident_weights"] = {"value": units * e2e_steps / res_s, "unit": unit, "inputs_kept_on_device": weights,
                                           "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for i, t in enumerate(h_in) if i not in weights)),
                                           "ms_per_step": 1e3 * res_s / e2e_steps}
                for i in weights:
                    session.set_resident(compiled, i, None)
            del h_in, h_out

        record = None
        if rank == 0:
            avg_ms = total_ms / steps if flush is None else float(np.mean(step_ms))
            note = None
            extra = {}
            if bound == "hbm":
                achieved = local_work["bytes"] / 1e9 / (avg_ms / 1e3)
                peak, peak_unit = self.peaks["hbm_gbs"], "GB/s"
            elif bound == "tensor":
                achieved = local_work["flops"] / 1e12 / (avg_ms / 1e3)
                peak, peak_unit = self.peaks["bf16_tflops"], "TFLOP/s"
                extra["peak_sustained"] = self.peaks["bf16_tflops_sustained"]
                # These kernels run at the 1000 W power cap, where the SM clock (sampled below) settles
                # well under its maximum: the same achieved rate against what the tensor pipes can do at
                # that clock (8192 dense bf16 flop per clock per SM: eight 128x128x16 MMAs take 512 cycles)
                mhz = (clocks or {}).get("sm_mhz")
                if mhz:
                    at_clock = 148 * 8192 * mhz * 1e6 / 1e12
                    extra["at_sampled_clock"] = {"sm_mhz": mhz, "tensor_peak": at_clock, "frac": achieved / at_clock}
            else:
                # FP32-bound: (guess, point) pairs per second against what a register-only loop of
                # CUDA's sinf plus the program's four other operations reaches on this GPU, and the
                # FP32 operations the kernel actually executes against the packed-FMA rate measured
                # here and the nominal rate (SMs x 128 lanes x 2 x the maximum SM clock)
                ceilings = self.fp32_ceilings()
                achieved = local_work["pairs"] / 1e9 / (avg_ms / 1e3)
                peak, peak_unit = ceilings["sinf_plus_4_flop_gpairs"], "Gpair/s"
                sm_max = (clocks or {}).get("sm_max_mhz") or 1965.0
                nominal = 148 * 128 * 2 * sm_max * 1e6 / 1e12
                executed = EXECUTED_FLOP_PER_PAIR[name] * achieved * 1e9 / 1e12
                extra["fp32"] = {"executed_flop_per_pair": EXECUTED_FLOP_PER_PAIR[name], "executed_tflops": executed,
                                 "measured_packed_fma_tflops": ceilings["packed_fma_tflops"], "nominal_fp32_tflops": nominal,
                                 "frac_of_measured_packed_fma": executed / ceilings["packed_fma_tflops"],
                                 "frac_of_nominal_fp32": executed / nominal,
                                 "recorded_flop_per_pair": local_work["flops"] / local_work["pairs"],
                                 "hbm_bytes": local_work["bytes"]}
                note = ("FP32-bound by construction (the broadcast product is never materialised: %d bytes of HBM traffic). "
                        "peak = pairs/s of a register-only sinf + 4 flop loop measured in this run; the kernel's own packed "
                        "sine is cheaper than sinf, so frac can exceed 1" % int(local_work["bytes"]))
            roofline = {"bound": bound, "achieved": achieved, "peak": peak, "unit": peak_unit, "frac": achieved / peak,
                        "traffic": NCU_TRAFFIC[name](cfg_sizes(cfg)) if name in NCU_TRAFFIC else None,
                        "peak_source": self.peaks["source"] if bound != "fp32" else "measured in this run",
                        "kernel_ms": avg_ms, "launches_per_step": work["launches"]}
            roofline.update(extra)
            if note:
                roofline["note"] = note
            cpu = None
            if with_cpu and world == 1:
                v, cores, sample, _, _ = cpu_sample(name, inputs, 1, budget_s=15.0)
                cpu = {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample}
            config = config_record(name, global_sizes, world, scaling if world > 1 else "weak", args.small,
                                   l2_rule)
            record = {"piece_specs": [repr(t) for t in program.input_types],
                      "plan": compiled.plan_summary().strip().split("\n"), "metric": metric, "value": value, "unit": unit, "ms_per_step": total_ms / steps, "steps": steps,
                      "warmup": warmup, "dtype": cfg.dtype, "config": config, "roofline": roofline,
                      "kernel_ms": {"min": float(min(step_ms)), "median": float(np.median(step_ms)), "mean": avg_ms},
                      "clocks": clocks, "parity": parity, "cpu_baseline": cpu, "e2e": e2e,
                      "gpu_launches": work["launches"] * steps, "wall_ms_per_step": 1e3 * wall / steps}
        session.deinit()
        del d_in, d_out, in_sets, out_sets
        torch.cuda.empty_cache()
        return record

    def finish(self):
        self.sampler.stop()
        if self.world > 1:
            self.dist.destroy_process_group()


def cfg_sizes(cfg):
    return [(n, e) for s in cfg.specs for n, e in s.dims]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="time this program alone (default: softmax_layernorm as the headline and, on one GPU, the "
                         "other four benchmark programs under `workloads`)")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--small", action="store_true", help="reduced sizes (profiling captures only; not a bench value)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle spot checks (profiling captures)")
    ap.add_argument("--weak", action="store_true",
                    help="with --gpus N > 1: every rank runs a full one-GPU problem (weak scaling) instead of 1/N of it")
    ap.add_argument("--strong", action="store_true", help="accepted for compatibility: strong scaling is the default")
    args = ap.parse_args()
    name = args.workload or "softmax_layernorm"
    if args.impl == "reference":
        reference_arm(args, name)
        return

    runner = Runner(args)
    world, rank = runner.world, runner.rank
    scaling = "weak" if (args.weak or world == 1) else "strong"
    head = runner.run(name, scaling, args.steps, args.warmup, with_e2e=not args.no_e2e, with_cpu=not args.no_cpu_baseline)
    others = {}
    weak = None
    if args.workload is None and world == 1 and not args.small:
        for other in SECONDARY:
            rec = runner.run(other, scaling, max(args.steps, 20), args.warmup, with_e2e=False, with_cpu=False)
            if rank == 0:
                others[other] = {"metric": rec["metric"], "value": rec["value"], "unit": rec["unit"], "kernel_ms": rec["kernel_ms"],
                                 "steps": rec["steps"], "roofline": rec["roofline"], "clocks": rec["clocks"], "parity": rec["parity"],
                                 "dtype": rec["dtype"], "specs": rec["config"]["specs"], "plan": rec["plan"],
                                 "gpu_launches": rec["gpu_launches"]}
    if world > 1 and scaling == "strong":
        # for the record: the same ranks with a full one-GPU problem each
        rec = runner.run(name, "weak", args.steps, args.warmup, with_e2e=False, with_cpu=False)
        if rank == 0:
            weak = {"value": rec["value"], "unit": rec["unit"], "ms_per_step": rec["ms_per_step"], "specs": rec["config"]["specs"]}
    if rank == 0:
        line = {"metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": args.steps,
                "warmup": head["warmup"], "ms_per_step": head["ms_per_step"], "higher_is_better": True,
                "scaling": scaling, "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic",
                "config": head["config"], "roofline": head["roofline"], "cpu_baseline": head["cpu_baseline"], "e2e": head["e2e"],
                "gpu_launches": runner.launches, "clocks": head["clocks"], "parity": head["parity"],
                "wall_ms_per_step": head["wall_ms_per_step"], "ms_min": head["kernel_ms"]["min"],
                "ms_median": head["kernel_ms"]["median"], "plan": head["plan"], "piece_specs": head["piece_specs"]}
        if others:
            line["workloads"] = others
        if weak:
            line["weak"] = weak
        print(json.dumps(line))
    runner.finish()


if __name__ == "__main__":
    main()
