"""Seeded synthetic inputs, input specs and work figures of the benchmark programs, in plain numpy.

This module imports nothing from the package and never touches the native library, so a process
that only wants the inputs (the CPU-timed reference arm of the benchmark, fixture scripts) can load
it by file path without mapping libaccy_b200.so.  `accy_b200.configs` builds its recorded programs
on top of the same tables, so both sides see the same bytes.

Inputs come from numpy's PCG64 `default_rng`; "N(0, s)" means standard deviation s; bf16 values
are carried as uint16 bit patterns (round-to-nearest-even from the f32 draw).  The large bf16
operands of one configuration are drawn from separate streams, `default_rng([seed, index])`, so
that they can be generated on separate host threads (numpy releases the interpreter lock while it
draws); the bytes depend on the seed and the index only, not on the threading.
"""
import math
from concurrent.futures import ThreadPoolExecutor

import numpy as np

# default extents of the five benchmark configurations, plus the derived value-and-slope program
SIZES = {
    "mismatch": [("guess", 8192), ("point", 65536)],
    "refine": [("guess", 8192), ("point", 65536)],
    "softmax_layernorm": [("row", 32768), ("col", 4096)],
    "matmul": [("m", 8192), ("n", 8192), ("k", 8192)],
    "attention": [("batch", 8), ("head", 32), ("seq", 4096), ("dim", 128)],
    "mlp": [("token", 16384), ("d", 4096), ("h", 16384)],
}
SEEDS = {"mismatch": 0, "refine": 0, "softmax_layernorm": 1, "matmul": 2, "attention": 3, "mlp": 4}
DTYPES = {"mismatch": "f32", "refine": "f32", "softmax_layernorm": "f32", "matmul": "bf16", "attention": "bf16", "mlp": "bf16"}


def f32_to_bf16_bits(a):
    """round-to-nearest-even f32 -> bf16 bit patterns (uint16)"""
    a = np.ascontiguousarray(a, dtype=np.float32)
    w = a.view(np.uint32)
    if not np.isfinite(a).all():
        # infinities and NaNs: the rounding increment is computed in 64 bits so it cannot wrap
        w = w.astype(np.uint64)
        return ((w + 0x7FFF + ((w >> 16) & 1)) >> 16).astype(np.uint16)
    return ((w + (np.uint32(0x7FFF) + ((w >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _normal_bf16(seed, index, shape, scale):
    draw = np.random.default_rng([seed, index]).standard_normal(shape, dtype=np.float32)
    if scale != 1.0:
        draw *= np.float32(scale)
    return f32_to_bf16_bits(draw)


def _drawn_together(seed, requests):
    """[(shape, scale), ...] -> bf16 bit patterns, one stream and (for large operands) one thread each"""
    if sum(int(np.prod(shape)) for shape, _ in requests) < (1 << 22):
        return [_normal_bf16(seed, i, shape, scale) for i, (shape, scale) in enumerate(requests)]
    with ThreadPoolExecutor(max_workers=len(requests)) as pool:
        futures = [pool.submit(_normal_bf16, seed, i, shape, scale) for i, (shape, scale) in enumerate(requests)]
        return [f.result() for f in futures]


def sizes_of(name, *extents):
    """The config's (axis, extent) list with the given extents in place of the defaults (in order)."""
    out = list(SIZES[name])
    for i, e in enumerate(extents):
        if e is not None:
            out[i] = (out[i][0], int(e))
    return out


def specs(name, sizes, keys=None):
    """Input specs as (dtype, [(axis, extent), ...]) in parameter order."""
    s = dict(sizes)
    if name in ("mismatch", "refine"):
        return [("f32", [("guess", s["guess"])]), ("f32", [("point", s["point"])]), ("f32", [("point", s["point"])])]
    if name == "softmax_layernorm":
        return [("f32", [("row", s["row"]), ("col", s["col"])])]
    if name == "matmul":
        return [("bf16", [("m", s["m"]), ("k", s["k"])]), ("bf16", [("k", s["k"]), ("n", s["n"])])]
    if name == "attention":
        keys = s["seq"] if keys is None else keys
        q = [("batch", s["batch"]), ("head", s["head"]), ("seq", s["seq"]), ("dim", s["dim"])]
        kv = [("batch", s["batch"]), ("head", s["head"]), ("key", keys), ("dim", s["dim"])]
        return [("bf16", q), ("bf16", kv), ("bf16", kv)]
    if name == "mlp":
        return [("bf16", [("token", s["token"]), ("d", s["d"])]), ("bf16", [("d", s["d"]), ("h", s["h"])]), ("bf16", [("h", s["h"])]),
                ("bf16", [("h", s["h"]), ("d", s["d"])]), ("bf16", [("d", s["d"])]), ("bf16", [("d", s["d"])])]
    raise KeyError(name)


def spec_text(spec):
    """The text form a recorded type prints as, e.g. f32[row=32768, col=4096]."""
    dtype, dims = spec
    return "%s[%s]" % (dtype, ", ".join("%s=%d" % d for d in dims))


def inputs(name, sizes, seed=None, keys=None):
    """The seeded input arrays of a configuration (bf16 as uint16 bit patterns)."""
    s = dict(sizes)
    seed = SEEDS[name] if seed is None else seed
    rng = np.random.default_rng(seed)
    if name in ("mismatch", "refine"):
        frequency = rng.uniform(0.0, 6.0, s["guess"]).astype(np.float32)
        time = (0.25 * np.arange(s["point"])).astype(np.float32)
        noise = np.random.default_rng([seed, 1]).normal(0.0, 0.01, s["point"])
        sample = (np.sin(3.0 * time.astype(np.float64)) + noise).astype(np.float32)
        return [frequency, time, sample]
    if name == "softmax_layernorm":
        return [rng.standard_normal((s["row"], s["col"]), dtype=np.float32) * np.float32(3.0)]
    if name == "matmul":
        scale = 1.0 / math.sqrt(s["k"])
        return _drawn_together(seed, [((s["m"], s["k"]), scale), ((s["k"], s["n"]), scale)])
    if name == "attention":
        keys = s["seq"] if keys is None else keys
        return _drawn_together(seed, [((s["batch"], s["head"], n, s["dim"]), 1.0) for n in (s["seq"], keys, keys)])
    if name == "mlp":
        x, w1, w2 = _drawn_together(seed, [((s["token"], s["d"]), 1.0), ((s["d"], s["h"]), 0.02), ((s["h"], s["d"]), 0.02)])
        return [x, w1, np.zeros(s["h"], np.uint16), w2, np.zeros(s["d"], np.uint16), f32_to_bf16_bits(np.ones(s["d"], np.float32))]
    raise KeyError(name)


def work(name, sizes, causal=True, keys=None):
    """Algorithmic work per pass: bytes that must cross HBM once, contraction flops, (row, column) pairs."""
    s = dict(sizes)
    if name == "mismatch":
        g, p = s["guess"], s["point"]
        return {"bytes": 4.0 * (g + 2 * p + g), "flops": 5.0 * g * p, "pairs": float(g) * p}
    if name == "refine":
        g, p = s["guess"], s["point"]
        return {"bytes": 4.0 * (g + 2 * p + 2 * g), "flops": 11.0 * g * p, "pairs": float(g) * p}
    if name == "softmax_layernorm":
        return {"bytes": 8.0 * s["row"] * s["col"], "flops": 0.0, "pairs": float(s["row"]) * s["col"]}
    if name == "matmul":
        m, n, k = s["m"], s["n"], s["k"]
        return {"bytes": 2.0 * (m * k + k * n + m * n), "flops": 2.0 * m * n * k, "pairs": 0.0}
    if name == "attention":
        keys = s["seq"] if keys is None else keys
        pairs = s["seq"] * (s["seq"] + 1) / 2.0 if causal else float(s["seq"]) * keys
        bh = s["batch"] * s["head"]
        return {"bytes": 4.0 * 2 * bh * s["seq"] * s["dim"], "flops": 4.0 * s["dim"] * pairs * bh, "pairs": 0.0}
    if name == "mlp":
        t, d, h = s["token"], s["d"], s["h"]
        return {"bytes": 2.0 * (2 * t * d + 2 * d * h + 2 * t * h), "flops": 4.0 * t * d * h, "pairs": 0.0}
    raise KeyError(name)
