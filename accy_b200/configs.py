"""The five benchmark programs, written against the recording API exactly as a user of the
reference would write them with `tensor.define` / `Value` methods, plus seeded synthetic inputs.

Each `Config` gives: the body, the specs at a chosen size, the axis the program shards along with
no exchange between shards, input generators, and the algorithmic work figures used for roofline
reporting.  Inputs are synthetic (numpy PCG64 `default_rng(seed)`); "N(0, s)" means standard
deviation s.
"""
import math

import numpy as np

from . import tensor as T


def f32_to_bf16_bits(a):
    """round-to-nearest-even f32 -> bf16 bit patterns (uint16)"""
    w = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    w = w + 0x7FFF + ((w >> 16) & 1)
    return (w >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- bodies -------------------------------------------------------------------------------
def mismatch_body(builder, args):
    """README `mismatch` vectorised over guesses: sum_point (sin(frequency*time) - sample)^2."""
    frequency, time, sample = args
    gap = frequency.mul(time).sin().sub(sample)
    return gap.mul(gap).sum("point")


def softmax_layernorm_body(builder, args):
    x = args[0]
    shifted = x.sub(x.max("col"))
    e = shifted.exp()
    y = e.div(e.sum("col"))
    centred = y.sub(y.mean("col"))
    variance = centred.mul(centred).mean("col")
    return centred.div(variance.add(builder.scalar("f32", 1e-5)).sqrt())


def matmul_body(builder, args):
    a, b = args
    return a.contract(b, "k")


def make_attention_body(scale, causal=True):
    def body(builder, args):
        q, k, v = args
        dtype = q.ty.dtype
        scores = q.contract(k, "dim").mul(builder.scalar(dtype, scale))
        if causal:
            dims = [d for d in scores.ty.dims if d[0] in ("seq", "key")]
            qi = builder.iota("i32", dims, "seq")
            ki = builder.iota("i32", dims, "key")
            mask = qi.compare("ge", ki)
            scores = mask.select(scores, builder.scalar(dtype, -math.inf))
        e = scores.sub(scores.max("key")).exp()
        p = e.div(e.sum("key"))
        return p.contract(v, "key")
    return body


def mlp_body(builder, args):
    x, w1, b1, w2, b2, g = args
    dtype = x.ty.dtype
    c = lambda v: builder.scalar(dtype, v)  # noqa: E731
    h = x.contract(w1, "d").add(b1)
    cube = h.mul(h).mul(h)
    inner = h.add(cube.mul(c(0.044715))).mul(c(0.7978845608028654))
    act = h.mul(c(0.5)).mul(inner.tanh().add(c(1.0)))
    y = act.contract(w2, "h").add(b2)
    rms = y.mul(y).mean("d").add(c(1e-6)).sqrt()
    return y.div(rms).mul(g)


# ---- configs ------------------------------------------------------------------------------
class Config:
    def __init__(self, name, body, specs, shard_axis, make_inputs, work, tolerance, dtype):
        self.name = name
        self.body = body
        self.specs = specs
        self.shard_axis = shard_axis
        self.make_inputs = make_inputs  # () -> list of numpy arrays (bf16 as uint16 bit patterns)
        self.work = work                # {"bytes":…, "flops":…, "pairs":…}
        self.tolerance = tolerance
        self.dtype = dtype

    def program(self):
        return T.define(self.name, self.specs, self.body)


def mismatch(guesses=8192, points=65536, seed=0):
    def inputs():
        rng = np.random.default_rng(seed)
        frequency = rng.uniform(0.0, 6.0, guesses).astype(np.float32)
        time = (0.25 * np.arange(points)).astype(np.float32)
        noise = np.random.default_rng([seed, 1]).normal(0.0, 0.01, points)
        sample = (np.sin(3.0 * time.astype(np.float64)) + noise).astype(np.float32)
        return [frequency, time, sample]
    specs = [T.spec("f32", guess=guesses), T.spec("f32", point=points), T.spec("f32", point=points)]
    work = {"bytes": 4.0 * (guesses + 2 * points + guesses), "flops": 5.0 * guesses * points,
            "pairs": float(guesses) * points}
    return Config("mismatch", mismatch_body, specs, "guess", inputs, work, 1e-5, "f32")


def softmax_layernorm(rows=32768, cols=4096, seed=1):
    def inputs():
        rng = np.random.default_rng(seed)
        return [rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(3.0)]
    specs = [T.spec("f32", row=rows, col=cols)]
    work = {"bytes": 8.0 * rows * cols, "flops": 0.0, "pairs": float(rows) * cols}
    return Config("softmax_layernorm", softmax_layernorm_body, specs, "row", inputs, work, 1e-5, "f32")


def matmul(m=8192, n=8192, k=8192, seed=2):
    def inputs():
        rng = np.random.default_rng(seed)
        a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(math.sqrt(k))
        b = rng.standard_normal((k, n), dtype=np.float32) / np.float32(math.sqrt(k))
        return [f32_to_bf16_bits(a), f32_to_bf16_bits(b)]
    specs = [T.spec("bf16", m=m, k=k), T.spec("bf16", k=k, n=n)]
    work = {"bytes": 2.0 * (m * k + k * n + m * n), "flops": 2.0 * m * n * k, "pairs": 0.0}
    return Config("matmul", matmul_body, specs, "m", inputs, work, 2e-2, "bf16")


def attention(batch=8, head=32, seq=4096, dim=128, causal=True, seed=3, keys=None):
    keys = seq if keys is None else keys   # a different key length (non-causal only): cross attention
    def inputs():
        rng = np.random.default_rng(seed)
        return [f32_to_bf16_bits(rng.standard_normal((batch, head, n, dim), dtype=np.float32)) for n in (seq, keys, keys)]
    specs = [T.spec("bf16", batch=batch, head=head, seq=seq, dim=dim),
             T.spec("bf16", batch=batch, head=head, key=keys, dim=dim),
             T.spec("bf16", batch=batch, head=head, key=keys, dim=dim)]
    pairs = seq * (seq + 1) / 2.0 if causal else float(seq) * keys
    work = {"bytes": 4.0 * 2 * batch * head * seq * dim, "flops": 4.0 * dim * pairs * batch * head, "pairs": 0.0}
    body = make_attention_body(1.0 / math.sqrt(dim), causal)
    return Config("attention", body, specs, "batch", inputs, work, 2e-2, "bf16")


def mlp(tokens=16384, d=4096, h=16384, seed=4):
    def inputs():
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((tokens, d), dtype=np.float32)
        w1 = rng.standard_normal((d, h), dtype=np.float32) * np.float32(0.02)
        w2 = rng.standard_normal((h, d), dtype=np.float32) * np.float32(0.02)
        return [f32_to_bf16_bits(x), f32_to_bf16_bits(w1), np.zeros(h, np.uint16), f32_to_bf16_bits(w2),
                np.zeros(d, np.uint16), f32_to_bf16_bits(np.ones(d, np.float32))]
    specs = [T.spec("bf16", token=tokens, d=d), T.spec("bf16", d=d, h=h), T.spec("bf16", h=h),
             T.spec("bf16", h=h, d=d), T.spec("bf16", d=d), T.spec("bf16", d=d)]
    work = {"bytes": 2.0 * (2 * tokens * d + 2 * d * h + 2 * tokens * h), "flops": 4.0 * tokens * d * h, "pairs": 0.0}
    return Config("mlp", mlp_body, specs, "token", inputs, work, 2e-2, "bf16")


class DerivedConfig(Config):
    """A config whose program is derived from a recorded one instead of recorded directly."""

    def __init__(self, derive, *args):
        Config.__init__(self, *args)
        self.derive = derive

    def program(self):
        return self.derive()


def refine(guesses=8192, points=65536, seed=0):
    """The README's gradient-descent program at the mismatch configuration's size: value and slope
    (d/d frequency) of the one-guess mismatch, mapped over guesses:
    define(mismatch).valueAndGrad(wrt 0).vmap(guess).  Two outputs f32[guess]."""
    base = mismatch(guesses, points, seed)

    def derive():
        one = T.define("mismatch", [T.spec("f32"), T.spec("f32", point=points), T.spec("f32", point=points)], mismatch_body)
        return one.value_and_grad([0]).vmap(guesses, [T.mapped_axis(0), None, None], axis_name="guess")
    work = {"bytes": 4.0 * (guesses + 2 * points + 2 * guesses), "flops": 11.0 * guesses * points,
            "pairs": float(guesses) * points}
    return DerivedConfig(derive, "refine", mismatch_body, base.specs, "guess", base.make_inputs, work, 1e-5, "f32")


BASELINE = {"refine": refine, "mismatch": mismatch, "softmax_layernorm": softmax_layernorm, "matmul": matmul,
            "attention": attention, "mlp": mlp}
