"""The five benchmark programs, written against the recording API exactly as a user of the
reference would write them with `tensor.define` / `Value` methods, plus seeded synthetic inputs.

Each `Config` gives: the body, the specs at a chosen size, the axis the program shards along with
no exchange between shards, input generators, and the algorithmic work figures used for roofline
reporting.  Inputs are synthetic (numpy PCG64 `default_rng(seed)`); "N(0, s)" means standard
deviation s.
"""
import math

import numpy as np

from . import synthetic
from . import tensor as T


from .synthetic import bf16_bits_to_f32, f32_to_bf16_bits  # noqa: F401  (re-exported)


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


def _specs(name, sizes, keys=None):
    return [T.spec(dtype, **dict(dims)) for dtype, dims in synthetic.specs(name, sizes, keys)]


def mismatch(guesses=8192, points=65536, seed=0):
    sizes = synthetic.sizes_of("mismatch", guesses, points)
    return Config("mismatch", mismatch_body, _specs("mismatch", sizes), "guess",
                  lambda: synthetic.inputs("mismatch", sizes, seed), synthetic.work("mismatch", sizes), 1e-5, "f32")


def softmax_layernorm(rows=32768, cols=4096, seed=1):
    sizes = synthetic.sizes_of("softmax_layernorm", rows, cols)
    return Config("softmax_layernorm", softmax_layernorm_body, _specs("softmax_layernorm", sizes), "row",
                  lambda: synthetic.inputs("softmax_layernorm", sizes, seed), synthetic.work("softmax_layernorm", sizes),
                  1e-5, "f32")


def matmul(m=8192, n=8192, k=8192, seed=2):
    sizes = synthetic.sizes_of("matmul", m, n, k)
    return Config("matmul", matmul_body, _specs("matmul", sizes), "m", lambda: synthetic.inputs("matmul", sizes, seed),
                  synthetic.work("matmul", sizes), 2e-2, "bf16")


def attention(batch=8, head=32, seq=4096, dim=128, causal=True, seed=3, keys=None):
    keys = seq if keys is None else keys   # a different key length (non-causal only): cross attention
    sizes = synthetic.sizes_of("attention", batch, head, seq, dim)
    body = make_attention_body(1.0 / math.sqrt(dim), causal)
    return Config("attention", body, _specs("attention", sizes, keys), "batch",
                  lambda: synthetic.inputs("attention", sizes, seed, keys), synthetic.work("attention", sizes, causal, keys),
                  2e-2, "bf16")


def mlp(tokens=16384, d=4096, h=16384, seed=4):
    sizes = synthetic.sizes_of("mlp", tokens, d, h)
    return Config("mlp", mlp_body, _specs("mlp", sizes), "token", lambda: synthetic.inputs("mlp", sizes, seed),
                  synthetic.work("mlp", sizes), 2e-2, "bf16")


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
    work = synthetic.work("refine", synthetic.sizes_of("refine", guesses, points))
    return DerivedConfig(derive, "refine", mismatch_body, base.specs, "guess", base.make_inputs, work, 1e-5, "f32")


BASELINE = {"refine": refine, "mismatch": mismatch, "softmax_layernorm": softmax_layernorm, "matmul": matmul,
            "attention": attention, "mlp": mlp}
