"""f32 elementwise programs are bit-identical to the reference's arithmetic.

The reference's CPU code rounds every recorded f32 operation on its own (mulss / addss / divss /
sqrtss, no FMA contraction: deps/lib/compiler/choir/src/backends/x64/scalar.zig:310,736), and an
elementwise program has no reduction order that could excuse a difference.  The row kernels use
packed f32x2 instructions, keep a recorded multiply from being merged with a following addition,
and divide a row by a per-row value through a reciprocal and two fused correction steps; these
tests hold all of that to the bits of the oracle's `mode="ref"` evaluation (one C float operation
per recorded op, compiled without contraction).

Beside the hand-written programs, seeded random ones: elementwise programs over broadcast operands,
and programs that mix in max / min reductions (order-independent, so still exact to the bit).

Operands: ordinary magnitudes (1e-10 .. 1e10), zeros of both signs, per-row divisors that include
powers of two, an all-ones significand, a subnormal and zero.  Not covered: NaN payloads (x86 and
the GPU produce different quiet-NaN bit patterns), transcendental functions (different libm), and
quotients of numerators below 2^-103, where the correction steps' residual is not exactly
representable and the last bit of a quotient can differ from a true division.
"""
import numpy as np
import pytest

from accy_b200 import tensor
from oracle import oracle

pytestmark = pytest.mark.gpu
T = tensor


def wide_values(rng, shape):
    """values across twenty orders of magnitude, both signs, with a sprinkling of zeros"""
    x = rng.standard_normal(shape) * np.power(10.0, rng.uniform(-10.0, 10.0, shape))
    x = x.astype(np.float32)
    flat = x.reshape(-1)
    flat[rng.integers(0, flat.size, max(1, flat.size // 97))] = 0.0
    flat[rng.integers(0, flat.size, max(1, flat.size // 101))] = -0.0
    return x


def moderate_values(rng, shape):
    return rng.uniform(-4.0, 4.0, shape).astype(np.float32)


def divisors(rng, rows):
    d = (rng.uniform(0.5, 8.0, rows) * rng.choice([-1.0, 1.0], rows)).astype(np.float32)
    special = [1.0, -2.0, 3.0, np.float32(1.9999999), 1e-35, 1e-40, 3e37, 0.0, 0.25, 7.0]
    d[:len(special)] = np.array(special, np.float32)
    return d


def row_divide_inputs(rng):
    x = wide_values(rng, (64, 1024))
    x[7][x[7] == 0] = 1.0    # the row divided by zero holds no zero (0/0 is NaN, whose bits differ by platform)
    return [x, divisors(rng, 64)]


CASES = {
    # a product that feeds an addition: the multiply keeps its own rounding
    "product_then_sum": ([T.spec("f32", n=1 << 20)] * 3, lambda b, a: a[0].mul(a[1]).add(a[2]),
                         lambda rng: [moderate_values(rng, 1 << 20) for _ in range(3)]),
    "product_then_difference_wide": ([T.spec("f32", n=300001)] * 3, lambda b, a: a[2].sub(a[0].mul(a[1])),
                                     lambda rng: [wide_values(rng, 300001), moderate_values(rng, 300001), wide_values(rng, 300001)]),
    # products of products, then a sum of two products
    "products_of_products": ([T.spec("f32", r=96, c=512)] * 3,
                             lambda b, a: a[0].mul(a[1]).mul(a[2]).add(a[0].mul(a[2])),
                             lambda rng: [moderate_values(rng, (96, 512)) for _ in range(3)]),
    # a row scaled by a per-row value and shifted by a per-column value (broadcast operands)
    "row_scale_column_shift": ([T.spec("f32", r=64, c=1024), T.spec("f32", r=64), T.spec("f32", c=1024)],
                               lambda b, a: a[0].mul(a[1]).add(a[2]),
                               lambda rng: [moderate_values(rng, (64, 1024)), moderate_values(rng, 64), moderate_values(rng, 1024)]),
    # the packed division by a per-row value (reciprocal + two fused corrections) and the ordinary one
    "row_divide": ([T.spec("f32", r=64, c=1024), T.spec("f32", r=64)], lambda b, a: a[0].div(a[1]), row_divide_inputs),
    "row_divide_long_rows": ([T.spec("f32", r=10, c=40000), T.spec("f32", r=10)], lambda b, a: a[0].div(a[1]),
                             lambda rng: [moderate_values(rng, (10, 40000)), divisors(rng, 10)]),
    "elementwise_divide": ([T.spec("f32", n=200000)] * 2, lambda b, a: a[0].div(a[1]),
                           lambda rng: [wide_values(rng, 200000), moderate_values(rng, 200000) + np.float32(5.0)]),
    "centred_and_scaled": ([T.spec("f32", r=32, c=2048), T.spec("f32", r=32), T.spec("f32", r=32)],
                           lambda b, a: a[0].sub(a[1]).div(a[2].mul(a[2]).add(b.scalar("f32", 1e-5)).sqrt()),
                           lambda rng: [moderate_values(rng, (32, 2048)), moderate_values(rng, 32), moderate_values(rng, 32)]),
    "sqrt_abs_neg": ([T.spec("f32", n=100003)], lambda b, a: a[0].abs().sqrt().neg().add(a[0]),
                     lambda rng: [wide_values(rng, 100003)]),
    "max_min": ([T.spec("f32", n=70001)] * 3, lambda b, a: a[0].max(a[1]).sub(a[1].min(a[2]).mul(a[0])),
                lambda rng: [moderate_values(rng, 70001) for _ in range(3)]),
    "select_by_comparison": ([T.spec("f32", r=40, c=768)] * 3,
                             lambda b, a: a[0].compare("gt", a[1]).select(a[0].mul(a[2]), a[1].add(a[2])),
                             lambda rng: [moderate_values(rng, (40, 768)) for _ in range(3)]),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_f32_elementwise_program_equals_the_oracle_bit_for_bit(gpu_session, name):
    specs, body, make = CASES[name]
    program = tensor.define("exact_" + name, specs, body)
    inputs = make(np.random.default_rng(len(name) * 7 + 1))
    compiled = gpu_session.compile(program)
    out = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    gpu_session.invoke(compiled, inputs, [out])
    gpu_session.release(compiled)
    want = np.asarray(oracle.run(program.wire, inputs, mode="ref")[0], np.float32).reshape(-1)
    got = out.view(np.float32)
    finite_or_inf = ~np.isnan(want)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    differing = np.flatnonzero(got.view(np.uint32)[finite_or_inf] != want.view(np.uint32)[finite_or_inf])
    assert differing.size == 0, "%d of %d elements differ, first at %d: gpu %r oracle %r" % (
        differing.size, want.size, differing[0], got[finite_or_inf][differing[0]], want[finite_or_inf][differing[0]])


def random_program(seed):
    """A seeded random f32 elementwise program over [r, c] with per-row, per-column and scalar operands:
    (specs, body, inputs).  Operations: add sub mul div max min neg abs sqrt(abs) select(compare)."""
    rng = np.random.default_rng(1000 + seed)
    r = int(rng.choice([1, 3, 17, 64, 257]))
    c = int(rng.choice([1, 5, 128, 1000, 4096, 4100]))
    kinds = ["full", "full"] + [str(k) for k in rng.choice(["full", "row", "col"], int(rng.integers(1, 3)))]
    specs, inputs = [], []
    for kind in kinds:
        if kind == "full":
            specs.append(T.spec("f32", r=r, c=c)); shape = (r, c)
        elif kind == "row":
            specs.append(T.spec("f32", r=r)); shape = (r,)
        else:
            specs.append(T.spec("f32", c=c)); shape = (c,)
        x = rng.uniform(-4.0, 4.0, shape).astype(np.float32)
        flat = x.reshape(-1)
        flat[rng.integers(0, flat.size, max(1, flat.size // 50))] = rng.choice([0.0, -0.0, 1.0, -1.0, 0.5, 2.0])
        inputs.append(x)
    steps = []   # (op, operand indices into the value list, constant)
    n_values = len(kinds)
    for _ in range(int(rng.integers(4, 10))):
        op = str(rng.choice(["add", "sub", "mul", "div", "max", "min", "neg", "abs", "sqrt", "select", "scalar_mul", "scalar_add"]))
        picks = [int(p) for p in rng.integers(0, n_values, 4)]
        steps.append((op, picks, float(np.float32(rng.uniform(-3.0, 3.0))), str(rng.choice(["lt", "le", "gt", "ge"]))))
        n_values += 1

    def body(b, a):
        values = list(a)
        for op, p, const, cmp in steps:
            x, y, z, w = (values[i] for i in p)
            if op in ("add", "sub", "mul", "max", "min"):
                v = getattr(x, op)(y)
            elif op == "div":
                v = x.div(y.abs().add(b.scalar("f32", 0.25)))     # divisors stay away from zero
            elif op == "neg":
                v = x.neg()
            elif op == "abs":
                v = x.abs()
            elif op == "sqrt":
                v = x.abs().sqrt()
            elif op == "select":
                v = x.compare(cmp, y).select(z, w)
            elif op == "scalar_mul":
                v = x.mul(b.scalar("f32", const))
            else:
                v = x.add(b.scalar("f32", const))
            values.append(v)
        # every input takes part, and the result has the full shape
        out = values[-1]
        for v in a:
            out = out.add(v)
        return out

    return specs, body, inputs


@pytest.mark.parametrize("seed", range(24))
def test_random_f32_elementwise_programs_equal_the_oracle_bit_for_bit(gpu_session, seed):
    """Seeded random programs (shapes from 1 x 1 to 257 x 4100, broadcast operands, signed zeros among the
    values): every element has the bits of the one-rounding-per-operation evaluation."""
    specs, body, inputs = random_program(seed)
    program = tensor.define("random_exact_%d" % seed, specs, body)
    compiled = gpu_session.compile(program)
    out = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    gpu_session.invoke(compiled, inputs, [out])
    gpu_session.release(compiled)
    want = np.asarray(oracle.run(program.wire, inputs, mode="ref")[0], np.float32).reshape(-1)
    got = out.view(np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    differing = np.flatnonzero(got.view(np.uint32)[ok] != want.view(np.uint32)[ok])
    assert differing.size == 0, "%d of %d elements differ, first at %d: gpu %r oracle %r" % (
        differing.size, want.size, differing[0], got[ok][differing[0]], want[ok][differing[0]])


def random_reduce_program(seed):
    """A seeded random f32 program over [r, c] that mixes elementwise operations with max / min
    reductions over c, over r or over both (whose results broadcast back by name): (specs, body, inputs).
    A maximum or minimum does not depend on the order of the fold, so these programs, too, have one
    right answer to the bit.  The inputs hold no zeros: the sign of a zero maximum would depend on
    the order in which +0 and -0 meet."""
    rng = np.random.default_rng(5000 + seed)
    r = int(rng.choice([1, 5, 64, 300]))
    c = int(rng.choice([1, 7, 256, 1000, 5000]))
    kinds = ["full", "full", str(rng.choice(["row", "col"]))]
    specs, inputs = [], []
    for kind in kinds:
        shape = {"full": (r, c), "row": (r,), "col": (c,)}[kind]
        specs.append(T.spec("f32", **({"r": r, "c": c} if kind == "full" else ({"r": r} if kind == "row" else {"c": c}))))
        x = rng.uniform(0.125, 4.0, shape) * rng.choice([-1.0, 1.0], shape)
        inputs.append(x.astype(np.float32))
    dims_of = [{"full": ("r", "c"), "row": ("r",), "col": ("c",)}[k] for k in kinds]
    steps = []
    for _ in range(int(rng.integers(5, 11))):
        op = str(rng.choice(["add", "sub", "mul", "max", "min", "neg", "abs", "select", "scalar_mul", "reduce", "reduce", "reduce"]))
        picks = [int(p) for p in rng.integers(0, len(dims_of), 4)]
        how = (str(rng.choice(["max", "min"])), str(rng.choice(["c", "r", "rc"])), float(np.float32(rng.uniform(-3.0, 3.0))),
               str(rng.choice(["lt", "le", "gt", "ge"])))
        if op == "reduce":
            have = dims_of[picks[0]]
            axes = tuple(a for a in how[1] if a in have)
            if not axes:
                op = "neg"
                dims_of.append(have)
            else:
                how = (how[0], axes) + how[2:]
                dims_of.append(tuple(a for a in have if a not in axes))
        elif op in ("neg", "abs", "scalar_mul"):
            dims_of.append(dims_of[picks[0]])
        elif op == "select":
            dims_of.append(tuple(a for a in ("r", "c") if any(a in dims_of[p] for p in picks)))
        else:
            dims_of.append(tuple(a for a in ("r", "c") if a in dims_of[picks[0]] or a in dims_of[picks[1]]))
        steps.append((op, picks, how))

    def body(b, a):
        values = list(a)
        for op, p, how in steps:
            x, y, z, w = (values[i] for i in p)
            if op in ("add", "sub", "mul", "max", "min"):
                v = getattr(x, op)(y)
            elif op == "neg":
                v = x.neg()
            elif op == "abs":
                v = x.abs()
            elif op == "select":
                v = x.compare(how[3], y).select(z, w)
            elif op == "scalar_mul":
                v = x.mul(b.scalar("f32", how[2]))
            else:
                v = getattr(x, how[0])(list(how[1]))
            values.append(v)
        out = values[-1]
        for v in a:
            out = out.add(v)
        return out

    return specs, body, inputs


@pytest.mark.parametrize("seed", range(24))
def test_random_f32_programs_with_max_and_min_reductions_equal_the_oracle_bit_for_bit(gpu_session, seed):
    specs, body, inputs = random_reduce_program(seed)
    program = tensor.define("random_reduce_%d" % seed, specs, body)
    compiled = gpu_session.compile(program)
    out = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    gpu_session.invoke(compiled, inputs, [out])
    gpu_session.release(compiled)
    want = np.asarray(oracle.run(program.wire, inputs, mode="ref")[0], np.float32).reshape(-1)
    got = out.view(np.float32)
    assert not np.isnan(want).any()
    differing = np.flatnonzero(got.view(np.uint32) != want.view(np.uint32))
    assert differing.size == 0, "%d of %d elements differ, first at %d: gpu %r oracle %r" % (
        differing.size, want.size, differing[0], got[differing[0]], want[differing[0]])
