"""f32 elementwise programs are bit-identical to the reference's arithmetic.

The reference's CPU code rounds every recorded f32 operation on its own (mulss / addss / divss /
sqrtss, no FMA contraction: deps/lib/compiler/choir/src/backends/x64/scalar.zig:310,736), and an
elementwise program has no reduction order that could excuse a difference.  The row kernels use
packed f32x2 instructions, keep a recorded multiply from being merged with a following addition,
and divide a row by a per-row value through a reciprocal and two fused correction steps; these
tests hold all of that to the bits of the oracle's `mode="ref"` evaluation (one C float operation
per recorded op, compiled without contraction).

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
