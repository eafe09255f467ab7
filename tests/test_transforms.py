"""grad / valueAndGrad / vmap of recorded programs (the reference's src/tensor/grad.zig,
src/tensor/batch.zig; the README's "refine eight frequency guesses" example).

CPU: the derived programs are evaluated with the oracle and checked against the README's known
answers, against central finite differences in f64, and (vmap) against the unmapped program run
once per index; error names follow the reference.  GPU: the same derived programs run through the
C ABI and are compared with the oracle (f32: 1e-5 relative to the f64 answer, on top of the
reference-order error itself)."""
import numpy as np
import pytest

from accy_b200 import tensor
from oracle import oracle

T = tensor


def mismatch(b, a):
    frequency, time, sample = a
    gap = frequency.mul(time).sin().sub(sample)
    return gap.mul(gap).sum("point")


def scalar(value):
    """the oracle hands rank-0 results back as arrays of one element"""
    return float(np.asarray(value).reshape(-1)[0])


def tone_samples(points=16):
    time = (0.25 * np.arange(points)).astype(np.float32)
    sample = np.sin(3.0 * time.astype(np.float64)).astype(np.float32)
    return time, sample


def one_guess_program(points=16):
    return tensor.define("mismatch", [T.spec("f32"), T.spec("f32", point=points), T.spec("f32", point=points)], mismatch)


# ---------------------------------------------------------------------------------------------
# known answers (README.md:142-153, 247-313)
# ---------------------------------------------------------------------------------------------
def test_value_and_slope_known_answers():
    time, sample = tone_samples()
    both = one_guess_program().value_and_grad([0])
    assert [repr(t) for t in both.output_types] == ["f32[]", "f32[]"]
    value, slope = oracle.run(both.wire, [np.float32(2.5), time, sample])
    assert abs(scalar(value) - 8.656) < 1e-3
    assert abs(scalar(slope) - (-31.29)) < 1e-2
    value, slope = oracle.run(both.wire, [np.float32(3.0), time, sample])
    assert abs(scalar(value)) < 1e-9
    only = one_guess_program().grad([0])
    assert len(only.output_types) == 1
    assert scalar(oracle.run(only.wire, [np.float32(2.5), time, sample])[0]) == pytest.approx(-31.29, abs=1e-2)


def descend(run, steps=100):
    frequency = np.array([0.5, 1.5, 2.5, 3.5, 4.5, 5.5, 6.5, 7.5], np.float32)
    value = None
    for _ in range(steps):
        value, slope = run(frequency)
        frequency = (frequency - np.float32(0.005) * slope).astype(np.float32)
    return frequency, value


def refine_program():
    return one_guess_program().value_and_grad([0]).vmap(8, [T.mapped_axis(0), None, None], axis_name="guess")


def check_descent(frequency, value):
    assert abs(frequency[2] - 3.0) < 1e-6 and abs(frequency[3] - 3.0) < 1e-6
    assert value[2] < 1e-6 and value[3] < 1e-6
    others = np.delete(value, [2, 3])
    assert others.min() > 7.9 and others.max() < 14.6


def test_refine_eight_frequency_guesses_with_the_oracle():
    each = refine_program()
    assert [repr(t) for t in each.input_types] == ["f32[guess=8]", "f32[point=16]", "f32[point=16]"]
    assert [repr(t) for t in each.output_types] == ["f32[guess=8]", "f32[guess=8]"]
    time, sample = tone_samples()
    check_descent(*descend(lambda f: oracle.run(each.wire, [f, time, sample])))


def test_c_restatement_of_the_refine_program_equals_its_evaluation():
    """bench.py's CPU leg for `--workload refine` runs oracle_mismatch_slope_f32 (oracle/ref_order.c);
    it must be the derived program's own arithmetic in the reference's order: bit for bit what the
    oracle's evaluator gives for valueAndGrad + vmap of the recorded mismatch."""
    import ctypes
    from accy_b200 import configs
    cfg = configs.refine(6, 256)
    inputs = cfg.make_inputs()
    want_value, want_slope = oracle.run(cfg.program().wire, inputs)
    value, slope = np.zeros(6, np.float32), np.zeros(6, np.float32)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)  # noqa: E731
    size = ctypes.c_size_t
    oracle.lib().oracle_mismatch_slope_f32(ptr(inputs[0]), ptr(inputs[1]), ptr(inputs[2]), ptr(value), ptr(slope),
                                           size(6), size(256), size(0), size(6))
    assert np.array_equal(value, want_value) and np.array_equal(slope, want_slope)


def test_function_keeps_its_derived_programs():
    """src/tensor/function.zig: derived functions hang off the root, whatever they were derived from."""
    f = tensor.Function.define("mismatch", [T.spec("f32"), T.spec("f32", point=16), T.spec("f32", point=16)], mismatch)
    both = f.value_and_grad([0])
    each = both.vmap(8, [T.mapped_axis(0), None, None], axis_name="guess")
    assert both.root is f and each.root is f and f.derived == [both, each]
    assert each.graph.wire == refine_program().wire
    with pytest.raises(AssertionError):
        each.deinit()
    f.deinit()
    assert f.derived == []


@pytest.mark.gpu
def test_function_compile_cuda_runs_the_readme_example():
    f = tensor.Function.define("mismatch", [T.spec("f32"), T.spec("f32", point=16), T.spec("f32", point=16)], mismatch)
    each = f.value_and_grad([0]).vmap(8, [T.mapped_axis(0), None, None], axis_name="guess")
    cuda = each.compile_cuda()
    time, sample = tone_samples()
    value, slope = np.empty(8, np.float32), np.empty(8, np.float32)

    def run(frequency):
        cuda.launch([frequency, time, sample], [value, slope])
        return value.copy(), slope.copy()
    check_descent(*descend(run))
    cuda.deinit()
    f.deinit()


@pytest.mark.gpu
def test_refine_eight_frequency_guesses_on_the_device(gpu_session):
    each = refine_program()
    compiled = gpu_session.compile(each)
    time, sample = tone_samples()
    value, slope = np.empty(8, np.float32), np.empty(8, np.float32)

    def run(frequency):
        gpu_session.invoke(compiled, [frequency, time, sample], [value, slope])
        return value.copy(), slope.copy()
    check_descent(*descend(run))
    gpu_session.release(compiled)


# ---------------------------------------------------------------------------------------------
# gradients against finite differences
# ---------------------------------------------------------------------------------------------
def attention_loss(b, a):
    q, k, v = a
    scores = q.contract(k.rename("token", "key"), "channel").mul(b.scalar(q.ty.dtype, 0.5))
    centered = scores.sub(scores.max("key"))
    weights = centered.exp()
    probs = weights.div(weights.sum("key"))
    mixed = probs.contract(v.rename("token", "key"), "key")
    return mixed.mul(mixed).sum(["token", "channel"])


def relu_mask_loss(b, a):
    x = a[0]
    zero = b.full(x.ty.dtype, x.ty.dims, 0.0)
    kept = x.compare("gt", zero).select(x.mul(x), x.neg())
    return kept.sum(["r", "c"])


def unary_zoo(b, a):
    x, y = a  # x in (0.5, 2), y any sign
    dt = x.ty.dtype
    total = x.log().add(x.sqrt()).add(x.exp().mul(b.scalar(dt, 0.1))).add(y.tanh()).add(y.abs())
    total = total.add(y.mul(b.scalar(dt, 0.3)).tan()).add(y.cos()).add(y.sin().neg())
    return total.sum("n")


def binary_zoo(b, a):
    x, y = a  # x in (0.5, 2), y any sign
    dt = x.ty.dtype
    total = x.div(y.mul(y).add(b.scalar(dt, 1.0))).add(x.pow(b.scalar(dt, 3.0))).add(x.pow(y))
    total = total.add(x.max(y)).add(x.min(y).mul(b.scalar(dt, 2.0))).sub(x.mul(y))
    return total.sum("n")


def extrema_loss(b, a):
    x = a[0]
    return x.max("c").mul(x.min("c")).sum("r").add(x.max(["r", "c"]))


def layout_loss(b, a):
    x, w = a  # x[a,b,c], w[c,a]
    merged = x.merge(["b", "c"], "bc").split("bc", b2=x.ty.dims[1][1], c2=x.ty.dims[2][1])
    mixed = merged.rename("c2", "c").mul(w)  # aligned by name: transposes w
    return mixed.mean(["a", "b2"]).mul(mixed.sum(["a", "b2"])).sum("c")


def mlp_loss(b, a):
    x, w1, w2 = a
    hidden = x.contract(w1, "d").tanh()
    return hidden.contract(w2, "h").mul(x).sum(["token", "d"])


def batched_dot_loss(b, a):
    return a[0].contract(a[1], "k").mul(a[2]).sum(["b", "m", "n"])


def broadcast_op_loss(b, a):
    scale, x = a
    return x.mul(scale.tanh().broadcast_op(**dict(x.ty.dims))).exp().sum("n")


def shared_scalar_loss(b, a):
    scale, x = a
    return x.mul(scale).exp().mean("n").div(scale)


GRAD_CASES = {
    "mismatch": (mismatch, [(), ("point", 16), ("point", 16)], [0, 2]),
    "attention": (attention_loss, [(("token", 5), ("channel", 3))] * 3, [0, 1, 2]),
    "relu_mask": (relu_mask_loss, [(("r", 6), ("c", 7))], [0]),
    "unary_zoo": (unary_zoo, [("n", 33), ("n", 33)], [0, 1]),
    "binary_zoo": (binary_zoo, [("n", 29), ("n", 29)], [1, 0]),
    "extrema": (extrema_loss, [(("r", 5), ("c", 9))], [0]),
    "layout": (layout_loss, [(("a", 3), ("b", 4), ("c", 5)), (("c", 5), ("a", 3))], [0, 1]),
    "mlp": (mlp_loss, [(("token", 6), ("d", 4)), (("d", 4), ("h", 8)), (("h", 8), ("d", 4))], [0, 1, 2]),
    "batched_dot": (batched_dot_loss, [(("b", 2), ("m", 3), ("k", 4)), (("b", 2), ("k", 4), ("n", 5)),
                                       (("b", 2), ("m", 3), ("n", 5))], [0, 1, 2]),
    "shared_scalar": (shared_scalar_loss, [(), ("n", 40)], [0, 1]),
    "broadcast_op": (broadcast_op_loss, [(), ("n", 21)], [0, 1]),
}


def dims_of(shape):
    if shape == ():
        return {}
    if isinstance(shape[0], str):
        return {shape[0]: shape[1]}
    return dict(shape)


def grad_inputs(name, shapes, dtype, seed=0):
    rng = np.random.default_rng(seed + len(name))
    out = []
    for i, shape in enumerate(shapes):
        extents = tuple(dims_of(shape).values())
        if name in ("unary_zoo", "binary_zoo") and i == 0 or name in ("shared_scalar", "broadcast_op") and i == 0:
            v = rng.uniform(0.5, 2.0, extents)
        else:
            v = rng.uniform(-1.5, 1.5, extents)
        out.append(np.asarray(v, dtype))
    return out


def define_case(name, dtype):
    body, shapes, wrt = GRAD_CASES[name]
    specs = [T.spec(dtype, **dims_of(s)) for s in shapes]
    return tensor.define(name, specs, body), shapes, wrt


@pytest.mark.parametrize("name", sorted(GRAD_CASES))
def test_gradient_matches_finite_differences(name):
    program, shapes, wrt = define_case(name, "f64")
    inputs = grad_inputs(name, shapes, np.float64)
    derived = program.value_and_grad(wrt)
    outs = oracle.run(derived.wire, inputs)
    value = scalar(oracle.run(program.wire, inputs)[0])
    assert scalar(outs[0]) == pytest.approx(value, rel=1e-14, abs=1e-300)
    for which, gradient in zip(wrt, outs[1:]):
        assert gradient.size == inputs[which].size and (inputs[which].ndim == 0 or gradient.shape == inputs[which].shape)
        flat = inputs[which].reshape(-1)
        numeric = np.empty(flat.size)
        for i in range(flat.size):
            keep = flat[i]
            h = 1e-6 * max(1.0, abs(keep))
            flat[i] = keep + h
            up = scalar(oracle.run(program.wire, inputs)[0])
            flat[i] = keep - h
            down = scalar(oracle.run(program.wire, inputs)[0])
            flat[i] = keep
            numeric[i] = (up - down) / (2 * h)
        scale = max(np.abs(numeric).max(), 1e-3)
        assert np.max(np.abs(gradient.reshape(-1) - numeric)) < 2e-6 * scale, (name, which)


def test_gradient_tie_conventions():
    """max / min give a tie to the left operand, abs'(0) = +1, every element equal to a reduced
    maximum receives the cotangent (src/tensor/autodiff.zig:766-770,808-815,346-370)."""
    two = [T.spec("f32", n=3), T.spec("f32", n=3)]
    x = np.array([1.0, 2.0, 3.0], np.float32)
    y = np.array([1.0, 5.0, 3.0], np.float32)
    gx, gy = oracle.run(tensor.define("m", two, lambda b, a: a[0].max(a[1]).sum("n")).grad([0, 1]).wire, [x, y])
    assert gx.tolist() == [1, 0, 1] and gy.tolist() == [0, 1, 0]
    gx, gy = oracle.run(tensor.define("m", two, lambda b, a: a[0].min(a[1]).sum("n")).grad([0, 1]).wire, [x, y])
    assert gx.tolist() == [1, 1, 1] and gy.tolist() == [0, 0, 0]
    one = [T.spec("f32", n=4)]
    z = np.array([-2.0, 0.0, 3.0, 3.0], np.float32)
    assert oracle.run(tensor.define("a", one, lambda b, a: a[0].abs().sum("n")).grad([0]).wire, [z])[0].tolist() == [-1, 1, 1, 1]
    assert oracle.run(tensor.define("r", one, lambda b, a: a[0].max("n")).grad([0]).wire, [z])[0].tolist() == [0, 0, 1, 1]


def test_gradient_of_an_unused_parameter_is_zero():
    program = tensor.define("u", [T.spec("f32", n=4), T.spec("f32", m=3)], lambda b, a: a[0].sum("n"))
    g0, g1 = oracle.run(program.grad([0, 1]).wire, [np.arange(4, dtype=np.float32), np.ones(3, np.float32)])
    assert g0.tolist() == [1, 1, 1, 1] and g1.tolist() == [0, 0, 0]


def test_transform_error_names():
    vector = tensor.define("v", [T.spec("f32", n=4)], lambda b, a: a[0].mul(a[0]))
    pair = tensor.define("p", [T.spec("f32", n=4)], lambda b, a: [a[0].sum("n"), a[0].max("n")])
    scalar = tensor.define("s", [T.spec("f32", n=4), T.spec("i32", n=4)], lambda b, a: a[0].sum("n"))
    for program, wrt, name in [(vector, [0], "GradientRequiresScalarOutput"), (pair, [0], "GradientRequiresScalarOutput"),
                               (scalar, [2], "ParameterOutOfRange"), (scalar, [0, 0], "DuplicateParameter"),
                               (scalar, [1], "NonDifferentiableParameter")]:
        with pytest.raises(tensor.TensorError) as info:
            program.grad(wrt)
        assert info.value.name == name
    for kwargs, name in [(dict(axis_size=-1, in_axes=[0, None]), "InvalidDimension"),
                         (dict(axis_size=2, in_axes=[0]), "InAxisCountMismatch"),
                         (dict(axis_size=2, in_axes=[2, None]), "AxisOutOfRange"),
                         (dict(axis_size=2, in_axes=[0, None], out_axis=1), "AxisOutOfRange")]:
        with pytest.raises(tensor.TensorError) as info:
            scalar.vmap(**kwargs)
        assert info.value.name == name


# ---------------------------------------------------------------------------------------------
# jvp (forward mode) against the gradient and against finite differences
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(GRAD_CASES))
def test_jvp_agrees_with_the_gradient(name):
    """For a scalar program the tangent along direction v is the sum over parameters of <grad, v>."""
    program, shapes, wrt = define_case(name, "f64")
    inputs = grad_inputs(name, shapes, np.float64)
    forward = program.jvp(wrt)
    ordered = sorted(wrt)                      # tangent inputs come in parameter order
    assert [repr(t) for t in forward.input_types] == [repr(t) for t in program.input_types] + \
        [repr(program.input_types[i]) for i in ordered]
    assert len(forward.output_types) == 2
    rng = np.random.default_rng(17)
    directions = [rng.uniform(-1.0, 1.0, inputs[i].shape) for i in ordered]
    value, tangent = oracle.run(forward.wire, inputs + directions)
    assert scalar(value) == pytest.approx(scalar(oracle.run(program.wire, inputs)[0]), rel=1e-14)
    gradients = oracle.run(program.grad(ordered).wire, inputs)
    expected = sum(float(np.sum(g.reshape(-1) * d.reshape(-1))) for g, d in zip(gradients, directions))
    scale = sum(float(np.sum(np.abs(g.reshape(-1) * d.reshape(-1)))) for g, d in zip(gradients, directions))
    assert abs(scalar(tangent) - expected) < 1e-11 * max(scale, 1e-3)


def test_jvp_of_a_program_with_several_array_outputs():
    def body(b, a):
        x, w = a
        e = x.sub(x.max("c")).exp()
        return [e.div(e.sum("c")), x.contract(w, "c").tanh(), w.mul(w)]
    specs = [T.spec("f64", r=4, c=6), T.spec("f64", c=6, k=3)]
    program = tensor.define("several", specs, body)
    rng = np.random.default_rng(2)
    x, w = rng.uniform(-1, 1, (4, 6)), rng.uniform(-1, 1, (6, 3))
    dx = rng.uniform(-1, 1, (4, 6))
    forward = program.jvp([0])
    assert len(forward.input_types) == 3 and len(forward.output_types) == 6
    outs = oracle.run(forward.wire, [x, w, dx])
    h = 1e-6
    up = oracle.run(program.wire, [x + h * dx, w])
    down = oracle.run(program.wire, [x - h * dx, w])
    for primal, tangent, u, d, plain in zip(outs[:3], outs[3:], up, down, oracle.run(program.wire, [x, w])):
        np.testing.assert_allclose(primal, plain, rtol=1e-14)
        np.testing.assert_allclose(tangent, (u - d) / (2 * h), rtol=1e-6, atol=1e-8)
    assert not outs[5].any()                  # w*w does not depend on x: its tangent is zeros
    # an integer output has a zero tangent of its own type (autodiff.zig:222-233 emits zeros for compare / iota)
    mask = tensor.define("mask", [T.spec("f64", n=5)], lambda b, a: [a[0].exp(), b.iota("i32", [("n", 5)], "n")])
    primal, count, tangent, none = oracle.run(mask.jvp([0]).wire, [np.zeros(5), np.ones(5)])
    assert tangent.tolist() == [1, 1, 1, 1, 1] and none.dtype == np.int32 and not none.any() and count.tolist() == [0, 1, 2, 3, 4]
    with pytest.raises(tensor.TensorError) as info:
        program.jvp([2])
    assert info.value.name == "ParameterOutOfRange"


def test_transformations_compose():
    """Derived programs are ordinary programs: the gradient of a gradient, the jvp of a gradient
    (a Hessian-vector product) and the vmap of that."""
    one = tensor.define("mismatch", [T.spec("f64"), T.spec("f64", point=16), T.spec("f64", point=16)], mismatch)
    time = 0.25 * np.arange(16)
    sample = np.sin(3.0 * time)
    first = one.grad([0])
    slope = lambda f: scalar(oracle.run(first.wire, [np.float64(f), time, sample])[0])  # noqa: E731
    curvature = scalar(oracle.run(first.grad([0]).wire, [np.float64(2.5), time, sample])[0])
    assert curvature == pytest.approx((slope(2.5 + 1e-6) - slope(2.5 - 1e-6)) / 2e-6, rel=1e-7)
    product = first.jvp([0])
    got = oracle.run(product.wire, [np.float64(2.5), time, sample, np.float64(-2.0)])
    assert scalar(got[0]) == pytest.approx(slope(2.5), rel=1e-14)
    assert scalar(got[1]) == pytest.approx(-2.0 * curvature, rel=1e-13)
    guesses = np.array([2.0, 2.5, 3.0, 3.5])
    slopes, products = oracle.run(product.vmap(4, [0, None, None, 0]).wire, [guesses, time, sample, np.ones(4)])
    np.testing.assert_allclose(slopes, [slope(f) for f in guesses], rtol=1e-13, atol=1e-12)
    assert products[1] == pytest.approx(curvature, rel=1e-13)


# ---------------------------------------------------------------------------------------------
# vmap against one run per index
# ---------------------------------------------------------------------------------------------
def row_softmax(b, a):
    x = a[0]
    e = x.sub(x.max("c")).exp()
    return e.div(e.sum("c"))


VMAP_CASES = {
    # body, per-instance shapes, in_axes, out_axis
    "mismatch_over_guesses": (mismatch, [(), ("point", 16), ("point", 16)], [0, None, None], 0),
    "softmax_rows_axis_last": (row_softmax, [("c", 12)], [1], 1),
    "softmax_matrix_axis_middle": (row_softmax, [(("r", 3), ("c", 12))], [1], 2),
    "dot_lhs_only": (lambda b, a: a[0].contract(a[1], "k"), [(("m", 3), ("k", 4)), (("k", 4), ("n", 5))], [0, None], 0),
    "dot_rhs_only": (lambda b, a: a[0].contract(a[1], "k"), [(("m", 3), ("k", 4)), (("k", 4), ("n", 5))], [None, 2], 1),
    "dot_both": (lambda b, a: a[0].contract(a[1], "k"), [(("m", 3), ("k", 4)), (("k", 4), ("n", 5))], [1, 0], 2),
    "batched_dot_rhs_only": (lambda b, a: a[0].contract(a[1], "k"),
                             [(("b", 2), ("m", 3), ("k", 4)), (("b", 2), ("k", 4), ("n", 5))], [None, 1], 0),
    "unmapped_output": (lambda b, a: [a[0].mul(a[1]), a[1].exp()], [("n", 6), ("n", 6)], [0, None], 1),
    "select_and_transpose": (relu_mask_loss, [(("r", 6), ("c", 7))], [2], 0),
    "layout_vmapped": (layout_loss, [(("a", 3), ("b", 4), ("c", 5)), (("c", 5), ("a", 3))], [3, 0], 0),
    "broadcast_op_mapped_scalar": (broadcast_op_loss, [(), ("n", 21)], [0, None], 0),
    "attention_gradient": (None, [(("token", 5), ("channel", 3))] * 3, [0, 0, None], 0),
}
VMAP_EXTENT = 4


def define_vmap_case(name, dtype):
    body, shapes, in_axes, out_axis = VMAP_CASES[name]
    specs = [T.spec(dtype, **dims_of(s)) for s in shapes]
    if body is None:
        single = tensor.define(name, specs, attention_loss).value_and_grad([0, 2])
    else:
        single = tensor.define(name, specs, body)
    return single, single.vmap(VMAP_EXTENT, in_axes, out_axis=out_axis, axis_name="instance"), shapes, in_axes, out_axis


def vmap_inputs(name, shapes, in_axes, dtype):
    rng = np.random.default_rng(len(name))
    stacked = []
    for shape, axis in zip(shapes, in_axes):
        extents = list(dims_of(shape).values())
        if axis is not None:
            extents.insert(axis, VMAP_EXTENT)
        stacked.append(np.asarray(rng.uniform(-1.5, 1.5, tuple(extents)), dtype))
    return stacked


def per_index_outputs(single, stacked, in_axes, out_axis, mode="ref"):
    rows = []
    for i in range(VMAP_EXTENT):
        inputs = [x if axis is None else np.ascontiguousarray(np.take(x, i, axis=axis)) for x, axis in zip(stacked, in_axes)]
        rows.append(oracle.run(single.wire, inputs, mode=mode))
    return [np.stack([row[o] for row in rows], axis=out_axis) for o in range(len(rows[0]))]


@pytest.mark.parametrize("name", sorted(VMAP_CASES))
def test_vmap_equals_one_run_per_index(name):
    single, mapped, shapes, in_axes, out_axis = define_vmap_case(name, "f64")
    stacked = vmap_inputs(name, shapes, in_axes, np.float64)
    got = oracle.run(mapped.wire, stacked)
    want = per_index_outputs(single, stacked, in_axes, out_axis)
    assert len(got) == len(want) == len(mapped.output_types)
    for g, w, ty in zip(got, want, mapped.output_types):
        assert g.shape == w.shape == tuple(e for _, e in ty.dims)
        assert ty.dims[out_axis] == ("instance", VMAP_EXTENT)
        np.testing.assert_allclose(g, w, rtol=1e-12, atol=1e-13)


def test_vmap_default_axis_name():
    single = tensor.define("d", [T.spec("f32", n=4)], lambda b, a: a[0].neg())
    mapped = single.vmap(3, [0])
    assert repr(mapped.input_types[0]) == "f32[#batch=3, n=4]"
    assert "#batch=3" in oracle.describe(mapped.wire)
    again = mapped.vmap(2, [0])
    assert repr(again.input_types[0]) == "f32[#batch1=2, #batch=3, n=4]"
    assert "#batch1=2" in oracle.describe(again.wire)


# ---------------------------------------------------------------------------------------------
# the derived programs on the CUDA target
# ---------------------------------------------------------------------------------------------
JVP_DEVICE_CASES = ["jvp_attention", "jvp_mlp", "jvp_binary_zoo", "jvp_extrema"]
DEVICE_CASES = sorted(GRAD_CASES) + sorted(VMAP_CASES) + JVP_DEVICE_CASES


def derived_case(name):
    if name.startswith("jvp_"):
        program, shapes, wrt = define_case(name[4:], "f32")
        inputs = grad_inputs(name[4:], shapes, np.float32)
        rng = np.random.default_rng(23)
        directions = [rng.uniform(-1.0, 1.0, inputs[i].shape).astype(np.float32) for i in sorted(wrt)]
        return program.jvp(wrt), inputs + directions
    if name in GRAD_CASES:
        program, shapes, wrt = define_case(name, "f32")
        return program.value_and_grad(wrt), grad_inputs(name, shapes, np.float32)
    _, mapped, shapes, in_axes, _ = define_vmap_case(name, "f32")
    return mapped, vmap_inputs(name, shapes, in_axes, np.float32)


@pytest.mark.parametrize("name", DEVICE_CASES)
def test_derived_programs_compile_for_sm100a(cpu_session, name):
    program, _ = derived_case(name)
    compiled = cpu_session.compile(program)
    assert compiled.work()["launches"] >= 1
    cpu_session.release(compiled)


def test_large_refine_program_is_one_fused_pass(cpu_session):
    """value and slope for 8192 guesses x 65536 points: the [guess, point] intermediates are never
    materialised (each output is a fused reduction over the region)."""
    program = one_guess_program(65536).value_and_grad([0]).vmap(8192, [0, None, None], axis_name="guess")
    compiled = cpu_session.compile(program)
    work = compiled.work()
    assert work["launches"] == 1 and work["pairs"] == 8192 * 65536
    assert work["bytes"] == 4 * (8192 + 2 * 65536 + 2 * 8192)  # inputs and the two outputs, nothing else
    assert "reduces=2" in compiled.plan_summary()
    cpu_session.release(compiled)


@pytest.mark.gpu
@pytest.mark.parametrize("name", DEVICE_CASES)
def test_derived_programs_match_oracle(gpu_session, name):
    program, inputs = derived_case(name)
    compiled = gpu_session.compile(program)
    outs = [np.empty(d.byte_size, np.uint8) for d in compiled.output_descriptors()]
    gpu_session.invoke(compiled, inputs, outs)
    gpu_session.release(compiled)
    expected = oracle.run(program.wire, inputs, mode="ref")
    exact = oracle.run(program.wire, inputs, mode="f64")
    for got_raw, want, ex in zip(outs, expected, exact):
        got = got_raw.view(np.float32).astype(np.float64)
        want64 = want.reshape(-1).astype(np.float64)
        ex64 = np.asarray(ex, np.float64).reshape(-1)
        floor = max(np.abs(ex64).max() * 1e-3, 1e-30)
        err_gpu = np.max(np.abs(got - ex64) / np.maximum(np.abs(ex64), floor))
        err_ref = np.max(np.abs(want64 - ex64) / np.maximum(np.abs(ex64), floor))
        assert err_gpu < 1e-5 + err_ref, (name, err_gpu, err_ref)


@pytest.mark.gpu
def test_large_refine_program_on_the_device(gpu_session):
    guesses, points = 512, 65536
    program = one_guess_program(points).value_and_grad([0]).vmap(guesses, [0, None, None], axis_name="guess")
    rng = np.random.default_rng(5)
    frequency = rng.uniform(0.0, 6.0, guesses).astype(np.float32)
    time = (0.25 * np.arange(points)).astype(np.float32)
    sample = (np.sin(3.0 * time.astype(np.float64)) + rng.normal(0.0, 0.01, points)).astype(np.float32)
    compiled = gpu_session.compile(program)
    value, slope = np.empty(guesses, np.float32), np.empty(guesses, np.float32)
    gpu_session.invoke(compiled, [frequency, time, sample], [value, slope])
    gpu_session.release(compiled)
    phase = frequency.astype(np.float64)[:, None] * time.astype(np.float64)[None, :]
    phase = (frequency[:, None] * time[None, :]).astype(np.float64)  # the f32 product, as recorded
    gap = np.sin(phase) - sample.astype(np.float64)
    want_value = (gap * gap).sum(axis=1)
    want_slope = (2.0 * gap * np.cos(phase) * time.astype(np.float64)).sum(axis=1)
    assert np.max(np.abs(value - want_value) / want_value) < 1e-5
    # the slope is a cancelling sum of terms of size |time| * |gap|: compare on that scale
    scale = (2.0 * np.abs(gap * np.cos(phase)) * time.astype(np.float64)).sum(axis=1)
    assert np.max(np.abs(slope - want_slope) / scale) < 1e-5


@pytest.mark.gpu
def test_bf16_mlp_gradient_runs_on_tensor_cores(gpu_session):
    """Every contraction of the gradient program (x^T g, g W^T, ...) stays on tcgen05: transposed
    operands are read through strides (K-major or MN-major tiles), not copied."""
    from accy_b200 import configs
    specs = [T.spec("bf16", token=384, d=128), T.spec("bf16", d=128, h=256), T.spec("bf16", h=256, d=128)]
    program = tensor.define("mlp_loss", specs, mlp_loss).grad([0, 1, 2])
    rng = np.random.default_rng(21)
    inputs = [configs.f32_to_bf16_bits((rng.standard_normal([e for _, e in sp.dims]) * scale).astype(np.float32))
              for sp, scale in zip(specs, (1.0, 0.1, 0.1))]
    compiled = gpu_session.compile(program)
    summary = compiled.plan_summary()
    assert summary.count("tcgen05") >= 5 and " simt" not in summary, summary
    outs = [np.empty(d.byte_size, np.uint8) for d in compiled.output_descriptors()]
    gpu_session.invoke(compiled, inputs, outs)
    gpu_session.release(compiled)
    for got_raw, want in zip(outs, oracle.run(program.wire, inputs, mode="wide")):
        got = configs.bf16_bits_to_f32(got_raw.view(np.uint16)).astype(np.float64)
        want64 = configs.bf16_bits_to_f32(want).reshape(-1).astype(np.float64)
        rms = np.sqrt(np.mean(want64 ** 2))
        assert np.max(np.abs(got - want64) / (np.abs(want64) + rms)) < 2e-2
