"""Programs beyond the five benchmark configurations: other reductions, multi-output programs,
plain elementwise programs, masks, transposed and reshaped operands, integer and f64 values.
Each is compiled on CPU (plan + NVRTC) and, on a GPU, run through the C ABI and compared with the
oracle.  f32 tolerance 1e-5 relative (floor: 1e-6 of the largest magnitude, 1e-3 where values cancel)."""
import numpy as np
import pytest

from accy_b200 import tensor
from oracle import oracle
from parity_checks import check_three_distances

T = tensor


def value_and_slope(b, a):
    """mismatch and its derivative w.r.t. frequency: two reductions over one fused region"""
    frequency, time, sample = a
    phase = frequency.mul(time)
    gap = phase.sin().sub(sample)
    value = gap.mul(gap).sum("point")
    slope = gap.mul(phase.cos()).mul(time).mul(b.scalar("f32", 2.0)).sum("point")
    return [value, slope]


def sine_and_cosine(x):
    return [x.sin(), x.cos()]


def masked_fill(b, a):
    x = a[0]
    dims = x.ty.dims
    keep = b.iota("i32", dims, "r").compare("ge", b.iota("i32", dims, "c"))
    return keep.select(x, b.scalar("f32", -1.0))


CASES = {
    "sum_to_scalar": ([T.spec("f32", n=100003)], lambda b, a: a[0].sum("n")),
    "sum_over_leading_axis": ([T.spec("f32", a=300, b=200)], lambda b, a: a[0].sum("a")),
    "max_over_two_axes": ([T.spec("f32", a=7, b=33, c=65)], lambda b, a: a[0].max(["b", "c"])),
    "min_of_interior_axis": ([T.spec("f32", a=5, b=40, c=24)], lambda b, a: a[0].min("b")),
    "value_and_slope": ([T.spec("f32", guess=24), T.spec("f32", point=4096), T.spec("f32", point=4096)], value_and_slope),
    "outer_elementwise": ([T.spec("f32", n=257), T.spec("f32", m=129), T.spec("f32", n=257, m=129)],
                          lambda b, a: a[0].mul(a[1]).add(a[2]).tanh()),
    "flat_elementwise": ([T.spec("f32", n=1 << 20)], lambda b, a: a[0].mul(a[0]).add(b.scalar("f32", 1.0)).sqrt().log()),
    "lower_triangle_mask": ([T.spec("f32", r=96, c=96)], masked_fill),
    "transposed_operand": ([T.spec("f32", a=64, b=48), T.spec("f32", b=48, a=64)], lambda b, a: a[0].add(a[1])),
    "merge_then_reduce": ([T.spec("f32", a=6, b=10, c=50)], lambda b, a: a[0].merge(["b", "c"], "bc").exp().sum("bc")),
    "split_axis": ([T.spec("f32", n=600)], lambda b, a: a[0].split("n", p=20, q=30).sum("q")),
    "int_arithmetic": ([T.spec("i32", n=1000), T.spec("i32", n=1000)], lambda b, a: a[0].mul(a[1]).sub(a[0]).max(a[1])),
    "double_precision": ([T.spec("f64", r=40, c=300)], lambda b, a: a[0].sub(a[0].mean("c")).abs().sum("c")),
    "bf16_rowsum": ([T.spec("bf16", r=128, c=512)], lambda b, a: a[0].mul(a[0]).sum("c")),
    "scalar_program": ([T.spec("f32"), T.spec("f32")], lambda b, a: a[0].div(a[1]).cos()),
    "passthrough_and_duplicate": ([T.spec("f32", n=100)], lambda b, a: [a[0], a[0].neg(), a[0]]),
    # the `broadcast` operation (Builder.broadcastOp): a rank-0 value repeated to the dims
    "broadcast_op": ([T.spec("f32"), T.spec("f32", r=40, c=50)],
                     lambda b, a: a[1].mul(a[0].exp().broadcast_op(r=40, c=50)).sum("c")),
    # a sine and a cosine of the same value: the joint routine, both results stored
    "sine_and_cosine": ([T.spec("f32", n=4096)], lambda b, a: sine_and_cosine(a[0].mul(b.scalar("f32", 40.0)))),
    "two_stage_reduce": ([T.spec("f32", a=50, b=70)], lambda b, a: a[0].sum("b").max("a")),
    # Value.reduce with a recorded start value that is not the reducer's own (Builder.reduceWith): the
    # reference folds it in once per result (reduction.zig:839-863), whatever the thread count
    "sum_from_five": ([T.spec("f32", r=64, c=1024)], lambda b, a: a[0].reduce(b.scalar("f32", 5.0), "sum", "c")),
    "sum_from_five_in_column_splits": ([T.spec("f32", r=3, c=1 << 18)],
                                       lambda b, a: a[0].reduce(b.scalar("f32", 5.0), "sum", "c")),
    "max_from_one_and_min_from_zero": ([T.spec("f32", r=40, c=300)],
                                       lambda b, a: [a[0].mul(b.scalar("f32", 0.25)).reduce(b.scalar("f32", 1.0), "max", "c"),
                                                     a[0].reduce(b.scalar("f32", 0.0), "min", "c")]),
    "int_sum_from_seven": ([T.spec("i32", r=9, c=1000)], lambda b, a: a[0].reduce(b.scalar("i32", 7), "sum", "c")),
    "row_pipeline_with_start_values": ([T.spec("f32", r=32, c=512)],
                                       lambda b, a: a[0].sub(a[0].reduce(b.scalar("f32", 0.5), "max", "c")).exp()
                                       .div(a[0].exp().reduce(b.scalar("f32", 3.0), "sum", "c"))),
    "softmax_then_colsum": ([T.spec("f32", r=64, c=128)],
                            lambda b, a: a[0].sub(a[0].max("c")).exp().div(a[0].sub(a[0].max("c")).exp().sum("c")).sum("r")),
}


def make_inputs(specs, seed):
    rng = np.random.default_rng(seed)
    out = []
    for s in specs:
        shape = tuple(e for _, e in s.dims)
        if s.dtype == "f32":
            out.append(rng.uniform(-2.0, 2.0, shape).astype(np.float32))
        elif s.dtype == "f64":
            out.append(rng.uniform(-2.0, 2.0, shape))
        elif s.dtype == "i32":
            out.append(rng.integers(-1000, 1000, shape, dtype=np.int32))
        elif s.dtype == "bf16":
            w = rng.uniform(-2.0, 2.0, shape).astype(np.float32).view(np.uint32)
            out.append((w >> 16).astype(np.uint16))
    return out


@pytest.mark.parametrize("name", sorted(CASES))
def test_compiles_for_sm100a(cpu_session, name):
    specs, body = CASES[name]
    program = tensor.define(name, specs, body)
    compiled = cpu_session.compile(program)
    assert compiled.work()["launches"] >= 1
    assert oracle.describe(program.wire)
    cpu_session.release(compiled)


def test_recorded_start_value_is_folded_once_per_row(cpu_session):
    """Per-thread accumulators start from the reducer's identity; the recorded 5.0 (0x40a00000)
    appears in one fold behind the tree, and with column splits only in the combine kernel."""
    for name in ("sum_from_five", "sum_from_five_in_column_splits"):
        specs, body = CASES[name]
        compiled = cpu_session.compile(tensor.define(name, specs, body))
        sources = {n: src for n, src, _ in compiled.kernels()}
        cpu_session.release(compiled)
        main = [src for n, src in sources.items() if not n.endswith("_combine")]
        combine = [src for n, src in sources.items() if n.endswith("_combine")]
        assert len(main) == 1
        assert "acc_" in main[0] and " = __uint_as_float(0x0u);" in main[0]
        assert "= __uint_as_float(0x40a00000u);" not in main[0]
        holder = combine[0] if combine else main[0]
        assert holder.count("0x40a00000u") == 1 and "fold<0, float>(__uint_as_float(0x40a00000u)," in holder
        if combine:
            assert "0x40a00000u" not in main[0]


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_matches_oracle(gpu_session, name):
    specs, body = CASES[name]
    program = tensor.define(name, specs, body)
    inputs = make_inputs(specs, seed=len(name))
    if name == "scalar_program":
        inputs = [np.array(1.5, np.float32), np.array(0.7, np.float32)]
    compiled = gpu_session.compile(program)
    outs = [np.empty(d.byte_size, np.uint8) for d in compiled.output_descriptors()]
    gpu_session.invoke(compiled, inputs, outs)
    gpu_session.release(compiled)
    mode = "wide" if any(s.dtype == "bf16" for s in specs) else "ref"
    expected = oracle.run(program.wire, inputs, mode=mode)
    exact = oracle.run(program.wire, inputs, mode="f64")
    for got_raw, want, ex, ty in zip(outs, expected, exact, program.output_types):
        if ty.dtype == "i32":
            assert np.array_equal(got_raw.view(np.int32), want.reshape(-1))
            continue
        if ty.dtype == "bf16":
            got = (got_raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
            want64 = (want.reshape(-1).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
            assert np.max(np.abs(got - want64) / (np.abs(want64) + np.sqrt(np.mean(want64 ** 2)))) < 2e-2
            continue
        got = got_raw.view(np.float64 if ty.dtype == "f64" else np.float32).astype(np.float64)
        want64 = want.reshape(-1).astype(np.float64)
        ex64 = np.asarray(ex, np.float64).reshape(-1)
        floor_frac = 1e-3 if name in ("value_and_slope", "softmax_then_colsum", "row_pipeline_with_start_values") else 1e-6
        check_three_distances(name, got, want64, ex64, floor_frac, tol=1e-12 if ty.dtype == "f64" else 1e-5)


# Zero-extent axes: the reference's type rules allow them (only negative extents are refused);
# a fold over an empty axis gives the init value, a contraction over an empty axis gives zeros.
EMPTY_CASES = {
    "empty_elementwise": ([T.spec("f32", n=0)], lambda b, a: a[0].mul(a[0])),
    "sum_over_empty_axis": ([T.spec("f32", r=4, c=0)], lambda b, a: a[0].sum("c")),
    "max_over_empty_axis": ([T.spec("f32", r=4, c=0)], lambda b, a: a[0].max("c")),
    "mean_then_arithmetic": ([T.spec("f32", r=3, c=0), T.spec("f32", r=3)], lambda b, a: a[0].sum("c").add(a[1]).exp()),
    "empty_rows": ([T.spec("f32", r=0, c=8)], lambda b, a: a[0].sum("c")),
    "empty_contraction": ([T.spec("f32", m=3, k=0), T.spec("f32", k=0, n=2)], lambda b, a: a[0].contract(a[1], "k")),
    "empty_and_full_outputs": ([T.spec("f32", n=0), T.spec("f32", m=5)], lambda b, a: [a[0].neg(), a[1].mul(a[1])]),
}


@pytest.mark.parametrize("name", sorted(EMPTY_CASES))
def test_zero_extent_programs_compile(cpu_session, name):
    specs, body = EMPTY_CASES[name]
    compiled = cpu_session.compile(tensor.define(name, specs, body))
    sizes = [d.byte_size for d in compiled.output_descriptors()]
    assert compiled.work()["launches"] == (0 if not any(sizes) else compiled.work()["launches"])
    cpu_session.release(compiled)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(EMPTY_CASES))
def test_zero_extent_programs_match_oracle(gpu_session, name):
    specs, body = EMPTY_CASES[name]
    program = tensor.define(name, specs, body)
    inputs = make_inputs(specs, seed=7)
    compiled = gpu_session.compile(program)
    outs = [np.full(d.byte_size, 0xAB, np.uint8) for d in compiled.output_descriptors()]
    gpu_session.invoke(compiled, inputs, outs)
    gpu_session.release(compiled)
    expected = oracle.run(program.wire, inputs, mode="ref")
    for got, want in zip(outs, expected):
        assert np.array_equal(got.view(np.float32), np.asarray(want, np.float32).reshape(-1))


def random_sum_program(seed):
    """A seeded random f32 program over [r, c] with sums, means, maxima and softmax-like groups over c,
    over r or over both, broadcast back by name: (specs, body, inputs).  All values stay positive, so
    no sum cancels and a relative tolerance means something for every element."""
    rng = np.random.default_rng(9000 + seed)
    r = int(rng.choice([1, 4, 48, 300]))
    c = int(rng.choice([1, 9, 256, 1000, 6000]))
    kinds = ["full", "full", str(rng.choice(["row", "col"]))]
    specs, inputs = [], []
    for kind in kinds:
        shape = {"full": (r, c), "row": (r,), "col": (c,)}[kind]
        specs.append(T.spec("f32", **({"r": r, "c": c} if kind == "full" else ({"r": r} if kind == "row" else {"c": c}))))
        inputs.append(rng.uniform(0.25, 2.0, shape).astype(np.float32))
    dims_of = [{"full": ("r", "c"), "row": ("r",), "col": ("c",)}[k] for k in kinds]
    steps = []
    for _ in range(int(rng.integers(4, 9))):
        op = str(rng.choice(["add", "mul", "div", "max", "min", "sqrt", "scale", "reduce", "reduce", "softmax"]))
        picks = [int(p) for p in rng.integers(0, len(dims_of), 2)]
        how = (str(rng.choice(["sum", "mean", "max"])), str(rng.choice(["c", "r", "rc"])), float(np.float32(rng.uniform(0.25, 1.5))))
        if op in ("reduce", "softmax"):
            have = dims_of[picks[0]]
            axes = tuple(a for a in how[1] if a in have)
            if not axes:
                op = "sqrt"
                dims_of.append(have)
            else:
                how = (how[0], axes, how[2])
                dims_of.append(have if op == "softmax" else tuple(a for a in have if a not in axes))
        elif op in ("sqrt", "scale"):
            dims_of.append(dims_of[picks[0]])
        else:
            dims_of.append(tuple(a for a in ("r", "c") if a in dims_of[picks[0]] or a in dims_of[picks[1]]))
        steps.append((op, picks, how))

    def body(b, a):
        values = list(a)
        for op, p, how in steps:
            x, y = values[p[0]], values[p[1]]
            if op in ("add", "mul", "div", "max", "min"):
                v = getattr(x, op)(y)
            elif op == "sqrt":
                v = x.sqrt()
            elif op == "scale":
                v = x.mul(b.scalar("f32", how[2]))
            elif op == "reduce":
                v = getattr(x, how[0])(list(how[1]))
            else:   # exp(x - max) / sum(exp(x - max)) over the axes, shifted so that it stays positive
                e = x.sub(x.max(list(how[1]))).exp()
                v = e.div(e.sum(list(how[1]))).add(b.scalar("f32", 0.125))
            values.append(v)
        out = values[-1]
        for v in a:
            out = out.add(v)
        return out

    return specs, body, inputs


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(20))
def test_random_programs_with_sums_match_oracle(gpu_session, seed):
    specs, body, inputs = random_sum_program(seed)
    program = tensor.define("random_sums_%d" % seed, specs, body)
    compiled = gpu_session.compile(program)
    out = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    gpu_session.invoke(compiled, inputs, [out])
    gpu_session.release(compiled)
    ref = np.asarray(oracle.run(program.wire, inputs, mode="ref")[0], np.float64).reshape(-1)
    exact = np.asarray(oracle.run(program.wire, inputs, mode="f64")[0], np.float64).reshape(-1)
    assert np.isfinite(exact).all()
    check_three_distances("random_sums_%d" % seed, out.view(np.float32).astype(np.float64), ref, exact, 1e-6)


def test_schedules_of_folds_over_a_leading_axis_and_of_flat_programs(cpu_session):
    """A fold over a leading axis of a row-major buffer runs with one thread per kept column (256
    neighbouring columns per CTA, the folded axis cut into slices); an elementwise-only flat program gets
    one chunk per CTA; the many partials of a one-row fold are combined by a warp."""
    def plan(name, specs, body):
        compiled = cpu_session.compile(tensor.define(name, specs, body))
        summary, kernels = compiled.plan_summary(), {n: src for n, src, _ in compiled.kernels()}
        cpu_session.release(compiled)
        return summary, kernels
    summary, _ = plan("column_sums", [T.spec("f32", r=16384, c=4096)], lambda b, a: a[0].sum("r"))
    assert "rows=4096 cols=16384" in summary and "tpr=1 rpc=256" in summary and "splits=64" in summary
    summary, _ = plan("interior_sums", [T.spec("f32", a=256, b=256, c=1024)], lambda b, a: a[0].sum("b"))
    assert "tpr=1 rpc=256" in summary
    # the same fold over the trailing axis keeps 256 threads on a row
    summary, _ = plan("row_sums", [T.spec("f32", r=16384, c=4096)], lambda b, a: a[0].sum("c"))
    assert "tpr=256" in summary and "splits=1 " in summary
    summary, _ = plan("flat", [T.spec("f32", n=1 << 26)] * 3, lambda b, a: a[0].mul(a[1]).add(a[2]))
    assert "chunks=16384 splits=16384" in summary
    summary, kernels = plan("total", [T.spec("f32", n=1 << 26)], lambda b, a: a[0].mul(a[0]).sum("n"))
    assert "splits=863" in summary
    combine = [src for n, src in kernels.items() if n.endswith("_combine")]
    assert len(combine) == 1 and "__shfl_xor_sync" in combine[0].split("extern \"C\"")[-1]
    # few partials per row: one thread per row folds them in order
    _, kernels = plan("few_partials", [T.spec("f32", r=16, c=1 << 16)], lambda b, a: a[0].sum("c"))
    combine = [src for n, src in kernels.items() if n.endswith("_combine")]
    assert len(combine) == 1 and "__shfl_xor_sync" not in combine[0].split("extern \"C\"")[-1]


def test_a_fold_over_a_leading_axis_that_is_used_further_gets_its_own_kernel(cpu_session):
    """Centring over axis 0: the column means come from a kernel of their own (one thread per column)
    and the subtraction runs along the rows; the same program over axis 1 stays one fused row kernel;
    two column folds that are both outputs still share one pass over the input."""
    def kernels_of(name, specs, body):
        compiled = cpu_session.compile(tensor.define(name, specs, body))
        lines = [l.strip() for l in compiled.plan_summary().strip().split("\n") if l.strip().startswith("row kernel")]
        cpu_session.release(compiled)
        return lines
    lines = kernels_of("centre_columns", [T.spec("f32", r=8192, c=8192)], lambda b, a: a[0].sub(a[0].mean("r")))
    assert len(lines) == 2 and "reduces=1 tpr=1 rpc=256" in lines[0] and "reduces=0 tpr=256" in lines[1] and "vec=4" in lines[1]
    lines = kernels_of("centre_rows", [T.spec("f32", r=8192, c=8192)], lambda b, a: a[0].sub(a[0].mean("c")))
    assert len(lines) == 1 and "reduces=1 tpr=256" in lines[0]
    lines = kernels_of("two_column_folds", [T.spec("f32", r=8192, c=8192)], lambda b, a: [a[0].sum("r"), a[0].mul(a[0]).sum("r")])
    assert len(lines) == 1 and "reduces=2 tpr=1 rpc=256" in lines[0] and "outputs=2" in lines[0]


def test_a_value_recorded_twice_is_computed_once(cpu_session):
    """x.max(r) written out for two uses is one fold kernel, and a contraction recorded twice is one GEMM."""
    def kernels_of(name, specs, body):
        compiled = cpu_session.compile(tensor.define(name, specs, body))
        lines = [l.strip() for l in compiled.plan_summary().strip().split("\n") if l.strip().startswith(("row kernel", "gemm"))]
        cpu_session.release(compiled)
        return lines
    lines = kernels_of("softmax_over_axis_0", [T.spec("f32", r=4096, c=4096)],
                       lambda b, a: a[0].sub(a[0].max("r")).exp().div(a[0].sub(a[0].max("r")).exp().sum("r")))
    assert len(lines) == 3 and sum("reduces=1" in l for l in lines) == 2
    lines = kernels_of("same_product_twice", [T.spec("bf16", m=256, k=256), T.spec("bf16", k=256, n=256)],
                       lambda b, a: a[0].contract(a[1], "k").add(a[0].contract(a[1], "k")))
    assert sum(l.startswith("gemm") for l in lines) == 1


def test_a_fold_over_rows_and_columns_joins_the_row_kernel_of_its_operand(cpu_session):
    """The sum over both axes at the end of a layer-norm loss is taken along the rows first: the row means,
    the row variances and the rows' shares of the loss come out of one kernel that reads the inputs once;
    a second, small kernel adds up the 8192 shares."""
    def loss(b, a):
        x, gain, target = a
        centred = x.sub(x.mean("c"))
        y = centred.div(centred.mul(centred).mean("c").add(b.scalar("f32", 1e-5)).sqrt()).mul(gain)
        d = y.sub(target)
        return d.mul(d).sum(["r", "c"])
    specs = [T.spec("f32", r=8192, c=4096), T.spec("f32", c=4096), T.spec("f32", r=8192, c=4096)]
    compiled = cpu_session.compile(tensor.define("layer_norm_loss", specs, loss))
    lines = [l.strip() for l in compiled.plan_summary().strip().split("\n") if l.strip().startswith("row kernel")]
    cpu_session.release(compiled)
    assert len(lines) == 2
    assert "rows=8192 cols=4096 reduces=3" in lines[0] and "rows=1 cols=8192 reduces=1" in lines[1]
    # innermost extents below 64 are folded as recorded
    compiled = cpu_session.compile(tensor.define("narrow", [T.spec("f32", r=4096, c=8)], lambda b, a: a[0].sum(["r", "c"])))
    lines = [l.strip() for l in compiled.plan_summary().strip().split("\n") if l.strip().startswith("row kernel")]
    cpu_session.release(compiled)
    assert len(lines) == 1 and "cols=32768" in lines[0]


def test_row_statistics_needed_elsewhere_leave_the_kernel_that_computes_them_anyway(cpu_session):
    """value_and_grad of the layer-norm loss: the gradient with respect to x needs the row means and
    variances; the gradient of the gain, a fold over the rows, needs them too.  They are written by the first
    kernel instead of being computed again from x by kernels of their own, and the rows' shares of the
    value (a fold over the same columns of an operand with the same dims) join that kernel too."""
    def loss(b, a):
        x, gain, target = a
        centred = x.sub(x.mean("c"))
        y = centred.div(centred.mul(centred).mean("c").add(b.scalar("f32", 1e-5)).sqrt()).mul(gain)
        d = y.sub(target)
        return d.mul(d).sum(["r", "c"])
    specs = [T.spec("f32", r=8192, c=4096), T.spec("f32", c=4096), T.spec("f32", r=8192, c=4096)]
    compiled = cpu_session.compile(tensor.define("layer_norm_loss", specs, loss).value_and_grad([0, 1]))
    lines = [l.strip() for l in compiled.plan_summary().strip().split("\n") if l.strip().startswith("row kernel")]
    cpu_session.release(compiled)
    # the rows' shares of the value join the same kernel: x and the target are read by two kernels, not five
    assert len(lines) == 3
    assert "rows=8192 cols=4096" in lines[0] and "reduces=5" in lines[0] and "outputs=4" in lines[0]
    assert "rows=4096 cols=8192" in lines[1] and "tpr=1 rpc=256" in lines[1]
    assert "rows=1 cols=8192" in lines[2]


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(12))
def test_random_gradient_and_multi_output_programs_match_oracle(gpu_session, seed):
    """The random programs above once more, as a scalar loss under value_and_grad (three outputs: the value
    and the gradients with respect to both full-shaped inputs) and as a program with up to four outputs of
    different shapes (the result, its square, its row sums, its column maxima): every output against the
    reference-order and the f64 evaluation of the very same derived program."""
    specs, body, inputs = random_sum_program(400 + seed)

    def loss(b, a):
        out = body(b, a)
        return out.sum([name for name, _ in out.ty.dims])

    def several(b, a):
        out = body(b, a)
        names = [name for name, _ in out.ty.dims]
        outs = [out, out.mul(out)]
        if "c" in names:
            outs.append(out.sum("c"))
        if "r" in names:
            outs.append(out.max("r"))
        return outs

    programs = [tensor.define("random_loss_%d" % seed, specs, loss).value_and_grad([0, 1]),
                tensor.define("random_outputs_%d" % seed, specs, several)]
    for program in programs:
        compiled = gpu_session.compile(program)
        outs = [np.empty(d.byte_size, np.uint8) for d in compiled.output_descriptors()]
        gpu_session.invoke(compiled, inputs, outs)
        gpu_session.release(compiled)
        ref = oracle.run(program.wire, inputs, mode="ref")
        exact = oracle.run(program.wire, inputs, mode="f64")
        for j, (got, want, ex) in enumerate(zip(outs, ref, exact)):
            check_three_distances("%s output %d" % (program.name, j),
                                  got.view(np.float32).astype(np.float64), np.asarray(want, np.float64).reshape(-1),
                                  np.asarray(ex, np.float64).reshape(-1), 1e-4)
