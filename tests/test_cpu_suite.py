"""CPU-side tests: recording rules, ACTP wire bytes, oracle known answers, fusion plans, kernel
compilation for sm_100a (NVRTC, no device needed), C ABI exports and host logic on the fake driver."""
import ctypes
import json
import os
import re
import struct

import numpy as np
import pytest

from accy_b200 import _native, configs, tensor
from accy_b200._native import lib
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def golden_bytes():
    with open(os.path.join(GOLDEN, "mismatch_2x16.actp"), "rb") as f:
        return f.read()


def known_answers():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        return json.load(f)


# ---------------------------------------------------------------------------------------------
# recording: named-axis rules and error names (examples/consumer/src/main.zig:230-249)
# ---------------------------------------------------------------------------------------------
def test_names_keep_guesses_and_points_apart_when_lengths_are_equal():
    p = tensor.define("mismatch", [tensor.spec("f32", guess=16), tensor.spec("f32", point=16),
                                   tensor.spec("f32", point=16)], configs.mismatch_body)
    assert p.output_types[0].dims == [("guess", 16)]


def test_different_lengths_are_refused_while_recording():
    with pytest.raises(tensor.TensorError) as e:
        tensor.define("mismatch", [tensor.spec("f32"), tensor.spec("f32", point=16), tensor.spec("f32", point=15)],
                      configs.mismatch_body)
    assert e.value.name == "AxisExtentMismatch"


def test_builder_error_names():
    b = tensor.Builder("t")
    x = b.input("f32", a=2, b=3)
    y = b.input("bf16", a=2)
    for fn, name in [(lambda: x.add(y), "DTypeMismatch"), (lambda: x.sum("nope"), "AxisNotFound"),
                     (lambda: x.sum(["a", "a"]), "DuplicateAxis"), (lambda: x.contract(y, "a"), "ContractDTypeMismatch"),
                     (lambda: b.input("f32", **{"#x": 2}), "AxisNameReserved"), (lambda: x.rename("a", "b"), "DuplicateAxis"),
                     (lambda: x.split("a", p=3, q=1), "SplitExtentMismatch")]:
        with pytest.raises(tensor.TensorError) as e:
            fn()
        assert e.value.name == name, name
    other = tensor.Builder("u")
    with pytest.raises(tensor.TensorError) as e:
        x.add(other.input("f32", a=2))
    assert e.value.name == "CrossBuilderValue"
    b.finish([x])
    with pytest.raises(tensor.TensorError) as e:
        x.neg()
    assert e.value.name == "BuilderFinished"


def test_union_order_alignment_and_contract_types():
    b = tensor.Builder("t")
    a = b.input("f32", n=4, m=3)
    c = b.input("f32", m=3, k=5)
    assert a.add(c).ty.dims == [("n", 4), ("m", 3), ("k", 5)]          # lhs dims first (algebra.zig:10-31)
    assert c.add(a).ty.dims == [("m", 3), ("k", 5), ("n", 4)]
    assert a.contract(c, "m").ty.dims == [("n", 4), ("k", 5)]
    q = b.input("bf16", batch=2, head=3, seq=4, dim=8)
    k = b.input("bf16", batch=2, head=3, key=5, dim=8)
    assert q.contract(k, "dim").ty.dims == [("batch", 2), ("head", 3), ("seq", 4), ("key", 5)]
    assert a.merge(["n", "m"], "nm").ty.dims == [("nm", 12)]
    assert a.split("n", p=2, q=2).ty.dims == [("p", 2), ("q", 2), ("m", 3)]
    assert a.mean("m").ty.dims == [("n", 4)]
    assert a.compare("lt", a).ty.dtype == "i1"


def test_recorded_op_lists_match_the_builder_rules():
    """Independent decoder (oracle) sees the op list the reference's Builder would record."""
    text = oracle.describe(configs.mismatch(8192, 65536).program().wire).splitlines()
    kinds = [line.split()[1] for line in text[:-1]]
    assert kinds == ["parameter", "parameter", "parameter", "broadcast_in_dim", "broadcast_in_dim", "binary", "unary",
                     "broadcast_in_dim", "binary", "binary", "constant", "reduce"]
    c2 = oracle.describe(configs.softmax_layernorm(8, 16).program().wire)
    assert c2.count(" reduce ") == 4 and c2.count("broadcast_in_dim") == 7
    c4 = oracle.describe(configs.attention(1, 2, 8, 4).program().wire)
    assert c4.count("dot_general") == 2 and c4.count("transpose") == 1 and c4.count("iota") == 2


# ---------------------------------------------------------------------------------------------
# ACTP wire bytes
# ---------------------------------------------------------------------------------------------
def reencode(data):
    buf = ctypes.create_string_buffer(len(data) + 4096)
    n = ctypes.c_size_t()
    err = ctypes.create_string_buffer(128)
    src = ctypes.create_string_buffer(bytes(data), len(data))
    status = lib.accy_b200_wire_reencode(ctypes.cast(src, ctypes.c_void_p), len(data), ctypes.cast(buf, ctypes.c_void_p),
                                         len(buf), ctypes.byref(n), ctypes.cast(err, ctypes.c_void_p), 128)
    return status, buf.raw[:n.value], err.value.decode()


def test_encoder_matches_hand_assembled_golden_bytes():
    program = configs.mismatch(2, 16).program()
    assert program.wire == golden_bytes()


def test_decode_reencode_round_trip_for_every_config():
    for cfg in (configs.mismatch(4, 32), configs.softmax_layernorm(4, 32), configs.matmul(8, 8, 8),
                configs.attention(1, 2, 8, 4), configs.mlp(4, 8, 16)):
        wire = cfg.program().wire
        status, again, _ = reencode(wire)
        assert status == 0 and again == wire
        assert oracle.describe(wire)  # the independent decoder accepts the same bytes


def test_both_decoders_derive_the_same_types():
    for cfg in (configs.softmax_layernorm(4, 32), configs.attention(1, 2, 8, 4), configs.mlp(4, 8, 16)):
        wire = cfg.program().wire
        buf = ctypes.create_string_buffer(1 << 16)
        n = ctypes.c_size_t()
        src = ctypes.create_string_buffer(wire, len(wire))
        assert lib.accy_b200_wire_describe(ctypes.cast(src, ctypes.c_void_p), len(wire), ctypes.cast(buf, ctypes.c_void_p),
                                           len(buf), ctypes.byref(n)) == 0
        assert buf.value.decode() == oracle.describe(wire)


def test_bad_bytes_are_refused_with_the_reference_error_names():
    good = golden_bytes()
    assert reencode(b"XXXX" + good[4:])[0::2] == (1, "BadMagic")
    status, _, name = reencode(good[:4] + struct.pack("<I", 2) + good[8:])
    assert (status, name) == (2, "UnsupportedVersion")
    assert reencode(good[:-3])[0::2] == (1, "InvalidArtifact")            # ends early
    assert reencode(good + b"\0")[0::2] == (1, "InvalidArtifact")         # trailing bytes
    assert reencode(good[:-4] + struct.pack("<I", 99))[0::2] == (1, "InvalidReference")
    # unknown kind code in the first operation
    at = 4 + 4 + 4 + len("mismatch") + 4
    assert reencode(good[:at] + struct.pack("<I", 77) + good[at + 4:])[0::2] == (1, "UnknownTag")


# ---------------------------------------------------------------------------------------------
# oracle pinned to the reference's shipped known answers
# ---------------------------------------------------------------------------------------------
def tone(points=16):
    time = (0.25 * np.arange(points)).astype(np.float32)
    return time, np.sin(3.0 * time.astype(np.float64)).astype(np.float32)


def test_oracle_mismatch_known_answers():
    ka = known_answers()["mismatch"]
    time, sample = tone(ka["points"])
    out = oracle.run(golden_bytes(), [np.array(ka["frequency"], np.float32), time, sample])[0]
    for got, want, tol in zip(out, ka["value"], ka["abs_tolerance"]):
        assert abs(float(got) - want) <= tol
    # f64 restatement of the definition (main.zig:188-198), relative 1e-5 (main.zig:208)
    exact = sum((np.sin(2.5 * float(t)) - float(s)) ** 2 for t, s in zip(time, sample))
    assert abs(float(out[0]) - exact) <= 1e-5 * exact


def test_oracle_eight_guesses_equal_eight_single_runs():
    time, sample = tone()
    starts = np.array([0.5, 1.0, 1.5, 2.0, 2.5, 3.5, 4.0, 4.5], np.float32)
    together = oracle.run(configs.mismatch(8, 16).program().wire, [starts, time, sample])[0]
    one = configs.mismatch(1, 16).program().wire
    for start, value in zip(starts, together):
        alone = oracle.run(one, [np.array([start], np.float32), time, sample])[0][0]
        assert abs(alone - value) <= 1e-6 * abs(alone)                  # main.zig:226


def test_oracle_dot_known_answer():
    ka = known_answers()["dot_f32_2x3_3x2"]
    program = tensor.define("dot", [tensor.spec("f32", m=2, k=3), tensor.spec("f32", k=3, n=2)], configs.matmul_body)
    out = oracle.run(program.wire, [np.array(ka["lhs"], np.float32), np.array(ka["rhs"], np.float32)])[0]
    assert out.reshape(-1).tolist() == ka["out"]


def test_oracle_config_loops_agree_with_the_program_evaluator():
    """The per-config C loops (used as the timed CPU baseline) compute what the generic evaluator does."""
    o = oracle.lib()
    size = ctypes.c_size_t

    def ptr(a):
        return a.ctypes.data_as(ctypes.c_void_p)
    cfg = configs.mismatch(5, 300)
    f, t, s = cfg.make_inputs()
    out = np.zeros(5, np.float32)
    o.oracle_mismatch_f32(ptr(f), ptr(t), ptr(s), ptr(out), size(5), size(300), size(0), size(5))
    assert np.array_equal(out, oracle.run(cfg.program().wire, [f, t, s])[0])
    cfg = configs.softmax_layernorm(6, 96)
    x = cfg.make_inputs()[0]
    out = np.zeros_like(x)
    o.oracle_softmax_layernorm_f32(ptr(x), ptr(out), size(6), size(96), ctypes.c_float(1e-5), size(0), size(6))
    assert np.array_equal(out, oracle.run(cfg.program().wire, [x])[0])
    cfg = configs.attention(1, 2, 24, 16)
    q, k, v = cfg.make_inputs()
    out = np.zeros((2, 24, 16), np.float32)
    scratch = np.zeros(24 * o.oracle_max_threads(), np.float32)
    scale = float(configs.bf16_bits_to_f32(configs.f32_to_bf16_bits(np.array([0.25], np.float32)))[0])
    o.oracle_attention_bf16(ptr(q), ptr(k), ptr(v), ptr(out), size(2), size(24), size(24), size(16),
                            ctypes.c_float(scale), ctypes.c_int(1), size(0), size(2), ptr(scratch))
    wide = configs.bf16_bits_to_f32(oracle.run(cfg.program().wire, [q, k, v], mode="wide")[0]).reshape(2, 24, 16)
    assert np.max(np.abs(out - wide)) < 2e-2
    cfg = configs.mlp(4, 16, 32)
    ins = cfg.make_inputs()
    out = np.zeros((4, 16), np.float32)
    hidden = np.zeros((4, 32), np.float32)
    o.oracle_mlp_bf16(*[ptr(a) for a in ins], ptr(out), ptr(hidden), size(4), size(16), size(32), ctypes.c_float(1e-6),
                      size(0), size(4))
    wide = configs.bf16_bits_to_f32(oracle.run(cfg.program().wire, ins, mode="wide")[0]).reshape(4, 16)
    assert np.max(np.abs(out - wide)) < 3e-2


# ---------------------------------------------------------------------------------------------
# the oracle against a second restatement written separately from the reference's text
# (tests/second_opinion.py): attention.zig:473-509, normalization.zig:372-398,560-590,
# elementwise.zig:125-135, dot.zig:2049-2115.  Both use one float32 operation per recorded
# operation; only the exp / tanh routines differ (numpy's against glibc's, an ulp apart at most),
# so results agree to a few ulp, up to 1e-5 (the f32 tolerance) where a weighted sum cancels.
# ---------------------------------------------------------------------------------------------
def _close(a, b, rel=1e-5):
    a, b = np.asarray(a, np.float64).reshape(-1), np.asarray(b, np.float64).reshape(-1)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3 * np.abs(b).max()))) < rel


def test_oracle_attention_agrees_with_a_second_restatement_on_the_reference_spec():
    """The reference's own SDPA spec (attention.zig:464-471: batch 2, queries 2, keys 3, qk 2, value 2)
    and a larger causal case, f32, through the program evaluator and through the C loop."""
    import second_opinion
    for (batch, nq, nk, qk, nv, causal) in [(2, 2, 3, 2, 2, False), (3, 9, 9, 8, 5, True), (1, 6, 11, 4, 3, False)]:
        rng = np.random.default_rng(nq * 10 + nk)
        # eighths in [-2, 2]: exact in bf16 too, so the bf16 C loop sees the very same numbers
        q = (rng.integers(-16, 17, (batch, nq, qk)) / 8.0).astype(np.float32)
        k = (rng.integers(-16, 17, (batch, nk, qk)) / 8.0).astype(np.float32)
        v = (rng.integers(-16, 17, (batch, nk, nv)) / 8.0).astype(np.float32)
        want = second_opinion.sdpa(q, k, v, causal)
        scale = float(np.float32(1.0 / np.sqrt(float(qk))))

        def body(b, a, scale=scale, causal=causal):
            scores = a[0].contract(a[1], "dim").mul(b.scalar("f32", scale))
            if causal:
                dims = [d for d in scores.ty.dims if d[0] in ("seq", "key")]
                mask = b.iota("i32", dims, "seq").compare("ge", b.iota("i32", dims, "key"))
                scores = mask.select(scores, b.scalar("f32", -np.inf))
            e = scores.sub(scores.max("key")).exp()
            return e.div(e.sum("key")).contract(a[2].rename("dim", "value"), "key")
        program = tensor.define("sdpa_spec", [tensor.spec("f32", batch=batch, seq=nq, dim=qk),
                                              tensor.spec("f32", batch=batch, key=nk, dim=qk),
                                              tensor.spec("f32", batch=batch, key=nk, dim=nv)], body)
        got = oracle.run(program.wire, [q, k, v], mode="ref")[0].reshape(batch, nq, nv)
        assert _close(got, want)
        if qk == nv:
            continue   # the C loop takes one dim for keys and values: checked on the square cases below
    # the C loop (bf16 bit patterns in, f32 out) on inputs that are exact in bf16
    o = oracle.lib()
    size = ctypes.c_size_t
    for (batch, n, dim, causal) in [(2, 3, 2, False), (2, 12, 8, True)]:
        rng = np.random.default_rng(n)
        q, k, v = [(rng.integers(-16, 17, (batch, n, dim)) / 8.0).astype(np.float32) for _ in range(3)]
        bits = [configs.f32_to_bf16_bits(a) for a in (q, k, v)]
        assert all(np.array_equal(configs.bf16_bits_to_f32(b), a) for a, b in zip((q, k, v), bits))
        out = np.zeros((batch, n, dim), np.float32)
        scratch = np.zeros(n * o.oracle_max_threads(), np.float32)
        o.oracle_attention_bf16(*[b.ctypes.data_as(ctypes.c_void_p) for b in bits], out.ctypes.data_as(ctypes.c_void_p),
                                size(batch), size(n), size(n), size(dim), ctypes.c_float(float(np.float32(1.0 / np.sqrt(float(dim))))),
                                ctypes.c_int(1 if causal else 0), size(0), size(batch), scratch.ctypes.data_as(ctypes.c_void_p))
        assert _close(out, second_opinion.sdpa(q, k, v, causal))
        rows = oracle.attention_rows(bits[0], bits[1], bits[2], [0, batch - 1], [n - 1, 1],
                                     float(np.float32(1.0 / np.sqrt(float(dim)))), causal)
        assert np.array_equal(rows, np.stack([out[0, n - 1], out[batch - 1, 1]]))


def test_oracle_row_formulas_agree_with_a_second_restatement():
    import second_opinion
    rng = np.random.default_rng(77)
    x = (rng.standard_normal((5, 48)) * 3.0).astype(np.float32)
    want = np.stack([second_opinion.row_layer_norm(second_opinion.row_softmax(row), 1e-5) for row in x])
    cfg = configs.softmax_layernorm(5, 48)
    got = oracle.run(cfg.program().wire, [x], mode="ref")[0]
    # softmax values are ~1/48 and their centred form cancels two digits: 1e-4 of the output's scale
    assert float(np.max(np.abs(got - want))) < 1e-4 * float(np.abs(want).max())
    o = oracle.lib()
    out = np.zeros_like(x)
    o.oracle_softmax_layernorm_f32(x.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(5),
                                   ctypes.c_size_t(48), ctypes.c_float(1e-5), ctypes.c_size_t(0), ctypes.c_size_t(5))
    assert float(np.max(np.abs(out - want))) < 1e-4 * float(np.abs(want).max())
    # softmax alone, where nothing cancels
    soft = tensor.define("softmax", [tensor.spec("f32", row=5, col=48)],
                         lambda b, a: a[0].sub(a[0].max("col")).exp().div(a[0].sub(a[0].max("col")).exp().sum("col")))
    assert _close(oracle.run(soft.wire, [x], mode="ref")[0], np.stack([second_opinion.row_softmax(r) for r in x]))


def test_oracle_mlp_and_gelu_agree_with_a_second_restatement():
    import second_opinion
    rng = np.random.default_rng(78)
    tokens, d, h = 3, 8, 16
    # sixteenths: exact in bf16
    x = (rng.integers(-32, 33, (tokens, d)) / 16.0).astype(np.float32)
    w1 = (rng.integers(-16, 17, (d, h)) / 16.0).astype(np.float32)
    w2 = (rng.integers(-16, 17, (h, d)) / 16.0).astype(np.float32)
    b1 = (rng.integers(-8, 9, h) / 16.0).astype(np.float32)
    b2 = (rng.integers(-8, 9, d) / 16.0).astype(np.float32)
    g = (rng.integers(8, 25, d) / 16.0).astype(np.float32)
    want = second_opinion.mlp_rms(x, w1, b1, w2, b2, g, 1e-6)
    bits = [configs.f32_to_bf16_bits(a) for a in (x, w1, b1, w2, b2, g)]
    got = oracle.mlp_rows(*bits, rows=[0, 1, 2])
    assert _close(got, want)
    # the same program in f32 through the generic evaluator (every op rounded on its own)
    program = tensor.define("mlp_f32", [tensor.spec("f32", token=tokens, d=d), tensor.spec("f32", d=d, h=h), tensor.spec("f32", h=h),
                                        tensor.spec("f32", h=h, d=d), tensor.spec("f32", d=d), tensor.spec("f32", d=d)],
                            configs.mlp_body)
    ref = oracle.run(program.wire, [x, w1, b1, w2, b2, g], mode="ref")[0]
    assert _close(ref, want)
    # tanh-GELU alone over a range of arguments
    values = np.linspace(-6.0, 6.0, 97).astype(np.float32)
    gelu = tensor.define("gelu", [tensor.spec("f32", n=97)],
                         lambda b, a: a[0].mul(b.scalar("f32", 0.5)).mul(
                             a[0].add(a[0].mul(a[0]).mul(a[0]).mul(b.scalar("f32", 0.044715))).mul(b.scalar("f32", 0.7978845608028654)).tanh()
                             .add(b.scalar("f32", 1.0))))
    got = np.asarray(oracle.run(gelu.wire, [values], mode="ref")[0], np.float64)
    want = np.array([second_opinion.gelu_tanh(v) for v in values], np.float64)
    # gate = tanh + 1 cancels for negative arguments, so an ulp of tanh (the two libraries' tanh
    # differ by that much) is an absolute 2^-24 * |x|: allow two of them
    assert np.all(np.abs(got - want) <= 2.0 ** -23 * np.maximum(np.abs(values.astype(np.float64)), 1.0))
    # the k-serial dot, bit for bit
    a = rng.standard_normal((4, 37)).astype(np.float32)
    b = rng.standard_normal((37, 5)).astype(np.float32)
    dot = tensor.define("dot", [tensor.spec("f32", m=4, k=37), tensor.spec("f32", k=37, n=5)], configs.matmul_body)
    assert np.array_equal(oracle.run(dot.wire, [a, b], mode="ref")[0], second_opinion.dot_serial(a, b))


# ---------------------------------------------------------------------------------------------
# fusion plans and sm_100a compilation (NVRTC, compile-only session)
# ---------------------------------------------------------------------------------------------
def plan_of(session, cfg, **kw):
    compiled = session.compile(cfg.program())
    summary, work, kernels = compiled.plan_summary(), compiled.work(), compiled.kernels()
    session.release(compiled)
    return summary, work, kernels


def test_mismatch_is_one_fused_reduction_kernel(cpu_session):
    summary, work, kernels = plan_of(cpu_session, configs.mismatch())
    assert work["launches"] == 1 and len(kernels) == 1
    assert "rows=8192 cols=65536 reduces=1" in summary and "vec=4" in summary
    assert work["bytes"] == 589824 and work["pairs"] == 536870912
    assert "sinf(" in kernels[0][1] and "--fmad=false" in kernels[0][2]


def test_few_guesses_use_the_deterministic_two_pass_combine(cpu_session):
    summary, work, kernels = plan_of(cpu_session, configs.mismatch(4, 1 << 20))
    assert work["launches"] == 2 and "splits=" in summary
    assert [k[0].endswith("_combine") for k in kernels] == [False, True]
    assert "atomic" not in kernels[0][1] and "atomic" not in kernels[1][1]


def test_softmax_layernorm_is_one_row_kernel_with_the_row_in_registers(cpu_session):
    summary, work, kernels = plan_of(cpu_session, configs.softmax_layernorm())
    assert work["launches"] == 1 and "reduces=4" in summary and "chunks=1" in summary
    assert work["bytes"] == 1073741824


def test_matmul_uses_the_tcgen05_kernel(cpu_session):
    summary, work, kernels = plan_of(cpu_session, configs.matmul())
    assert "tcgen05" in summary and work["flops"] == 2.0 * 8192 ** 3
    src = kernels[0][1]
    # a CTA pair per 256-row tile: paired MMAs, every TMA load without cluster multicast (each CTA
    # loads its own operand halves; only the MMA-completion signal goes to both CTAs)
    assert "tcgen05.mma.cta_group::2.kind::f16" in src and "__cluster_dims__(2, 1, 1)" in src
    loads = [line for line in src.split("\n") if "cp.async.bulk.tensor" in line]
    assert loads and not any("multicast" in line for line in loads)
    # one 128-row block: the one-CTA kernel
    summary, work, kernels = plan_of(cpu_session, configs.matmul(128, 512, 256))
    src = kernels[0][1]
    assert "tcgen05.mma.cta_group::1.kind::f16" in src and "cp.async.bulk.tensor.3d" in src and "__cluster_dims__" not in src
    assert "multicast" not in src


def test_mlp_fuses_gelu_into_the_first_gemm_and_rmsnorm_into_one_row_kernel(cpu_session):
    summary, work, kernels = plan_of(cpu_session, configs.mlp())
    lines = summary.strip().split("\n")
    assert len(lines) == 3 and work["launches"] == 3
    assert "epilogue_nodes=16" in lines[0] and "tcgen05" in lines[0] and "tcgen05" in lines[1]
    assert lines[2].startswith("row kernel") and "reduces=1" in lines[2]
    assert "fast_tanh(" in kernels[0][1]


def test_odd_shapes_fall_back_to_the_exact_order_simt_dot(cpu_session):
    summary, _, kernels = plan_of(cpu_session, configs.matmul(96, 80, 72))
    # separate multiply and add in the source of either SIMT kernel (one thread per output, or tiled)
    assert "simt" in summary and ("acc = acc + prod" in kernels[0][1] or "acc[i][j] = acc[i][j] + prod" in kernels[0][1])


def test_unsupported_programs_are_refused_not_emulated(cpu_session):
    def body(b, a):
        return a[0].pow(a[0])
    program = tensor.define("ipow", [tensor.spec("i32", n=8)], body)
    with pytest.raises(tensor.SessionError) as e:
        cpu_session.compile(program)
    assert e.value.name == "compile_failed"


def test_compile_only_session_cannot_launch(cpu_session):
    cfg = configs.mismatch(2, 16)
    compiled = cpu_session.compile(cfg.program())
    with pytest.raises(tensor.SessionError) as e:
        cpu_session.invoke(compiled, cfg.make_inputs(), [np.zeros(2, np.float32)])
    assert e.value.name == "launch_failed"
    cpu_session.release(compiled)


# ---------------------------------------------------------------------------------------------
# C ABI surface and host logic (fake driver)
# ---------------------------------------------------------------------------------------------
def test_library_exports_every_symbol_the_header_declares():
    with open(os.path.join(ROOT, "include", "accy_b200.h")) as f:
        header = f.read()
    declared = set(re.findall(r"\b(accy_b200_[a-z0-9_]+)\s*\(", header))
    declared.discard("accy_b200_observer")
    raw = ctypes.CDLL(_native.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), name
    assert declared == set(_native.PROTOTYPES), declared ^ set(_native.PROTOTYPES)


@pytest.fixture
def fake_driver():
    lib.accy_b200_test_use_fake_driver(1)
    yield
    lib.accy_b200_test_use_fake_driver(0)


def test_invoke_flow_on_the_fake_driver(fake_driver):
    session = tensor.Session(device=0)
    cfg = configs.mismatch(8, 16)
    phases = []
    session.set_observer(lambda phase, ns: phases.append(phase))
    compiled = session.compile(cfg.program())
    descs = compiled.input_descriptors() + compiled.output_descriptors()
    assert [d.byte_size for d in descs] == [32, 64, 64, 32] and all(d.alignment == 256 for d in descs)
    out = np.zeros(8, np.float32)
    session.invoke(compiled, cfg.make_inputs(), [out])
    assert lib.accy_b200_test_fake_call_count(b"cuLaunchKernel") == 1
    assert lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync") == 3
    assert {"decode", "plan", "kernel_compile", "load", "h2d_enqueue", "launch_enqueue", "d2h_and_sync"} <= set(phases)
    # exact sizes and no overlap (binding.zig:125-128, session.zig:176-178)
    with pytest.raises(tensor.SessionError) as e:
        session.invoke(compiled, cfg.make_inputs(), [np.zeros(7, np.float32)])
    assert e.value.name == "invalid_buffer"
    ins = cfg.make_inputs()
    with pytest.raises(tensor.SessionError) as e:
        session.invoke(compiled, ins, [ins[0]])
    assert e.value.name == "invalid_buffer"
    with pytest.raises(tensor.SessionError) as e:
        session.invoke(compiled, ins[:2], [out])
    assert e.value.name == "invalid_buffer"
    # stale handles are refused after release (session.zig:58-64)
    session.release(compiled)
    with pytest.raises(tensor.SessionError) as e:
        session.invoke(compiled, ins, [out])
    assert e.value.name == "invalid_handle"
    session.deinit()


def test_launch_timing_events_are_recorded_only_on_request(fake_driver):
    """The two events behind last_kernel_ms cost a stream of back-to-back invokes a few microseconds
    each, so an invoke records them only after time_launches(True)."""
    session = tensor.Session(device=0)
    cfg = configs.mismatch(8, 16)
    compiled = session.compile(cfg.program())
    out = np.zeros(8, np.float32)
    events = lambda: lib.accy_b200_test_fake_call_count(b"cuEventRecord")
    before = events()
    session.invoke(compiled, cfg.make_inputs(), [out])
    assert events() == before
    with pytest.raises(tensor.SessionError) as e:
        compiled.last_kernel_ms()
    assert e.value.name == "launch_failed" and "time_launches" in str(e.value)
    session.time_launches(True)
    session.invoke(compiled, cfg.make_inputs(), [out])
    assert events() == before + 2
    assert compiled.last_kernel_ms() >= 0.0
    session.time_launches(False)
    session.invoke(compiled, cfg.make_inputs(), [out])
    assert events() == before + 2
    session.deinit()


def test_multi_kernel_programs_replay_a_recorded_launch_sequence(fake_driver):
    """A plan of several kernels is captured as a CUDA graph by its first host invoke and replayed
    by the following ones: the kernels are enqueued once, later invokes submit the graph only."""
    session = tensor.Session(device=0)
    program = tensor.define("two_stage", [tensor.spec("f32", a=50, b=70)], lambda b, a: a[0].sum("b").max("a"))
    compiled = session.compile(program)
    launches = compiled.work()["launches"]
    assert launches >= 2
    count = lambda name: lib.accy_b200_test_fake_call_count(name)
    before = {n: count(n) for n in (b"cuLaunchKernel", b"cuGraphLaunch", b"cuStreamBeginCapture", b"cuGraphInstantiateWithFlags")}
    x = np.ones((50, 70), np.float32)
    out = np.zeros(1, np.float32)
    for _ in range(3):
        session.invoke(compiled, [x], [out])
    assert count(b"cuLaunchKernel") - before[b"cuLaunchKernel"] == launches
    assert count(b"cuStreamBeginCapture") - before[b"cuStreamBeginCapture"] == 1
    assert count(b"cuGraphInstantiateWithFlags") - before[b"cuGraphInstantiateWithFlags"] == 1
    assert count(b"cuGraphLaunch") - before[b"cuGraphLaunch"] == 3
    # a failed replay falls back to plain launches and stops using the graph
    lib.accy_b200_test_fake_fail(b"cuGraphLaunch", 0)
    session.invoke(compiled, [x], [out])
    lib.accy_b200_test_fake_fail(b"cuGraphLaunch", -1)
    assert count(b"cuLaunchKernel") - before[b"cuLaunchKernel"] == 2 * launches
    session.invoke(compiled, [x], [out])
    assert count(b"cuLaunchKernel") - before[b"cuLaunchKernel"] == 3 * launches
    session.release(compiled)
    session.deinit()


def test_resident_inputs_are_copied_once(fake_driver):
    """set_resident uploads an input once; invokes that pass None for it copy only the others,
    a wrong size is refused, and dropping the copy makes None invalid again."""
    session = tensor.Session(device=0)
    compiled = session.compile(configs.mismatch(2, 16).program())
    freq = np.array([2.5, 3.0], np.float32)
    time = (0.25 * np.arange(16)).astype(np.float32)
    sample = np.sin(3 * time).astype(np.float32)
    out = np.zeros(2, np.float32)
    with pytest.raises(tensor.SessionError) as err:
        session.set_resident(compiled, 1, time[:8])
    assert err.value.name == "invalid_buffer"
    with pytest.raises(tensor.SessionError):
        session.set_resident(compiled, 3, time)
    copies = lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync")
    session.set_resident(compiled, 1, time)
    session.set_resident(compiled, 2, sample)
    assert lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync") - copies == 2
    copies = lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync")
    session.invoke(compiled, [freq, None, None], [out])
    session.invoke(compiled, [freq, None, sample], [out])   # a pointer overrides the resident copy for that call
    assert lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync") - copies == 3
    session.set_resident(compiled, 1, None)
    with pytest.raises(tensor.SessionError) as err:
        session.invoke(compiled, [freq, None, None], [out])
    assert err.value.name == "invalid_buffer"
    session.deinit()


def test_compiled_kernels_are_reused_across_sessions():
    """A program compiled a second time (another session, same process) takes its kernels from the
    process-wide cache keyed by source text: the kernel_compile phase all but disappears."""
    program = configs.mismatch(7, 4099).program()   # extents no other test uses
    spent = []
    for _ in range(2):
        session = tensor.Session(device=-1)
        phases = {}
        session.set_observer(lambda phase, ns: phases.__setitem__(phase, phases.get(phase, 0) + ns))
        session.compile(program)
        spent.append(phases["kernel_compile"])
        session.deinit()
    assert spent[1] * 5 < spent[0]


def test_compiled_kernels_are_reused_across_processes(tmp_path):
    """ACCY_B200_KERNEL_CACHE_DIR keeps compiled kernels on disk: a second process compiles the same
    program without running NVRTC; a damaged file is ignored and rewritten."""
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from accy_b200 import tensor, configs\n"
            "from accy_b200._native import lib\n"
            "s = tensor.Session(device=-1)\n"
            "c = s.compile(configs.mismatch(5, 4111).program())\n"
            "print('nvrtc_runs', lib.accy_b200_test_fake_call_count(b'nvrtcCompileProgram'))\n") % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ACCY_B200_KERNEL_CACHE_DIR=str(tmp_path))

    def runs():
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, out.stderr
        return int(out.stdout.split("nvrtc_runs")[1])
    assert runs() >= 1
    files = sorted(tmp_path.glob("accy_*.cubin"))
    assert files and not list(tmp_path.glob("*.tmp*"))
    assert runs() == 0
    files[0].write_bytes(files[0].read_bytes()[:100])
    assert runs() >= 1
    assert files[0].stat().st_size > 100
    assert runs() == 0


def test_failed_launch_poisons_the_session(fake_driver):
    session = tensor.Session(device=0)
    cfg = configs.mismatch(8, 16)
    compiled = session.compile(cfg.program())
    out = np.zeros(8, np.float32)
    lib.accy_b200_test_fake_fail(b"cuLaunchKernel", 0)
    with pytest.raises(tensor.SessionError) as e:
        session.invoke(compiled, cfg.make_inputs(), [out])
    assert e.value.name == "launch_failed" and "ILLEGAL_ADDRESS" in e.value.message
    lib.accy_b200_test_fake_fail(b"cuLaunchKernel", -1)
    with pytest.raises(tensor.SessionError) as e:
        session.invoke(compiled, cfg.make_inputs(), [out])
    assert "poisoned" in e.value.message
    session.deinit()


def test_a_kernel_that_gives_up_on_a_wait_poisons_the_session(fake_driver):
    """The tcgen05 kernels bound every wait; when one runs out the kernel writes a code into the
    session's device status word and returns.  The host reads the word after synchronising: a
    non-zero code is `launch_failed`, the results are not handed out as valid, and the session
    refuses further launches (stream poisoning, runtime.zig:279-314)."""
    session = tensor.Session(device=0)
    cfg = configs.matmul(256, 256, 256)
    compiled = session.compile(cfg.program())
    out = np.zeros(256 * 256, np.uint16)
    session.invoke(compiled, cfg.make_inputs(), [out])          # a clean run first
    launches = lib.accy_b200_test_fake_call_count(b"cuLaunchKernel")
    lib.accy_b200_test_fake_device_status(1)
    with pytest.raises(tensor.SessionError) as e:
        session.invoke(compiled, cfg.make_inputs(), [out])
    assert e.value.name == "launch_failed" and "bounded wait" in e.value.message and "status 1" in e.value.message
    lib.accy_b200_test_fake_device_status(0)
    after = lib.accy_b200_test_fake_call_count(b"cuLaunchKernel")
    assert after == launches + 1
    for call in (lambda: session.invoke(compiled, cfg.make_inputs(), [out]),
                 lambda: session.invoke_device(compiled, [256, 512], [768])):
        with pytest.raises(tensor.SessionError) as e:
            call()
        assert e.value.name == "launch_failed" and "poisoned" in e.value.message
    assert lib.accy_b200_test_fake_call_count(b"cuLaunchKernel") == after   # nothing reached the device
    session.deinit()
    # a new session on the same device starts clean
    fresh = tensor.Session(device=0)
    again = fresh.compile(cfg.program())
    fresh.invoke(again, cfg.make_inputs(), [out])
    fresh.deinit()


def test_at_most_64_programs_per_session(cpu_session):
    held = []
    wire = configs.mismatch(1, 4).program().wire
    session = tensor.Session(device=-1)
    for _ in range(64):
        held.append(session.compile(wire))
    with pytest.raises(tensor.SessionError) as e:
        session.compile(wire)
    assert e.value.name == "too_many_programs"
    session.release(held.pop())
    held.append(session.compile(wire))
    session.deinit()


def test_large_host_invokes_stream_through_the_device_in_chunks(fake_driver):
    """Programs with enough data are re-recorded for a slice of their outermost axis and run chunk
    by chunk on three streams; replicated inputs are copied once."""
    session = tensor.Session(device=0)
    cfg = configs.softmax_layernorm(4096, 4096)           # 64 MiB in + 64 MiB out
    compiled = session.compile(cfg.program())
    x = np.zeros((4096, 4096), np.float32)
    out = np.zeros_like(x)
    before = lib.accy_b200_test_fake_call_count(b"cuLaunchKernel")
    copies = lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync")
    session.invoke(compiled, [x], [out])
    assert lib.accy_b200_test_fake_call_count(b"cuLaunchKernel") - before == 8
    assert lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync") - copies == 8
    session.deinit()
    single = tensor.Session(device=0, single_shot_invoke=1)
    compiled = single.compile(cfg.program())
    before = lib.accy_b200_test_fake_call_count(b"cuLaunchKernel")
    single.invoke(compiled, [x], [out])
    assert lib.accy_b200_test_fake_call_count(b"cuLaunchKernel") - before == 1
    single.deinit()


def test_shard_program_rules():
    piece, partial = tensor.shard_program(configs.mismatch(8, 64).program(), "guess", 4)
    assert not partial and piece.wire == configs.mismatch(4, 64).program().wire
    piece, partial = tensor.shard_program(configs.mismatch(8, 64).program(), "point", 16)
    assert partial and piece.input_types[1].dims == [("point", 16)]
    for cfg, axis in [(configs.softmax_layernorm(8, 32), "col"), (configs.matmul(16, 8, 8), "k"),
                      (configs.attention(4, 2, 8, 4), "seq")]:
        with pytest.raises(tensor.SessionError) as e:
            tensor.shard_program(cfg.program(), axis, 2)
        assert e.value.name == "compile_failed"
    for cfg, axis in [(configs.softmax_layernorm(8, 32), "row"), (configs.matmul(16, 8, 8), "m"),
                      (configs.attention(4, 2, 8, 4), "batch"), (configs.mlp(8, 8, 16), "token")]:
        piece, partial = tensor.shard_program(cfg.program(), axis, 2)
        assert not partial and piece.output_types[0].dims[0] == (axis, 2)


def test_one_process_runs_the_pieces_on_several_devices(fake_driver):
    """accy_b200_sharded_*: one session per device, every device gets its piece; checked on the
    recording fake driver (launches and copies per device), refusals with their reasons."""
    cfg = configs.mismatch(8, 64)
    multi = tensor.MultiCuda(cfg.program(), "guess", [0, 1, 2, 3])
    out = np.zeros(8, np.float32)
    launches = lib.accy_b200_test_fake_call_count(b"cuLaunchKernel")
    uploads = lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync")
    downloads = lib.accy_b200_test_fake_call_count(b"cuMemcpyDtoHAsync")
    multi.launch(cfg.make_inputs(), [out])
    assert lib.accy_b200_test_fake_call_count(b"cuLaunchKernel") - launches == 4            # one piece per device
    assert lib.accy_b200_test_fake_call_count(b"cuMemcpyHtoDAsync") - uploads == 4 * 3      # frequency block, time, sample
    assert lib.accy_b200_test_fake_call_count(b"cuMemcpyDtoHAsync") - downloads >= 4        # a block of the result each
    # wrong sizes are those of the whole program
    with pytest.raises(tensor.SessionError) as e:
        multi.launch(cfg.make_inputs(), [np.zeros(2, np.float32)])
    assert e.value.name == "invalid_buffer" and "32 bytes" in e.value.message
    multi.deinit()
    # the summed axis: pieces hold partial sums (two launches each: column-split fold and its combine, or one)
    partial = tensor.MultiCuda(cfg.program(), "point", [0, 1])
    partial.launch(cfg.make_inputs(), [out])
    partial.deinit()
    for axis, devices, reason in [("guess", [0, 1, 2], "does not divide"), ("nothing", [0, 1], "no value carries")]:
        with pytest.raises(tensor.SessionError) as e:
            tensor.MultiCuda(cfg.program(), axis, devices)
        assert e.value.name == "compile_failed" and reason in e.value.message
    with pytest.raises(tensor.SessionError) as e:
        tensor.MultiCuda(configs.softmax_layernorm(8, 32).program(), "col", [0, 1])
    assert e.value.name == "compile_failed"


def test_reference_arm_of_the_bench_runs_without_the_native_library():
    """`bench.py --impl reference` times the CPU restatement only: it must print one JSON line with
    the native arm's metric, unit and `config.specs`, and must not map libaccy_b200.so (its inputs
    come from accy_b200/synthetic.py loaded by file path)."""
    import subprocess
    import sys
    root = ROOT
    probe = ("import runpy, sys\n"
             "sys.argv = ['bench.py', '--impl', 'reference', '--small', '--steps', '1', '--warmup', '1']\n"
             "runpy.run_path(%r, run_name='__main__')\n"
             "maps = open('/proc/self/maps').read()\n"
             "print('NATIVE_MAPPED' if 'libaccy_b200' in maps else 'NATIVE_ABSENT', file=sys.stderr)\n"
             "print('ORACLE_MAPPED' if 'libaccy_oracle' in maps else 'ORACLE_ABSENT', file=sys.stderr)\n") % os.path.join(root, "bench.py")
    done = subprocess.run([sys.executable, "-c", probe], capture_output=True, text=True, cwd=root, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    assert "NATIVE_ABSENT" in done.stderr and "ORACLE_MAPPED" in done.stderr
    line = json.loads(done.stdout.strip().split("\n")[-1])
    assert line["impl"] == "reference" and line["metric"] == "fused_reduce_hbm_gbs" and line["unit"] == "GB/s"
    assert line["config"]["workload"] == "softmax_layernorm" and line["config"]["specs"] == ["f32[row=8192, col=4096]"]
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["single_core"]["cores"] == 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0 and line["value"] > 0


def test_synthetic_inputs_are_the_configs_inputs():
    """accy_b200/synthetic.py (plain numpy, loadable by path) and accy_b200.configs give the same bytes and specs."""
    import importlib.util
    path = os.path.join(ROOT, "accy_b200", "synthetic.py")
    spec = importlib.util.spec_from_file_location("synthetic_by_path", path)
    synthetic = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(synthetic)
    for name, cfg in [("mismatch", configs.mismatch(6, 40)), ("softmax_layernorm", configs.softmax_layernorm(4, 8)),
                      ("matmul", configs.matmul(8, 16, 24)), ("attention", configs.attention(1, 2, 8, 4)), ("mlp", configs.mlp(4, 8, 16))]:
        sizes = [(n, e) for n, e in synthetic.SIZES[name]]
        dims = {n: e for s in cfg.specs for n, e in s.dims}
        sizes = [(n, dims[n]) for n, _ in sizes]
        assert [synthetic.spec_text(s) for s in synthetic.specs(name, sizes)] == [repr(t) for t in cfg.program().input_types]
        for a, b in zip(synthetic.inputs(name, sizes), cfg.make_inputs()):
            assert a.dtype == b.dtype and np.array_equal(a, b)
        assert synthetic.work(name, sizes) == cfg.work
