"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle on the same seeded inputs.

Tolerances (stated by the benchmark definition): f32 reductions 1e-5 relative; bf16 matmul and
attention 2e-2 relative against an f32 computation on the same bf16-rounded inputs.  "Relative" is
taken against max(|expected|, floor), so elements that cancel to nearly zero are not held to an
impossible standard: for f32 programs the floor is a small fraction of the output's largest
magnitude; bf16 programs are checked the way `allclose` does with the absolute term tied to the
output's scale: |got - want| <= 2e-2 * (|want| + rms(want)).  Rounding an intermediate activation
or the softmax weights to bf16, which any bf16 tensor-core kernel must do, alone moves elements
that are smaller than the typical magnitude by more than 2% of their own value.
"""
import numpy as np
import pytest

from accy_b200 import configs, tensor
from oracle import oracle
from parity_checks import check_three_distances

pytestmark = pytest.mark.gpu


def run_gpu(session, cfg, inputs):
    program = cfg.program()
    compiled = session.compile(program)
    outs = [np.empty(d.byte_size, np.uint8) for d in compiled.output_descriptors()]
    session.invoke(compiled, inputs, outs)
    session.release(compiled)
    return program, outs


def rel_err(got, want, floor_frac):
    want = want.astype(np.float64)
    got = got.astype(np.float64)
    floor = max(np.abs(want).max() * floor_frac, 1e-30)
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))


def rel_err_bf16(got, want):
    want = want.astype(np.float64).reshape(-1)
    got = got.astype(np.float64).reshape(-1)
    rms = max(float(np.sqrt(np.mean(want * want))), 1e-30)
    return float(np.max(np.abs(got - want) / (np.abs(want) + rms)))


@pytest.mark.parametrize("guesses,points", [(1, 16), (8, 16), (3, 17), (64, 4096), (5, 100000), (2, 1 << 20), (512, 8192),
                                            # enough guesses for two rows per thread; an odd count leaves the last thread one row
                                            (2501, 20000), (3000, 12289)])
def test_mismatch_matches_oracle(gpu_session, guesses, points):
    cfg = configs.mismatch(guesses, points)
    inputs = cfg.make_inputs()
    program, outs = run_gpu(gpu_session, cfg, inputs)
    got = outs[0].view(np.float32)
    ref = oracle.run(program.wire, inputs)[0]
    exact = oracle.run(program.wire, inputs, mode="f64")[0]
    # The serial f32 fold of the reference carries its own rounding error of about sqrt(n)*eps, and
    # the f32 product frequency * time is up to 0.004 rad away from the product in f64 (which alone
    # moves a sum over 20000 points by 3e-5): the GPU's tree-shaped fold must be as close to the f64
    # result as the reference-order oracle is, up to 1e-5 relative.
    check_three_distances("mismatch %dx%d" % (guesses, points), got, ref, exact, 1e-6)


def test_value_and_slope_with_two_rows_per_thread(gpu_session):
    """The derived value-and-slope program (two reductions, a sine and a cosine of one phase) at a
    size where every thread folds two guesses at once and shares the time and sample vectors."""
    cfg = configs.refine(2601, 16384)
    inputs = cfg.make_inputs()
    program = cfg.program()
    compiled = gpu_session.compile(program)
    assert "rows_per_thread=2" in compiled.plan_summary()
    outs = [np.empty(2601, np.float32), np.empty(2601, np.float32)]
    gpu_session.invoke(compiled, inputs, outs)
    gpu_session.release(compiled)
    refs = oracle.run(program.wire, inputs)
    exacts = oracle.run(program.wire, inputs, mode="f64")
    for label, got, ref, exact in zip(("value", "slope"), outs, refs, exacts):
        check_three_distances("refine 2601x16384 " + label, got, ref, exact, 1e-3 if label == "slope" else 1e-6)


def test_mismatch_readme_constants(gpu_session):
    cfg = configs.mismatch(2, 16)
    time = (0.25 * np.arange(16)).astype(np.float32)
    sample = np.sin(3.0 * time.astype(np.float64)).astype(np.float32)
    program, outs = run_gpu(gpu_session, cfg, [np.array([2.5, 3.0], np.float32), time, sample])
    got = outs[0].view(np.float32)
    assert abs(got[0] - 8.656) < 1e-3      # README.md:151-153
    assert abs(got[1]) < 1e-9              # examples/consumer/src/main.zig:210


@pytest.mark.parametrize("rows,cols", [(1, 4), (7, 33), (256, 1024), (100, 4096), (16, 8192), (4, 40000), (3, 1000)])
def test_softmax_layernorm_matches_oracle(gpu_session, rows, cols):
    cfg = configs.softmax_layernorm(rows, cols)
    inputs = cfg.make_inputs()
    program, outs = run_gpu(gpu_session, cfg, inputs)
    got = outs[0].view(np.float32).reshape(rows, cols)
    ref = oracle.run(program.wire, inputs)[0]
    exact = oracle.run(program.wire, inputs, mode="f64")[0]
    check_three_distances("softmax_layernorm %dx%d" % (rows, cols), got, ref, exact, 1e-3)


@pytest.mark.parametrize("m,n,k", [(2, 2, 3), (96, 80, 72), (256, 256, 256), (128, 384, 192)])
def test_matmul_bf16_matches_f32_reference(gpu_session, m, n, k):
    cfg = configs.matmul(m, n, k)
    inputs = cfg.make_inputs()
    program, outs = run_gpu(gpu_session, cfg, inputs)
    got = configs.bf16_bits_to_f32(outs[0].view(np.uint16)).reshape(m, n)
    ref = oracle.run(program.wire, inputs, mode="wide")[0]
    assert rel_err_bf16(got, configs.bf16_bits_to_f32(ref)) < 2e-2


def test_dot_f32_known_answer(gpu_session):
    # src/executable/fragment.zig:1193-1205: [2,3]x[3,2] of 1..6 and 7..12
    def body(b, a):
        return a[0].contract(a[1], "k")
    program = tensor.define("dot", [tensor.spec("f32", m=2, k=3), tensor.spec("f32", k=3, n=2)], body)
    compiled = gpu_session.compile(program)
    out = np.zeros(4, np.float32)
    gpu_session.invoke(compiled, [np.arange(1, 7, dtype=np.float32), np.arange(7, 13, dtype=np.float32)], [out])
    assert out.tolist() == [58.0, 64.0, 139.0, 154.0]


@pytest.mark.parametrize("batch,head,seq,dim,causal", [(1, 1, 48, 32, False), (1, 2, 64, 32, True), (2, 2, 256, 128, True),
                                                        (1, 2, 256, 128, False), (1, 3, 1024, 128, True),
                                                        (2, 1, 512, 128, False), (1, 1, 2048, 128, True),
                                                        # more work items than SMs: CTAs take several items each
                                                        (4, 10, 1024, 128, True), (3, 26, 512, 128, False),
                                                        # head dim 64 in the fused kernel
                                                        (2, 2, 512, 64, True), (1, 3, 256, 64, False), (2, 40, 512, 64, True)])
def test_attention_matches_f32_reference(gpu_session, batch, head, seq, dim, causal):
    cfg = configs.attention(batch, head, seq, dim, causal)
    inputs = cfg.make_inputs()
    program, outs = run_gpu(gpu_session, cfg, inputs)
    got = configs.bf16_bits_to_f32(outs[0].view(np.uint16))
    ref = configs.bf16_bits_to_f32(oracle.run(program.wire, inputs, mode="wide")[0]).reshape(-1)
    assert rel_err_bf16(got, ref) < 2e-2


F32_GEMMS = {
    "ragged_bias": ([tensor.spec("f32", m=1000, k=333), tensor.spec("f32", k=333, n=517), tensor.spec("f32", n=517)],
                    lambda b, a: a[0].contract(a[1], "k").add(a[2])),
    "batched_k_major_b": ([tensor.spec("f32", g=3, m=130, k=77), tensor.spec("f32", g=3, n=200, k=77)], lambda b, a: a[0].contract(a[1], "k")),
    "m_contiguous_a": ([tensor.spec("f32", k=96, m=256), tensor.spec("f32", k=96, n=128)], lambda b, a: a[0].contract(a[1], "k")),
    "small": ([tensor.spec("f32", m=50, k=30), tensor.spec("f32", k=30, n=70)], lambda b, a: a[0].contract(a[1], "k")),
    "short_k": ([tensor.spec("f32", m=256, k=5), tensor.spec("f32", k=5, n=256)], lambda b, a: a[0].contract(a[1], "k")),
}


@pytest.mark.parametrize("name", sorted(F32_GEMMS))
def test_f32_matmul_is_bit_exact(gpu_session, name):
    """f32 contractions keep the reference's arithmetic (k folded serially, separate multiply and
    add roundings, dot.zig:2049-2115) in the tiled kernel too: the bits equal the oracle's."""
    specs, body = F32_GEMMS[name]
    program = tensor.define("gemm_f32_" + name, specs, body)
    rng = np.random.default_rng(17)
    inputs = [rng.standard_normal([e for _, e in sp.dims]).astype(np.float32) for sp in specs]
    compiled = gpu_session.compile(program)
    size = compiled.output_descriptors()[0].byte_size
    out = np.full(size + 4096, 0x5A, np.uint8)
    gpu_session.invoke(compiled, inputs, [out[:size]])
    gpu_session.release(compiled)
    assert np.all(out[size:] == 0x5A)
    want = oracle.run(program.wire, inputs, mode="ref")[0].astype(np.float32).reshape(-1)
    assert np.array_equal(out[:size].view(np.float32).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", ["i32", "u32"])
def test_integer_contraction_wraps_like_the_oracle(gpu_session, dtype):
    """i32 / u32 contractions (the reference's dot lowering takes them) with values large enough
    to overflow: exact wrap-around arithmetic, followed by an elementwise op in its own kernel."""
    np_t = np.int32 if dtype == "i32" else np.uint32
    program = tensor.define("int_dot_" + dtype, [tensor.spec(dtype, g=2, m=40, k=33), tensor.spec(dtype, g=2, k=33, n=50),
                                                  tensor.spec(dtype, n=50)],
                            lambda b, a: a[0].contract(a[1], "k").add(a[2]))
    rng = np.random.default_rng(23)
    inputs = [rng.integers(0, 2 ** 31 - 1, shape, dtype=np.int64).astype(np_t) for shape in ((2, 40, 33), (2, 33, 50), (50,))]
    compiled = gpu_session.compile(program)
    out = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    gpu_session.invoke(compiled, inputs, [out])
    gpu_session.release(compiled)
    want = oracle.run(program.wire, inputs, mode="ref")[0]
    assert np.array_equal(out.view(np_t), np.asarray(want).astype(np_t).reshape(-1))


RAGGED_GEMMS = {
    "ragged_all": ([tensor.spec("bf16", m=300, k=200), tensor.spec("bf16", k=200, n=392)], lambda b, a: a[0].contract(a[1], "k")),
    "ragged_bias_tanh": ([tensor.spec("bf16", m=1000, k=72), tensor.spec("bf16", k=72, n=1032), tensor.spec("bf16", n=1032)],
                         lambda b, a: a[0].contract(a[1], "k").add(a[2]).tanh()),
    "one_tile_plus_a_bit": ([tensor.spec("bf16", m=129, k=64), tensor.spec("bf16", k=64, n=136)], lambda b, a: a[0].contract(a[1], "k")),
    "batched_k_major_b": ([tensor.spec("bf16", g=3, m=200, k=136), tensor.spec("bf16", g=3, n=150, k=136)],
                          lambda b, a: a[0].contract(a[1], "k")),
    "f32_output_odd_n": ([tensor.spec("bf16", m=130, k=128), tensor.spec("bf16", n=131, k=128)], lambda b, a: a[0].contract(a[1], "k")),
    # lhs stored [k, m] (what the gradient of a contraction with respect to its rhs reads): M-major A tiles
    "transposed_a": ([tensor.spec("bf16", k=200, m=304), tensor.spec("bf16", k=200, n=392)], lambda b, a: a[0].contract(a[1], "k")),
    "transposed_a_k_major_b": ([tensor.spec("bf16", k=136, m=264), tensor.spec("bf16", n=150, k=136)],
                               lambda b, a: a[0].contract(a[1], "k")),
    "batched_transposed_a": ([tensor.spec("bf16", g=2, k=128, m=200), tensor.spec("bf16", g=2, k=128, n=256)],
                             lambda b, a: a[0].contract(a[1], "k")),
}


@pytest.mark.parametrize("name", sorted(RAGGED_GEMMS))
def test_ragged_matmul_on_tensor_cores(gpu_session, name):
    """Extents that are not multiples of the 128 x 128/256 x 64 tile stay on tcgen05: loads past
    the end read zeros, stores are guarded (bytes after the output stay untouched)."""
    specs, body = RAGGED_GEMMS[name]
    program = tensor.define("gemm_" + name, specs, body)
    rng = np.random.default_rng(13)
    inputs = [configs.f32_to_bf16_bits((rng.standard_normal([e for _, e in sp.dims]) / 8.0).astype(np.float32)) for sp in specs]
    compiled = gpu_session.compile(program)
    assert "tcgen05" in compiled.plan_summary()
    size = compiled.output_descriptors()[0].byte_size
    out = np.full(size + 4096, 0x5A, np.uint8)
    gpu_session.invoke(compiled, inputs, [out[:size]])
    gpu_session.release(compiled)
    assert np.all(out[size:] == 0x5A)
    got = configs.bf16_bits_to_f32(out[:size].view(np.uint16))
    ref = configs.bf16_bits_to_f32(oracle.run(program.wire, inputs, mode="wide")[0]).reshape(-1)
    assert rel_err_bf16(got, ref) < 2e-2


F16_PROGRAMS = {
    # f16 is the 16-bit float the reference's own dot lowering accepts (f32 accumulate, narrowed
    # once at the end, kernelization/lowering/dot.zig:2004-2015); here it runs on tcgen05
    "plain": ([tensor.spec("f16", m=256, k=192), tensor.spec("f16", k=192, n=384)], lambda b, a: a[0].contract(a[1], "k")),
    "bias_tanh": ([tensor.spec("f16", m=128, k=256), tensor.spec("f16", k=256, n=256), tensor.spec("f16", n=256)],
                  lambda b, a: a[0].contract(a[1], "k").add(a[2]).tanh()),
    "batched_k_major_b": ([tensor.spec("f16", g=3, m=128, k=128), tensor.spec("f16", g=3, n=128, k=128)],
                          lambda b, a: a[0].contract(a[1], "k")),
}


@pytest.mark.parametrize("name", sorted(F16_PROGRAMS))
def test_f16_matmul_on_tensor_cores(gpu_session, name):
    specs, body = F16_PROGRAMS[name]
    program = tensor.define("f16_" + name, specs, body)
    rng = np.random.default_rng(11)
    inputs = [(rng.standard_normal([e for _, e in sp.dims]) / 8.0).astype(np.float16) for sp in specs]
    compiled = gpu_session.compile(program)
    assert "tcgen05" in compiled.plan_summary()
    out = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    gpu_session.invoke(compiled, inputs, [out])
    gpu_session.release(compiled)
    want = oracle.run(program.wire, inputs, mode="wide")[0].astype(np.float64).reshape(-1)
    got = out.view(np.float16).astype(np.float64)
    rms = max(float(np.sqrt(np.mean(want * want))), 1e-30)
    assert float(np.max(np.abs(got - want) / (np.abs(want) + rms))) < 2e-3   # f16 keeps 11 significant bits


@pytest.mark.parametrize("causal", [True, False])
def test_f16_attention(gpu_session, causal):
    """The fused attention kernel with f16 operands (P is written to TMEM as f16)."""
    import math
    specs = [tensor.spec("f16", batch=2, head=3, seq=512, dim=128), tensor.spec("f16", batch=2, head=3, key=512, dim=128),
             tensor.spec("f16", batch=2, head=3, key=512, dim=128)]
    program = tensor.define("attention_f16", specs, configs.make_attention_body(1.0 / math.sqrt(128), causal))
    rng = np.random.default_rng(5)
    inputs = [rng.standard_normal([e for _, e in sp.dims]).astype(np.float16) for sp in specs]
    compiled = gpu_session.compile(program)
    assert "attention:" in compiled.plan_summary()
    out = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    gpu_session.invoke(compiled, inputs, [out])
    gpu_session.release(compiled)
    want = oracle.run(program.wire, inputs, mode="wide")[0].astype(np.float64).reshape(-1)
    got = out.view(np.float16).astype(np.float64)
    rms = max(float(np.sqrt(np.mean(want * want))), 1e-30)
    assert float(np.max(np.abs(got - want) / (np.abs(want) + rms))) < 4e-3


@pytest.mark.parametrize("seq,keys,dim,causal", [(1000, 1000, 128, True), (700, 700, 64, True), (600, 600, 128, True),
                                                  (384, 200, 128, False), (300, 300, 64, False), (129, 129, 128, True)])
def test_ragged_attention_lengths(gpu_session, seq, keys, dim, causal):
    """Sequence lengths that are not multiples of the 128-row tile still run in the fused kernel:
    loads past the end read zeros, the last key block is masked, stores past the end are dropped."""
    cfg = configs.attention(2, 3, seq, dim, causal, keys=keys)
    inputs = cfg.make_inputs()
    program = cfg.program()
    compiled = gpu_session.compile(program)
    assert "attention:" in compiled.plan_summary()
    guard = 0x5A
    out = np.full(compiled.output_descriptors()[0].byte_size + 4096, guard, np.uint8)
    gpu_session.invoke(compiled, inputs, [out[:-4096]])
    gpu_session.release(compiled)
    assert np.all(out[-4096:] == guard)
    got = configs.bf16_bits_to_f32(out[:-4096].view(np.uint16))
    ref = configs.bf16_bits_to_f32(oracle.run(program.wire, inputs, mode="wide")[0]).reshape(-1)
    assert rel_err_bf16(got, ref) < 2e-2


@pytest.mark.parametrize("seq,keys", [(256, 128), (512, 384), (256, 1152)])
def test_cross_attention_key_lengths(gpu_session, seq, keys):
    """Non-causal attention whose key length differs from the query length: a single key block
    (the tile's first S is also its last), an odd number of blocks, more key blocks than queries."""
    cfg = configs.attention(1, 3, seq, 128, False, keys=keys)
    inputs = cfg.make_inputs()
    program, outs = run_gpu(gpu_session, cfg, inputs)
    assert "attention:" in gpu_session.compile(program).plan_summary()
    got = configs.bf16_bits_to_f32(outs[0].view(np.uint16))
    ref = configs.bf16_bits_to_f32(oracle.run(program.wire, inputs, mode="wide")[0]).reshape(-1)
    assert rel_err_bf16(got, ref) < 2e-2


def random_attention(seed):
    """seeded random attention shapes: (batch, heads, queries, head dim, causal, keys)"""
    rng = np.random.default_rng(3000 + seed)
    causal = bool(rng.random() < 0.5)
    dim = int(rng.choice([64, 128]))
    batch, heads = int(rng.integers(1, 3)), int(rng.integers(1, 4))
    seq = int(rng.integers(128, 900))
    if rng.random() < 0.5:
        seq = seq // 128 * 128
    keys = None
    if not causal and rng.random() < 0.6:
        keys = int(rng.integers(128, 900))
    return batch, heads, seq, dim, causal, keys


@pytest.mark.parametrize("seed", range(16))
def test_random_attention_shapes_match_the_oracle(gpu_session, seed):
    """Query and key lengths that are and are not multiples of the 128-row tiles and 128-key blocks, both
    head dims, causal and not, cross attention: the fused kernel against the f32 SDPA restatement."""
    batch, heads, seq, dim, causal, keys = random_attention(seed)
    cfg = configs.attention(batch, heads, seq, dim, causal, keys=keys, seed=100 + seed)
    inputs = cfg.make_inputs()
    program = cfg.program()
    compiled = gpu_session.compile(program)
    assert "attention:" in compiled.plan_summary()
    size = compiled.output_descriptors()[0].byte_size
    out = np.full(size + 4096, 0x5A, np.uint8)
    gpu_session.invoke(compiled, inputs, [out[:size]])
    gpu_session.release(compiled)
    assert np.all(out[size:] == 0x5A)
    got = configs.bf16_bits_to_f32(out[:size].view(np.uint16))
    ref = configs.bf16_bits_to_f32(oracle.run(program.wire, inputs, mode="wide")[0]).reshape(-1)
    err = rel_err_bf16(got, ref)
    print("batch %d heads %d queries %d dim %d causal %s keys %s: err %.3g" % (batch, heads, seq, dim, causal, keys, err))
    assert err < 2e-2


def test_attention_repeated_launches_agree(gpu_session):
    """The persistent attention kernel hands out work through a device counter that every launch
    must leave cleared: three launches of one compiled program give the same bytes."""
    cfg = configs.attention(2, 40, 512, 128, True)   # 160 work items
    inputs = cfg.make_inputs()
    compiled = gpu_session.compile(cfg.program())
    results = []
    for _ in range(3):
        out = np.zeros(compiled.output_descriptors()[0].byte_size, np.uint8)
        gpu_session.invoke(compiled, inputs, [out])
        results.append(out)
    gpu_session.release(compiled)
    assert results[0].any()
    assert np.array_equal(results[0], results[1]) and np.array_equal(results[0], results[2])


@pytest.mark.parametrize("tokens,d,h", [(8, 16, 32), (256, 256, 512), (128, 512, 1024)])
def test_mlp_matches_f32_reference(gpu_session, tokens, d, h):
    cfg = configs.mlp(tokens, d, h)
    inputs = cfg.make_inputs()
    program, outs = run_gpu(gpu_session, cfg, inputs)
    got = configs.bf16_bits_to_f32(outs[0].view(np.uint16))
    ref = configs.bf16_bits_to_f32(oracle.run(program.wire, inputs, mode="wide")[0]).reshape(-1)
    assert rel_err_bf16(got, ref) < 2e-2


def test_softmax_layernorm_full_size_properties(gpu_session):
    """BASELINE size: every output row has zero mean and unit variance (up to the eps term),
    and a sample of rows matches the oracle."""
    import ctypes
    cfg = configs.softmax_layernorm()
    inputs = cfg.make_inputs()
    program, outs = run_gpu(gpu_session, cfg, inputs)
    got = outs[0].view(np.float32).reshape(32768, 4096)
    assert np.all(np.isfinite(got))
    assert np.abs(got.mean(axis=1, dtype=np.float64)).max() < 1e-4
    rows = np.concatenate([[0, 1, 4097, 16384, 32767], np.random.default_rng(19).integers(0, 32768, 251)])
    sub = np.ascontiguousarray(inputs[0][rows])
    ref = np.zeros_like(sub)
    lib = oracle.lib()
    lib.oracle_softmax_layernorm_f32(sub.ctypes.data_as(ctypes.c_void_p), ref.ctypes.data_as(ctypes.c_void_p),
                                     ctypes.c_size_t(len(rows)), ctypes.c_size_t(4096), ctypes.c_float(1e-5),
                                     ctypes.c_size_t(0), ctypes.c_size_t(len(rows)))
    # the exact rows: softmax then layer-norm in f64
    x = sub.astype(np.float64)
    e = np.exp(x - x.max(axis=1, keepdims=True))
    y = e / e.sum(axis=1, keepdims=True)
    c = y - y.mean(axis=1, keepdims=True)
    exact = c / np.sqrt((c * c).mean(axis=1, keepdims=True) + 1e-5)
    check_three_distances("softmax_layernorm 32768x4096, 256 rows", got[rows], ref, exact, 1e-3)


def test_mismatch_full_size_sample(gpu_session):
    import ctypes
    cfg = configs.mismatch()
    inputs = cfg.make_inputs()
    program, outs = run_gpu(gpu_session, cfg, inputs)
    got = outs[0].view(np.float32)
    assert np.all(np.isfinite(got)) and np.all(got >= 0)
    exact = np.zeros(16, np.float64)
    f = np.ascontiguousarray(inputs[0][:16])
    oracle.lib().oracle_mismatch_f64(f.ctypes.data_as(ctypes.c_void_p), inputs[1].ctypes.data_as(ctypes.c_void_p),
                                     inputs[2].ctypes.data_as(ctypes.c_void_p), exact.ctypes.data_as(ctypes.c_void_p),
                                     ctypes.c_size_t(16), ctypes.c_size_t(65536))
    assert rel_err(got[:16], exact, 1e-6) < 1e-5
    # 64 guesses spread over the whole output against the reference-order f32 fold as well
    picks = np.linspace(0, 8191, 64).astype(np.int64)
    f = np.ascontiguousarray(inputs[0][picks])
    ref = np.zeros(64, np.float32)
    exact = np.zeros(64, np.float64)
    args = (inputs[1].ctypes.data_as(ctypes.c_void_p), inputs[2].ctypes.data_as(ctypes.c_void_p))
    oracle.lib().oracle_mismatch_f32(f.ctypes.data_as(ctypes.c_void_p), args[0], args[1], ref.ctypes.data_as(ctypes.c_void_p),
                                     ctypes.c_size_t(64), ctypes.c_size_t(65536), ctypes.c_size_t(0), ctypes.c_size_t(64))
    oracle.lib().oracle_mismatch_f64(f.ctypes.data_as(ctypes.c_void_p), args[0], args[1], exact.ctypes.data_as(ctypes.c_void_p),
                                     ctypes.c_size_t(64), ctypes.c_size_t(65536))
    check_three_distances("mismatch 8192x65536, 64 guesses", got[picks], ref, exact, 1e-6)


@pytest.mark.parametrize("make,kept", [(lambda: configs.mlp(256, 256, 512), [1, 2, 3, 4, 5]),
                                       (lambda: configs.mlp(4096, 2048, 4096), [1, 2, 3, 4, 5]),
                                       (lambda: configs.softmax_layernorm(8192, 4096), [0])])
def test_resident_inputs_give_the_same_bytes(gpu_session, make, kept):
    """Inputs kept on the device by set_resident (weights; or, in the streamed invoke, an input
    that carries the chunked axis and is then read in place) give the same output bytes."""
    cfg = make()
    inputs = cfg.make_inputs()
    compiled = gpu_session.compile(cfg.program())
    want = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    gpu_session.invoke(compiled, inputs, [want])
    for i in kept:
        gpu_session.set_resident(compiled, i, inputs[i])
    got = np.zeros_like(want)
    gpu_session.invoke(compiled, [None if i in kept else a for i, a in enumerate(inputs)], [got])
    assert np.array_equal(got, want)
    got[:] = 0
    gpu_session.invoke(compiled, [None if i in kept else a for i, a in enumerate(inputs)], [got])
    assert np.array_equal(got, want)
    gpu_session.release(compiled)


def test_launch_timing_is_off_until_asked_for():
    """last_kernel_ms (the device vtable's elapsed_event_ns, deps/lib/compiler/gpu/src/contract.zig:2048-2085)
    answers only after time_launches(True); the measured time of a 268 MB row program lies between what
    HBM allows and a millisecond, and the result bytes do not depend on the switch."""
    session = tensor.Session(device=0)
    cfg = configs.softmax_layernorm(8192, 4096)
    inputs = cfg.make_inputs()
    compiled = session.compile(cfg.program())
    plain = np.empty(compiled.output_descriptors()[0].byte_size, np.uint8)
    session.invoke(compiled, inputs, [plain])
    with pytest.raises(tensor.SessionError) as e:
        compiled.last_kernel_ms()
    assert e.value.name == "launch_failed"
    session.time_launches(True)
    timed = np.zeros_like(plain)
    session.invoke(compiled, inputs, [timed])
    assert np.array_equal(plain, timed)
    import torch
    x = torch.from_numpy(inputs[0]).cuda()
    out = torch.empty(plain.size, dtype=torch.uint8, device="cuda")
    session.invoke_device(compiled, [x.data_ptr()], [out.data_ptr()])
    session.synchronize()
    ms = compiled.last_kernel_ms()
    assert 0.03 < ms < 1.0, ms
    assert np.array_equal(out.cpu().numpy(), plain)
    session.deinit()


@pytest.mark.parametrize("make", [lambda: configs.softmax_layernorm(8192, 4096), lambda: configs.mlp(4096, 2048, 4096),
                                  lambda: configs.attention(8, 4, 1024, 128)])
def test_chunked_host_invoke_equals_single_shot(make):
    """The streamed (chunked, three-lane) host invoke returns the same bytes as one launch over the whole input."""
    cfg = make()
    inputs = cfg.make_inputs()
    results = []
    for single in (0, 1):
        session = tensor.Session(device=0, single_shot_invoke=single)
        compiled = session.compile(cfg.program())
        outs = [np.empty(d.byte_size, np.uint8) for d in compiled.output_descriptors()]
        session.invoke(compiled, inputs, outs)
        session.invoke(compiled, inputs, outs)   # buffers are reused across invocations
        results.append(outs[0].copy())
        session.deinit()
    assert np.array_equal(results[0], results[1])


def _ulps(got, want64):
    want32 = want64.astype(np.float32)
    return np.abs(got.astype(np.float64) - want64) / np.abs(np.spacing(want32)).astype(np.float64)


def test_packed_sine_and_cosine_are_accurate_to_two_ulp(gpu_session):
    """The row kernels' own sine / cosine (packed FP32, no library call): each alone, and the joint
    routine used when a program takes both of the same value.  Against f64 over |x| <= 1e5, near
    multiples of pi/2, on the mismatch configuration's phases, and beyond 1e5 (where the thread
    falls back to sinf / cosf); infinities give NaN and NaN stays NaN."""
    rng = np.random.default_rng(31)
    n = 1 << 20
    parts = [rng.uniform(-100.0, 100.0, n // 4), rng.uniform(-1e5, 1e5, n // 4),
             np.pi / 2 * rng.integers(-63000, 63000, n // 4) + rng.uniform(-1e-3, 1e-3, n // 4),
             rng.uniform(0.0, 6.0, n // 4).astype(np.float32) * (0.25 * rng.integers(0, 65536, n // 4)).astype(np.float32)]
    x = np.concatenate(parts).astype(np.float32)
    x[:8] = [0.0, -0.0, 3.0e5, -7.5e6, np.inf, -np.inf, np.nan, 1.0e5]
    x64 = x.astype(np.float64)
    finite = np.isfinite(x)
    spec = [tensor.spec("f32", n=n)]
    programs = {"sine": lambda b, a: a[0].sin(), "cosine": lambda b, a: a[0].cos(),
                "both": lambda b, a: [a[0].sin(), a[0].cos()]}
    for name, body in programs.items():
        program = tensor.define("packed_" + name, spec, body)
        compiled = gpu_session.compile(program)
        assert ("w0 ?" in compiled.kernels()[0][1]) == (name == "both")   # the joint routine only where both are asked for
        outs = [np.empty(n, np.float32) for _ in program.output_types]
        gpu_session.invoke(compiled, [x], outs)
        gpu_session.release(compiled)
        wants = {"sine": [np.sin], "cosine": [np.cos], "both": [np.sin, np.cos]}[name]
        for got, fn in zip(outs, wants):
            with np.errstate(invalid="ignore"):
                want = fn(x64)
            assert np.all(np.isnan(got[~finite]))
            assert _ulps(got[finite], want[finite]).max() < 2.0, name


def test_packed_exp_is_accurate_to_three_ulp(gpu_session):
    """The row kernels' own exp (2^x of the special-function unit with the argument's rounding error
    carried into the result): against f64 over the whole finite range, at the overflow and
    underflow edges, and for infinities and NaN (where the thread falls back to expf).  Results
    below 2^-126 may be flushed to zero (expf returns subnormal numbers there)."""
    rng = np.random.default_rng(37)
    n = 1 << 20
    x = np.concatenate([rng.uniform(-104.0, 89.0, n // 2), rng.uniform(-30.0, 0.0, n // 4), rng.standard_normal(n // 4) * 3.0]).astype(np.float32)
    x[:16] = [0.0, -0.0, np.inf, -np.inf, np.nan, 88.7, 88.73, 89.0, -87.0, -87.4, -90.0, -103.0, -110.0, 1e30, -1e30, 1.0]
    program = tensor.define("packed_exp", [tensor.spec("f32", n=n)], lambda b, a: a[0].exp())
    compiled = gpu_session.compile(program)
    assert "ex2_ftz(-nh0)" in compiled.kernels()[0][1]
    got = np.empty(n, np.float32)
    gpu_session.invoke(compiled, [x], [got])
    gpu_session.release(compiled)
    with np.errstate(over="ignore", invalid="ignore"):
        want = np.exp(x.astype(np.float64))
    assert np.isnan(got[4]) and got[2] == np.inf and got[3] == 0.0 and got[13] == np.inf and got[14] == 0.0
    assert got[0] == 1.0 and got[1] == 1.0
    overflow = want > float(np.finfo(np.float32).max)
    assert np.all(got[overflow & ~np.isnan(want)] == np.inf)
    normal = np.isfinite(want) & (want >= 2.0 ** -126) & ~overflow
    assert _ulps(got[normal], want[normal]).max() < 3.0
    tiny = np.isfinite(want) & (want < 2.0 ** -126)
    assert np.all(np.abs(got[tiny].astype(np.float64) - want[tiny]) <= 2.0 ** -126)
    print("packed exp: max %.2f ulp, mean %.3f ulp" % (_ulps(got[normal], want[normal]).max(), _ulps(got[normal], want[normal]).mean()))
