"""GPU parity of the tcgen05 kernels on the paths the benchmark runs: CTAs (or CTA pairs, where two
CTAs share a 256-row tile through cta_group::2) that take several output tiles (both accumulator
buffers, accumulator phases 0 and 1), k extents that wrap the shared-memory stage ring several
times, and the five BASELINE sizes themselves by sampled rows.

The oracle side evaluates only the sampled rows (`oracle.matmul_rows`, `attention_rows`,
`mlp_rows`: the same k-serial f32 folds of dot.zig:2049-2115 and the SDPA restatement of
src/kernel/library/attention.zig:473-509), so the full-size cases stay within seconds of CPU time.
Rows are spread so that every row block of the output, and with it every tile of every CTA's walk,
has rows under comparison; all columns of a sampled row are compared.

Tolerance: bf16 2e-2 as |got - want| <= 2e-2 * (|want| + rms(want)), f32 row programs 1e-5.
"""
import math

import numpy as np
import pytest

from accy_b200 import configs, tensor
from oracle import oracle

pytestmark = pytest.mark.gpu


def bf16(a):
    return configs.f32_to_bf16_bits(np.asarray(a, np.float32))


def widen(bits):
    return configs.bf16_bits_to_f32(bits)


def rel_err_bf16(got, want):
    want = np.asarray(want, np.float64).reshape(-1)
    got = np.asarray(got, np.float64).reshape(-1)
    rms = max(float(np.sqrt(np.mean(want * want))), 1e-30)
    return float(np.max(np.abs(got - want) / (np.abs(want) + rms)))


def spread_rows(extent, block, per_block, seed):
    """`per_block` rows of every `block`-row block (first and last row of the block among them)"""
    rng = np.random.default_rng(seed)
    rows = []
    for lo in range(0, extent, block):
        hi = min(extent, lo + block)
        pick = {lo, hi - 1}
        while len(pick) < min(per_block, hi - lo):
            pick.add(int(rng.integers(lo, hi)))
        rows.extend(sorted(pick))
    return np.array(rows, np.uint64)


def run(session, program, inputs, guard=4096):
    compiled = session.compile(program)
    summary = compiled.plan_summary()
    size = compiled.output_descriptors()[0].byte_size
    out = np.full(size + guard, 0x5A, np.uint8)
    session.invoke(compiled, inputs, [out[:size]])
    session.release(compiled)
    assert np.all(out[size:] == 0x5A), "bytes behind the output were written"
    return out[:size], summary


# name: (lhs dims, rhs dims, contracted axis); every case has more tiles than the GPU has SMs and
# more k-blocks than the stage ring has stages
MULTI_TILE_GEMMS = {
    # 16 x 16 tiles of 128 x 256, 16 k-blocks
    "plain_256_tiles": ((("m", 2048), ("k", 1024)), (("k", 1024), ("n", 4096))),
    # n is not a multiple of 256: 128 x 128 tiles, 16 x 17 of them
    "n_not_multiple_of_256": ((("m", 2048), ("k", 1024)), (("k", 1024), ("n", 2176))),
    # nothing is a multiple of the tile: 16 x 24 tiles with ragged edges, the last k-block is partial
    "ragged_everywhere": ((("m", 2000), ("k", 1000)), (("k", 1000), ("n", 3000))),
    # rhs stored [n, k] (K-major B)
    "k_major_rhs": ((("m", 1536), ("k", 832)), (("n", 4096), ("k", 832))),
    # lhs stored [k, m] (M-major A tiles, what gradients of contractions read)
    "transposed_lhs": ((("k", 1024), ("m", 2048)), (("k", 1024), ("n", 4096))),
    # one 128-row block: the one-CTA kernel (no CTA pair), 150 tiles of 128 x 256, 9 k-blocks
    "single_row_block_many_columns": ((("m", 128), ("k", 576)), (("k", 576), ("n", 38400))),
    # 257 rows: the second CTA pair's lower CTA has one row inside the matrix, the rest of its tile is outside
    "one_row_past_a_pair": ((("m", 257), ("k", 640)), (("k", 640), ("n", 19456))),
}


@pytest.mark.parametrize("name", sorted(MULTI_TILE_GEMMS))
def test_gemm_with_several_tiles_per_cta_matches_oracle(gpu_session, name):
    lhs_dims, rhs_dims = MULTI_TILE_GEMMS[name]
    program = tensor.define("gemm_" + name, [tensor.spec("bf16", **dict(lhs_dims)), tensor.spec("bf16", **dict(rhs_dims))],
                            lambda b, a: a[0].contract(a[1], "k"))
    rng = np.random.default_rng(len(name))
    lhs = bf16(rng.standard_normal([e for _, e in lhs_dims]) / 8.0)
    rhs = bf16(rng.standard_normal([e for _, e in rhs_dims]) / 8.0)
    out, summary = run(gpu_session, program, [lhs, rhs])
    assert "tcgen05" in summary
    m, n = dict(lhs_dims)["m"], dict(rhs_dims)["n"]
    got = widen(out.view(np.uint16)).reshape(m, n)
    a_mk = lhs if lhs_dims[0][0] == "m" else np.ascontiguousarray(lhs.T)
    b_kn = rhs if rhs_dims[0][0] == "k" else np.ascontiguousarray(rhs.T)
    rows = spread_rows(m, 128, 6, seed=3)
    want = oracle.matmul_rows(a_mk, b_kn, rows)
    assert rel_err_bf16(got[rows.astype(np.int64)], widen(bf16(want))) < 2e-2
    # every row, every column, against a second computation (f64 product of the widened inputs):
    # no tile of any CTA's walk may be skipped, repeated or written to the wrong place
    full = (widen(a_mk).astype(np.float64) @ widen(b_kn).astype(np.float64))
    assert rel_err_bf16(got, full) < 2e-2


def test_batched_gemm_with_several_tiles_per_cta_matches_oracle(gpu_session):
    """6 batches of 8 x 4 tiles (192 tiles), 9 k-blocks, rhs K-major in three of the comparisons' worth."""
    g, m, k, n = 6, 1024, 576, 1024
    program = tensor.define("gemm_batched", [tensor.spec("bf16", g=g, m=m, k=k), tensor.spec("bf16", g=g, k=k, n=n)],
                            lambda b, a: a[0].contract(a[1], "k"))
    rng = np.random.default_rng(41)
    lhs = bf16(rng.standard_normal((g, m, k)) / 8.0)
    rhs = bf16(rng.standard_normal((g, k, n)) / 8.0)
    out, summary = run(gpu_session, program, [lhs, rhs])
    assert "tcgen05" in summary
    got = widen(out.view(np.uint16)).reshape(g, m, n)
    rows = spread_rows(m, 128, 4, seed=5)
    for b in range(g):
        want = oracle.matmul_rows(lhs[b], rhs[b], rows)
        assert rel_err_bf16(got[b][rows.astype(np.int64)], widen(bf16(want))) < 2e-2, b
        full = widen(lhs[b]).astype(np.float64) @ widen(rhs[b]).astype(np.float64)
        assert rel_err_bf16(got[b], full) < 2e-2, b


def test_mlp_with_several_tiles_per_cta_matches_oracle(gpu_session):
    """GEMM + bias + GELU epilogue (256 tiles), second GEMM (64 tiles, 64 k-blocks), RMSNorm."""
    cfg = configs.mlp(2048, 1024, 4096)
    inputs = cfg.make_inputs()
    rng = np.random.default_rng(9)
    inputs[2] = bf16(rng.standard_normal(4096) * 0.1)       # non-zero biases and norm weights
    inputs[4] = bf16(rng.standard_normal(1024) * 0.1)
    inputs[5] = bf16(1.0 + rng.standard_normal(1024) * 0.1)
    out, summary = run(gpu_session, cfg.program(), inputs)
    assert summary.count("tcgen05") >= 2
    got = widen(out.view(np.uint16)).reshape(2048, 1024)
    rows = spread_rows(2048, 128, 4, seed=7)
    want = oracle.mlp_rows(*inputs, rows=rows)
    assert rel_err_bf16(got[rows.astype(np.int64)], want) < 2e-2
    assert np.all(np.isfinite(got))


# ---- the BASELINE sizes themselves ----------------------------------------------------------
def test_matmul_full_size_sampled_rows(gpu_session):
    """C3, bf16 8192^3: 2048 tiles (13.8 per CTA), 128 k-blocks.  Two rows of each of the 64 row
    blocks, all 8192 columns, against the k-serial f32 oracle; plus a checksum over every row."""
    cfg = configs.matmul()
    a, b = cfg.make_inputs()
    out, summary = run(gpu_session, cfg.program(), [a, b])
    assert "tcgen05" in summary
    got = widen(out.view(np.uint16)).reshape(8192, 8192)
    rows = spread_rows(8192, 128, 2, seed=11)
    want = oracle.matmul_rows(a, b, rows)
    assert rel_err_bf16(got[rows.astype(np.int64)], widen(bf16(want))) < 2e-2
    # linearity: C.1 = A.(B.1) for every row (catches a tile written to the wrong rows or never written)
    row_sums = got.astype(np.float64).sum(axis=1)
    expect = widen(a).astype(np.float64) @ widen(b).astype(np.float64).sum(axis=1)
    scale = np.sqrt(8192.0) * float(np.sqrt(np.mean(got.astype(np.float64) ** 2)))
    assert np.max(np.abs(row_sums - expect)) < 2e-2 * scale


def test_attention_full_size_sampled_rows(gpu_session):
    """C4, bf16 batch 8 x head 32 x seq 4096 x dim 128, causal: 4096 work items (27.7 per CTA), up
    to 32 key blocks.  Heads 0, 101 and 255 (the last items of the work queue), two query rows of
    each 128-row tile, against the SDPA oracle."""
    cfg = configs.attention()
    q, k, v = cfg.make_inputs()
    out, summary = run(gpu_session, cfg.program(), [q, k, v])
    assert "attention:" in summary
    got = widen(out.view(np.uint16)).reshape(256, 4096, 128)
    assert np.all(np.isfinite(got))
    queries = spread_rows(4096, 128, 2, seed=13)
    heads = np.repeat(np.array([0, 101, 255], np.uint64), len(queries))
    rows = np.tile(queries, 3)
    want = oracle.attention_rows(q.reshape(256, 4096, 128), k.reshape(256, 4096, 128), v.reshape(256, 4096, 128),
                                 heads, rows, 1.0 / math.sqrt(128.0), causal=True)
    picked = got[heads.astype(np.int64), rows.astype(np.int64)]
    assert rel_err_bf16(picked, want) < 2e-2
    # every head: query 0 attends to key 0 only, so its output row is V[0]
    assert np.array_equal(out.view(np.uint16).reshape(256, 4096, 128)[:, 0, :], v.reshape(256, 4096, 128)[:, 0, :])


def test_mlp_full_size_sampled_tokens(gpu_session):
    """C5, bf16 tokens 16384, d 4096, h 16384: 8192 + 2048 tiles.  One token of each of the 128 row
    blocks against the oracle; every output row has unit mean square (RMSNorm with weight one)."""
    cfg = configs.mlp()
    inputs = cfg.make_inputs()
    out, summary = run(gpu_session, cfg.program(), inputs)
    assert summary.count("tcgen05") >= 2
    got = widen(out.view(np.uint16)).reshape(16384, 4096)
    rng = np.random.default_rng(17)
    rows = np.array([lo + int(rng.integers(0, 128)) for lo in range(0, 16384, 128)], np.uint64)
    want = oracle.mlp_rows(*inputs, rows=rows)
    assert rel_err_bf16(got[rows.astype(np.int64)], want) < 2e-2
    mean_square = (got.astype(np.float64) ** 2).mean(axis=1)
    assert np.all(np.abs(mean_square - 1.0) < 2e-2)


@pytest.mark.parametrize("make", [lambda: configs.matmul(2304, 1024, 2048),          # nine tile pairs, 32 k-blocks each
                                  lambda: configs.matmul(1000, 1032, 264),           # ragged in m, n and k
                                  lambda: configs.attention(1, 37, 2048, 128, True), # 296 work items on 148 CTAs
                                  lambda: configs.mlp(1024, 1024, 2048)])
def test_repeated_device_launches_give_identical_bytes(make):
    """The tensor-core kernels keep state between launches of one compiled program (stage-ring and
    accumulator phases, the work counter of the persistent attention kernel) and run with whatever
    timing the GPU gives them: twenty back-to-back launches on device buffers, each into a cleared
    output, give the bytes of the first."""
    import torch
    cfg = make()
    inputs = cfg.make_inputs()
    session = tensor.Session(device=0)
    compiled = session.compile(cfg.program())
    d_in = [torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda() for a in inputs]
    nbytes = compiled.output_descriptors()[0].byte_size
    first = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    outs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(20)]
    torch.cuda.synchronize()   # the session launches on a stream of its own
    session.invoke_device(compiled, [t.data_ptr() for t in d_in], [first.data_ptr()])
    session.synchronize()
    assert first.any()
    for out in outs:
        session.invoke_device(compiled, [t.data_ptr() for t in d_in], [out.data_ptr()])
    session.synchronize()
    for out in outs:
        assert torch.equal(out, first)
    session.deinit()


def random_gemm(seed):
    """A seeded random bf16 contraction: extents from 1 to about 700 (multiples of eight and not),
    either operand stored either way round, an optional leading batch axis, an optional epilogue
    (bias, bias + tanh, scale, bias added to a product with a second matrix): (specs, body)."""
    rng = np.random.default_rng(7000 + seed)
    def extent():
        e = int(rng.integers(1, 700))
        return e if rng.random() < 0.4 else max(8, e // 8 * 8)
    m, n, k = extent(), extent(), extent()
    g = int(rng.choice([0, 0, 2, 3]))
    lhs = [("m", m), ("k", k)] if rng.random() < 0.6 else [("k", k), ("m", m)]
    rhs = [("k", k), ("n", n)] if rng.random() < 0.6 else [("n", n), ("k", k)]
    if g:
        lhs, rhs = [("g", g)] + lhs, [("g", g)] + rhs
    epilogue = str(rng.choice(["none", "bias", "bias_tanh", "scale", "residual"]))
    specs = [tensor.spec("bf16", **dict(lhs)), tensor.spec("bf16", **dict(rhs))]
    if epilogue in ("bias", "bias_tanh"):
        specs.append(tensor.spec("bf16", n=n))
    if epilogue == "residual":
        specs.append(tensor.spec("bf16", **dict(([("g", g)] if g else []) + [("m", m), ("n", n)])))

    def body(b, a):
        y = a[0].contract(a[1], "k")
        if epilogue == "bias":
            y = y.add(a[2])
        elif epilogue == "bias_tanh":
            y = y.add(a[2]).tanh()
        elif epilogue == "scale":
            y = y.mul(b.scalar("bf16", 0.5))
        elif epilogue == "residual":
            y = y.add(a[2])
        return y

    return specs, body, "m%d n%d k%d g%d %s %s %s" % (m, n, k, g, "".join(d for d, _ in lhs), "".join(d for d, _ in rhs), epilogue)


@pytest.mark.parametrize("seed", range(24))
def test_random_bf16_contractions_match_the_oracle(gpu_session, seed):
    """Whatever kernel the planner picks for the shape (the two-CTA or the one-CTA tcgen05 kernel, or the
    exact-order SIMT kernel where a TMA rule keeps the tensor cores out), the result matches the f32
    evaluation on the bf16-rounded inputs and nothing behind the output is written."""
    specs, body, label = random_gemm(seed)
    program = tensor.define("random_gemm_%d" % seed, specs, body)
    rng = np.random.default_rng(seed)
    inputs = [bf16(rng.standard_normal([e for _, e in sp.dims]) / 4.0) for sp in specs]
    out, summary = run(gpu_session, program, inputs)
    want = widen(oracle.run(program.wire, inputs, mode="wide")[0]).reshape(-1)
    got = widen(out.view(np.uint16))
    err = rel_err_bf16(got, want)
    print(label, "->", "tcgen05" if "accy_gemm_tc" in summary else "simt", "err %.3g" % err)
    assert err < 2e-2, (label, err)
