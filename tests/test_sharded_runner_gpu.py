"""accy_b200_sharded_* on the GPU: one process cuts a program into pieces, runs them side by side
(one session and one host thread per piece) and returns the whole program's result in the caller's
buffers.  With two or more GPUs the pieces go to different devices; on a one-GPU machine the same
ordinal is named several times, which exercises everything but the second device.  Results are
compared with the CPU oracle: sliced outputs bit for bit against the single-device run as well."""
import numpy as np
import pytest

from accy_b200 import configs, tensor
from oracle import oracle
from parity_checks import check_three_distances

pytestmark = pytest.mark.gpu


def device_list(pieces):
    import torch
    count = max(1, torch.cuda.device_count())
    return [d % count for d in range(pieces)]


def single(cfg, inputs):
    outs = [np.empty(t.byte_count(), np.uint8) for t in cfg.program().output_types]
    tensor.run_cuda(cfg.program(), inputs, outs, device=0)
    return outs


@pytest.mark.parametrize("pieces", [2, 4])
def test_rows_are_cut_with_no_exchange(pieces):
    cfg = configs.softmax_layernorm(1024, 2048)
    inputs = cfg.make_inputs()
    multi = tensor.MultiCuda(cfg.program(), "row", device_list(pieces))
    out = np.zeros(1024 * 2048, np.float32)
    multi.launch(inputs, [out])
    multi.launch(inputs, [out])          # buffers and kernels are reused
    multi.deinit()
    assert np.array_equal(out.view(np.uint8), single(cfg, inputs)[0])   # a row does not care which piece it is in
    program = cfg.program()
    check_three_distances("sharded softmax_layernorm x%d" % pieces, out, oracle.run(program.wire, inputs)[0],
                          oracle.run(program.wire, inputs, mode="f64")[0], 1e-3)


def test_guesses_are_cut_and_vectors_replicated():
    cfg = configs.mismatch(96, 20000)
    inputs = cfg.make_inputs()
    multi = tensor.MultiCuda(cfg.program(), "guess", device_list(3))
    out = np.zeros(96, np.float32)
    multi.launch(inputs, [out])
    multi.deinit()
    program = cfg.program()
    check_three_distances("sharded mismatch by guess", out, oracle.run(program.wire, inputs)[0],
                          oracle.run(program.wire, inputs, mode="f64")[0], 1e-6)


def test_the_summed_axis_gives_partial_sums_combined_in_device_order():
    cfg = configs.mismatch(24, 1 << 16)
    inputs = cfg.make_inputs()
    results = []
    for _ in range(2):
        multi = tensor.MultiCuda(cfg.program(), "point", device_list(4))
        out = np.zeros(24, np.float32)
        multi.launch(inputs, [out])
        multi.deinit()
        results.append(out)
    assert np.array_equal(results[0], results[1])      # fixed order of the host-side fold: run-to-run identical
    program = cfg.program()
    check_three_distances("sharded mismatch by point", results[0], oracle.run(program.wire, inputs)[0],
                          oracle.run(program.wire, inputs, mode="f64")[0], 1e-6)


def test_column_maxima_combine_exactly():
    program = tensor.define("column_max", [tensor.spec("f32", row=512, col=300)], lambda b, a: a[0].max("row"))
    x = np.random.default_rng(9).standard_normal((512, 300)).astype(np.float32)
    multi = tensor.MultiCuda(program, "row", device_list(4))
    out = np.zeros(300, np.float32)
    multi.launch([x], [out])
    multi.deinit()
    assert np.array_equal(out, x.max(axis=0))


def test_bf16_matmul_rows_on_tensor_cores():
    cfg = configs.matmul(1024, 512, 256)
    inputs = cfg.make_inputs()
    multi = tensor.MultiCuda(cfg.program(), "m", device_list(2))
    out = np.zeros(1024 * 512, np.uint16)
    multi.launch(inputs, [out])
    multi.deinit()
    assert np.array_equal(out.view(np.uint8), single(cfg, inputs)[0])
