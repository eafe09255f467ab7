"""Two ranks on two GPUs (NCCL): each runs its piece of a sharded program through the C ABI; a program
that folds over the sharded axis ends with one all-reduce of its partial results.  Skipped on a
machine with fewer than two GPUs (the host logic is covered on CPU by test_multi_rank_cpu.py)."""
import os
import socket

import numpy as np
import pytest

from accy_b200 import configs, shard, tensor
from oracle import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case(name):
    if name == "points_sum":
        cfg = configs.mismatch(64, 8192)
        return cfg.program(), cfg.make_inputs(), "point"
    if name == "guesses_blocks":
        cfg = configs.mismatch(64, 8192)
        return cfg.program(), cfg.make_inputs(), "guess"
    which = "max" if name == "rows_max" else "min"
    program = tensor.define("column_" + which, [tensor.spec("f32", row=512, col=1024)],
                            lambda b, a: getattr(a[0].mul(a[0]).sub(a[0]), which)("row"))
    return program, [np.random.default_rng(9).standard_normal((512, 1024)).astype(np.float32)], "row"


def _rank_main(rank, world, port, case, result_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        program, inputs, axis = _case(case)
        runner = shard.ShardedCuda(program, axis, rank, world, device=rank)
        plan = runner.plan
        local_inputs = plan.local_inputs(rank, inputs)
        outs = [np.empty(length, np.uint8) for _, length in plan.output_slices(rank)]
        runner.launch(local_inputs, outs)
        np.save(os.path.join(result_dir, "rank%d.npy" % rank), outs[0].view(np.float32))
        runner.deinit()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["points_sum", "guesses_blocks", "rows_max", "rows_min"])
def test_two_gpus_reproduce_the_single_device_result(case, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)
    program, inputs, _ = _case(case)
    full = oracle.run(program.wire, inputs)[0].reshape(-1)
    exact = np.asarray(oracle.run(program.wire, inputs, mode="f64")[0], np.float64).reshape(-1)
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npy" % r)) for r in range(world)]
    if case == "guesses_blocks":
        got = np.concatenate(parts)
    else:
        assert np.array_equal(parts[0], parts[1])   # every rank holds the combined result
        got = parts[0]
    if case.startswith("rows_"):
        assert np.array_equal(got, full)            # extremes do not depend on the split
    else:
        err_ref = np.max(np.abs(full - exact) / np.abs(exact))
        assert np.max(np.abs(got - exact) / np.abs(exact)) < 1e-5 + err_ref
