"""The N>1 path on CPU: two gloo ranks shard a program, run their pieces and (when the sharded axis
is the summed one) all-reduce the partial sums.  No GPU is involved: the host logic under test is
the shard plan, the per-rank slices and the collective; the pieces are evaluated by the CPU oracle,
which here stands in for the device."""
import os
import socket

import numpy as np
import pytest

from accy_b200 import configs, shard
from oracle import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, case, result_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg, axis = _case(case)
        program = cfg.program()
        inputs = cfg.make_inputs()
        plan = shard.ShardPlan(program, axis, world)
        local = plan.local_inputs(rank, inputs)
        outs = oracle.run(plan.piece.wire, [bytes(b) for b in local])
        if plan.partial_sum:
            shard.all_reduce_partials(outs, plan.piece.output_types, fold=plan.partial_sum.name)
        np.save(os.path.join(result_dir, "rank%d.npy" % rank), outs[0])
        with open(os.path.join(result_dir, "rank%d.txt" % rank), "w") as f:
            f.write("%d %s %s" % (int(plan.partial_sum), plan.output_slices(rank), plan.input_slices(rank)))
    finally:
        dist.destroy_process_group()


def _case(name):
    if name == "rows":
        return configs.softmax_layernorm(8, 64), "row"
    if name == "guesses":
        return configs.mismatch(6, 128), "guess"
    if name == "column_maxima":
        return _ColumnExtreme("max"), "row"
    if name == "column_minima":
        return _ColumnExtreme("min"), "row"
    if name == "column_maxima_from_start":
        return _ColumnExtreme("max", start=0.25), "row"
    return configs.mismatch(6, 128), "point"


class _ColumnExtreme:
    """max / min over the sharded axis: the ranks' partial extremes combine with the same operation"""

    def __init__(self, which, start=None):
        self.which = which
        self.start = start

    def program(self):
        from accy_b200 import tensor
        if self.start is not None:
            # a recorded start value: every rank takes it in again, which an extreme does not mind
            return tensor.define("column_" + self.which, [tensor.spec("f32", row=8, col=16)],
                                 lambda b, a: a[0].reduce(b.scalar("f32", self.start), self.which, "row"))
        return tensor.define("column_" + self.which, [tensor.spec("f32", row=8, col=16)],
                             lambda b, a: getattr(a[0], self.which)("row"))

    def make_inputs(self):
        return [np.random.default_rng(3).standard_normal((8, 16)).astype(np.float32)]


@pytest.mark.parametrize("case", ["rows", "guesses", "points", "column_maxima", "column_minima", "column_maxima_from_start"])
def test_two_ranks_reproduce_the_single_device_result(case, tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)
    cfg, axis = _case(case)
    full = oracle.run(cfg.program().wire, cfg.make_inputs())[0]
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npy" % r)) for r in range(world)]
    if case.startswith("column_"):
        # extremes are exact whatever the split
        assert np.array_equal(parts[0], full) and np.array_equal(parts[1], full)
    elif case == "points":
        # the summed axis was split: every rank holds the all-reduced total
        for p in parts:
            assert np.allclose(p, full, rtol=1e-5)
        assert np.array_equal(parts[0], parts[1])
    else:
        # independent pieces: rank r holds rows [r*n/2, (r+1)*n/2) bit for bit
        assert np.array_equal(np.concatenate(parts, axis=0), full)


def test_shard_plan_slices():
    program = configs.mismatch(8, 64).program()
    plan = shard.ShardPlan(program, "guess", 4)
    assert not plan.partial_sum and plan.local_extent == 2
    assert plan.input_slices(3) == [(24, 8), (0, 256), (0, 256)]      # frequency sliced, time/sample replicated
    assert plan.output_slices(1) == [(8, 8)]
    plan = shard.ShardPlan(program, "point", 2)
    assert plan.partial_sum
    assert plan.input_slices(1) == [(0, 32), (128, 128), (128, 128)]
    assert plan.output_slices(1) == [(0, 32)]
    with pytest.raises(Exception):
        shard.ShardPlan(program, "guess", 3)


def test_a_sum_from_a_non_zero_start_is_not_cut_along_its_axis():
    """Every piece would add the recorded start value again and the all-reduce would add the pieces:
    total + world * start.  The shard planner refuses the axis; the kept axis still shards."""
    from accy_b200 import tensor
    program = tensor.define("sum_from_five", [tensor.spec("f32", row=8, col=16)],
                            lambda b, a: a[0].reduce(b.scalar("f32", 5.0), "sum", "row"))
    with pytest.raises(tensor.SessionError) as e:
        shard.ShardPlan(program, "row", 2)
    assert "initial value" in str(e.value)
    kept = tensor.define("row_sums_from_five", [tensor.spec("f32", row=8, col=16)],
                         lambda b, a: a[0].reduce(b.scalar("f32", 5.0), "sum", "col"))
    plan = shard.ShardPlan(kept, "row", 2)
    assert not plan.partial_sum
    x = np.random.default_rng(5).standard_normal((8, 16)).astype(np.float32)
    full = oracle.run(kept.wire, [x])[0]
    halves = [oracle.run(plan.piece.wire, [np.ascontiguousarray(x[r * 4:(r + 1) * 4])])[0] for r in range(2)]
    assert np.array_equal(np.concatenate(halves), full)
