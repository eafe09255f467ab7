"""Running one recorded program across the GPUs of a box: one process (rank) per GPU.

The reference executes on a single device and has no collective of any kind, so this module has
no counterpart there.  A program is cut along a named batch-like axis with
`tensor.shard_program`; each rank compiles the piece for its own block of the axis and runs it on
its own rows, with no exchange between ranks.  Only when the chosen axis is the one the program
folds over (sum, max or min as its last step) do the ranks hold partial results, which one
all-reduce with the same operation combines (NCCL on GPUs, gloo in the CPU tests of the host logic).
"""
import numpy as np

from . import tensor


class ShardPlan:
    """Which slice of every input and output a rank owns when `program` is cut along `axis`."""

    def __init__(self, program, axis, world):
        self.program = program
        self.axis = axis
        self.world = world
        extent = None
        for t in list(program.input_types) + list(program.output_types):
            for name, e in t.dims:
                if name == axis:
                    extent = e
        if extent is None:
            raise tensor.SessionError(7, "no input or output carries axis '%s'" % axis)
        if extent % world != 0:
            raise tensor.SessionError(7, "axis '%s' of extent %d does not divide over %d ranks" % (axis, extent, world))
        self.extent = extent
        self.local_extent = extent // world
        self.piece, self.partial_sum = tensor.shard_program(program, axis, self.local_extent)

    def _slice(self, ty, rank):
        """(byte offset, byte length) of rank's block of a buffer of type `ty`."""
        total = ty.byte_count()
        if not ty.dims or ty.dims[0][0] != self.axis:
            return 0, total            # replicated: every rank holds the whole buffer
        per = total // self.world
        return rank * per, per

    def input_slices(self, rank):
        return [self._slice(t, rank) for t in self.program.input_types]

    def output_slices(self, rank):
        if self.partial_sum:
            return [(0, t.byte_count()) for t in self.program.output_types]
        return [self._slice(t, rank) for t in self.program.output_types]

    def local_inputs(self, rank, inputs):
        """Views of this rank's block of each full input (numpy arrays or bytes-like)."""
        out = []
        for buf, (offset, length) in zip(inputs, self.input_slices(rank)):
            raw = np.ascontiguousarray(buf).reshape(-1).view(np.uint8) if isinstance(buf, np.ndarray) else \
                np.frombuffer(buf, np.uint8)
            out.append(raw[offset:offset + length])
        return out


class ShardedCuda:
    """The multi-GPU counterpart of `tensor.Cuda`: rank `rank` of `world` runs its piece on `device`.

    `launch(local_inputs, local_outputs)` takes this rank's blocks (see ShardPlan); when the plan
    yields partial sums it finishes with one all-reduce over `group` (torch.distributed)."""

    def __init__(self, program, axis, rank, world, device=0, group=None):
        self.plan = ShardPlan(program, axis, world)
        self.rank = rank
        self.group = group
        self.executor = tensor.Cuda(self.plan.piece, device=device)

    def launch(self, local_inputs, local_outputs):
        self.executor.launch(local_inputs, local_outputs)
        if self.plan.partial_sum and self.plan.world > 1:
            all_reduce_partials(local_outputs, self.plan.piece.output_types, self.group, fold=self.plan.partial_sum.name)

    def deinit(self):
        self.executor.deinit()


_TORCH_DTYPES = {"f32": "float32", "f64": "float64", "i32": "int32", "i64": "int64"}


def all_reduce_partials(outputs, types, group=None, fold="sum"):
    """Combines the per-rank partial results in place: one all-reduce per output buffer, adding
    them or taking their maximum / minimum (`fold`, ShardPlan.partial_sum.name)."""
    import torch
    import torch.distributed as dist
    for buf, ty in zip(outputs, types):
        if ty.dtype not in _TORCH_DTYPES:
            raise tensor.SessionError(7, "partial sums of dtype %s cannot be all-reduced" % ty.dtype)
        if isinstance(buf, torch.Tensor):
            t = buf.view(getattr(torch, _TORCH_DTYPES[ty.dtype]))
        else:
            t = torch.from_numpy(np.asarray(buf).reshape(-1).view(getattr(np, _TORCH_DTYPES[ty.dtype])))
        op = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[fold]
        if not t.is_cuda and "nccl" in str(dist.get_backend(group)):
            # host buffers (what `launch` fills) with an NCCL group: the collective runs on device memory
            staged = t.cuda()
            dist.all_reduce(staged, op=op, group=group)
            t.copy_(staged)
        else:
            dist.all_reduce(t, op=op, group=group)
