"""Host-side mirror of the reference's `accy.tensor` interface for the B200 target.

Recording: `define(name, specs, body)` calls `body(builder, args)` on placeholder `Value`s with
named axes and records every operation, as the reference's `tensor.define` does
(src/tensor/trace/define.zig:8-19); `Value` has the reference's methods with the same names and
argument meaning (src/tensor/trace/value.zig:13-155) and `Builder` its constructors
(src/tensor/trace/builder.zig: `scalar`, `full`, `iota`).  Failures raise `TensorError` whose
`name` is the reference's Zig error name (e.g. "AxisExtentMismatch").

Execution: `run_cuda(program, inputs, outputs)` has `runCpu`'s byte-slice contract
(src/tensor/execute.zig:54-63): inputs in parameter order, outputs in output order, each buffer
exactly the declared byte size; `Cuda(program)` / `.launch` / `.deinit` mirror `Cpu`
(execute.zig:9-51); `Session` mirrors `tensor.session.Session` (src/tensor/session/session.zig).
All of them go through the C ABI of libaccy_b200.so and run CUDA kernels only.
"""
import ctypes
import struct

import numpy as np

from . import _native
from ._native import lib

DTYPES = ["i1", "i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "f16", "bf16", "f32", "f64", "key"]
DTYPE_SIZE = {"i1": 1, "i8": 1, "i16": 2, "i32": 4, "i64": 8, "u8": 1, "u16": 2, "u32": 4, "u64": 8,
              "f16": 2, "bf16": 2, "f32": 4, "f64": 8, "key": 8}
UNARY = ["neg", "abs", "exp", "log", "sqrt", "tanh", "sin", "cos", "tan"]
BINARY = ["add", "sub", "mul", "div", "max", "min", "pow"]
REDUCER = ["sum", "max", "min"]
COMPARE = ["lt", "le", "gt", "ge", "eq", "ne"]
STATUS = ["ok", "invalid_program", "unsupported_version", "invalid_handle", "invalid_buffer",
          "too_many_programs", "out_of_memory", "compile_failed", "launch_failed"]


class TensorError(Exception):
    """A recording failure; `name` is the reference's error name."""

    def __init__(self, name):
        super().__init__(name)
        self.name = name


class SessionError(Exception):
    """A session failure; `status` is the stable status number, `name` its reference name."""

    def __init__(self, status, message):
        super().__init__("%s: %s" % (STATUS[status] if status < len(STATUS) else status, message))
        self.status = status
        self.name = STATUS[status] if status < len(STATUS) else str(status)
        self.message = message


class Spec:
    """dtype + ordered named axes: the reference's `tensor.spec(.f32, .{ .guess = 8 })`."""

    def __init__(self, dtype, dims):
        self.dtype = dtype
        self.dims = list(dims)


def spec(dtype, **dims):
    return Spec(dtype, list(dims.items()))


def _names_extents(dims):
    dims = list(dims.items()) if isinstance(dims, dict) else list(dims)
    names = (ctypes.c_char_p * max(1, len(dims)))(*[n.encode() for n, _ in dims])
    extents = (ctypes.c_int64 * max(1, len(dims)))(*[int(e) for _, e in dims])
    return names, extents, len(dims)


def _axes(axes):
    if isinstance(axes, str):
        axes = [axes]
    axes = list(axes)
    return (ctypes.c_char_p * max(1, len(axes)))(*[a.encode() for a in axes]), len(axes)


class Type:
    def __init__(self, dtype, dims):
        self.dtype = dtype
        self.dims = dims  # list of (name, extent)

    def byte_count(self):
        n = DTYPE_SIZE[self.dtype]
        for _, e in self.dims:
            n *= e
        return n

    def __repr__(self):
        return "%s[%s]" % (self.dtype, ", ".join("%s=%d" % d for d in self.dims))


def _type_from_descriptor(d):
    return Type(DTYPES[d.dtype], [(d.names[i].decode(), d.extents[i]) for i in range(d.rank)])


class Builder:
    def __init__(self, name):
        self._h = ctypes.c_void_p()
        status = lib.accy_b200_builder_create(name.encode(), ctypes.byref(self._h))
        if status:
            raise MemoryError("builder")
        self.finished = False

    def __del__(self):
        if getattr(self, "_h", None):
            lib.accy_b200_builder_destroy(self._h)
            self._h = None

    def _emit(self, fn, *args):
        out = ctypes.c_uint32()
        status = fn(self._h, *args, ctypes.byref(out))
        if status:
            raise TensorError(lib.accy_b200_builder_last_error(self._h).decode())
        return Value(self, out.value)

    def _check(self, other):
        if not isinstance(other, Value) or other.builder is not self:
            raise TensorError("CrossBuilderValue")
        return other.id

    # constructors (builder.zig:89-123, 192-281, 283-300)
    def input(self, dtype, **dims):
        return self.input_spec(spec(dtype, **dims))

    def input_spec(self, s):
        names, extents, rank = _names_extents(s.dims)
        return self._emit(lib.accy_b200_builder_input, DTYPES.index(s.dtype), names, extents, rank)

    def inputs(self, specs):
        return [self.input_spec(s) for s in specs]

    def scalar(self, dtype, value):
        payload = _scalar_bytes(dtype, value)
        names, extents, rank = _names_extents([])
        return self._emit(lib.accy_b200_builder_constant, DTYPES.index(dtype), names, extents, 0, payload, len(payload))

    def constant(self, dtype, dims, array_bytes):
        names, extents, rank = _names_extents(dims)
        return self._emit(lib.accy_b200_builder_constant, DTYPES.index(dtype), names, extents, rank,
                          bytes(array_bytes), len(array_bytes))

    def full(self, dtype, dims, fill):
        names, extents, rank = _names_extents(dims)
        return self._emit(lib.accy_b200_builder_full, DTYPES.index(dtype), names, extents, rank, float(fill))

    def iota(self, dtype, dims, axis):
        names, extents, rank = _names_extents(dims)
        return self._emit(lib.accy_b200_builder_iota, DTYPES.index(dtype), names, extents, rank, axis.encode())

    def type_of(self, value_id):
        d = _native.Descriptor()
        status = lib.accy_b200_builder_value_type(self._h, value_id, ctypes.byref(d))
        if status:
            raise TensorError(lib.accy_b200_builder_last_error(self._h).decode())
        return _type_from_descriptor(d)

    def finish(self, outputs):
        ids = (ctypes.c_uint32 * max(1, len(outputs)))(*[self._check(o) for o in outputs])
        data = ctypes.POINTER(ctypes.c_uint8)()
        length = ctypes.c_size_t()
        status = lib.accy_b200_builder_finish(self._h, ids, len(outputs), ctypes.byref(data), ctypes.byref(length))
        if status:
            raise TensorError(lib.accy_b200_builder_last_error(self._h).decode())
        self.finished = True
        return ctypes.string_at(data, length.value)


def _scalar_bytes(dtype, value):
    if dtype == "f32":
        return struct.pack("<f", value)
    if dtype == "f64":
        return struct.pack("<d", value)
    if dtype == "bf16":  # truncation, as the reference's Bf16.fromF32 (gpu/abi/src/dtype.zig:6-9)
        return struct.pack("<H", struct.unpack("<I", struct.pack("<f", value))[0] >> 16)
    if dtype == "f16":
        return np.float16(value).tobytes()
    if dtype == "i1":
        return struct.pack("<B", 1 if value else 0)
    fmt = {"i8": "<b", "i16": "<h", "i32": "<i", "i64": "<q", "u8": "<B", "u16": "<H", "u32": "<I", "u64": "<Q"}[dtype]
    return struct.pack(fmt, value)


class Value:
    """A recorded value with named axes (src/tensor/trace/value.zig)."""

    def __init__(self, builder, value_id):
        self.builder = builder
        self.id = value_id
        self._ty = None

    @property
    def ty(self):
        if self._ty is None:
            self._ty = self.builder.type_of(self.id)
        return self._ty

    def _bin(self, op, rhs):
        b = self.builder
        return b._emit(lib.accy_b200_builder_binary, BINARY.index(op), self.id, b._check(rhs))

    def add(self, rhs): return self._bin("add", rhs)
    def sub(self, rhs): return self._bin("sub", rhs)
    def mul(self, rhs): return self._bin("mul", rhs)
    def div(self, rhs): return self._bin("div", rhs)
    def pow(self, rhs): return self._bin("pow", rhs)

    def _reduce(self, reducer, axes):
        names, count = _axes(axes)
        return self.builder._emit(lib.accy_b200_builder_reduce, self.id, REDUCER.index(reducer), names, count)

    def reduce(self, init, reducer, axes):
        """Value.reduce (value.zig:60-61): fold over `axes` with `reducer`, starting from the rank-0 value `init`."""
        names, count = _axes(axes)
        b = self.builder
        return b._emit(lib.accy_b200_builder_reduce_with, self.id, b._check(init), REDUCER.index(reducer), names, count)

    def max(self, other):
        return self._bin("max", other) if isinstance(other, Value) else self._reduce("max", other)

    def min(self, other):
        return self._bin("min", other) if isinstance(other, Value) else self._reduce("min", other)

    def sum(self, axes): return self._reduce("sum", axes)

    def mean(self, axes):
        names, count = _axes(axes)
        return self.builder._emit(lib.accy_b200_builder_mean, self.id, names, count)

    def contract(self, rhs, axes):
        names, count = _axes(axes)
        return self.builder._emit(lib.accy_b200_builder_contract, self.id, self.builder._check(rhs), names, count)

    def rename(self, old_name, new_name):
        return self.builder._emit(lib.accy_b200_builder_rename, self.id, old_name.encode(), new_name.encode())

    def split(self, axis, **parts):
        names, extents, rank = _names_extents(list(parts.items()))
        return self.builder._emit(lib.accy_b200_builder_split, self.id, axis.encode(), names, extents, rank)

    def merge(self, axes, merged_name):
        names, count = _axes(axes)
        return self.builder._emit(lib.accy_b200_builder_merge, self.id, names, count, merged_name.encode())

    def broadcast(self, **added):
        names, extents, rank = _names_extents(list(added.items()))
        return self.builder._emit(lib.accy_b200_builder_broadcast, self.id, names, extents, rank)

    def broadcast_op(self, **dims):
        """Builder.broadcastOp (builder.zig:487-497): this rank-0 value repeated to `dims`."""
        names, extents, rank = _names_extents(list(dims.items()))
        return self.builder._emit(lib.accy_b200_builder_broadcast_op, self.id, names, extents, rank)

    def _un(self, op):
        return self.builder._emit(lib.accy_b200_builder_unary, UNARY.index(op), self.id)

    def neg(self): return self._un("neg")
    def abs(self): return self._un("abs")
    def exp(self): return self._un("exp")
    def log(self): return self._un("log")
    def sqrt(self): return self._un("sqrt")
    def tanh(self): return self._un("tanh")
    def sin(self): return self._un("sin")
    def cos(self): return self._un("cos")
    def tan(self): return self._un("tan")

    def compare(self, direction, rhs):
        b = self.builder
        return b._emit(lib.accy_b200_builder_compare, COMPARE.index(direction), self.id, b._check(rhs))

    def select(self, on_true, on_false):
        b = self.builder
        return b._emit(lib.accy_b200_builder_select, self.id, b._check(on_true), b._check(on_false))


class Program:
    """A finished recording: its ACTP wire bytes plus the parameter and output types."""

    def __init__(self, name, wire, input_types, output_types):
        self.name = name
        self.wire = wire
        self.input_types = input_types
        self.output_types = output_types

    def deinit(self):
        pass

    # -- derived programs (src/tensor/function.zig: grad / valueAndGrad / vmap return programs) --
    def grad(self, wrt):
        """tensor.grad (src/tensor/grad.zig:19-33): gradients of the one scalar output with respect
        to the parameter indices `wrt`, in that order."""
        return _derive_grad(self, wrt, keep_value=False)

    def value_and_grad(self, wrt):
        """tensor.valueAndGrad (src/tensor/grad.zig:35-49): outputs = value, then the gradients."""
        return _derive_grad(self, wrt, keep_value=True)

    def jvp(self, wrt):
        """tensor.jvp (src/tensor/autodiff.zig:725-732): inputs + one tangent per parameter in `wrt`
        (parameter order); outputs + their tangents."""
        wrt = [int(i) for i in wrt]
        indices = (ctypes.c_uint64 * max(1, len(wrt)))(*wrt)

        def call(src, length, out, capacity, n, err, err_capacity):
            return lib.accy_b200_wire_jvp(src, length, indices, len(wrt), out, capacity, n, err, err_capacity)
        wire = _transformed(call, self)
        return Program(self.name, wire, *_io_types(wire))

    def vmap(self, axis_size, in_axes, out_axis=0, axis_name=""):
        """tensor.vmap (src/tensor/batch.zig:14-47).  in_axes: per input the position of the new
        axis (`mapped_axis(k)` or an int) or None for an input shared by every instance."""
        return _derive_vmap(self, axis_size, in_axes, out_axis, axis_name)


def mapped_axis(index):
    """batch.zig:29 `mapped`: the new axis sits at position `index` of that input."""
    return int(index)


def _transformed(call, program):
    wire = program.wire
    src = ctypes.create_string_buffer(wire, len(wire))
    capacity = 4 * len(wire) + 65536
    err = ctypes.create_string_buffer(512)
    for _ in range(2):
        out = ctypes.create_string_buffer(capacity)
        n = ctypes.c_size_t()
        status = call(ctypes.cast(src, ctypes.c_void_p), len(wire), ctypes.cast(out, ctypes.c_void_p), capacity,
                      ctypes.byref(n), ctypes.cast(err, ctypes.c_void_p), 512)
        if status == 4 and n.value > capacity:  # invalid_buffer: the derived program is larger
            capacity = n.value
            continue
        break
    if status:
        name = err.value.decode(errors="replace")
        if status == 1:
            raise TensorError(name)
        raise SessionError(status, name)
    return out.raw[:n.value]


def _io_types(wire):
    """(input types, output types) of ACTP bytes, read back from the library's own decoding
    (accy_b200_wire_describe: one "id kind dtype[name=extent,...] operands" line per operation,
    then "outputs %id ...")."""
    src = ctypes.create_string_buffer(wire, len(wire))
    capacity = 64 * len(wire) + 65536
    out = ctypes.create_string_buffer(capacity)
    n = ctypes.c_size_t()
    status = lib.accy_b200_wire_describe(ctypes.cast(src, ctypes.c_void_p), len(wire), ctypes.cast(out, ctypes.c_void_p),
                                         capacity, ctypes.byref(n))
    if status:
        raise SessionError(status, "cannot describe the derived program")
    types, inputs, outputs = {}, [], []
    for line in out.raw[:n.value].decode().splitlines():
        fields = line.split(" ")
        if fields[0] == "outputs":
            outputs = [types[int(f[1:])] for f in fields[1:]]
            continue
        dtype, _, rest = fields[2].partition("[")
        dims = []
        for item in filter(None, rest.rstrip("]").split(",")):
            name, _, extent = item.rpartition("=")
            dims.append((name, int(extent)))
        types[int(fields[0])] = Type(dtype, dims)
        if fields[1] == "parameter":
            inputs.append(types[int(fields[0])])
    return inputs, outputs


def _derive_grad(program, wrt, keep_value):
    wrt = [int(i) for i in wrt]
    indices = (ctypes.c_uint64 * max(1, len(wrt)))(*wrt)

    def call(src, length, out, capacity, n, err, err_capacity):
        return lib.accy_b200_wire_grad(src, length, indices, len(wrt), 1 if keep_value else 0, out, capacity, n,
                                       err, err_capacity)
    wire = _transformed(call, program)
    return Program(program.name, wire, *_io_types(wire))


def _derive_vmap(program, axis_size, in_axes, out_axis, axis_name):
    axes = [-1 if a is None else int(a) for a in in_axes]
    c_axes = (ctypes.c_int64 * max(1, len(axes)))(*axes)

    def call(src, length, out, capacity, n, err, err_capacity):
        return lib.accy_b200_wire_vmap(src, length, int(axis_size), c_axes, len(axes), int(out_axis),
                                       axis_name.encode(), out, capacity, n, err, err_capacity)
    wire = _transformed(call, program)
    return Program(program.name, wire, *_io_types(wire))


def define(name, specs, body):
    """tensor.define (src/tensor/trace/define.zig:8-19): records `body` on placeholders."""
    builder = Builder(name)
    args = builder.inputs(specs)
    result = body(builder, args)
    outputs = list(result) if isinstance(result, (list, tuple)) else [result]
    input_types = [a.ty for a in args]
    output_types = [o.ty for o in outputs]
    wire = builder.finish(outputs)
    return Program(name, wire, input_types, output_types)


class PartialFold(int):
    """How the pieces' outputs combine: 0 (falsy) = independent blocks, 1 = add, 2 = maximum, 3 = minimum."""

    @property
    def name(self):
        return (None, "sum", "max", "min")[int(self)]


def shard_program(program, axis, extent):
    """Re-records `program` with `extent` for the named axis so it can run as independent pieces
    (one rank per GPU, or one chunk at a time).  Returns (piece, partial_sum): when partial_sum
    is True every output of a piece is a partial sum over the axis and the pieces must be added
    (one all-reduce); otherwise piece i's outputs are rows [i*extent, (i+1)*extent) of the full
    outputs (partial_sum.name says how the pieces combine: "sum", "max" or "min").  Raises SessionError("compile_failed") when an operation mixes values across the axis."""
    wire = program.wire if isinstance(program, Program) else bytes(program)
    src = ctypes.create_string_buffer(wire, len(wire))
    out = ctypes.create_string_buffer(len(wire) + 65536)
    n = ctypes.c_size_t()
    partial = ctypes.c_uint32()
    err = ctypes.create_string_buffer(512)
    status = lib.accy_b200_wire_shard(ctypes.cast(src, ctypes.c_void_p), len(wire), axis.encode(), int(extent),
                                      ctypes.cast(out, ctypes.c_void_p), len(out), ctypes.byref(n), ctypes.byref(partial),
                                      ctypes.cast(err, ctypes.c_void_p), 512)
    if status:
        raise SessionError(status, err.value.decode(errors="replace"))
    piece_wire = out.raw[:n.value]

    def resize(types):
        return [Type(t.dtype, [(name, extent if name == axis else e) for name, e in t.dims]) for t in types]
    name = program.name if isinstance(program, Program) else "shard"
    inputs = resize(program.input_types) if isinstance(program, Program) else []
    outputs = resize(program.output_types) if isinstance(program, Program) else []
    return Program(name, piece_wire, inputs, outputs), PartialFold(partial.value)


# ---------------------------------------------------------------------------------------------
# execution
# ---------------------------------------------------------------------------------------------
class CompiledProgram:
    def __init__(self, session, handle):
        self.session = session
        self.handle = handle

    def _descriptors(self, is_output):
        n_in = ctypes.c_uint32()
        n_out = ctypes.c_uint32()
        self.session._check(lib.accy_b200_session_io_counts(self.session._h, self.handle, ctypes.byref(n_in), ctypes.byref(n_out)))
        out = []
        for i in range(n_out.value if is_output else n_in.value):
            d = _native.Descriptor()
            self.session._check(lib.accy_b200_session_describe(self.session._h, self.handle, 1 if is_output else 0, i, ctypes.byref(d)))
            t = _type_from_descriptor(d)
            t.byte_size = d.byte_size
            t.alignment = d.alignment
            out.append(t)
        return out

    def input_descriptors(self):
        return self._descriptors(False)

    def output_descriptors(self):
        return self._descriptors(True)

    def plan_summary(self):
        return lib.accy_b200_session_plan_summary(self.session._h, self.handle).decode()

    def work(self):
        w = _native.Work()
        self.session._check(lib.accy_b200_session_work(self.session._h, self.handle, ctypes.byref(w)))
        return {"bytes": w.bytes, "flops": w.flops, "pairs": w.pairs, "launches": w.launches}

    def kernels(self):
        count = ctypes.c_uint32()
        self.session._check(lib.accy_b200_session_kernel_count(self.session._h, self.handle, ctypes.byref(count)))
        out = []
        for i in range(count.value):
            name = ctypes.c_char_p()
            options = ctypes.c_char_p()
            src = lib.accy_b200_session_kernel_source(self.session._h, self.handle, i, ctypes.byref(name), ctypes.byref(options))
            out.append((name.value.decode(), src.decode(), options.value.decode()))
        return out

    def last_kernel_ms(self):
        ms = ctypes.c_float()
        self.session._check(lib.accy_b200_session_last_kernel_ms(self.session._h, self.handle, ctypes.byref(ms)))
        return ms.value


def _buffer_address(buf, writable):
    """(address, byte length, keepalive) of a bytes-like object, numpy array or torch CPU tensor."""
    if hasattr(buf, "data_ptr") and hasattr(buf, "element_size"):
        return buf.data_ptr(), buf.numel() * buf.element_size(), buf
    if isinstance(buf, np.ndarray):
        if not buf.flags["C_CONTIGUOUS"]:
            raise SessionError(4, "numpy buffers must be C-contiguous")
        return buf.ctypes.data, buf.nbytes, buf
    if isinstance(buf, (bytes, bytearray, memoryview)):
        if writable:
            arr = (ctypes.c_char * len(buf)).from_buffer(buf)
        else:
            arr = (ctypes.c_char * len(buf)).from_buffer_copy(buf) if isinstance(buf, bytes) else (ctypes.c_char * len(buf)).from_buffer(buf)
        return ctypes.addressof(arr), len(buf), arr
    raise SessionError(4, "unsupported buffer type %r" % type(buf))


class Session:
    """tensor.session.Session (src/tensor/session/session.zig:88-246) on a B200."""

    def __init__(self, device=0, **overrides):
        opts = _native.Options()
        opts.device = device
        for k, v in overrides.items():
            setattr(opts, k, v)
        self._h = ctypes.c_void_p()
        status = lib.accy_b200_session_create(ctypes.byref(opts), ctypes.byref(self._h))
        if status:
            raise SessionError(status, "session_create")
        self._observer = None

    def deinit(self):
        if self._h:
            lib.accy_b200_session_destroy(self._h)
            self._h = None

    def __del__(self):
        if lib is not None:   # module globals are cleared at interpreter shutdown
            self.deinit()

    def _check(self, status):
        if status:
            raise SessionError(status, lib.accy_b200_session_last_error(self._h).decode(errors="replace"))

    def set_observer(self, fn):
        """fn(phase_name, nanoseconds), as FragmentInstrumentation.observe (src/executable/phase.zig)."""
        self._observer = _native.OBSERVER(lambda ctx, phase, ns: fn(phase.decode(), ns)) if fn else _native.OBSERVER()
        self._check(lib.accy_b200_session_set_observer(self._h, self._observer, None))

    def time_launches(self, enable=True):
        """Record CUDA events around every invoke's kernels, for `Compiled.last_kernel_ms` (off by default:
        the events cost a stream of back-to-back invokes a few microseconds each)."""
        self._check(lib.accy_b200_session_time_launches(self._h, 1 if enable else 0))

    def compile(self, wire_bytes):
        wire_bytes = wire_bytes.wire if isinstance(wire_bytes, Program) else bytes(wire_bytes)
        handle = ctypes.c_uint64()
        buf = ctypes.create_string_buffer(wire_bytes, len(wire_bytes))
        self._check(lib.accy_b200_session_compile(self._h, ctypes.cast(buf, ctypes.c_void_p), len(wire_bytes), ctypes.byref(handle)))
        return CompiledProgram(self, handle.value)

    def invoke(self, compiled, inputs, outputs):
        keep = []
        in_ptrs = (ctypes.c_void_p * max(1, len(inputs)))()
        in_sizes = (ctypes.c_size_t * max(1, len(inputs)))()
        for i, b in enumerate(inputs):
            if b is None:   # an input kept on the device by set_resident
                in_ptrs[i], in_sizes[i] = None, compiled.input_descriptors()[i].byte_size
                continue
            addr, size, k = _buffer_address(b, False)
            in_ptrs[i], in_sizes[i] = addr, size
            keep.append(k)
        out_ptrs = (ctypes.c_void_p * max(1, len(outputs)))()
        out_sizes = (ctypes.c_size_t * max(1, len(outputs)))()
        for j, b in enumerate(outputs):
            addr, size, k = _buffer_address(b, True)
            out_ptrs[j], out_sizes[j] = addr, size
            keep.append(k)
        self._check(lib.accy_b200_session_invoke(self._h, compiled.handle, in_ptrs, in_sizes, len(inputs),
                                                 out_ptrs, out_sizes, len(outputs)))

    def set_resident(self, compiled, index, data):
        """Keeps input `index` of the program on the device across invokes (weights); later
        `invoke` calls pass None for it.  `data` None drops the device copy."""
        if data is None:
            self._check(lib.accy_b200_session_set_resident(self._h, compiled.handle, index, None, 0))
            return
        addr, size, keep = _buffer_address(data, False)
        self._check(lib.accy_b200_session_set_resident(self._h, compiled.handle, index, addr, size))
        del keep

    def invoke_device(self, compiled, input_ptrs, output_ptrs, stream=None):
        ins = (ctypes.c_uint64 * max(1, len(input_ptrs)))(*input_ptrs)
        outs = (ctypes.c_uint64 * max(1, len(output_ptrs)))(*output_ptrs)
        self._check(lib.accy_b200_session_invoke_device(self._h, compiled.handle, ins, len(input_ptrs), outs,
                                                        len(output_ptrs), ctypes.c_void_p(stream or 0)))

    def synchronize(self, stream=None):
        self._check(lib.accy_b200_session_synchronize(self._h, ctypes.c_void_p(stream or 0)))

    def release(self, compiled):
        self._check(lib.accy_b200_session_release(self._h, compiled.handle))


class MultiCuda:
    """One recorded program over several GPUs of a box from one process (`accy_b200_sharded_*`):
    the program is cut along `axis` into one piece per device, `launch` takes the buffers of the
    WHOLE program (as `Cuda.launch` does) and drives all devices at once.  The reference runs on
    one device only; this has no counterpart there."""

    def __init__(self, program, axis, devices, **overrides):
        opts = _native.Options()
        for k, v in overrides.items():
            setattr(opts, k, v)
        ordinals = (ctypes.c_int32 * len(devices))(*devices)
        self._h = ctypes.c_void_p()
        status = lib.accy_b200_sharded_create(ordinals, len(devices), ctypes.byref(opts), ctypes.byref(self._h))
        if status:
            raise SessionError(status, "sharded_create")
        wire_bytes = program.wire if isinstance(program, Program) else bytes(program)
        handle = ctypes.c_uint64()
        buf = ctypes.create_string_buffer(wire_bytes, len(wire_bytes))
        try:
            self._check(lib.accy_b200_sharded_compile(self._h, ctypes.cast(buf, ctypes.c_void_p), len(wire_bytes), axis.encode(),
                                                      ctypes.byref(handle)))
        except SessionError:
            self.deinit()
            raise
        self.handle = handle.value

    def _check(self, status):
        if status:
            raise SessionError(status, lib.accy_b200_sharded_last_error(self._h).decode(errors="replace"))

    def launch(self, inputs, outputs):
        keep = []
        in_ptrs = (ctypes.c_void_p * max(1, len(inputs)))()
        in_sizes = (ctypes.c_size_t * max(1, len(inputs)))()
        for i, b in enumerate(inputs):
            addr, size, k = _buffer_address(b, False)
            in_ptrs[i], in_sizes[i] = addr, size
            keep.append(k)
        out_ptrs = (ctypes.c_void_p * max(1, len(outputs)))()
        out_sizes = (ctypes.c_size_t * max(1, len(outputs)))()
        for j, b in enumerate(outputs):
            addr, size, k = _buffer_address(b, True)
            out_ptrs[j], out_sizes[j] = addr, size
            keep.append(k)
        self._check(lib.accy_b200_sharded_invoke(self._h, self.handle, in_ptrs, in_sizes, len(inputs), out_ptrs, out_sizes,
                                                 len(outputs)))

    def deinit(self):
        if self._h:
            lib.accy_b200_sharded_destroy(self._h)
            self._h = None

    def __del__(self):
        if lib is not None:
            self.deinit()


class Cuda:
    """The B200 counterpart of the reference's `Cpu` executor (src/tensor/execute.zig:9-51):
    compile once in `__init__`, `launch` many times, `deinit` to free."""

    def __init__(self, program, device=0, **overrides):
        self.session = Session(device=device, **overrides)
        self.compiled = self.session.compile(program)

    def launch(self, inputs, outputs):
        self.session.invoke(self.compiled, inputs, outputs)

    def launch_device(self, input_ptrs, output_ptrs, stream=None):
        self.session.invoke_device(self.compiled, input_ptrs, output_ptrs, stream)

    def deinit(self):
        self.session.deinit()


class Function:
    """tensor.Function (src/tensor/function.zig:10-83): a recording together with the programs
    derived from it.  `grad`, `value_and_grad` and `vmap` return Functions that the root keeps, so
    one `deinit` on the root releases them all; `compile_cuda` stands where `compileCpu` does."""

    def __init__(self, program, root=None):
        self.graph = program
        self.root = root
        self.derived = []

    @classmethod
    def define(cls, name, specs, body):
        return cls(define(name, specs, body))

    def _adopt(self, program):
        root = self.root or self
        child = Function(program, root)
        root.derived.append(child)
        return child

    def grad(self, wrt):
        return self._adopt(self.graph.grad(wrt))

    def value_and_grad(self, wrt):
        return self._adopt(self.graph.value_and_grad(wrt))

    def jvp(self, wrt):
        return self._adopt(self.graph.jvp(wrt))

    def vmap(self, axis_size, in_axes, out_axis=0, axis_name=""):
        return self._adopt(self.graph.vmap(axis_size, in_axes, out_axis, axis_name))

    def compile_cuda(self, device=0, **overrides):
        return Cuda(self.graph, device=device, **overrides)

    def deinit(self):
        assert self.root is None, "derived functions are released by their root"
        for child in self.derived:
            child.graph.deinit()
        self.derived = []
        self.graph.deinit()


def run_cuda(program, inputs, outputs, device=0):
    """runCpu's contract (src/tensor/execute.zig:54-63) on a B200: compile, run, free."""
    executor = Cuda(program, device=device)
    try:
        executor.launch(inputs, outputs)
    finally:
        executor.deinit()
