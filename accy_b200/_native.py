"""ctypes binding of libaccy_b200.so: one prototype per symbol declared in include/accy_b200.h."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libaccy_b200.so")

MAX_RANK = 8

c_u32 = ctypes.c_uint32
c_u64 = ctypes.c_uint64
c_size = ctypes.c_size_t
c_p = ctypes.c_void_p
c_str = ctypes.c_char_p
P = ctypes.POINTER


class Options(ctypes.Structure):
    _fields_ = [("device", ctypes.c_int32), ("threads_per_row", ctypes.c_int32),
                ("vectors_per_thread", ctypes.c_int32), ("column_splits", ctypes.c_int32),
                ("force_simt_gemm", ctypes.c_int32), ("row_min_blocks", ctypes.c_int32),
                ("single_shot_invoke", ctypes.c_int32)]


class Descriptor(ctypes.Structure):
    _fields_ = [("dtype", c_u32), ("rank", c_u32), ("extents", ctypes.c_int64 * MAX_RANK),
                ("names", c_str * MAX_RANK), ("byte_size", c_size), ("alignment", c_u32)]


class Work(ctypes.Structure):
    _fields_ = [("bytes", ctypes.c_double), ("flops", ctypes.c_double), ("pairs", ctypes.c_double),
                ("launches", c_u32), ("reserved", c_u32)]


OBSERVER = ctypes.CFUNCTYPE(None, c_p, c_str, c_u64)

# name -> (restype, argtypes); the CPU test-suite checks that every one of these is exported
PROTOTYPES = {
    "accy_b200_version": (c_str, []),
    "accy_b200_session_create": (c_u32, [P(Options), P(c_p)]),
    "accy_b200_session_destroy": (None, [c_p]),
    "accy_b200_session_compile": (c_u32, [c_p, c_p, c_size, P(c_u64)]),
    "accy_b200_session_io_counts": (c_u32, [c_p, c_u64, P(c_u32), P(c_u32)]),
    "accy_b200_session_describe": (c_u32, [c_p, c_u64, c_u32, c_u32, P(Descriptor)]),
    "accy_b200_session_invoke": (c_u32, [c_p, c_u64, P(c_p), P(c_size), c_u32, P(c_p), P(c_size), c_u32]),
    "accy_b200_session_invoke_device": (c_u32, [c_p, c_u64, P(c_u64), c_u32, P(c_u64), c_u32, c_p]),
    "accy_b200_session_set_resident": (c_u32, [c_p, c_u64, c_u32, c_p, c_size]),
    "accy_b200_session_synchronize": (c_u32, [c_p, c_p]),
    "accy_b200_session_release": (c_u32, [c_p, c_u64]),
    "accy_b200_session_set_observer": (c_u32, [c_p, OBSERVER, c_p]),
    "accy_b200_session_last_error": (c_str, [c_p]),
    "accy_b200_session_plan_summary": (c_str, [c_p, c_u64]),
    "accy_b200_session_work": (c_u32, [c_p, c_u64, P(Work)]),
    "accy_b200_session_kernel_count": (c_u32, [c_p, c_u64, P(c_u32)]),
    "accy_b200_session_kernel_source": (c_str, [c_p, c_u64, c_u32, P(c_str), P(c_str)]),
    "accy_b200_session_time_launches": (c_u32, [c_p, c_u32]),
    "accy_b200_session_last_kernel_ms": (c_u32, [c_p, c_u64, P(ctypes.c_float)]),
    "accy_b200_builder_create": (c_u32, [c_str, P(c_p)]),
    "accy_b200_builder_destroy": (None, [c_p]),
    "accy_b200_builder_last_error": (c_str, [c_p]),
    "accy_b200_builder_input": (c_u32, [c_p, c_u32, P(c_str), P(ctypes.c_int64), c_u32, P(c_u32)]),
    "accy_b200_builder_constant": (c_u32, [c_p, c_u32, P(c_str), P(ctypes.c_int64), c_u32, c_p, c_size, P(c_u32)]),
    "accy_b200_builder_full": (c_u32, [c_p, c_u32, P(c_str), P(ctypes.c_int64), c_u32, ctypes.c_double, P(c_u32)]),
    "accy_b200_builder_iota": (c_u32, [c_p, c_u32, P(c_str), P(ctypes.c_int64), c_u32, c_str, P(c_u32)]),
    "accy_b200_builder_unary": (c_u32, [c_p, c_u32, c_u32, P(c_u32)]),
    "accy_b200_builder_binary": (c_u32, [c_p, c_u32, c_u32, c_u32, P(c_u32)]),
    "accy_b200_builder_compare": (c_u32, [c_p, c_u32, c_u32, c_u32, P(c_u32)]),
    "accy_b200_builder_select": (c_u32, [c_p, c_u32, c_u32, c_u32, P(c_u32)]),
    "accy_b200_builder_reduce": (c_u32, [c_p, c_u32, c_u32, P(c_str), c_u32, P(c_u32)]),
    "accy_b200_builder_reduce_with": (c_u32, [c_p, c_u32, c_u32, c_u32, P(c_str), c_u32, P(c_u32)]),
    "accy_b200_builder_mean": (c_u32, [c_p, c_u32, P(c_str), c_u32, P(c_u32)]),
    "accy_b200_builder_contract": (c_u32, [c_p, c_u32, c_u32, P(c_str), c_u32, P(c_u32)]),
    "accy_b200_builder_rename": (c_u32, [c_p, c_u32, c_str, c_str, P(c_u32)]),
    "accy_b200_builder_split": (c_u32, [c_p, c_u32, c_str, P(c_str), P(ctypes.c_int64), c_u32, P(c_u32)]),
    "accy_b200_builder_merge": (c_u32, [c_p, c_u32, P(c_str), c_u32, c_str, P(c_u32)]),
    "accy_b200_builder_broadcast": (c_u32, [c_p, c_u32, P(c_str), P(ctypes.c_int64), c_u32, P(c_u32)]),
    "accy_b200_builder_broadcast_op": (c_u32, [c_p, c_u32, P(c_str), P(ctypes.c_int64), c_u32, P(c_u32)]),
    "accy_b200_builder_value_type": (c_u32, [c_p, c_u32, P(Descriptor)]),
    "accy_b200_builder_finish": (c_u32, [c_p, P(c_u32), c_u32, P(P(ctypes.c_uint8)), P(c_size)]),
    "accy_b200_wire_reencode": (c_u32, [c_p, c_size, c_p, c_size, P(c_size), c_p, c_size]),
    "accy_b200_wire_shard": (c_u32, [c_p, c_size, c_str, ctypes.c_int64, c_p, c_size, P(c_size), P(c_u32), c_p, c_size]),
    "accy_b200_wire_grad": (c_u32, [c_p, c_size, P(c_u64), c_u32, c_u32, c_p, c_size, P(c_size), c_p, c_size]),
    "accy_b200_wire_jvp": (c_u32, [c_p, c_size, P(c_u64), c_u32, c_p, c_size, P(c_size), c_p, c_size]),
    "accy_b200_wire_vmap": (c_u32, [c_p, c_size, ctypes.c_int64, P(ctypes.c_int64), c_u32, c_u32, c_str, c_p, c_size,
                            P(c_size), c_p, c_size]),
    "accy_b200_wire_describe": (c_u32, [c_p, c_size, c_p, c_size, P(c_size)]),
    "accy_b200_sharded_create": (c_u32, [P(ctypes.c_int32), c_u32, P(Options), P(c_p)]),
    "accy_b200_sharded_destroy": (None, [c_p]),
    "accy_b200_sharded_device_count": (c_u32, [c_p]),
    "accy_b200_sharded_compile": (c_u32, [c_p, c_p, c_size, c_str, P(c_u64)]),
    "accy_b200_sharded_invoke": (c_u32, [c_p, c_u64, P(c_p), P(c_size), c_u32, P(c_p), P(c_size), c_u32]),
    "accy_b200_sharded_release": (c_u32, [c_p, c_u64]),
    "accy_b200_sharded_last_error": (c_str, [c_p]),
    "accy_b200_mismatch_noalloc": (c_u32, [c_p, c_p, c_p, c_p, c_u64, c_u64, c_u32, c_p, c_p, c_size]),
    "accy_b200_probe_fp32_rates": (c_u32, [c_p, P(ctypes.c_double), P(ctypes.c_double), c_p, c_size]),
    "accy_b200_test_use_fake_driver": (None, [ctypes.c_int32]),
    "accy_b200_test_fake_fail": (None, [c_str, ctypes.c_int32]),
    "accy_b200_test_fake_device_status": (None, [ctypes.c_int32]),
    "accy_b200_test_fake_call_count": (c_u32, [c_str]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "accy_b200: native library %s is missing. Build it with `python accy_b200/build.py` "
            "(or __graft_entry__.build()). There is no Python or CPU fallback." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()
