/*
 * accy_b200.h -- C ABI of the B200 (sm_100a) execution target for recorded Accy tensor programs.
 *
 * The library is a drop-in for the reference's CPU execution path: a recorded program goes in as
 * the reference's own "ACTP" version 1 wire bytes, inputs and outputs are dense row-major
 * little-endian buffers of exactly the declared byte size, in parameter order and output order.
 * Plain pointers and sizes only; every function returns a status number whose values 0..8 are
 * the reference's stable session codes.
 *
 * Reference interfaces each group replaces (paths inside a-tiny-project/accy):
 *   session_*   src/tensor/session/session.zig:33-56 (Status), :120-161 (compile), :163-171
 *               (input/outputDescriptors), :181-213 (invoke), :218-226 (release);
 *               src/tensor/execute.zig:9-63 (runCpu / Cpu.init / Cpu.launch / Cpu.deinit)
 *   builder_*   src/tensor/trace/builder.zig:62-1047 and src/tensor/trace/value.zig:13-155
 *               (named-axis recording), src/tensor/wire/encode.zig:28-60 (encode)
 *   invoke_device / synchronize / elapsed
 *               deps/lib/compiler/gpu/src/contract.zig:2048-2085 (launch on caller buffers,
 *               synchronize, elapsed_event_ns of the device vtable)
 */
#ifndef ACCY_B200_H
#define ACCY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status numbers: src/tensor/session/session.zig:33-56.  Once assigned a number keeps its meaning. */
enum {
  ACCY_B200_OK = 0,
  ACCY_B200_INVALID_PROGRAM = 1,
  ACCY_B200_UNSUPPORTED_VERSION = 2,
  ACCY_B200_INVALID_HANDLE = 3,
  ACCY_B200_INVALID_BUFFER = 4,
  ACCY_B200_TOO_MANY_PROGRAMS = 5,
  ACCY_B200_OUT_OF_MEMORY = 6,
  ACCY_B200_COMPILE_FAILED = 7,
  ACCY_B200_LAUNCH_FAILED = 8
};

/* Element type codes: src/tensor/wire/format.zig:101-103. */
enum {
  ACCY_B200_I1 = 0, ACCY_B200_I8, ACCY_B200_I16, ACCY_B200_I32, ACCY_B200_I64, ACCY_B200_U8,
  ACCY_B200_U16, ACCY_B200_U32, ACCY_B200_U64, ACCY_B200_F16, ACCY_B200_BF16, ACCY_B200_F32,
  ACCY_B200_F64, ACCY_B200_KEY
};

#define ACCY_B200_MAX_PROGRAMS 64u /* session.zig:16 */
#define ACCY_B200_MAX_RANK 8u
#define ACCY_B200_BUFFER_ALIGNMENT 256u /* deps/lib/compiler/gpu/src/cuda.zig:241-245 */

typedef struct accy_b200_session accy_b200_session;
typedef struct accy_b200_builder accy_b200_builder;

/* Session options (role of FragmentCompilerOptions, src/executable/fragment.zig:75-102). */
typedef struct accy_b200_options {
  int32_t device;             /* CUDA ordinal; -1 = compile only, no device is touched */
  int32_t threads_per_row;    /* schedule override for row kernels, 0 = automatic */
  int32_t vectors_per_thread; /* schedule override, 0 = automatic */
  int32_t column_splits;      /* schedule override, 0 = automatic */
  int32_t force_simt_gemm;    /* 1 = never use the tcgen05 kernels (exact k-serial order) */
  int32_t row_min_blocks;     /* schedule override: resident CTAs per SM requested of row kernels, 0 = automatic */
  int32_t single_shot_invoke; /* 1 = host-buffer invoke never streams the program through the GPU in chunks */
} accy_b200_options;

/* One input or output slot: session.zig:66-74 (Descriptor). */
typedef struct accy_b200_descriptor {
  uint32_t dtype;
  uint32_t rank;
  int64_t extents[ACCY_B200_MAX_RANK];
  const char* names[ACCY_B200_MAX_RANK]; /* valid until the program is released */
  size_t byte_size;
  uint32_t alignment;
} accy_b200_descriptor;

/* Work a compiled program does per invocation, for roofline reporting. */
typedef struct accy_b200_work {
  double bytes;   /* inputs read once + outputs written once */
  double flops;   /* contraction flops (causal count for masked attention) */
  double pairs;   /* elementwise/reduction evaluations of the row kernels */
  uint32_t launches; /* kernel launches per invocation */
  uint32_t reserved;
} accy_b200_work;

typedef void (*accy_b200_observer)(void* context, const char* phase, uint64_t nanoseconds);

/* ---- session: Session.init / deinit (session.zig:99-118) ---- */
uint32_t accy_b200_session_create(const accy_b200_options* options, accy_b200_session** session);
void accy_b200_session_destroy(accy_b200_session* session);

/* Session.compile (session.zig:120-161): decode ACTP bytes, plan, emit and compile the sm_100a
 * kernels, load them.  The bytes may be freed when the call returns. */
uint32_t accy_b200_session_compile(accy_b200_session* session, const uint8_t* actp, size_t length,
                                   uint64_t* handle);
/* Session.inputDescriptors / outputDescriptors (session.zig:163-171). */
uint32_t accy_b200_session_io_counts(accy_b200_session* session, uint64_t handle, uint32_t* inputs,
                                     uint32_t* outputs);
uint32_t accy_b200_session_describe(accy_b200_session* session, uint64_t handle, uint32_t is_output,
                                    uint32_t index, accy_b200_descriptor* descriptor);
/* Session.invoke (session.zig:181-213) == Cpu.launch (execute.zig:44-51): host buffers, sizes
 * must match the descriptors exactly, outputs must not overlap inputs or each other; copies to
 * and from the device happen inside the call, which returns after the results are in place. */
uint32_t accy_b200_session_invoke(accy_b200_session* session, uint64_t handle,
                                  const void* const* inputs, const size_t* input_sizes,
                                  uint32_t input_count, void* const* outputs,
                                  const size_t* output_sizes, uint32_t output_count);
/* The same launch on buffers already in device memory (the vtable's launch on caller-allocated
 * buffers, contract.zig:2048-2085): no copies, asynchronous on `stream` (a CUstream, or NULL for
 * the session's own stream).  Pointers must be 256-byte aligned.  Launches of one handle must not
 * overlap on the device (put them on one stream or order them with events): they share the
 * program's temporaries, scratch and work counters. */
uint32_t accy_b200_session_invoke_device(accy_b200_session* session, uint64_t handle,
                                         const uint64_t* input_ptrs, uint32_t input_count,
                                         const uint64_t* output_ptrs, uint32_t output_count,
                                         void* stream);
/* Keeps one input of a compiled program in device memory across invokes: `data` (exactly the
 * descriptor's byte size) is copied to the device once; later accy_b200_session_invoke calls may
 * pass NULL for that input (its size is still given) and the resident copy is used, so weights are
 * not sent again with every call.  A non-NULL pointer in a later invoke overrides the resident copy
 * for that call.  `data` == NULL drops the resident copy.  The reference keeps compiled programs
 * and their buffers in Cpu / FragmentCompilerCache (src/tensor/execute.zig:14-51,
 * src/executable/compiler.zig:39-153) but copies every input per launch; this call has no
 * counterpart there. */
uint32_t accy_b200_session_set_resident(accy_b200_session* session, uint64_t handle, uint32_t input_index,
                                        const void* data, size_t size);
uint32_t accy_b200_session_synchronize(accy_b200_session* session, void* stream);
/* Session.release (session.zig:218-226): the handle is refused from then on. */
uint32_t accy_b200_session_release(accy_b200_session* session, uint64_t handle);
/* FragmentInstrumentation.observe (src/executable/phase.zig:3-50): phase name and duration. */
uint32_t accy_b200_session_set_observer(accy_b200_session* session, accy_b200_observer observer,
                                        void* context);
/* Session.last_cause (session.zig:93-97), as text.  Valid until the next call on the session. */
const char* accy_b200_session_last_error(accy_b200_session* session);
/* Fusion decisions, work figures and generated CUDA source of a compiled program. */
const char* accy_b200_session_plan_summary(accy_b200_session* session, uint64_t handle);
uint32_t accy_b200_session_work(accy_b200_session* session, uint64_t handle, accy_b200_work* work);
uint32_t accy_b200_session_kernel_count(accy_b200_session* session, uint64_t handle, uint32_t* count);
const char* accy_b200_session_kernel_source(accy_b200_session* session, uint64_t handle, uint32_t index,
                                            const char** name, const char** options);
/* Device time of the most recent invoke's kernels, ms (elapsed_event_ns of the device vtable,
 * deps/lib/compiler/gpu/src/contract.zig:2048-2085).  The two CUDA events around the launch list
 * are recorded only after accy_b200_session_time_launches(session, 1): in a stream of back-to-back
 * invokes they cost a few microseconds each, so they are off by default, and last_kernel_ms then
 * answers LAUNCH_FAILED. */
uint32_t accy_b200_session_time_launches(accy_b200_session* session, uint32_t enable);
uint32_t accy_b200_session_last_kernel_ms(accy_b200_session* session, uint64_t handle, float* ms);

/* ---- builder: tensor.define recording (builder.zig, value.zig) ----
 * Values are the dense ids of the recorded operations.  A failed call returns INVALID_PROGRAM and
 * accy_b200_builder_last_error gives the reference's error name (e.g. "AxisExtentMismatch"). */
uint32_t accy_b200_builder_create(const char* name, accy_b200_builder** builder);
void accy_b200_builder_destroy(accy_b200_builder* builder);
const char* accy_b200_builder_last_error(accy_b200_builder* builder);
uint32_t accy_b200_builder_input(accy_b200_builder* b, uint32_t dtype, const char* const* names,
                                 const int64_t* extents, uint32_t rank, uint32_t* value);
uint32_t accy_b200_builder_constant(accy_b200_builder* b, uint32_t dtype, const char* const* names,
                                    const int64_t* extents, uint32_t rank, const void* payload,
                                    size_t payload_bytes, uint32_t* value);
uint32_t accy_b200_builder_full(accy_b200_builder* b, uint32_t dtype, const char* const* names,
                                const int64_t* extents, uint32_t rank, double fill, uint32_t* value);
uint32_t accy_b200_builder_iota(accy_b200_builder* b, uint32_t dtype, const char* const* names,
                                const int64_t* extents, uint32_t rank, const char* axis, uint32_t* value);
uint32_t accy_b200_builder_unary(accy_b200_builder* b, uint32_t op, uint32_t x, uint32_t* value);
uint32_t accy_b200_builder_binary(accy_b200_builder* b, uint32_t op, uint32_t lhs, uint32_t rhs, uint32_t* value);
uint32_t accy_b200_builder_compare(accy_b200_builder* b, uint32_t direction, uint32_t lhs, uint32_t rhs, uint32_t* value);
uint32_t accy_b200_builder_select(accy_b200_builder* b, uint32_t pred, uint32_t on_true, uint32_t on_false, uint32_t* value);
uint32_t accy_b200_builder_reduce(accy_b200_builder* b, uint32_t x, uint32_t reducer, const char* const* axes,
                                  uint32_t axis_count, uint32_t* value);
/* Builder.reduceWith (src/tensor/trace/builder.zig:589-603; Value.reduce, value.zig:60-61): a fold over
 * the named axes that starts from the rank-0 value `init` instead of the reducer's own start value. */
uint32_t accy_b200_builder_reduce_with(accy_b200_builder* b, uint32_t x, uint32_t init, uint32_t reducer,
                                       const char* const* axes, uint32_t axis_count, uint32_t* value);
uint32_t accy_b200_builder_mean(accy_b200_builder* b, uint32_t x, const char* const* axes, uint32_t axis_count,
                                uint32_t* value);
uint32_t accy_b200_builder_contract(accy_b200_builder* b, uint32_t lhs, uint32_t rhs, const char* const* axes,
                                    uint32_t axis_count, uint32_t* value);
uint32_t accy_b200_builder_rename(accy_b200_builder* b, uint32_t x, const char* old_name, const char* new_name,
                                  uint32_t* value);
uint32_t accy_b200_builder_split(accy_b200_builder* b, uint32_t x, const char* axis, const char* const* names,
                                 const int64_t* extents, uint32_t parts, uint32_t* value);
uint32_t accy_b200_builder_merge(accy_b200_builder* b, uint32_t x, const char* const* axes, uint32_t axis_count,
                                 const char* merged, uint32_t* value);
uint32_t accy_b200_builder_broadcast(accy_b200_builder* b, uint32_t x, const char* const* names,
                                     const int64_t* extents, uint32_t rank, uint32_t* value);
/* Builder.broadcastOp (builder.zig:487-497): the `broadcast` operation, a rank-0 value repeated to
 * the given dims (the target runs it for rank-0 operands, which is what the reference's own
 * transformations give it, batch.zig:698-722). */
uint32_t accy_b200_builder_broadcast_op(accy_b200_builder* b, uint32_t x, const char* const* names,
                                        const int64_t* extents, uint32_t rank, uint32_t* value);
uint32_t accy_b200_builder_value_type(accy_b200_builder* b, uint32_t value, accy_b200_descriptor* descriptor);
/* Builder.finish + wire.encode: the ACTP bytes stay valid until the builder is destroyed. */
uint32_t accy_b200_builder_finish(accy_b200_builder* b, const uint32_t* outputs, uint32_t output_count,
                                  const uint8_t** actp, size_t* length);

/* ---- wire: decode + re-encode (round-trip check of foreign ACTP bytes) ---- */
uint32_t accy_b200_wire_reencode(const uint8_t* actp, size_t length, uint8_t* out, size_t capacity,
                                 size_t* out_length, char* error_name, size_t error_capacity);
/* Re-records a program with extent `extent` for the named axis, for running it as independent
 * pieces (one per GPU, or one per chunk).  No counterpart in the reference, which runs on one
 * device.  Refused (COMPILE_FAILED, reason in `error`) when an operation mixes values across the
 * axis.  *partial_sum is 0 when piece i's outputs are block i of the full outputs; 1, 2 or 3 when
 * every output is a sum, maximum or minimum over the axis: the pieces' outputs must then be
 * combined with that operation (one all-reduce). */
uint32_t accy_b200_wire_shard(const uint8_t* actp, size_t length, const char* axis, int64_t extent, uint8_t* out,
                              size_t capacity, size_t* out_length, uint32_t* partial_sum, char* error,
                              size_t error_capacity);
/* ---- program transformations (src/tensor/grad.zig:19-49 `grad` / `valueAndGrad`,
 * src/tensor/batch.zig:14-47 `vmap`; src/tensor/function.zig chains them) ----
 * Both take ACTP bytes and write the derived program's ACTP bytes to `out` (*out_length is set even
 * when `capacity` is too small: INVALID_BUFFER, call again with a larger buffer).  A refusal
 * returns INVALID_PROGRAM with the reference's error name in `error`: GradientRequiresScalarOutput,
 * ParameterOutOfRange, DuplicateParameter, NonDifferentiableParameter, UnsupportedDerivative;
 * InvalidDimension, InAxisCountMismatch, AxisOutOfRange.
 *
 * grad: the program must have one rank-0 floating-point output.  The derived program takes the
 * same inputs and returns [the value, when keep_value != 0,] then the gradient with respect to
 * each parameter index in `wrt`, in that order, each typed like its parameter. */
uint32_t accy_b200_wire_grad(const uint8_t* actp, size_t length, const uint64_t* wrt, uint32_t wrt_count,
                             uint32_t keep_value, uint8_t* out, size_t capacity, size_t* out_length, char* error,
                             size_t error_capacity);
/* jvp (src/tensor/autodiff.zig:725-732): forward mode, any number and rank of outputs.  The derived
 * program takes the source's inputs followed by one tangent per parameter listed in `wrt` (in
 * parameter order, typed like the parameter) and returns the source's outputs followed by their
 * tangents (zeros for an output no listed parameter reaches). */
uint32_t accy_b200_wire_jvp(const uint8_t* actp, size_t length, const uint64_t* wrt, uint32_t wrt_count, uint8_t* out,
                            size_t capacity, size_t* out_length, char* error, size_t error_capacity);
/* vmap: runs the program once per index of a new axis of extent axis_size.  in_axes[i] is the
 * position of the new axis in input i (batch.zig `mapped(axis)`), or -1 for an input shared by
 * every instance (`.none`); every output carries the new axis at out_axis (outputs that do not
 * depend on a mapped input are repeated along it).  axis_name NULL or "" selects "#batch". */
uint32_t accy_b200_wire_vmap(const uint8_t* actp, size_t length, int64_t axis_size, const int64_t* in_axes,
                             uint32_t in_axis_count, uint32_t out_axis, const char* axis_name, uint8_t* out,
                             size_t capacity, size_t* out_length, char* error, size_t error_capacity);
/* Operation list of decoded bytes as text, one op per line: "id kind dtype[name=extent,...] ...". */
uint32_t accy_b200_wire_describe(const uint8_t* actp, size_t length, char* out, size_t capacity,
                                 size_t* out_length);

/* ---- one program over several GPUs, from one process ----
 * No counterpart in the reference, which runs on one device and has no collective
 * (deps/lib/compiler/gpu/src/runtime/cuda/runtime.zig:56-85 opens one ordinal).  The program is cut
 * along the named axis into one piece per device (the analysis and the pieces of accy_b200_wire_shard);
 * each device gets a session of its own and a host thread per invoke.  Buffers and sizes are those of
 * the WHOLE program, as Session.invoke would take them (session.zig:163-226): buffers that carry the
 * axis are used in place, block d by device d; the others are read by every device; when the axis is
 * the one the outputs fold over, the devices' partial results are combined on the host in device
 * order (sum, maximum or minimum, as recorded).  The axis extent must divide by the device count.
 * `devices` may name one ordinal several times (pieces then share that GPU). */
typedef struct accy_b200_sharded accy_b200_sharded;
uint32_t accy_b200_sharded_create(const int32_t* devices, uint32_t device_count, const accy_b200_options* options,
                                  accy_b200_sharded** sharded);
void accy_b200_sharded_destroy(accy_b200_sharded* sharded);
uint32_t accy_b200_sharded_device_count(accy_b200_sharded* sharded);
uint32_t accy_b200_sharded_compile(accy_b200_sharded* sharded, const uint8_t* actp, size_t length, const char* axis,
                                   uint64_t* handle);
uint32_t accy_b200_sharded_invoke(accy_b200_sharded* sharded, uint64_t handle, const void* const* inputs,
                                  const size_t* input_sizes, uint32_t input_count, void* const* outputs,
                                  const size_t* output_sizes, uint32_t output_count);
uint32_t accy_b200_sharded_release(accy_b200_sharded* sharded, uint64_t handle);
const char* accy_b200_sharded_last_error(accy_b200_sharded* sharded);

/* ---- allocation-free entry point ----
 * No counterpart in the reference.  For hosts that may not allocate device memory while running
 * (a service whose pool owns the whole device, a real-time loop, a fixed stream schedule): the
 * two-pass column-split "mismatch" reduction, out[g] = sum_p (sin(frequency[g]*time[p]) -
 * sample[p])^2 in f32, with its partial sums kept in a 1 MiB array built into the library's device
 * image instead of an allocated scratch buffer.  All four pointers are device pointers the caller
 * already owns; `stream` is a CUstream/cudaStream_t (NULL = default stream); `splits` is the
 * number of column splits wanted (clamped to the number of 4096-point chunks).  Limit:
 * guesses * splits <= 262144, otherwise ACCY_B200_INVALID_BUFFER with a message in `error`.
 * The call is asynchronous on `stream`.  Calls on one device share the array: issue them one
 * after another, never overlapping.  The first call on a device looks up the array's device
 * address; make it outside stream capture.  A CUDA runtime error that the caller's own earlier calls
 * left pending on the calling thread is returned (and cleared) as ACCY_B200_LAUNCH_FAILED with a
 * message that says so, and nothing is launched; each of the two launches is checked by itself. */
uint32_t accy_b200_mismatch_noalloc(const float* frequency, const float* time, const float* sample, float* out,
                                    uint64_t guesses, uint64_t points, uint32_t splits, void* stream,
                                    char* error, size_t error_capacity);

/* ---- measurement support ----
 * No counterpart in the reference (which ships no benchmarks, src/root.zig:76-78).  Runs two
 * register-only micro-kernels on the current CUDA device and `stream` and returns the ceilings the
 * FP32-bound row kernels are reported against: (guess, point) pairs per second of a loop that does
 * nothing but `sinf(f * t) - s`, square and add with CUDA's own sinf ("sinf + 4 flop"), and the
 * flop/s of independent packed fma.rn.f32x2 chains.  Allocates nothing; synchronises `stream`. */
uint32_t accy_b200_probe_fp32_rates(void* stream, double* sinf_pairs_per_second, double* packed_fma_flops,
                                    char* error, size_t error_capacity);

/* ---- test support: a recording fake of the CUDA driver (the reference tests its CUDA backend
 * the same way, deps/lib/compiler/gpu/src/runtime/cuda/runtime.zig:643-1031) ---- */
void accy_b200_test_use_fake_driver(int32_t enable);
void accy_b200_test_fake_fail(const char* driver_function, int32_t after_calls);
uint32_t accy_b200_test_fake_call_count(const char* driver_function);
/* The fake's device status word reads as `value` from now on (0 = as stored): stands for a kernel
 * whose bounded wait ran out (runtime.zig:279-314 is the reference's poisoning after a failed call). */
void accy_b200_test_fake_device_status(int32_t value);

const char* accy_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ACCY_B200_H */
