// One recorded program over several GPUs of a box, from one process, behind the C ABI.
//
// The reference runs on one device and has no collective of any kind (no counterpart there); this
// is the host-side runner of the pieces that `accy_b200_wire_shard` cuts: the program is cut along
// a named batch-like axis into one piece per device, every device gets its own session (context,
// stream, buffers, compiled kernels), and a host-buffer invoke drives all devices at once, one
// host thread per device:
//   * inputs and outputs that carry the axis (as their outermost dim, which the shard analysis
//     requires) are contiguous byte ranges of the caller's buffers: device d reads and writes
//     block d in place, nothing is gathered or scattered;
//   * inputs that do not carry the axis are replicated: every device reads the whole buffer;
//   * when the axis is the one the program folds over (its outputs are sums, maxima or minima over
//     it), every device produces a full-shape partial result; they are combined on the host in
//     device order with the outputs' own reducer, so the result does not depend on timing.
// No exchange between devices happens on the data path.  Processes that keep their data on the
// devices (one rank per GPU) use the session API directly and an all-reduce of their own for the
// partial case (accy_b200/shard.py does that with NCCL).
#include <cstring>
#include <mutex>
#include <thread>

#include "../../include/accy_b200.h"
#include "plan.hpp"

using namespace accy;

namespace {

struct ShardedEntry {
  bool live = false;
  uint32_t generation = 0;
  std::vector<uint64_t> handles;        // per device
  std::vector<size_t> input_bytes;      // of the whole program
  std::vector<bool> input_sliced;       // carries the axis: device d owns block d
  std::vector<size_t> output_bytes;
  std::vector<DType> output_dtypes;
  uint32_t partial_fold = 0;            // 0: outputs are sliced; 1 add, 2 maximum, 3 minimum over the devices' partials
};

template <typename T>
void foldInto(T* into, const T* from, size_t n, uint32_t how) {
  for (size_t i = 0; i < n; ++i) {
    if (how == 1) into[i] = into[i] + from[i];
    else if (how == 2) into[i] = into[i] > from[i] ? into[i] : from[i];
    else into[i] = into[i] < from[i] ? into[i] : from[i];
  }
}

bool foldBuffers(DType dtype, void* into, const void* from, size_t bytes, uint32_t how) {
  switch (dtype) {
    case DType::f32: foldInto(static_cast<float*>(into), static_cast<const float*>(from), bytes / 4, how); return true;
    case DType::f64: foldInto(static_cast<double*>(into), static_cast<const double*>(from), bytes / 8, how); return true;
    case DType::i32: {
      // wrap-around addition like the kernels' own integer sums
      if (how == 1) foldInto(static_cast<uint32_t*>(into), static_cast<const uint32_t*>(from), bytes / 4, how);
      else foldInto(static_cast<int32_t*>(into), static_cast<const int32_t*>(from), bytes / 4, how);
      return true;
    }
    case DType::u32: foldInto(static_cast<uint32_t*>(into), static_cast<const uint32_t*>(from), bytes / 4, how); return true;
    case DType::i64: {
      if (how == 1) foldInto(static_cast<uint64_t*>(into), static_cast<const uint64_t*>(from), bytes / 8, how);
      else foldInto(static_cast<int64_t*>(into), static_cast<const int64_t*>(from), bytes / 8, how);
      return true;
    }
    default: return false;
  }
}

}  // namespace

struct accy_b200_sharded {
  std::vector<accy_b200_session*> sessions;
  std::mutex mutex;
  std::string last_error;
  ShardedEntry entries[ACCY_B200_MAX_PROGRAMS];
};

namespace {

uint32_t failWith(accy_b200_sharded* s, uint32_t status, const std::string& message) {
  s->last_error = message;
  return status;
}

ShardedEntry* entryOf(accy_b200_sharded* s, uint64_t handle) {
  const uint32_t index = static_cast<uint32_t>(handle & 0xffffffffu), generation = static_cast<uint32_t>(handle >> 32);
  if (index >= ACCY_B200_MAX_PROGRAMS) return nullptr;
  ShardedEntry& e = s->entries[index];
  return (e.live && e.generation == generation) ? &e : nullptr;
}

}  // namespace

extern "C" {

uint32_t accy_b200_sharded_create(const int32_t* devices, uint32_t device_count, const accy_b200_options* options,
                                  accy_b200_sharded** out) {
  if (!out || !devices || device_count == 0 || device_count > 64) return ACCY_B200_INVALID_BUFFER;
  auto* s = new accy_b200_sharded();
  for (uint32_t d = 0; d < device_count; ++d) {
    accy_b200_options o{};
    if (options) o = *options;
    o.device = devices[d];
    o.single_shot_invoke = 1;   // the pieces already run side by side; no chunked streaming inside a piece
    accy_b200_session* session = nullptr;
    uint32_t status = accy_b200_session_create(&o, &session);
    if (status != ACCY_B200_OK) {
      for (accy_b200_session* made : s->sessions) accy_b200_session_destroy(made);
      delete s;
      return status;
    }
    s->sessions.push_back(session);
  }
  *out = s;
  return ACCY_B200_OK;
}

void accy_b200_sharded_destroy(accy_b200_sharded* s) {
  if (!s) return;
  for (accy_b200_session* session : s->sessions) accy_b200_session_destroy(session);
  delete s;
}

const char* accy_b200_sharded_last_error(accy_b200_sharded* s) { return s ? s->last_error.c_str() : ""; }

uint32_t accy_b200_sharded_compile(accy_b200_sharded* s, const uint8_t* actp, size_t length, const char* axis,
                                   uint64_t* handle) {
  if (!s) return ACCY_B200_INVALID_HANDLE;
  std::lock_guard<std::mutex> lock(s->mutex);
  if (!actp || !handle) return failWith(s, ACCY_B200_INVALID_BUFFER, "null argument");
  try {
    const std::string name = axis ? axis : "";
    Program program = decodeProgram(actp, length);
    ShardInfo info = analyseShardAxis(program, name);
    if (!info.shardable) return failWith(s, ACCY_B200_COMPILE_FAILED, "axis '" + name + "' cannot be sharded: " + info.reason);
    const int64_t devices = static_cast<int64_t>(s->sessions.size());
    if (info.extent % devices != 0)
      return failWith(s, ACCY_B200_COMPILE_FAILED, "axis '" + name + "' of extent " + std::to_string(info.extent) +
                                                       " does not divide over " + std::to_string(devices) + " devices");
    uint32_t index = 0;
    while (index < ACCY_B200_MAX_PROGRAMS && s->entries[index].live) ++index;
    if (index == ACCY_B200_MAX_PROGRAMS) return failWith(s, ACCY_B200_TOO_MANY_PROGRAMS, "too many programs");
    const std::vector<uint8_t> piece = encodeProgram(shardProgram(program, name, info.extent / devices));
    ShardedEntry e;
    for (uint32_t id : program.parameters) {
      const Type& t = program.typeOf(id);
      e.input_bytes.push_back(t.byteCount());
      e.input_sliced.push_back(findDim(t.dims, name) >= 0);
    }
    for (uint32_t id : program.outputs) {
      e.output_bytes.push_back(program.typeOf(id).byteCount());
      e.output_dtypes.push_back(program.typeOf(id).dtype);
    }
    e.partial_fold = info.partial_sum ? info.partial_fold : 0u;
    if (e.partial_fold) {
      char scratch[8] = {0};
      for (DType d : e.output_dtypes)
        if (!foldBuffers(d, scratch, scratch, 0, e.partial_fold))
          return failWith(s, ACCY_B200_COMPILE_FAILED, "partial results of this element type cannot be combined");
    }
    for (accy_b200_session* session : s->sessions) {
      uint64_t h = 0;
      uint32_t status = accy_b200_session_compile(session, piece.data(), piece.size(), &h);
      if (status != ACCY_B200_OK) {
        std::string why = accy_b200_session_last_error(session);
        for (size_t d = 0; d < e.handles.size(); ++d) accy_b200_session_release(s->sessions[d], e.handles[d]);
        return failWith(s, status, why);
      }
      e.handles.push_back(h);
    }
    e.live = true;
    e.generation = s->entries[index].generation + 1;
    s->entries[index] = e;
    *handle = (static_cast<uint64_t>(e.generation) << 32) | index;
    return ACCY_B200_OK;
  } catch (const PlanError& err) {
    return failWith(s, ACCY_B200_COMPILE_FAILED, err.what());
  } catch (const std::exception& err) {
    return failWith(s, ACCY_B200_INVALID_PROGRAM, err.what());
  }
}

uint32_t accy_b200_sharded_invoke(accy_b200_sharded* s, uint64_t handle, const void* const* inputs,
                                  const size_t* input_sizes, uint32_t input_count, void* const* outputs,
                                  const size_t* output_sizes, uint32_t output_count) {
  if (!s) return ACCY_B200_INVALID_HANDLE;
  std::lock_guard<std::mutex> lock(s->mutex);
  ShardedEntry* e = entryOf(s, handle);
  if (!e) return failWith(s, ACCY_B200_INVALID_HANDLE, "stale or unknown handle");
  if (input_count != e->input_bytes.size() || output_count != e->output_bytes.size())
    return failWith(s, ACCY_B200_INVALID_BUFFER, "wrong number of buffers");
  if ((input_count && (!inputs || !input_sizes)) || (output_count && (!outputs || !output_sizes)))
    return failWith(s, ACCY_B200_INVALID_BUFFER, "null buffer array");
  for (uint32_t i = 0; i < input_count; ++i)
    if (input_sizes[i] != e->input_bytes[i] || (!inputs[i] && e->input_bytes[i]))
      return failWith(s, ACCY_B200_INVALID_BUFFER, "input " + std::to_string(i) + " must be exactly " + std::to_string(e->input_bytes[i]) + " bytes");
  for (uint32_t j = 0; j < output_count; ++j)
    if (output_sizes[j] != e->output_bytes[j] || (!outputs[j] && e->output_bytes[j]))
      return failWith(s, ACCY_B200_INVALID_BUFFER, "output " + std::to_string(j) + " must be exactly " + std::to_string(e->output_bytes[j]) + " bytes");
  const size_t devices = s->sessions.size();
  // partial results of devices 1.. land in host buffers of their own; device 0 writes the caller's
  std::vector<std::vector<std::vector<unsigned char>>> partials(devices);
  std::vector<uint32_t> status(devices, ACCY_B200_OK);
  std::vector<std::string> message(devices);
  std::vector<std::thread> threads;
  for (size_t d = 0; d < devices; ++d) {
    threads.emplace_back([&, d] {
     try {
      std::vector<const void*> in(input_count);
      std::vector<size_t> in_size(input_count);
      std::vector<void*> out(output_count);
      std::vector<size_t> out_size(output_count);
      for (uint32_t i = 0; i < input_count; ++i) {
        const size_t piece = e->input_sliced[i] ? e->input_bytes[i] / devices : e->input_bytes[i];
        in_size[i] = piece;
        in[i] = e->input_sliced[i] ? static_cast<const char*>(inputs[i]) + d * piece : inputs[i];
      }
      if (e->partial_fold && d > 0) partials[d].resize(output_count);
      for (uint32_t j = 0; j < output_count; ++j) {
        if (e->partial_fold) {
          out_size[j] = e->output_bytes[j];
          if (d == 0) out[j] = outputs[j];
          else {
            partials[d][j].resize(e->output_bytes[j] ? e->output_bytes[j] : 1);
            out[j] = partials[d][j].data();
          }
        } else {
          const size_t piece = e->output_bytes[j] / devices;
          out_size[j] = piece;
          out[j] = static_cast<char*>(outputs[j]) + d * piece;
        }
      }
      status[d] = accy_b200_session_invoke(s->sessions[d], e->handles[d], in.data(), in_size.data(), input_count, out.data(),
                                           out_size.data(), output_count);
      if (status[d] != ACCY_B200_OK) message[d] = accy_b200_session_last_error(s->sessions[d]);
     } catch (const std::bad_alloc&) {
      status[d] = ACCY_B200_OUT_OF_MEMORY;
      message[d] = "out of host memory for the partial results";
     } catch (const std::exception& err) {
      status[d] = ACCY_B200_LAUNCH_FAILED;
      message[d] = err.what();
     }
    });
  }
  for (std::thread& t : threads) t.join();
  for (size_t d = 0; d < devices; ++d)
    if (status[d] != ACCY_B200_OK) return failWith(s, status[d], "device " + std::to_string(d) + ": " + message[d]);
  if (e->partial_fold)
    for (size_t d = 1; d < devices; ++d)
      for (uint32_t j = 0; j < output_count; ++j)
        foldBuffers(e->output_dtypes[j], outputs[j], partials[d][j].data(), e->output_bytes[j], e->partial_fold);
  return ACCY_B200_OK;
}

uint32_t accy_b200_sharded_release(accy_b200_sharded* s, uint64_t handle) {
  if (!s) return ACCY_B200_INVALID_HANDLE;
  std::lock_guard<std::mutex> lock(s->mutex);
  ShardedEntry* e = entryOf(s, handle);
  if (!e) return failWith(s, ACCY_B200_INVALID_HANDLE, "stale or unknown handle");
  for (size_t d = 0; d < e->handles.size(); ++d) accy_b200_session_release(s->sessions[d], e->handles[d]);
  e->live = false;
  e->handles.clear();
  return ACCY_B200_OK;
}

uint32_t accy_b200_sharded_device_count(accy_b200_sharded* s) { return s ? static_cast<uint32_t>(s->sessions.size()) : 0u; }

}  // extern "C"
