// C ABI: sessions (compile / describe / invoke / release), the Builder mirror and wire helpers.
//
// A session plays the role of the reference's tensor.session.Session
// (src/tensor/session/session.zig:88-246): a table of at most 64 compiled programs addressed by
// generation-counted handles, stable status numbers, caller-owned buffers.  Per program it owns
// what the reference's LoadedFragment owns (src/executable/fragment.zig:711-757): the loaded
// kernels, the planned device slots and the launch list.  There is no CPU fallback anywhere:
// without a CUDA device the session can only compile.
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <sstream>

#include "../../include/accy_b200.h"
#include "driver.hpp"
#include "plan.hpp"
#include "program.hpp"

using namespace accy;

namespace {

uint64_t nowNs() {
  return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(
                                   std::chrono::steady_clock::now().time_since_epoch()).count());
}

struct LoadedKernel {
  std::vector<char> cubin;
  CUmodule_t module = nullptr;
  CUfunction_t function = nullptr;
  std::string options;
};

struct Entry {
  bool live = false;
  uint32_t generation = 0;
  Program program;
  Plan plan;
  std::vector<LoadedKernel> kernels;
  std::vector<CUdeviceptr_t> owned;      // per slot: device memory owned by the session (0 = none)
  std::vector<CUdeviceptr_t> bound;      // per slot: pointer used by the current launch
  bool staging_ready = false;            // input/output slots have session-owned device buffers
  std::vector<CUdeviceptr_t> resident;   // per parameter: device copy kept across invokes (0 = none)
  std::vector<std::vector<std::string>> names;  // descriptor name storage
  CUevent_t ev_begin = nullptr, ev_end = nullptr;
  bool timed = false;
  // The launch list recorded once as a CUDA graph and replayed while the bound pointers stay the
  // same (a host invoke always binds the program's own buffers).
  CUgraphExec_t graph = nullptr;
  std::vector<CUdeviceptr_t> graph_bound;
  int graph_recordings = 0;              // re-recordings so far; callers that change pointers every time stop being recorded
  // Encoded tensor maps, one per (launch, argument), kept while the pointer they were encoded for
  // stays bound: a steady invoke loop does no cuTensorMapEncodeTiled on its launch path.
  struct CachedMap {
    CUdeviceptr_t base = 0;
    bool valid = false;
    TensorMap map;
  };
  std::vector<std::vector<CachedMap>> map_cache;
  // Chunked host invoke: the program re-recorded for a slice of its outermost batch-like axis,
  // loaded three times (three lanes = three streams with their own buffers) so that the copy in
  // of chunk i+1, the kernels of chunk i and the copy out of chunk i-1 overlap.
  struct Pipeline {
    bool tried = false, ready = false;
    int chunks = 1;
    std::vector<std::unique_ptr<Entry>> lanes;
    std::vector<CUstream_t> streams;
    std::vector<bool> input_sharded;           // per parameter: carries the chunked axis
    std::vector<CUdeviceptr_t> shared_inputs;  // per parameter: one device copy of a replicated input
    CUevent_t shared_ready = nullptr;
  } pipeline;
};

struct StatusError {
  uint32_t status;
  std::string message;
};

}  // namespace

struct accy_b200_session {
  accy_b200_options options{};
  std::mutex mutex;
  Entry entries[ACCY_B200_MAX_PROGRAMS];
  std::string last_error;
  accy_b200_observer observer = nullptr;
  void* observer_context = nullptr;
  bool device_ready = false;
  bool poisoned = false;  // a launch failed: later launches are refused (runtime.zig:279-314)
  CUdevice_t device = 0;
  CUcontext_t context = nullptr;
  CUstream_t stream = nullptr;
  int sm_count = 148;
  bool time_launches = false;      // accy_b200_session_time_launches
  CUdeviceptr_t status_word = 0;  // device int the tcgen05 kernels set when a bounded wait gives up

  void observe(const char* phase, uint64_t begin_ns) {
    if (observer) observer(observer_context, phase, nowNs() - begin_ns);
  }

  void check(CUresult_t r, const char* what, uint32_t status = ACCY_B200_LAUNCH_FAILED) {
    if (r == 0) return;
    if (r == 2) status = ACCY_B200_OUT_OF_MEMORY;
    throw StatusError{status, std::string(what) + " failed: " + driverErrorName(r)};
  }

  void ensureDevice() {
    if (device_ready) return;
    if (options.device < 0) throw StatusError{ACCY_B200_LAUNCH_FAILED, "session was created without a device (compile only)"};
    const DriverTable* d;
    try {
      d = &driver();
    } catch (const std::exception& e) {
      throw StatusError{ACCY_B200_LAUNCH_FAILED, e.what()};
    }
    check(d->cuDeviceGet(&device, options.device), "cuDeviceGet");
    check(d->cuDevicePrimaryCtxRetain(&context, device), "cuDevicePrimaryCtxRetain");
    check(d->cuCtxSetCurrent(context), "cuCtxSetCurrent");
    check(d->cuStreamCreate(&stream, 1 /* non-blocking */), "cuStreamCreate");
    int sms = 0;
    if (d->cuDeviceGetAttribute(&sms, 16 /* MULTIPROCESSOR_COUNT */, device) == 0 && sms > 0) sm_count = sms;
    check(d->cuMemAlloc(&status_word, 256), "cuMemAlloc");
    check(d->cuMemsetD8Async(status_word, 0, 256, stream), "cuMemsetD8Async");
    check(d->cuStreamSynchronize(stream), "cuStreamSynchronize");
    device_ready = true;
  }

  // Reads the device status word after a synchronize: non-zero means a kernel gave up on a bounded
  // wait (its results are invalid); the session is poisoned like after any failed launch.
  void checkDeviceStatus(CUstream_t on) {
    const DriverTable& d = driver();
    int host = 0;
    check(d.cuMemcpyDtoHAsync(&host, status_word, sizeof(host), on), "cuMemcpyDtoHAsync");
    check(d.cuStreamSynchronize(on), "cuStreamSynchronize");
    if (host != 0) {
      poisoned = true;
      throw StatusError{ACCY_B200_LAUNCH_FAILED, "a kernel gave up on a bounded wait (device status " + std::to_string(host) + ")"};
    }
  }

  // plan the entry's program and compile every kernel of the plan to an sm_100a cubin
  void planAndCompile(Entry& x) {
    uint64_t t0 = nowNs();
    ScheduleOverrides ov;
    ov.threads_per_row = options.threads_per_row;
    ov.vectors_per_thread = options.vectors_per_thread;
    ov.column_splits = options.column_splits;
    ov.force_simt_gemm = options.force_simt_gemm;
    ov.row_min_blocks = options.row_min_blocks;
    ov.sm_count = sm_count;
    x.plan = planProgram(x.program, ov);
    observe("plan", t0);
    t0 = nowNs();
    x.kernels.resize(x.plan.kernels.size());
    for (size_t k = 0; k < x.plan.kernels.size(); ++k) {
      const KernelSource& ks = x.plan.kernels[k];
      std::string log;
      try {
        x.kernels[k].cubin = compileToCubin(ks.source, ks.name, ks.options, &log);
      } catch (const std::exception& ex) {
        throw StatusError{ACCY_B200_COMPILE_FAILED, ex.what()};
      }
      std::ostringstream opts;
      for (const std::string& o : ks.options) opts << o << " ";
      x.kernels[k].options = opts.str();
    }
    observe("kernel_compile", t0);
  }

  void allocateStaging(Entry& x) {
    if (x.staging_ready) return;
    const DriverTable& d = driver();
    for (int slot : x.plan.input_slots)
      if (!x.owned[slot]) check(d.cuMemAlloc(&x.owned[slot], x.plan.slots[slot].bytes ? x.plan.slots[slot].bytes : 1), "cuMemAlloc");
    for (int slot : x.plan.output_slots)
      if (!x.owned[slot]) check(d.cuMemAlloc(&x.owned[slot], x.plan.slots[slot].bytes ? x.plan.slots[slot].bytes : 1), "cuMemAlloc");
    x.staging_ready = true;
  }

  // Builds the chunked variant of a program for the host-buffer invoke, when the program's
  // outermost output axis can be cut into independent pieces and there is enough data for the
  // overlap to pay.  Any failure simply leaves the single-shot path in place.
  void buildPipeline(Entry& e) {
    Entry::Pipeline& P = e.pipeline;
    P.tried = true;
    size_t io_bytes = 0;
    for (int slot : e.plan.input_slots) io_bytes += e.plan.slots[slot].bytes;
    for (int slot : e.plan.output_slots) io_bytes += e.plan.slots[slot].bytes;
    if (io_bytes < (64u << 20) || e.program.outputs.empty()) return;
    const Type& out0 = e.program.typeOf(e.program.outputs[0]);
    if (out0.rank() == 0) return;
    const std::string axis = out0.dims[0].name;
    ShardInfo info = analyseShardAxis(e.program, axis);
    if (!info.shardable || info.partial_sum) return;
    // 16 chunks at most: with 32 or 64 the end-to-end rate measured lower (C2 90 -> 89 -> 83 GB/s,
    // attention 68 -> 59 TFLOP/s); the copies in and out already run at what PCIe gives in both
    // directions at once
    int chunks = 16;
    while (chunks > 1 && (info.extent % chunks != 0 || io_bytes / chunks < (16u << 20))) chunks /= 2;
    if (chunks < 2) return;
    try {
      Entry piece;
      piece.program = shardProgram(e.program, axis, info.extent / chunks);
      planAndCompile(piece);
      const DriverTable& d = driver();
      for (int lane = 0; lane < 3; ++lane) {
        auto x = std::make_unique<Entry>();
        x->program = piece.program;
        x->plan = piece.plan;
        x->kernels.resize(piece.kernels.size());
        for (size_t k = 0; k < piece.kernels.size(); ++k) {
          x->kernels[k].cubin = piece.kernels[k].cubin;
          x->kernels[k].options = piece.kernels[k].options;
        }
        x->live = true;
        P.lanes.push_back(std::move(x));
        loadKernels(*P.lanes.back());
        CUstream_t st = nullptr;
        check(d.cuStreamCreate(&st, 1), "cuStreamCreate");
        P.streams.push_back(st);
      }
      P.input_sharded.assign(e.program.parameters.size(), false);
      P.shared_inputs.assign(e.program.parameters.size(), 0);
      for (size_t i = 0; i < e.program.parameters.size(); ++i) {
        const Type& t = e.program.typeOf(e.program.parameters[i]);
        P.input_sharded[i] = findDim(t.dims, axis) == 0;
        if (!P.input_sharded[i]) check(d.cuMemAlloc(&P.shared_inputs[i], t.byteCount() ? t.byteCount() : 1), "cuMemAlloc");
      }
      // lanes own chunk-sized staging for the sliced inputs and for every output
      for (auto& lane : P.lanes) {
        for (size_t i = 0; i < e.program.parameters.size(); ++i) {
          int slot = lane->plan.input_slots[i];
          if (P.input_sharded[i]) check(d.cuMemAlloc(&lane->owned[slot], lane->plan.slots[slot].bytes ? lane->plan.slots[slot].bytes : 1), "cuMemAlloc");
        }
        for (int slot : lane->plan.output_slots)
          check(d.cuMemAlloc(&lane->owned[slot], lane->plan.slots[slot].bytes ? lane->plan.slots[slot].bytes : 1), "cuMemAlloc");
        lane->staging_ready = true;
      }
      check(d.cuEventCreate(&P.shared_ready, 2 /* disable timing */), "cuEventCreate");
      P.chunks = chunks;
      P.ready = true;
    } catch (const StatusError&) {
      dropPipeline(e);
    } catch (const std::exception&) {
      dropPipeline(e);
    }
  }

  void dropPipeline(Entry& e) {
    Entry::Pipeline& P = e.pipeline;
    if (device_ready) {
      const DriverTable& d = driver();
      for (auto& lane : P.lanes)
        if (lane) unload(*lane);
      for (CUstream_t st : P.streams)
        if (st) d.cuStreamDestroy(st);
      for (CUdeviceptr_t p : P.shared_inputs)
        if (p) d.cuMemFree(p);
      if (P.shared_ready) d.cuEventDestroy(P.shared_ready);
    }
    bool tried = P.tried;
    P = Entry::Pipeline{};
    P.tried = tried;
  }

  void runPipelined(Entry& e, const void* const* inputs, void* const* outputs) {
    if (poisoned) throw StatusError{ACCY_B200_LAUNCH_FAILED, "session is poisoned by an earlier failed launch"};
    Entry::Pipeline& P = e.pipeline;
    const DriverTable& d = driver();
    uint64_t t0 = nowNs();
    for (size_t i = 0; i < P.input_sharded.size(); ++i) {
      if (P.input_sharded[i] || !inputs[i]) continue;
      size_t bytes = e.plan.slots[e.plan.input_slots[i]].bytes;
      if (bytes) check(d.cuMemcpyHtoDAsync(P.shared_inputs[i], inputs[i], bytes, P.streams[0]), "cuMemcpyHtoDAsync");
    }
    check(d.cuEventRecord(P.shared_ready, P.streams[0]), "cuEventRecord");
    for (size_t lane = 1; lane < P.streams.size(); ++lane)
      check(d.cuStreamWaitEvent(P.streams[lane], P.shared_ready, 0), "cuStreamWaitEvent");
    for (int c = 0; c < P.chunks; ++c) {
      Entry& x = *P.lanes[c % P.lanes.size()];
      CUstream_t st = P.streams[c % P.streams.size()];
      x.bound = x.owned;
      for (size_t i = 0; i < P.input_sharded.size(); ++i) {
        int slot = x.plan.input_slots[i];
        if (!P.input_sharded[i]) {
          // a zero-byte input may be NULL without ever having been made resident
          x.bound[slot] = inputs[i] ? P.shared_inputs[i] : (i < e.resident.size() ? e.resident[i] : 0);
          continue;
        }
        size_t bytes = x.plan.slots[slot].bytes;
        if (!inputs[i] && bytes) {
          // a resident input that carries the chunked axis: the chunk is a contiguous slice of it
          x.bound[slot] = e.resident[i] + static_cast<CUdeviceptr_t>(c) * bytes;
          continue;
        }
        if (bytes)
          check(d.cuMemcpyHtoDAsync(x.owned[slot], static_cast<const char*>(inputs[i]) + static_cast<size_t>(c) * bytes, bytes, st),
                "cuMemcpyHtoDAsync");
      }
      launchAll(x, st, false);
      for (size_t j = 0; j < x.plan.output_slots.size(); ++j) {
        int slot = x.plan.output_slots[j];
        size_t bytes = x.plan.slots[slot].bytes;
        if (bytes)
          check(d.cuMemcpyDtoHAsync(static_cast<char*>(outputs[j]) + static_cast<size_t>(c) * bytes, x.owned[slot], bytes, st),
                "cuMemcpyDtoHAsync");
      }
    }
    observe("pipeline_enqueue", t0);
    t0 = nowNs();
    for (CUstream_t st : P.streams) {
      CUresult_t r = d.cuStreamSynchronize(st);
      if (r != 0) {
        poisoned = true;
        check(r, "cuStreamSynchronize");
      }
    }
    checkDeviceStatus(P.streams[0]);
    e.timed = false;
    observe("pipeline_sync", t0);
  }

  Entry& entryOf(uint64_t handle) {
    uint32_t index = static_cast<uint32_t>(handle & 0xffffffffu);
    uint32_t generation = static_cast<uint32_t>(handle >> 32);
    if (index >= ACCY_B200_MAX_PROGRAMS) throw StatusError{ACCY_B200_INVALID_HANDLE, "handle index out of range"};
    Entry& e = entries[index];
    if (!e.live || e.generation != generation) throw StatusError{ACCY_B200_INVALID_HANDLE, "stale or unknown handle"};
    return e;
  }

  void loadKernels(Entry& e) {
    const DriverTable& d = driver();
    check(d.cuCtxSetCurrent(context), "cuCtxSetCurrent");
    for (size_t k = 0; k < e.kernels.size(); ++k) {
      LoadedKernel& lk = e.kernels[k];
      if (lk.function) continue;
      check(d.cuModuleLoadData(&lk.module, lk.cubin.data()), "cuModuleLoadData", ACCY_B200_COMPILE_FAILED);
      check(d.cuModuleGetFunction(&lk.function, lk.module, e.plan.kernels[k].name.c_str()), "cuModuleGetFunction",
            ACCY_B200_COMPILE_FAILED);
    }
    for (const Launch& l : e.plan.launches) {
      if (l.dynamic_smem > 48 * 1024)
        check(d.cuFuncSetAttribute(e.kernels[l.kernel].function, 8 /* MAX_DYNAMIC_SHARED_SIZE_BYTES */,
                                   static_cast<int>(l.dynamic_smem)),
              "cuFuncSetAttribute", ACCY_B200_COMPILE_FAILED);
    }
    // planned slots that are neither inputs nor outputs: temporaries, constants, scratch
    e.owned.assign(e.plan.slots.size(), 0);
    e.bound.assign(e.plan.slots.size(), 0);
    for (size_t s = 0; s < e.plan.slots.size(); ++s) {
      const Slot& slot = e.plan.slots[s];
      if (slot.role == Slot::Input || slot.role == Slot::Output) continue;
      check(d.cuMemAlloc(&e.owned[s], slot.bytes ? slot.bytes : 1), "cuMemAlloc");
      if (slot.role == Slot::Constant)
        check(d.cuMemcpyHtoDAsync(e.owned[s], slot.payload.data(), slot.payload.size(), stream), "cuMemcpyHtoDAsync");
      if (slot.zero_init && slot.bytes) check(d.cuMemsetD8Async(e.owned[s], 0, slot.bytes, stream), "cuMemsetD8Async");
    }
    check(d.cuStreamSynchronize(stream), "cuStreamSynchronize");
    check(d.cuEventCreate(&e.ev_begin, 0), "cuEventCreate");
    check(d.cuEventCreate(&e.ev_end, 0), "cuEventCreate");
  }

  void unload(Entry& e) {
    dropPipeline(e);
    if (device_ready) {
      const DriverTable& d = driver();
      d.cuCtxSetCurrent(context);
      for (CUdeviceptr_t p : e.owned)
        if (p) d.cuMemFree(p);
      for (CUdeviceptr_t p : e.resident)
        if (p) d.cuMemFree(p);
      for (LoadedKernel& k : e.kernels)
        if (k.module) d.cuModuleUnload(k.module);
      if (e.ev_begin) d.cuEventDestroy(e.ev_begin);
      if (e.ev_end) d.cuEventDestroy(e.ev_end);
      if (e.graph) d.cuGraphExecDestroy(e.graph);
    }
    uint32_t generation = e.generation + 1;
    e = Entry{};
    e.generation = generation;
  }

  // Launches the plan with e.bound holding a device pointer for every slot.  A plan of several
  // kernels is recorded as a CUDA graph on its first single-shot launch and replayed afterwards
  // (one submission instead of one per kernel; the reference's record_sequence / submit_sequence,
  // deps/lib/compiler/gpu/src/contract.zig:1929-1966).  ACCY_B200_NO_GRAPHS=1 turns this off.
  void launchAll(Entry& e, CUstream_t on, bool time_it) {
    if (poisoned) throw StatusError{ACCY_B200_LAUNCH_FAILED, "session is poisoned by an earlier failed launch"};
    const DriverTable& d = driver();
    // Events around the launch list cost the stream a few microseconds per invoke (each one
    // drains the kernels before it), so they are recorded only when the caller asked for timings.
    const bool record_events = time_it && time_launches;
    if (record_events) check(d.cuEventRecord(e.ev_begin, on), "cuEventRecord");
    static const bool graphs_off = std::getenv("ACCY_B200_NO_GRAPHS") != nullptr;
    const bool replayable = time_it && !graphs_off && e.plan.launches.size() >= 2 && e.graph_recordings < 4;
    bool submitted = false;
    if (replayable && e.graph && e.graph_bound == e.bound) {
      submitted = d.cuGraphLaunch(e.graph, on) == 0;
      if (!submitted) e.graph_recordings = 4;  // give up on graphs for this program, launch directly below
    } else if (replayable && d.cuStreamBeginCapture(on, 2 /* relaxed: other threads' calls do not matter */) == 0) {
      if (e.graph) d.cuGraphExecDestroy(e.graph);
      e.graph = nullptr;
      e.graph_recordings += 1;
      CUgraph_t recorded = nullptr;
      try {
        issueLaunches(e, on);
      } catch (...) {
        d.cuStreamEndCapture(on, &recorded);
        if (recorded) d.cuGraphDestroy(recorded);
        throw;
      }
      if (d.cuStreamEndCapture(on, &recorded) == 0 && recorded &&
          d.cuGraphInstantiateWithFlags(&e.graph, recorded, 0) == 0 && d.cuGraphLaunch(e.graph, on) == 0) {
        e.graph_bound = e.bound;
        submitted = true;
      } else {
        if (e.graph) d.cuGraphExecDestroy(e.graph);
        e.graph = nullptr;
        e.graph_recordings = 4;
      }
      if (recorded) d.cuGraphDestroy(recorded);
    }
    if (!submitted) issueLaunches(e, on);
    if (record_events) {
      check(d.cuEventRecord(e.ev_end, on), "cuEventRecord");
      e.timed = true;
    }
  }

  void issueLaunches(Entry& e, CUstream_t on) {
    const DriverTable& d = driver();
    if (e.map_cache.size() != e.plan.launches.size()) {
      e.map_cache.clear();
      e.map_cache.resize(e.plan.launches.size());
      for (size_t i = 0; i < e.plan.launches.size(); ++i) e.map_cache[i].resize(e.plan.launches[i].args.size());
    }
    for (size_t li = 0; li < e.plan.launches.size(); ++li) {
      const Launch& l = e.plan.launches[li];
      std::vector<uint64_t> values(l.args.size());
      std::vector<void*> ptrs(l.args.size());
      for (size_t a = 0; a < l.args.size(); ++a) {
        const KernelArg& arg = l.args[a];
        if (arg.tensor_map) {
          const KernelArg::Tma& t = arg.tma;
          Entry::CachedMap& cached = e.map_cache[li][a];
          if (!cached.valid || cached.base != e.bound[t.slot]) {
            const uint32_t elem_strides[5] = {1, 1, 1, 1, 1};
            const int dtype = t.elem_bytes == 2 ? 9 /* BFLOAT16 */ : (t.elem_bytes == 4 ? 7 /* FLOAT32 */ : 0);
            cached.valid = false;
            CUresult_t r = d.cuTensorMapEncodeTiled(&cached.map, dtype, static_cast<unsigned>(t.rank),
                                                    reinterpret_cast<void*>(e.bound[t.slot]), t.dims, t.strides, t.box,
                                                    elem_strides, 0, t.swizzle, 2 /* L2 128B promotion */, 0);
            check(r, "cuTensorMapEncodeTiled");
            cached.base = e.bound[t.slot];
            cached.valid = true;
          }
          ptrs[a] = &cached.map;
        } else if (arg.is_slot) {
          values[a] = arg.slot == -2 ? status_word : e.bound[arg.slot];
          ptrs[a] = &values[a];
        } else {
          values[a] = arg.scalar;
          ptrs[a] = &values[a];
        }
      }
      CUresult_t r = d.cuLaunchKernel(e.kernels[l.kernel].function, l.grid[0], l.grid[1], l.grid[2], l.block[0],
                                      l.block[1], l.block[2], l.dynamic_smem, on, ptrs.data(), nullptr);
      if (r != 0) {
        poisoned = true;
        throw StatusError{ACCY_B200_LAUNCH_FAILED, "cuLaunchKernel(" + l.label + ") failed: " + driverErrorName(r)};
      }
    }
  }
};

namespace {

template <typename F>
uint32_t guarded(accy_b200_session* s, F&& body) {
  if (!s) return ACCY_B200_INVALID_HANDLE;
  std::lock_guard<std::mutex> lock(s->mutex);
  try {
    body();
    return ACCY_B200_OK;
  } catch (const StatusError& e) {
    s->last_error = e.message;
    return e.status;
  } catch (const WireError& e) {
    s->last_error = e.what();
    return std::string(e.what()) == "UnsupportedVersion" ? ACCY_B200_UNSUPPORTED_VERSION : ACCY_B200_INVALID_PROGRAM;
  } catch (const TensorError& e) {
    s->last_error = e.what();
    return ACCY_B200_INVALID_PROGRAM;
  } catch (const PlanError& e) {
    s->last_error = e.what();
    return ACCY_B200_COMPILE_FAILED;
  } catch (const std::bad_alloc&) {
    s->last_error = "OutOfMemory";
    return ACCY_B200_OUT_OF_MEMORY;
  } catch (const std::exception& e) {
    s->last_error = e.what();
    return ACCY_B200_COMPILE_FAILED;
  }
}

void fillDescriptor(const Type& ty, accy_b200_descriptor* out, std::vector<std::string>* storage) {
  std::memset(out, 0, sizeof(*out));
  out->dtype = static_cast<uint32_t>(ty.dtype);
  out->rank = static_cast<uint32_t>(ty.rank());
  if (ty.rank() > ACCY_B200_MAX_RANK) throw StatusError{ACCY_B200_COMPILE_FAILED, "rank above 8"};
  if (storage) {
    storage->clear();
    for (const Dim& d : ty.dims) storage->push_back(d.name);
  }
  for (size_t i = 0; i < ty.rank(); ++i) {
    out->extents[i] = ty.dims[i].extent;
    out->names[i] = storage ? (*storage)[i].c_str() : nullptr;
  }
  out->byte_size = ty.byteCount();
  out->alignment = ACCY_B200_BUFFER_ALIGNMENT;
}

}  // namespace

extern "C" {

const char* accy_b200_version(void) { return "accy_b200 0.1 (sm_100a)"; }

uint32_t accy_b200_session_create(const accy_b200_options* options, accy_b200_session** session) {
  if (!session) return ACCY_B200_INVALID_HANDLE;
  auto* s = new (std::nothrow) accy_b200_session();
  if (!s) return ACCY_B200_OUT_OF_MEMORY;
  if (options) s->options = *options;
  *session = s;
  return ACCY_B200_OK;
}

void accy_b200_session_destroy(accy_b200_session* s) {
  if (!s) return;
  try {
    std::lock_guard<std::mutex> lock(s->mutex);
    for (Entry& e : s->entries)
      if (e.live) s->unload(e);
    if (s->device_ready) {
      const DriverTable& d = driver();
      d.cuCtxSetCurrent(s->context);
      if (s->status_word) d.cuMemFree(s->status_word);
      if (s->stream) d.cuStreamDestroy(s->stream);
      d.cuDevicePrimaryCtxRelease(s->device);
    }
  } catch (const std::exception&) {
    // the driver is gone (or was never there): nothing left to hand back
  }
  delete s;
}

uint32_t accy_b200_session_compile(accy_b200_session* s, const uint8_t* actp, size_t length, uint64_t* handle) {
  return guarded(s, [&] {
    if (!actp || !handle) throw StatusError{ACCY_B200_INVALID_PROGRAM, "null program bytes"};
    int free_index = -1;
    for (uint32_t i = 0; i < ACCY_B200_MAX_PROGRAMS; ++i)
      if (!s->entries[i].live) { free_index = static_cast<int>(i); break; }
    if (free_index < 0) throw StatusError{ACCY_B200_TOO_MANY_PROGRAMS, "64 programs are already held"};
    Entry& e = s->entries[free_index];
    uint32_t generation = e.generation;
    uint64_t t0 = nowNs();
    Entry fresh;
    fresh.generation = generation;
    fresh.program = decodeProgram(actp, length);
    s->observe("decode", t0);
    if (s->options.device >= 0) s->ensureDevice();
    t0 = nowNs();
    s->planAndCompile(fresh);
    fresh.names.resize(fresh.program.parameters.size() + fresh.program.outputs.size());
    e = std::move(fresh);
    e.live = true;
    if (s->options.device >= 0) {
      t0 = nowNs();
      try {
        s->loadKernels(e);
      } catch (...) {
        s->unload(e);
        throw;
      }
      s->observe("load", t0);
    }
    *handle = (static_cast<uint64_t>(e.generation) << 32) | static_cast<uint32_t>(free_index);
  });
}

uint32_t accy_b200_session_io_counts(accy_b200_session* s, uint64_t handle, uint32_t* inputs, uint32_t* outputs) {
  return guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    if (inputs) *inputs = static_cast<uint32_t>(e.program.parameters.size());
    if (outputs) *outputs = static_cast<uint32_t>(e.program.outputs.size());
  });
}

uint32_t accy_b200_session_describe(accy_b200_session* s, uint64_t handle, uint32_t is_output, uint32_t index,
                                    accy_b200_descriptor* descriptor) {
  return guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    const auto& ids = is_output ? e.program.outputs : e.program.parameters;
    if (!descriptor || index >= ids.size()) throw StatusError{ACCY_B200_INVALID_BUFFER, "descriptor index out of range"};
    size_t slot = is_output ? e.program.parameters.size() + index : index;
    fillDescriptor(e.program.typeOf(ids[index]), descriptor, &e.names[slot]);
  });
}

static void checkCounts(Entry& e, uint32_t input_count, uint32_t output_count) {
  if (input_count != e.program.parameters.size() || output_count != e.program.outputs.size())
    throw StatusError{ACCY_B200_INVALID_BUFFER, "input or output count does not match the program"};
}

uint32_t accy_b200_session_invoke(accy_b200_session* s, uint64_t handle, const void* const* inputs,
                                  const size_t* input_sizes, uint32_t input_count, void* const* outputs,
                                  const size_t* output_sizes, uint32_t output_count) {
  return guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    checkCounts(e, input_count, output_count);
    // exact sizes (binding.zig:125-128, fragment.zig:487-488) and no overlap (session.zig:176-178)
    struct Range { const char* lo; const char* hi; };
    std::vector<Range> ranges;
    for (uint32_t i = 0; i < input_count; ++i) {
      size_t want = e.plan.slots[e.plan.input_slots[i]].bytes;
      const bool kept = i < e.resident.size() && e.resident[i] != 0;
      if (!inputs || !input_sizes || input_sizes[i] != want || (!inputs[i] && want && !kept))
        throw StatusError{ACCY_B200_INVALID_BUFFER, "input " + std::to_string(i) + " must be exactly " + std::to_string(want) + " bytes"};
      if (inputs[i]) ranges.push_back({static_cast<const char*>(inputs[i]), static_cast<const char*>(inputs[i]) + want});
    }
    for (uint32_t j = 0; j < output_count; ++j) {
      size_t want = e.plan.slots[e.plan.output_slots[j]].bytes;
      if (!outputs || !output_sizes || output_sizes[j] != want || (!outputs[j] && want))
        throw StatusError{ACCY_B200_INVALID_BUFFER, "output " + std::to_string(j) + " must be exactly " + std::to_string(want) + " bytes"};
      const char* lo = static_cast<const char*>(outputs[j]);
      const char* hi = lo + want;
      for (const Range& r : ranges)
        if (lo < r.hi && r.lo < hi && want)
          throw StatusError{ACCY_B200_INVALID_BUFFER, "output " + std::to_string(j) + " overlaps another buffer"};
      ranges.push_back({lo, hi});
    }
    s->ensureDevice();
    const DriverTable& d = driver();
    s->check(d.cuCtxSetCurrent(s->context), "cuCtxSetCurrent");
    if (!e.pipeline.tried && !s->options.single_shot_invoke) s->buildPipeline(e);
    bool pipelined = e.pipeline.ready;
    for (uint32_t i = 0; pipelined && i < input_count; ++i) {
      // chunks of a resident input are used in place, which needs every chunk to start aligned
      size_t chunk = e.pipeline.lanes[0]->plan.slots[e.pipeline.lanes[0]->plan.input_slots[i]].bytes;
      if (!inputs[i] && e.pipeline.input_sharded[i] && chunk % ACCY_B200_BUFFER_ALIGNMENT) pipelined = false;
    }
    if (pipelined) {
      s->runPipelined(e, inputs, outputs);
      return;
    }
    // device-resident staging buffers are created once and kept with the program
    s->allocateStaging(e);
    e.bound = e.owned;
    uint64_t t0 = nowNs();
    for (uint32_t i = 0; i < input_count; ++i) {
      int slot = e.plan.input_slots[i];
      if (!inputs[i] && e.plan.slots[slot].bytes) {
        e.bound[slot] = e.resident[i];   // kept on the device by set_resident
        continue;
      }
      if (e.plan.slots[slot].bytes)
        s->check(d.cuMemcpyHtoDAsync(e.owned[slot], inputs[i], e.plan.slots[slot].bytes, s->stream), "cuMemcpyHtoDAsync");
    }
    s->observe("h2d_enqueue", t0);
    t0 = nowNs();
    s->launchAll(e, s->stream, true);
    s->observe("launch_enqueue", t0);
    t0 = nowNs();
    for (uint32_t j = 0; j < output_count; ++j) {
      int slot = e.plan.output_slots[j];
      if (e.plan.slots[slot].bytes)
        s->check(d.cuMemcpyDtoHAsync(outputs[j], e.owned[slot], e.plan.slots[slot].bytes, s->stream), "cuMemcpyDtoHAsync");
    }
    CUresult_t r = d.cuStreamSynchronize(s->stream);
    if (r != 0) {
      s->poisoned = true;
      s->check(r, "cuStreamSynchronize");
    }
    s->checkDeviceStatus(s->stream);
    s->observe("d2h_and_sync", t0);
  });
}

uint32_t accy_b200_session_invoke_device(accy_b200_session* s, uint64_t handle, const uint64_t* input_ptrs,
                                         uint32_t input_count, const uint64_t* output_ptrs, uint32_t output_count,
                                         void* stream) {
  return guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    checkCounts(e, input_count, output_count);
    if ((input_count && !input_ptrs) || (output_count && !output_ptrs))
      throw StatusError{ACCY_B200_INVALID_BUFFER, "null pointer array"};
    s->ensureDevice();
    const DriverTable& d = driver();
    s->check(d.cuCtxSetCurrent(s->context), "cuCtxSetCurrent");
    e.bound = e.owned;
    for (uint32_t i = 0; i < input_count; ++i) {
      if (input_ptrs[i] % ACCY_B200_BUFFER_ALIGNMENT) throw StatusError{ACCY_B200_INVALID_BUFFER, "input pointer is not 256-byte aligned"};
      e.bound[e.plan.input_slots[i]] = input_ptrs[i];
    }
    for (uint32_t j = 0; j < output_count; ++j) {
      if (output_ptrs[j] % ACCY_B200_BUFFER_ALIGNMENT) throw StatusError{ACCY_B200_INVALID_BUFFER, "output pointer is not 256-byte aligned"};
      e.bound[e.plan.output_slots[j]] = output_ptrs[j];
    }
    s->launchAll(e, stream ? static_cast<CUstream_t>(stream) : s->stream, true);
  });
}

uint32_t accy_b200_session_set_resident(accy_b200_session* s, uint64_t handle, uint32_t input_index, const void* data,
                                        size_t size) {
  return guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    if (input_index >= e.program.parameters.size()) throw StatusError{ACCY_B200_INVALID_BUFFER, "input index out of range"};
    s->ensureDevice();
    const DriverTable& d = driver();
    s->check(d.cuCtxSetCurrent(s->context), "cuCtxSetCurrent");
    e.resident.resize(e.program.parameters.size(), 0);
    // no launch of this program may still be reading the copy that is replaced
    s->check(d.cuStreamSynchronize(s->stream), "cuStreamSynchronize");
    for (CUstream_t st : e.pipeline.streams) s->check(d.cuStreamSynchronize(st), "cuStreamSynchronize");
    if (e.resident[input_index]) {
      d.cuMemFree(e.resident[input_index]);
      e.resident[input_index] = 0;
    }
    if (!data) return;
    size_t want = e.plan.slots[e.plan.input_slots[input_index]].bytes;
    if (size != want) throw StatusError{ACCY_B200_INVALID_BUFFER, "input " + std::to_string(input_index) + " must be exactly " + std::to_string(want) + " bytes"};
    s->check(d.cuMemAlloc(&e.resident[input_index], want ? want : 1), "cuMemAlloc");
    if (want) {
      s->check(d.cuMemcpyHtoDAsync(e.resident[input_index], data, want, s->stream), "cuMemcpyHtoDAsync");
      s->check(d.cuStreamSynchronize(s->stream), "cuStreamSynchronize");
    }
  });
}

uint32_t accy_b200_session_synchronize(accy_b200_session* s, void* stream) {
  return guarded(s, [&] {
    s->ensureDevice();
    const DriverTable& d = driver();
    CUstream_t on = stream ? static_cast<CUstream_t>(stream) : s->stream;
    CUresult_t r = d.cuStreamSynchronize(on);
    if (r != 0) {
      s->poisoned = true;
      s->check(r, "cuStreamSynchronize");
    }
    s->checkDeviceStatus(on);
  });
}

uint32_t accy_b200_session_release(accy_b200_session* s, uint64_t handle) {
  return guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    s->unload(e);
  });
}

uint32_t accy_b200_session_set_observer(accy_b200_session* s, accy_b200_observer observer, void* context) {
  return guarded(s, [&] {
    s->observer = observer;
    s->observer_context = context;
  });
}

const char* accy_b200_session_last_error(accy_b200_session* s) { return s ? s->last_error.c_str() : "null session"; }

const char* accy_b200_session_plan_summary(accy_b200_session* s, uint64_t handle) {
  const char* out = "";
  guarded(s, [&] { out = s->entryOf(handle).plan.summary.c_str(); });
  return out;
}

uint32_t accy_b200_session_work(accy_b200_session* s, uint64_t handle, accy_b200_work* work) {
  return guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    work->bytes = e.plan.work.bytes;
    work->flops = e.plan.work.flops;
    work->pairs = e.plan.work.pairs;
    work->launches = static_cast<uint32_t>(e.plan.launches.size());
    work->reserved = 0;
  });
}

uint32_t accy_b200_session_kernel_count(accy_b200_session* s, uint64_t handle, uint32_t* count) {
  return guarded(s, [&] { *count = static_cast<uint32_t>(s->entryOf(handle).plan.kernels.size()); });
}

const char* accy_b200_session_kernel_source(accy_b200_session* s, uint64_t handle, uint32_t index, const char** name,
                                            const char** options) {
  const char* out = nullptr;
  guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    if (index >= e.plan.kernels.size()) throw StatusError{ACCY_B200_INVALID_BUFFER, "kernel index out of range"};
    if (name) *name = e.plan.kernels[index].name.c_str();
    if (options) *options = e.kernels[index].options.c_str();
    out = e.plan.kernels[index].source.c_str();
  });
  return out;
}

uint32_t accy_b200_session_time_launches(accy_b200_session* s, uint32_t enable) {
  return guarded(s, [&] { s->time_launches = enable != 0; });
}

uint32_t accy_b200_session_last_kernel_ms(accy_b200_session* s, uint64_t handle, float* ms) {
  return guarded(s, [&] {
    Entry& e = s->entryOf(handle);
    if (!e.timed) throw StatusError{ACCY_B200_LAUNCH_FAILED, "no timed launch yet (timing is switched on by accy_b200_session_time_launches)"};
    const DriverTable& d = driver();
    s->check(d.cuEventSynchronize(e.ev_end), "cuEventSynchronize");
    s->check(d.cuEventElapsedTime(ms, e.ev_begin, e.ev_end), "cuEventElapsedTime");
  });
}

// ---------------------------------------------------------------------------------------------
// builder
// ---------------------------------------------------------------------------------------------
}  // extern "C"

struct accy_b200_builder {
  Builder builder;
  std::string last_error;
  std::vector<uint8_t> bytes;
  std::vector<std::string> names;
  explicit accy_b200_builder(const char* name) : builder(name ? name : "") {}
};

namespace {

template <typename F>
uint32_t built(accy_b200_builder* b, uint32_t* value, F&& body) {
  if (!b) return ACCY_B200_INVALID_HANDLE;
  try {
    uint32_t id = body();
    if (value) *value = id;
    return ACCY_B200_OK;
  } catch (const std::exception& e) {
    b->last_error = e.what();
    return ACCY_B200_INVALID_PROGRAM;
  }
}

std::vector<Dim> dimsOf(const char* const* names, const int64_t* extents, uint32_t rank) {
  std::vector<Dim> dims(rank);
  for (uint32_t i = 0; i < rank; ++i) dims[i] = Dim{names[i] ? names[i] : "", extents[i]};
  return dims;
}

std::vector<std::string> namesOf(const char* const* names, uint32_t count) {
  std::vector<std::string> out(count);
  for (uint32_t i = 0; i < count; ++i) out[i] = names[i] ? names[i] : "";
  return out;
}

DType dtypeOf(uint32_t code) {
  if (code >= kDTypeCount) throw TensorError("UnknownTag");
  return static_cast<DType>(code);
}

template <typename E>
E codeOf(uint32_t code, uint32_t count) {
  if (code >= count) throw TensorError("UnknownTag");
  return static_cast<E>(code);
}

}  // namespace

extern "C" {

uint32_t accy_b200_builder_create(const char* name, accy_b200_builder** builder) {
  if (!builder) return ACCY_B200_INVALID_HANDLE;
  *builder = new (std::nothrow) accy_b200_builder(name);
  return *builder ? ACCY_B200_OK : ACCY_B200_OUT_OF_MEMORY;
}

void accy_b200_builder_destroy(accy_b200_builder* b) { delete b; }

const char* accy_b200_builder_last_error(accy_b200_builder* b) { return b ? b->last_error.c_str() : "null builder"; }

uint32_t accy_b200_builder_input(accy_b200_builder* b, uint32_t dtype, const char* const* names, const int64_t* extents,
                                 uint32_t rank, uint32_t* value) {
  return built(b, value, [&] { return b->builder.input(dtypeOf(dtype), dimsOf(names, extents, rank)); });
}

uint32_t accy_b200_builder_constant(accy_b200_builder* b, uint32_t dtype, const char* const* names,
                                    const int64_t* extents, uint32_t rank, const void* payload, size_t payload_bytes,
                                    uint32_t* value) {
  return built(b, value, [&] {
    std::vector<Dim> dims = dimsOf(names, extents, rank);
    validateAuthoredDims(dims);
    return b->builder.constantBytes(Type{dtypeOf(dtype), dims}, static_cast<const uint8_t*>(payload), payload_bytes);
  });
}

uint32_t accy_b200_builder_full(accy_b200_builder* b, uint32_t dtype, const char* const* names, const int64_t* extents,
                                uint32_t rank, double fill, uint32_t* value) {
  return built(b, value, [&] {
    std::vector<Dim> dims = dimsOf(names, extents, rank);
    validateAuthoredDims(dims);
    return b->builder.fullFloat(Type{dtypeOf(dtype), dims}, fill);
  });
}

uint32_t accy_b200_builder_iota(accy_b200_builder* b, uint32_t dtype, const char* const* names, const int64_t* extents,
                                uint32_t rank, const char* axis, uint32_t* value) {
  return built(b, value, [&] { return b->builder.iota(dtypeOf(dtype), dimsOf(names, extents, rank), axis ? axis : ""); });
}

uint32_t accy_b200_builder_unary(accy_b200_builder* b, uint32_t op, uint32_t x, uint32_t* value) {
  return built(b, value, [&] { return b->builder.unary(codeOf<Unary>(op, 9), x); });
}

uint32_t accy_b200_builder_binary(accy_b200_builder* b, uint32_t op, uint32_t lhs, uint32_t rhs, uint32_t* value) {
  return built(b, value, [&] { return b->builder.alignedBinary(codeOf<Binary>(op, 7), lhs, rhs); });
}

uint32_t accy_b200_builder_compare(accy_b200_builder* b, uint32_t direction, uint32_t lhs, uint32_t rhs, uint32_t* value) {
  return built(b, value, [&] { return b->builder.alignedCompare(codeOf<Compare>(direction, 6), lhs, rhs); });
}

uint32_t accy_b200_builder_select(accy_b200_builder* b, uint32_t pred, uint32_t on_true, uint32_t on_false, uint32_t* value) {
  return built(b, value, [&] { return b->builder.alignedSelect(pred, on_true, on_false); });
}

uint32_t accy_b200_builder_reduce(accy_b200_builder* b, uint32_t x, uint32_t reducer, const char* const* axes,
                                  uint32_t axis_count, uint32_t* value) {
  return built(b, value, [&] { return b->builder.reduceNamed(x, codeOf<Reducer>(reducer, 3), namesOf(axes, axis_count)); });
}

uint32_t accy_b200_builder_reduce_with(accy_b200_builder* b, uint32_t x, uint32_t init, uint32_t reducer,
                                       const char* const* axes, uint32_t axis_count, uint32_t* value) {
  return built(b, value, [&] { return b->builder.reduceWith(x, init, codeOf<Reducer>(reducer, 3), namesOf(axes, axis_count)); });
}

uint32_t accy_b200_builder_mean(accy_b200_builder* b, uint32_t x, const char* const* axes, uint32_t axis_count, uint32_t* value) {
  return built(b, value, [&] { return b->builder.meanNamed(x, namesOf(axes, axis_count)); });
}

uint32_t accy_b200_builder_contract(accy_b200_builder* b, uint32_t lhs, uint32_t rhs, const char* const* axes,
                                    uint32_t axis_count, uint32_t* value) {
  return built(b, value, [&] { return b->builder.contract(lhs, rhs, namesOf(axes, axis_count)); });
}

uint32_t accy_b200_builder_rename(accy_b200_builder* b, uint32_t x, const char* old_name, const char* new_name, uint32_t* value) {
  return built(b, value, [&] { return b->builder.renameAxis(x, old_name ? old_name : "", new_name ? new_name : ""); });
}

uint32_t accy_b200_builder_split(accy_b200_builder* b, uint32_t x, const char* axis, const char* const* names,
                                 const int64_t* extents, uint32_t parts, uint32_t* value) {
  return built(b, value, [&] { return b->builder.splitAxis(x, axis ? axis : "", dimsOf(names, extents, parts)); });
}

uint32_t accy_b200_builder_merge(accy_b200_builder* b, uint32_t x, const char* const* axes, uint32_t axis_count,
                                 const char* merged, uint32_t* value) {
  return built(b, value, [&] { return b->builder.mergeAxes(x, namesOf(axes, axis_count), merged ? merged : ""); });
}

uint32_t accy_b200_builder_broadcast(accy_b200_builder* b, uint32_t x, const char* const* names, const int64_t* extents,
                                     uint32_t rank, uint32_t* value) {
  return built(b, value, [&] { return b->builder.broadcastAxes(x, dimsOf(names, extents, rank)); });
}

uint32_t accy_b200_builder_broadcast_op(accy_b200_builder* b, uint32_t x, const char* const* names,
                                        const int64_t* extents, uint32_t rank, uint32_t* value) {
  return built(b, value, [&] { return b->builder.broadcastOp(x, dimsOf(names, extents, rank)); });
}

uint32_t accy_b200_builder_value_type(accy_b200_builder* b, uint32_t value, accy_b200_descriptor* descriptor) {
  return built(b, nullptr, [&] {
    try {
      fillDescriptor(b->builder.typeOf(value), descriptor, &b->names);
    } catch (const StatusError& e) {
      throw std::runtime_error(e.message);
    }
    return 0u;
  });
}

uint32_t accy_b200_builder_finish(accy_b200_builder* b, const uint32_t* outputs, uint32_t output_count,
                                  const uint8_t** actp, size_t* length) {
  return built(b, nullptr, [&] {
    Program p = b->builder.finish(std::vector<uint32_t>(outputs, outputs + output_count));
    b->bytes = encodeProgram(p);
    *actp = b->bytes.data();
    *length = b->bytes.size();
    return 0u;
  });
}

uint32_t accy_b200_wire_reencode(const uint8_t* actp, size_t length, uint8_t* out, size_t capacity, size_t* out_length,
                                 char* error_name, size_t error_capacity) {
  try {
    Program p = decodeProgram(actp, length);
    std::vector<uint8_t> bytes = encodeProgram(p);
    if (out_length) *out_length = bytes.size();
    if (bytes.size() > capacity) return ACCY_B200_INVALID_BUFFER;
    std::memcpy(out, bytes.data(), bytes.size());
    return ACCY_B200_OK;
  } catch (const std::exception& e) {
    if (error_name && error_capacity) {
      std::strncpy(error_name, e.what(), error_capacity - 1);
      error_name[error_capacity - 1] = '\0';
    }
    return std::string(e.what()) == "UnsupportedVersion" ? ACCY_B200_UNSUPPORTED_VERSION : ACCY_B200_INVALID_PROGRAM;
  }
}

uint32_t accy_b200_wire_shard(const uint8_t* actp, size_t length, const char* axis, int64_t extent, uint8_t* out,
                              size_t capacity, size_t* out_length, uint32_t* partial_sum, char* error,
                              size_t error_capacity) {
  auto fail = [&](uint32_t status, const char* what) {
    if (error && error_capacity) {
      std::strncpy(error, what, error_capacity - 1);
      error[error_capacity - 1] = '\0';
    }
    return status;
  };
  try {
    Program p = decodeProgram(actp, length);
    ShardInfo info = analyseShardAxis(p, axis ? axis : "");
    Program piece = shardProgram(p, axis ? axis : "", extent);
    std::vector<uint8_t> bytes = encodeProgram(piece);
    if (out_length) *out_length = bytes.size();
    if (partial_sum) *partial_sum = info.partial_sum ? info.partial_fold : 0u;
    if (bytes.size() > capacity) return fail(ACCY_B200_INVALID_BUFFER, "output buffer too small");
    std::memcpy(out, bytes.data(), bytes.size());
    return ACCY_B200_OK;
  } catch (const PlanError& e) {
    return fail(ACCY_B200_COMPILE_FAILED, e.what());
  } catch (const std::exception& e) {
    return fail(ACCY_B200_INVALID_PROGRAM, e.what());
  }
}

namespace {
uint32_t transformedBytes(const std::function<Program()>& make, uint8_t* out, size_t capacity, size_t* out_length, char* error,
                          size_t error_capacity) {
  auto fail = [&](uint32_t status, const char* what) {
    if (error && error_capacity) {
      std::strncpy(error, what, error_capacity - 1);
      error[error_capacity - 1] = '\0';
    }
    return status;
  };
  try {
    std::vector<uint8_t> bytes = encodeProgram(make());
    if (out_length) *out_length = bytes.size();
    if (bytes.size() > capacity) return fail(ACCY_B200_INVALID_BUFFER, "output buffer too small");
    std::memcpy(out, bytes.data(), bytes.size());
    return ACCY_B200_OK;
  } catch (const std::exception& e) {
    return fail(ACCY_B200_INVALID_PROGRAM, e.what());
  }
}
}  // namespace

uint32_t accy_b200_wire_grad(const uint8_t* actp, size_t length, const uint64_t* wrt, uint32_t wrt_count,
                             uint32_t keep_value, uint8_t* out, size_t capacity, size_t* out_length, char* error,
                             size_t error_capacity) {
  return transformedBytes(
      [&] {
        Program p = decodeProgram(actp, length);
        std::vector<size_t> indices;
        for (uint32_t i = 0; i < wrt_count; ++i) indices.push_back(static_cast<size_t>(wrt[i]));
        return gradProgram(p, indices, keep_value != 0);
      },
      out, capacity, out_length, error, error_capacity);
}

uint32_t accy_b200_wire_jvp(const uint8_t* actp, size_t length, const uint64_t* wrt, uint32_t wrt_count, uint8_t* out,
                            size_t capacity, size_t* out_length, char* error, size_t error_capacity) {
  return transformedBytes(
      [&] {
        Program p = decodeProgram(actp, length);
        std::vector<size_t> indices;
        for (uint32_t i = 0; i < wrt_count; ++i) indices.push_back(static_cast<size_t>(wrt[i]));
        return jvpProgram(p, indices);
      },
      out, capacity, out_length, error, error_capacity);
}

uint32_t accy_b200_wire_vmap(const uint8_t* actp, size_t length, int64_t axis_size, const int64_t* in_axes,
                             uint32_t in_axis_count, uint32_t out_axis, const char* axis_name, uint8_t* out,
                             size_t capacity, size_t* out_length, char* error, size_t error_capacity) {
  return transformedBytes(
      [&] {
        Program p = decodeProgram(actp, length);
        std::vector<int64_t> axes(in_axes, in_axes + in_axis_count);
        return vmapProgram(p, axis_size, axes, out_axis, axis_name ? axis_name : "");
      },
      out, capacity, out_length, error, error_capacity);
}

uint32_t accy_b200_wire_describe(const uint8_t* actp, size_t length, char* out, size_t capacity, size_t* out_length) {
  try {
    Program p = decodeProgram(actp, length);
    std::ostringstream o;
    for (const Operation& op : p.ops) {
      o << op.id << " " << kindName(op.kind) << " " << dtypeName(op.result.dtype) << "[";
      for (size_t i = 0; i < op.result.dims.size(); ++i)
        o << (i ? "," : "") << op.result.dims[i].name << "=" << op.result.dims[i].extent;
      o << "]";
      for (uint32_t a : op.operands) o << " %" << a;
      o << "\n";
    }
    o << "outputs";
    for (uint32_t id : p.outputs) o << " %" << id;
    o << "\n";
    std::string text = o.str();
    if (out_length) *out_length = text.size();
    if (text.size() + 1 > capacity) return ACCY_B200_INVALID_BUFFER;
    std::memcpy(out, text.c_str(), text.size() + 1);
    return ACCY_B200_OK;
  } catch (const std::exception&) {
    return ACCY_B200_INVALID_PROGRAM;
  }
}

void accy_b200_test_use_fake_driver(int32_t enable) { useFakeDriver(enable != 0); }
void accy_b200_test_fake_fail(const char* driver_function, int32_t after_calls) {
  fakeFailAfter(driver_function ? driver_function : "", after_calls);
}
void accy_b200_test_fake_device_status(int32_t value) { fakeDeviceStatus(value); }
uint32_t accy_b200_test_fake_call_count(const char* driver_function) {
  // "nvrtcCompileProgram" counts real NVRTC runs of this process (cache hits, in memory or on disk, do not)
  if (driver_function && std::strcmp(driver_function, "nvrtcCompileProgram") == 0) return nvrtcCompileCount();
  return fakeCallCount(driver_function ? driver_function : "");
}

}  // extern "C"
