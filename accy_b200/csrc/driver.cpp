// Loader for the CUDA driver API and NVRTC, plus the recording fake driver used by host tests.
#include "driver.hpp"

#include <dlfcn.h>
#include <unistd.h>

#include <cstdio>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>

namespace accy {
namespace {

std::mutex g_mutex;
bool g_use_fake = false;
bool g_real_loaded = false;
DriverTable g_real{};
std::map<std::string, unsigned> g_fake_calls;
std::map<std::string, int> g_fake_fail;  // function -> remaining successful calls before failing
int g_fake_device_status = 0;            // what the next 4-byte device-to-host reads deliver (0 = the memory's own bytes)

template <typename F>
void bind(void* lib, F& slot, const char* symbol) {
  void* p = dlsym(lib, symbol);
  if (!p) throw std::runtime_error(std::string("CUDA driver symbol missing: ") + symbol);
  slot = reinterpret_cast<F>(p);
}

void loadReal() {
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) throw std::runtime_error("cannot load libcuda.so.1: the B200 target has no CPU fallback");
  bind(lib, g_real.cuInit, "cuInit");
  bind(lib, g_real.cuDeviceGet, "cuDeviceGet");
  bind(lib, g_real.cuDeviceGetCount, "cuDeviceGetCount");
  bind(lib, g_real.cuDeviceGetAttribute, "cuDeviceGetAttribute");
  bind(lib, g_real.cuDevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain");
  bind(lib, g_real.cuDevicePrimaryCtxRelease, "cuDevicePrimaryCtxRelease_v2");
  bind(lib, g_real.cuCtxSetCurrent, "cuCtxSetCurrent");
  bind(lib, g_real.cuModuleLoadData, "cuModuleLoadData");
  bind(lib, g_real.cuModuleUnload, "cuModuleUnload");
  bind(lib, g_real.cuModuleGetFunction, "cuModuleGetFunction");
  bind(lib, g_real.cuFuncSetAttribute, "cuFuncSetAttribute");
  bind(lib, g_real.cuLaunchKernel, "cuLaunchKernel");
  bind(lib, g_real.cuMemAlloc, "cuMemAlloc_v2");
  bind(lib, g_real.cuMemFree, "cuMemFree_v2");
  bind(lib, g_real.cuMemcpyHtoDAsync, "cuMemcpyHtoDAsync_v2");
  bind(lib, g_real.cuMemcpyDtoHAsync, "cuMemcpyDtoHAsync_v2");
  bind(lib, g_real.cuMemsetD8Async, "cuMemsetD8Async");
  bind(lib, g_real.cuStreamCreate, "cuStreamCreate");
  bind(lib, g_real.cuStreamDestroy, "cuStreamDestroy_v2");
  bind(lib, g_real.cuStreamSynchronize, "cuStreamSynchronize");
  bind(lib, g_real.cuStreamWaitEvent, "cuStreamWaitEvent");
  bind(lib, g_real.cuEventCreate, "cuEventCreate");
  bind(lib, g_real.cuEventDestroy, "cuEventDestroy_v2");
  bind(lib, g_real.cuEventRecord, "cuEventRecord");
  bind(lib, g_real.cuEventSynchronize, "cuEventSynchronize");
  bind(lib, g_real.cuEventElapsedTime, "cuEventElapsedTime");
  bind(lib, g_real.cuGetErrorName, "cuGetErrorName");
  bind(lib, g_real.cuTensorMapEncodeTiled, "cuTensorMapEncodeTiled");
  bind(lib, g_real.cuStreamBeginCapture, "cuStreamBeginCapture_v2");
  bind(lib, g_real.cuStreamEndCapture, "cuStreamEndCapture");
  bind(lib, g_real.cuGraphInstantiateWithFlags, "cuGraphInstantiateWithFlags");
  bind(lib, g_real.cuGraphLaunch, "cuGraphLaunch");
  bind(lib, g_real.cuGraphExecDestroy, "cuGraphExecDestroy");
  bind(lib, g_real.cuGraphDestroy, "cuGraphDestroy");
  CUresult_t r = g_real.cuInit(0);
  if (r != 0) throw std::runtime_error("cuInit failed: " + std::to_string(r));
  g_real_loaded = true;
}

// ---- fake driver: host memory stands for device memory, launches are only recorded ----
std::mutex g_fake_mutex;   // sessions of several devices call the fake from their own host threads
CUresult_t fakeResult(const char* fn) {
  std::lock_guard<std::mutex> lock(g_fake_mutex);
  g_fake_calls[fn] += 1;
  auto it = g_fake_fail.find(fn);
  if (it != g_fake_fail.end()) {
    if (it->second <= 0) return 700;  // CUDA_ERROR_ILLEGAL_ADDRESS, the reference maps it to DeviceLost
    it->second -= 1;
  }
  return 0;
}
CUresult_t f_cuInit(unsigned) { return fakeResult("cuInit"); }
CUresult_t f_cuDeviceGet(CUdevice_t* d, int o) { *d = o; return fakeResult("cuDeviceGet"); }
CUresult_t f_cuDeviceGetCount(int* n) { *n = 1; return fakeResult("cuDeviceGetCount"); }
CUresult_t f_cuDeviceGetAttribute(int* v, int attr, CUdevice_t) {
  *v = attr == 16 ? 148 : (attr == 75 ? 10 : (attr == 76 ? 0 : 0));
  return fakeResult("cuDeviceGetAttribute");
}
CUresult_t f_cuDevicePrimaryCtxRetain(CUcontext_t* c, CUdevice_t) { *c = reinterpret_cast<CUcontext_t>(0x1000); return fakeResult("cuDevicePrimaryCtxRetain"); }
CUresult_t f_cuDevicePrimaryCtxRelease(CUdevice_t) { return fakeResult("cuDevicePrimaryCtxRelease"); }
CUresult_t f_cuCtxSetCurrent(CUcontext_t) { return fakeResult("cuCtxSetCurrent"); }
CUresult_t f_cuModuleLoadData(CUmodule_t* m, const void*) { *m = reinterpret_cast<CUmodule_t>(0x2000); return fakeResult("cuModuleLoadData"); }
CUresult_t f_cuModuleUnload(CUmodule_t) { return fakeResult("cuModuleUnload"); }
CUresult_t f_cuModuleGetFunction(CUfunction_t* f, CUmodule_t, const char*) { *f = reinterpret_cast<CUfunction_t>(0x3000); return fakeResult("cuModuleGetFunction"); }
CUresult_t f_cuFuncSetAttribute(CUfunction_t, int, int) { return fakeResult("cuFuncSetAttribute"); }
CUresult_t f_cuLaunchKernel(CUfunction_t, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                            CUstream_t, void**, void**) { return fakeResult("cuLaunchKernel"); }
CUresult_t f_cuMemAlloc(CUdeviceptr_t* p, size_t n) {
  CUresult_t r = fakeResult("cuMemAlloc");
  if (r) return r;
  void* mem = nullptr;
  if (posix_memalign(&mem, 256, n ? n : 1) != 0) return 2;
  std::memset(mem, 0, n);
  *p = reinterpret_cast<CUdeviceptr_t>(mem);
  return 0;
}
CUresult_t f_cuMemFree(CUdeviceptr_t p) { free(reinterpret_cast<void*>(p)); return fakeResult("cuMemFree"); }
CUresult_t f_cuMemcpyHtoDAsync(CUdeviceptr_t d, const void* s, size_t n, CUstream_t) {
  CUresult_t r = fakeResult("cuMemcpyHtoDAsync");
  if (!r) std::memcpy(reinterpret_cast<void*>(d), s, n);
  return r;
}
CUresult_t f_cuMemcpyDtoHAsync(void* d, CUdeviceptr_t s, size_t n, CUstream_t) {
  CUresult_t r = fakeResult("cuMemcpyDtoHAsync");
  if (!r) std::memcpy(d, reinterpret_cast<void*>(s), n);
  // a kernel that gave up on a bounded wait leaves a code in the session's status word, which the
  // host reads back as one int: the fake delivers the injected code for such reads
  if (!r && n == sizeof(int) && g_fake_device_status != 0) std::memcpy(d, &g_fake_device_status, n);
  return r;
}
CUresult_t f_cuMemsetD8Async(CUdeviceptr_t d, unsigned char v, size_t n, CUstream_t) {
  std::memset(reinterpret_cast<void*>(d), v, n);
  return fakeResult("cuMemsetD8Async");
}
CUresult_t f_cuStreamCreate(CUstream_t* s, unsigned) { *s = reinterpret_cast<CUstream_t>(0x4000); return fakeResult("cuStreamCreate"); }
CUresult_t f_cuStreamDestroy(CUstream_t) { return fakeResult("cuStreamDestroy"); }
CUresult_t f_cuStreamSynchronize(CUstream_t) { return fakeResult("cuStreamSynchronize"); }
CUresult_t f_cuStreamWaitEvent(CUstream_t, CUevent_t, unsigned) { return fakeResult("cuStreamWaitEvent"); }
CUresult_t f_cuEventCreate(CUevent_t* e, unsigned) { *e = reinterpret_cast<CUevent_t>(0x5000); return fakeResult("cuEventCreate"); }
CUresult_t f_cuEventDestroy(CUevent_t) { return fakeResult("cuEventDestroy"); }
CUresult_t f_cuEventRecord(CUevent_t, CUstream_t) { return fakeResult("cuEventRecord"); }
CUresult_t f_cuEventSynchronize(CUevent_t) { return fakeResult("cuEventSynchronize"); }
CUresult_t f_cuEventElapsedTime(float* ms, CUevent_t, CUevent_t) { *ms = 0.0f; return fakeResult("cuEventElapsedTime"); }
CUresult_t f_cuGetErrorName(CUresult_t r, const char** s) {
  *s = r == 700 ? "CUDA_ERROR_ILLEGAL_ADDRESS" : "CUDA_ERROR_UNKNOWN";
  return 0;
}
CUresult_t f_cuTensorMapEncodeTiled(TensorMap* m, int, unsigned, void*, const uint64_t*, const uint64_t*,
                                    const uint32_t*, const uint32_t*, int, int, int, int) {
  std::memset(m, 0, sizeof(*m));
  return fakeResult("cuTensorMapEncodeTiled");
}

CUresult_t f_cuStreamBeginCapture(CUstream_t, int) { return fakeResult("cuStreamBeginCapture"); }
CUresult_t f_cuStreamEndCapture(CUstream_t, CUgraph_t* g) {
  *g = reinterpret_cast<CUgraph_t>(0x6000);
  return fakeResult("cuStreamEndCapture");
}
CUresult_t f_cuGraphInstantiateWithFlags(CUgraphExec_t* e, CUgraph_t, unsigned long long) {
  *e = reinterpret_cast<CUgraphExec_t>(0x7000);
  return fakeResult("cuGraphInstantiateWithFlags");
}
CUresult_t f_cuGraphLaunch(CUgraphExec_t, CUstream_t) { return fakeResult("cuGraphLaunch"); }
CUresult_t f_cuGraphExecDestroy(CUgraphExec_t) { return fakeResult("cuGraphExecDestroy"); }
CUresult_t f_cuGraphDestroy(CUgraph_t) { return fakeResult("cuGraphDestroy"); }

const DriverTable g_fake = {
    f_cuInit, f_cuDeviceGet, f_cuDeviceGetCount, f_cuDeviceGetAttribute, f_cuDevicePrimaryCtxRetain,
    f_cuDevicePrimaryCtxRelease, f_cuCtxSetCurrent, f_cuModuleLoadData, f_cuModuleUnload,
    f_cuModuleGetFunction, f_cuFuncSetAttribute, f_cuLaunchKernel, f_cuMemAlloc, f_cuMemFree,
    f_cuMemcpyHtoDAsync, f_cuMemcpyDtoHAsync, f_cuMemsetD8Async, f_cuStreamCreate, f_cuStreamDestroy,
    f_cuStreamSynchronize, f_cuStreamWaitEvent, f_cuEventCreate, f_cuEventDestroy, f_cuEventRecord,
    f_cuEventSynchronize, f_cuEventElapsedTime, f_cuGetErrorName, f_cuTensorMapEncodeTiled,
    f_cuStreamBeginCapture, f_cuStreamEndCapture, f_cuGraphInstantiateWithFlags, f_cuGraphLaunch,
    f_cuGraphExecDestroy, f_cuGraphDestroy};

// ---- NVRTC ----
struct Nvrtc {
  int (*createProgram)(void**, const char*, const char*, int, const char* const*, const char* const*);
  int (*compileProgram)(void*, int, const char* const*);
  int (*getCUBINSize)(void*, size_t*);
  int (*getCUBIN)(void*, char*);
  int (*getProgramLogSize)(void*, size_t*);
  int (*getProgramLog)(void*, char*);
  int (*destroyProgram)(void**);
  const char* (*getErrorString)(int);
  int (*version)(int*, int*);
  bool loaded = false;
} g_nvrtc;

void loadNvrtc() {
  // ACCY_B200_NVRTC names a specific file.  Otherwise the bare name comes first, so a process that
  // already holds an NVRTC (for instance the one bundled with PyTorch) shares it; the kernels guard
  // what newer PTX versions add (three-input max) by the compiler version.  Measured on the row
  // kernels, NVRTC 12.8 code was 1 % (softmax + layer norm) to 10 % (sin-heavy mismatch) faster than
  // 12.9 code, and equal on attention.
  const char* names[] = {getenv("ACCY_B200_NVRTC"), "libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12",
                         "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so"};
  void* lib = nullptr;
  for (const char* n : names) {
    if (!n || !*n) continue;
    lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    if (lib) break;
  }
  if (!lib) throw std::runtime_error("cannot load libnvrtc.so.12 (needed to build sm_100a kernels)");
  bind(lib, g_nvrtc.createProgram, "nvrtcCreateProgram");
  bind(lib, g_nvrtc.compileProgram, "nvrtcCompileProgram");
  bind(lib, g_nvrtc.getCUBINSize, "nvrtcGetCUBINSize");
  bind(lib, g_nvrtc.getCUBIN, "nvrtcGetCUBIN");
  bind(lib, g_nvrtc.getProgramLogSize, "nvrtcGetProgramLogSize");
  bind(lib, g_nvrtc.getProgramLog, "nvrtcGetProgramLog");
  bind(lib, g_nvrtc.destroyProgram, "nvrtcDestroyProgram");
  bind(lib, g_nvrtc.getErrorString, "nvrtcGetErrorString");
  bind(lib, g_nvrtc.version, "nvrtcVersion");
  g_nvrtc.loaded = true;
}

}  // namespace

const DriverTable& driver() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_use_fake) return g_fake;
  if (!g_real_loaded) loadReal();
  return g_real;
}

void useFakeDriver(bool enable) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_use_fake = enable;
  std::lock_guard<std::mutex> fake_lock(g_fake_mutex);
  g_fake_calls.clear();
  g_fake_fail.clear();
  g_fake_device_status = 0;
}

void fakeDeviceStatus(int value) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_fake_device_status = value;
}

void fakeFailAfter(const std::string& function, int calls) {
  std::lock_guard<std::mutex> lock(g_fake_mutex);
  if (calls < 0) g_fake_fail.erase(function);
  else g_fake_fail[function] = calls;
}

unsigned fakeCallCount(const std::string& function) {
  std::lock_guard<std::mutex> lock(g_fake_mutex);
  auto it = g_fake_calls.find(function);
  return it == g_fake_calls.end() ? 0 : it->second;
}

std::string driverErrorName(CUresult_t r) {
  const char* s = nullptr;
  try {
    driver().cuGetErrorName(r, &s);
  } catch (...) {
  }
  return s ? std::string(s) : ("CUresult " + std::to_string(r));
}

// Compiled kernels are kept for the life of the process, keyed by the exact source text and
// options (the reference keeps its JIT-compiled modules keyed by PTX text,
// deps/lib/compiler/gpu/src/cuda.zig): compiling a program a second time, in this or another
// session, costs a lookup instead of 0.3-1.4 s of NVRTC per kernel.  ACCY_B200_NO_KERNEL_CACHE=1
// turns it off.
namespace {
std::mutex g_cubin_mutex;
std::map<std::string, std::vector<char>> g_cubins;
size_t g_cubin_bytes = 0;
constexpr size_t kCubinCacheLimit = 256u << 20;

// The same cache on disk, for the next process: ACCY_B200_KERNEL_CACHE_DIR names a directory
// (nothing is written anywhere unless it is set).  One file per kernel, named by a hash of the
// compiler version, options and source; the file repeats that text in full and is used only if
// it matches, so a hash collision or a truncated file costs a recompilation, never a wrong kernel.
const char kDiskMagic[8] = {'A', 'C', 'C', 'Y', 'C', 'U', 'B', '1'};

std::string diskPath(const std::string& key) {
  const char* dir = getenv("ACCY_B200_KERNEL_CACHE_DIR");
  if (!dir || !*dir) return "";
  uint64_t h1 = 1469598103934665603ull, h2 = 0x9e3779b97f4a7c15ull;
  for (unsigned char ch : key) {
    h1 = (h1 ^ ch) * 1099511628211ull;
    h2 = (h2 + ch) * 0xff51afd7ed558ccdull;
    h2 ^= h2 >> 29;
  }
  char name[64];
  std::snprintf(name, sizeof name, "/accy_%016llx%016llx.cubin", static_cast<unsigned long long>(h1),
                static_cast<unsigned long long>(h2));
  return std::string(dir) + name;
}

bool readDisk(const std::string& path, const std::string& key, std::vector<char>* cubin) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) return false;
  bool ok = false;
  char magic[8];
  uint64_t key_size = 0, cubin_size = 0;
  if (std::fread(magic, 1, 8, f) == 8 && std::memcmp(magic, kDiskMagic, 8) == 0 &&
      std::fread(&key_size, 8, 1, f) == 1 && std::fread(&cubin_size, 8, 1, f) == 1 && key_size == key.size() &&
      cubin_size > 0 && cubin_size <= kCubinCacheLimit) {
    std::string stored(key_size, '\0');
    cubin->resize(cubin_size);
    ok = std::fread(&stored[0], 1, key_size, f) == key_size && stored == key &&
         std::fread(cubin->data(), 1, cubin_size, f) == cubin_size && std::fgetc(f) == EOF;
  }
  std::fclose(f);
  return ok;
}

void writeDisk(const std::string& path, const std::string& key, const std::vector<char>& cubin) {
  // written under a private name and renamed into place, so a reader never sees half a file
  const std::string tmp = path + ".tmp" + std::to_string(static_cast<long long>(getpid()));
  FILE* f = std::fopen(tmp.c_str(), "wb");
  if (!f) return;
  const uint64_t key_size = key.size(), cubin_size = cubin.size();
  bool ok = std::fwrite(kDiskMagic, 1, 8, f) == 8 && std::fwrite(&key_size, 8, 1, f) == 1 &&
            std::fwrite(&cubin_size, 8, 1, f) == 1 && std::fwrite(key.data(), 1, key.size(), f) == key.size() &&
            std::fwrite(cubin.data(), 1, cubin.size(), f) == cubin.size();
  ok = std::fclose(f) == 0 && ok;
  if (!ok || std::rename(tmp.c_str(), path.c_str()) != 0) std::remove(tmp.c_str());
}

unsigned g_nvrtc_runs = 0;
}  // namespace

unsigned nvrtcCompileCount() {
  std::lock_guard<std::mutex> lock(g_cubin_mutex);
  return g_nvrtc_runs;
}

std::vector<char> compileToCubin(const std::string& source, const std::string& name,
                                 const std::vector<std::string>& extra_options, std::string* log) {
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_nvrtc.loaded) loadNvrtc();
  }
  const char* no_cache = getenv("ACCY_B200_NO_KERNEL_CACHE");
  const bool cached = !(no_cache && *no_cache == '1');
  std::string key, disk;
  if (cached) {
    int major = 0, minor = 0;
    g_nvrtc.version(&major, &minor);
    key = "nvrtc " + std::to_string(major) + "." + std::to_string(minor) + '\n';
    for (const std::string& o : extra_options) key += o + '\n';
    key += '\0';
    key += source;
    std::lock_guard<std::mutex> lock(g_cubin_mutex);
    auto hit = g_cubins.find(key);
    if (hit != g_cubins.end()) {
      if (log) log->clear();
      return hit->second;
    }
    disk = diskPath(key);
    std::vector<char> stored;
    if (!disk.empty() && readDisk(disk, key, &stored)) {
      if (log) log->clear();
      if (g_cubin_bytes + stored.size() + key.size() <= kCubinCacheLimit && g_cubins.emplace(key, stored).second)
        g_cubin_bytes += stored.size() + key.size();
      return stored;
    }
  }
  {
    std::lock_guard<std::mutex> lock(g_cubin_mutex);
    g_nvrtc_runs += 1;
  }
  void* prog = nullptr;
  int rc = g_nvrtc.createProgram(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr);
  if (rc != 0) throw std::runtime_error(std::string("nvrtcCreateProgram: ") + g_nvrtc.getErrorString(rc));
  std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo"};
  for (const std::string& o : extra_options) opts.push_back(o);
  std::vector<const char*> raw;
  for (const std::string& o : opts) raw.push_back(o.c_str());
  rc = g_nvrtc.compileProgram(prog, static_cast<int>(raw.size()), raw.data());
  size_t log_size = 0;
  g_nvrtc.getProgramLogSize(prog, &log_size);
  std::string text(log_size, '\0');
  if (log_size > 1) g_nvrtc.getProgramLog(prog, &text[0]);
  if (log) *log = text;
  if (rc != 0) {
    g_nvrtc.destroyProgram(&prog);
    throw std::runtime_error("nvrtc failed for " + name + ": " + g_nvrtc.getErrorString(rc) + "\n" + text);
  }
  size_t size = 0;
  g_nvrtc.getCUBINSize(prog, &size);
  std::vector<char> cubin(size);
  g_nvrtc.getCUBIN(prog, cubin.data());
  g_nvrtc.destroyProgram(&prog);
  if (cached) {
    std::lock_guard<std::mutex> lock(g_cubin_mutex);
    if (g_cubin_bytes + cubin.size() + key.size() <= kCubinCacheLimit && g_cubins.emplace(key, cubin).second)
      g_cubin_bytes += cubin.size() + key.size();
    if (!disk.empty()) writeDisk(disk, key, cubin);
  }
  return cubin;
}

}  // namespace accy
