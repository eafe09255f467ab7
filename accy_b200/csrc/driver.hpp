// Dynamically loaded CUDA driver API and NVRTC tables.
//
// The library links against neither: libcuda.so.1 and libnvrtc.so.12 are dlopen'ed on first use,
// like the reference's own driver table (deps/lib/base/sys/src/cuda.zig, dlopen'd symbol list and
// CUresult mapping).  Every driver entry point goes through a table of function pointers that a
// recording fake can replace, which is how the host logic is tested on machines without a GPU
// (deps/lib/compiler/gpu/src/runtime/cuda/runtime.zig:643-1031 does the same with fakeCu*).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace accy {

typedef int CUresult_t;
typedef int CUdevice_t;
typedef uint64_t CUdeviceptr_t;
typedef struct CUctx_st* CUcontext_t;
typedef struct CUmod_st* CUmodule_t;
typedef struct CUfunc_st* CUfunction_t;
typedef struct CUstream_st* CUstream_t;
typedef struct CUevent_st* CUevent_t;
typedef struct CUgraph_st* CUgraph_t;
typedef struct CUgraphExec_st* CUgraphExec_t;

struct alignas(64) TensorMap {
  uint64_t opaque[16];
};

struct DriverTable {
  CUresult_t (*cuInit)(unsigned);
  CUresult_t (*cuDeviceGet)(CUdevice_t*, int);
  CUresult_t (*cuDeviceGetCount)(int*);
  CUresult_t (*cuDeviceGetAttribute)(int*, int, CUdevice_t);
  CUresult_t (*cuDevicePrimaryCtxRetain)(CUcontext_t*, CUdevice_t);
  CUresult_t (*cuDevicePrimaryCtxRelease)(CUdevice_t);
  CUresult_t (*cuCtxSetCurrent)(CUcontext_t);
  CUresult_t (*cuModuleLoadData)(CUmodule_t*, const void*);
  CUresult_t (*cuModuleUnload)(CUmodule_t);
  CUresult_t (*cuModuleGetFunction)(CUfunction_t*, CUmodule_t, const char*);
  CUresult_t (*cuFuncSetAttribute)(CUfunction_t, int, int);
  CUresult_t (*cuLaunchKernel)(CUfunction_t, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                               unsigned, CUstream_t, void**, void**);
  CUresult_t (*cuMemAlloc)(CUdeviceptr_t*, size_t);
  CUresult_t (*cuMemFree)(CUdeviceptr_t);
  CUresult_t (*cuMemcpyHtoDAsync)(CUdeviceptr_t, const void*, size_t, CUstream_t);
  CUresult_t (*cuMemcpyDtoHAsync)(void*, CUdeviceptr_t, size_t, CUstream_t);
  CUresult_t (*cuMemsetD8Async)(CUdeviceptr_t, unsigned char, size_t, CUstream_t);
  CUresult_t (*cuStreamCreate)(CUstream_t*, unsigned);
  CUresult_t (*cuStreamDestroy)(CUstream_t);
  CUresult_t (*cuStreamSynchronize)(CUstream_t);
  CUresult_t (*cuStreamWaitEvent)(CUstream_t, CUevent_t, unsigned);
  CUresult_t (*cuEventCreate)(CUevent_t*, unsigned);
  CUresult_t (*cuEventDestroy)(CUevent_t);
  CUresult_t (*cuEventRecord)(CUevent_t, CUstream_t);
  CUresult_t (*cuEventSynchronize)(CUevent_t);
  CUresult_t (*cuEventElapsedTime)(float*, CUevent_t, CUevent_t);
  CUresult_t (*cuGetErrorName)(CUresult_t, const char**);
  CUresult_t (*cuTensorMapEncodeTiled)(TensorMap*, int dtype, unsigned rank, void* base,
                                       const uint64_t* dims, const uint64_t* strides,
                                       const uint32_t* box, const uint32_t* elem_strides,
                                       int interleave, int swizzle, int l2, int oob);
  // launch sequences recorded once and replayed (the reference's record_sequence / submit_sequence,
  // deps/lib/compiler/gpu/src/contract.zig:1929-1966)
  CUresult_t (*cuStreamBeginCapture)(CUstream_t, int mode);
  CUresult_t (*cuStreamEndCapture)(CUstream_t, CUgraph_t*);
  CUresult_t (*cuGraphInstantiateWithFlags)(CUgraphExec_t*, CUgraph_t, unsigned long long flags);
  CUresult_t (*cuGraphLaunch)(CUgraphExec_t, CUstream_t);
  CUresult_t (*cuGraphExecDestroy)(CUgraphExec_t);
  CUresult_t (*cuGraphDestroy)(CUgraph_t);
};

// Returns the active table: the real driver (loaded on first call) or the fake.  Throws
// std::runtime_error when the real driver cannot be loaded.
const DriverTable& driver();
void useFakeDriver(bool enable);
void fakeFailAfter(const std::string& function, int calls);
unsigned fakeCallCount(const std::string& function);
void fakeDeviceStatus(int value);   // the code later reads of the device status word return (0 = none)
std::string driverErrorName(CUresult_t r);

// NVRTC: CUDA source -> sm_100a cubin.  Throws std::runtime_error carrying the compiler log.
unsigned nvrtcCompileCount();  // NVRTC runs so far in this process (cache hits do not count)
std::vector<char> compileToCubin(const std::string& source, const std::string& name,
                                 const std::vector<std::string>& extra_options, std::string* log);

}  // namespace accy
