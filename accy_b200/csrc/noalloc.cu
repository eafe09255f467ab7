// accy_b200_mismatch_noalloc: the column-split fused reduction without any allocation.
//
// Who this is for: hosts that must not allocate device memory while they run.  Examples are a
// service that hands its whole device-memory budget to its own pool at start-up (so a later
// cudaMalloc from a library would fail or fragment the pool), a real-time loop that cannot take
// the implicit device synchronisation an allocation may cause, and code between two fixed points
// of a stream schedule where the allocator is simply off limits.  The session API
// (accy_b200_session_*) allocates device buffers for temporaries and scratch when it loads a
// program; this entry point never does.
//
// What it computes: out[g] = sum_p (sin(frequency[g] * time[p]) - sample[p])^2 in f32, the
// "mismatch" program (README `mismatch` vectorised over guesses), with the same two-pass
// deterministic schedule the planner picks when there are too few guesses to fill the GPU: the
// points are cut into column splits, one CTA folds each (guess, split) cell, and a second kernel
// folds a guess's partials in split order.
//
// Where the partials live: in `g_partials` below, a fixed array in the library's own device
// image.  Every GPU that loads the library carries these kMaxPartials*4 bytes (1 MiB) until the
// process exits.  The size is the limit of the entry point: guesses * splits must not exceed
// kMaxPartials, larger calls are refused with ACCY_B200_INVALID_BUFFER and a message.
//
// Sharing: every call on a device uses the same array.  A call overwrites exactly the cells it
// later reads (no cell has to start at zero, nothing is accumulated across calls), so calls that
// run one after another on a stream are independent; two calls that overlap on the GPU (different
// streams, or different host threads) race on the array and must be serialised by the caller.
//
// Set-up: in host code the name `g_partials` is only a handle, not a device address.  The first
// call on each device asks the runtime for the real address (cudaGetSymbolAddress, with that
// device current) and caches it; make that first call outside any stream capture.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/accy_b200.h"

namespace {

constexpr int kMaxPartials = 262144;          // floats: 1 MiB per device
constexpr int kThreads = 256;
constexpr int kVec = 4;
constexpr int kVectorsPerThread = 4;
constexpr long long kChunk = (long long)kThreads * kVec * kVectorsPerThread;  // 4096 points
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_partials[kMaxPartials];

float* g_partials_address[kMaxDevices];       // per device, filled by the first call on it
std::mutex g_setup_mutex;

__device__ __forceinline__ float block_sum(float v, float* cells) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(0xffffffffu, v, off, 32);
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) cells[warp] = v;
  __syncthreads();
  float acc = cells[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) acc = acc + cells[w];
  return acc;
}

// one CTA per (guess, split): folds its range of chunks, writes one partial
__global__ void __launch_bounds__(kThreads)
mismatch_partials(const float* __restrict__ frequency, const float* __restrict__ time,
                  const float* __restrict__ sample, float* __restrict__ partials, long long points,
                  long long chunks_per_split, int splits) {
  __shared__ float cells[kThreads / 32];
  const long long g = blockIdx.x;
  const float f = frequency[g];
  const long long chunk_begin = (long long)blockIdx.y * chunks_per_split;
  const long long chunk_end = chunk_begin + chunks_per_split;
  float acc = 0.0f;
  for (long long ck = chunk_begin; ck < chunk_end; ++ck) {
    const long long base = ck * kChunk;
#pragma unroll
    for (int j = 0; j < kVectorsPerThread; ++j) {
      const long long p0 = base + (long long)(j * kThreads + threadIdx.x) * kVec;
#pragma unroll
      for (int e = 0; e < kVec; ++e) {
        const long long p = p0 + e;
        if (p < points) {
          const float gap = __fsub_rn(sinf(__fmul_rn(f, time[p])), sample[p]);
          acc = __fadd_rn(acc, __fmul_rn(gap, gap));
        }
      }
    }
  }
  const float total = block_sum(acc, cells);
  if (threadIdx.x == 0) partials[g * splits + blockIdx.y] = total;
}

// one thread per guess: folds the partials in split order
__global__ void __launch_bounds__(128)
mismatch_combine(const float* __restrict__ partials, float* __restrict__ out, long long guesses, int splits) {
  const long long g = (long long)blockIdx.x * 128 + threadIdx.x;
  if (g >= guesses) return;
  float acc = partials[g * splits];
  for (int s = 1; s < splits; ++s) acc = __fadd_rn(acc, partials[g * splits + s]);
  out[g] = acc;
}

uint32_t fail(char* error, size_t capacity, uint32_t status, const char* text) {
  if (error && capacity) snprintf(error, capacity, "%s", text);
  return status;
}

}  // namespace

extern "C" uint32_t accy_b200_mismatch_noalloc(const float* frequency, const float* time, const float* sample,
                                               float* out, uint64_t guesses, uint64_t points, uint32_t splits,
                                               void* stream, char* error, size_t error_capacity) {
  if (!frequency || !time || !sample || !out)
    return fail(error, error_capacity, ACCY_B200_INVALID_BUFFER, "null buffer");
  if (guesses == 0 || points == 0 || guesses > 0x7fffffffull)
    return fail(error, error_capacity, ACCY_B200_INVALID_BUFFER, "guesses and points must be positive (guesses < 2^31)");
  const long long chunks = (long long)((points + kChunk - 1) / kChunk);
  if (splits == 0) splits = 1;
  if ((long long)splits > chunks) splits = (uint32_t)chunks;
  if (splits > 65535u) splits = 65535u;
  const long long chunks_per_split = (chunks + splits - 1) / splits;
  splits = (uint32_t)((chunks + chunks_per_split - 1) / chunks_per_split);
  if (guesses * (uint64_t)splits > (uint64_t)kMaxPartials) {
    char text[160];
    snprintf(text, sizeof(text), "guesses * splits = %llu exceeds the built-in scratch of %d partials",
             (unsigned long long)(guesses * splits), kMaxPartials);
    return fail(error, error_capacity, ACCY_B200_INVALID_BUFFER, text);
  }
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail(error, error_capacity, ACCY_B200_LAUNCH_FAILED, "no current CUDA device");
  float* partials = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_partials_address[device]) {
      void* address = nullptr;
      cudaError_t rc = cudaGetSymbolAddress(&address, g_partials);
      if (rc != cudaSuccess)
        return fail(error, error_capacity, ACCY_B200_LAUNCH_FAILED, cudaGetErrorString(rc));
      g_partials_address[device] = static_cast<float*>(address);
    }
    partials = g_partials_address[device];
  }
  cudaStream_t on = static_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)guesses, splits);
  // An error the caller's own runtime calls left pending on this thread is not this call's: it is
  // handed back as such (and thereby cleared) before anything is launched.
  cudaError_t rc = cudaGetLastError();
  if (rc != cudaSuccess) {
    char text[200];
    snprintf(text, sizeof(text), "an earlier CUDA error was pending on this thread, nothing launched: %s", cudaGetErrorString(rc));
    return fail(error, error_capacity, ACCY_B200_LAUNCH_FAILED, text);
  }
  mismatch_partials<<<grid, kThreads, 0, on>>>(frequency, time, sample, partials, (long long)points,
                                                chunks_per_split, (int)splits);
  rc = cudaGetLastError();
  if (rc != cudaSuccess) return fail(error, error_capacity, ACCY_B200_LAUNCH_FAILED, cudaGetErrorString(rc));
  mismatch_combine<<<(unsigned)((guesses + 127) / 128), 128, 0, on>>>(partials, out, (long long)guesses, (int)splits);
  rc = cudaGetLastError();
  if (rc != cudaSuccess) return fail(error, error_capacity, ACCY_B200_LAUNCH_FAILED, cudaGetErrorString(rc));
  return ACCY_B200_OK;
}
