// accy_b200_probe_fp32_rates: two register-only micro-kernels that measure, on the current device,
// the instruction-throughput ceilings the FP32-bound row kernels are reported against.
//
//   * "sinf + 4 flop": what one (guess, point) pair of the mismatch program costs when written with
//     CUDA's own sinf and nothing else in the way: gap = sinf(frequency * time) - sample;
//     acc += gap * gap, with time and sample made up in registers (no memory traffic at all) and
//     phases over the benchmark's range (0 .. 98304 rad, below sinf's slow-path threshold).  The
//     figure is pairs per second; a kernel that reads its operands from memory and uses sinf
//     cannot beat it, one with a cheaper sine can.
//   * packed FMA: independent fma.rn.f32x2 chains, the FP32 pipe's peak in flop/s as this GPU
//     delivers it at its current clock.
//
// Both are timed with CUDA events on the caller's stream, best of three after a warm-up launch.
// Nothing is allocated: the kernels keep everything in registers and write one word to a file-scope
// device variable only under a condition that never holds (so the compiler keeps the arithmetic).
#include <cuda_runtime.h>

#include <cstdio>

#include "../../include/accy_b200.h"

namespace {

constexpr int kThreads = 256;
constexpr int kBlocksPerSm = 8;
constexpr int kPairsPerThread = 16384;    // sinf kernel: pairs per thread
constexpr int kFmaIterations = 8192;      // FMA kernel: iterations of 8 packed chains per thread

__device__ float g_sink;

__global__ void __launch_bounds__(kThreads) sinf_pairs(float frequency_step) {
  const float frequency = 0.001f + frequency_step * (float)(blockIdx.x * kThreads + threadIdx.x);
  float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
  float time = 0.25f * (float)(threadIdx.x & 31);
  const float sample = 0.125f;
#pragma unroll 4
  for (int i = 0; i < kPairsPerThread; i += 4) {
    const float g0 = sinf(frequency * time) - sample;
    const float g1 = sinf(frequency * (time + 0.25f)) - sample;
    const float g2 = sinf(frequency * (time + 0.5f)) - sample;
    const float g3 = sinf(frequency * (time + 0.75f)) - sample;
    acc0 += g0 * g0;
    acc1 += g1 * g1;
    acc2 += g2 * g2;
    acc3 += g3 * g3;
    time += 1.0f;
  }
  const float total = (acc0 + acc1) + (acc2 + acc3);
  if (total == -1.0f) g_sink = total;   // a sum of squares is never negative
}

__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long pk2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

__global__ void __launch_bounds__(kThreads) packed_fma(float seed) {
  const float s = seed + 1e-6f * (float)threadIdx.x;
  unsigned long long c0 = pk2(s, s + 1.0f), c1 = pk2(s + 2.0f, s + 3.0f), c2 = pk2(s + 4.0f, s + 5.0f),
                     c3 = pk2(s + 6.0f, s + 7.0f), c4 = pk2(s + 8.0f, s + 9.0f), c5 = pk2(s + 10.0f, s + 11.0f),
                     c6 = pk2(s + 12.0f, s + 13.0f), c7 = pk2(s + 14.0f, s + 15.0f);
  const unsigned long long a = pk2(0.999f, 1.001f), b = pk2(0.001f, -0.001f);
#pragma unroll 4
  for (int i = 0; i < kFmaIterations; ++i) {
    c0 = fma2(c0, a, b); c1 = fma2(c1, a, b); c2 = fma2(c2, a, b); c3 = fma2(c3, a, b);
    c4 = fma2(c4, a, b); c5 = fma2(c5, a, b); c6 = fma2(c6, a, b); c7 = fma2(c7, a, b);
  }
  const unsigned long long all = c0 ^ c1 ^ c2 ^ c3 ^ c4 ^ c5 ^ c6 ^ c7;
  if (all == 0x7fc000007fc00000ull) g_sink = seed;   // two quiet NaNs: never, with these operands
}

uint32_t fail(char* error, size_t capacity, const char* text) {
  if (error && capacity) snprintf(error, capacity, "%s", text);
  return ACCY_B200_LAUNCH_FAILED;
}

}  // namespace

extern "C" uint32_t accy_b200_probe_fp32_rates(void* stream, double* sinf_pairs_per_second, double* packed_fma_flops,
                                               char* error, size_t error_capacity) {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
    return fail(error, error_capacity, "no current CUDA device");
  cudaStream_t on = static_cast<cudaStream_t>(stream);
  cudaEvent_t begin, end;
  if (cudaEventCreate(&begin) != cudaSuccess || cudaEventCreate(&end) != cudaSuccess)
    return fail(error, error_capacity, "cudaEventCreate failed");
  const int blocks = sms * kBlocksPerSm;
  double best[2] = {0.0, 0.0};
  uint32_t status = ACCY_B200_OK;
  for (int which = 0; which < 2 && status == ACCY_B200_OK; ++which) {
    for (int rep = 0; rep < 4; ++rep) {   // rep 0 warms up
      cudaEventRecord(begin, on);
      if (which == 0) sinf_pairs<<<blocks, kThreads, 0, on>>>(6.0f / (float)(blocks * kThreads));
      else packed_fma<<<blocks, kThreads, 0, on>>>(1.0f);
      cudaEventRecord(end, on);
      cudaError_t rc = cudaEventSynchronize(end);
      if (rc == cudaSuccess) rc = cudaGetLastError();
      if (rc != cudaSuccess) {
        status = fail(error, error_capacity, cudaGetErrorString(rc));
        break;
      }
      float ms = 0.0f;
      cudaEventElapsedTime(&ms, begin, end);
      const double threads = (double)blocks * kThreads;
      const double units = which == 0 ? threads * kPairsPerThread : threads * kFmaIterations * 8.0 * 2.0 * 2.0;
      if (rep > 0 && ms > 0.0f && units / (ms * 1e-3) > best[which]) best[which] = units / (ms * 1e-3);
    }
  }
  cudaEventDestroy(begin);
  cudaEventDestroy(end);
  if (status != ACCY_B200_OK) return status;
  if (sinf_pairs_per_second) *sinf_pairs_per_second = best[0];
  if (packed_fma_flops) *packed_fma_flops = best[1];
  return ACCY_B200_OK;
}
