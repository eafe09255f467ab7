// Fused scaled-dot-product attention for sm_100a: O = softmax(scale * Q K^T [+ causal mask]) V.
//
// Replaces the reference's flash-attention lowering (src/preparation/kernelization/lowering/
// flash.zig:330-604: f32 only, head dim 64, non-causal, 32x32 tiles of scalar FMAs) and its
// library SDPA (src/kernel/library/attention.zig:389-441) with a tcgen05 kernel for bf16,
// head dim 128, optional causal mask, any number of leading batch axes:
//   * one CTA owns 256 consecutive queries of one (batch, head) as two 128-row tiles; K/V blocks
//     of 128 keys stream through a TMA ring and are shared by both tiles;
//   * S = Q K^T and O += P V run on the tensor cores (tcgen05.mma, f32 accumulators in TMEM:
//     S0, S1, O0, O1 = 4 x 128 columns); P is written back over S as bf16 and read by the second
//     MMA straight from TMEM;
//   * two softmax warpgroups (one per tile, one thread per query row, so row max and row sum need
//     no shuffles) work in ping-pong with the MMA issuer: while one tile's softmax runs the
//     tensor cores serve the other tile;
//   * online softmax in f32 in the log2 domain (ex2.approx of fma(s, scale*log2e, -m)); O is only
//     rescaled when a row's running max grows by more than 2^8, so the rescale through TMEM is rare;
//   * causal programs skip key blocks above the diagonal and mask only the diagonal block.
// Every mbarrier wait is bounded; on expiry the kernel sets the device status word and returns.
#include <cmath>
#include <sstream>

#include "plan.hpp"

namespace accy {

extern const char* kConvertPrelude;
extern const char* kTcPreludeShared;
bool attentionReady() { return true; }

namespace {

void replaceAll(std::string& s, const std::string& from, const std::string& to) {
  size_t at = 0;
  while ((at = s.find(from, at)) != std::string::npos) {
    s.replace(at, from.size(), to);
    at += to.size();
  }
}

const char* kAttentionTemplate = R"CUDA(
#define SEQ_Q @SEQ_Q@
#define SEQ_K @SEQ_K@
#define BATCH @BATCH@
#define CAUSAL @CAUSAL@
#define HEAD_DIM 128
#define TILE 128
#define KV_STAGES 2
#define TILE_BYTES (TILE * HEAD_DIM * 2)   // one 128 x 128 bf16 tile: two 64-wide boxes of 16 KB
#define HALF_BYTES (TILE * 64 * 2)
#define SCALE_LOG2 @SCALE_LOG2@f
#define RESCALE_THRESHOLD 8.0f
#define POLY_SHARE @POLY_SHARE@   // of every 8 pairs in the second half of a 64-column group
#define HALF_HANDOFF @HALF_HANDOFF@   // P is handed to the MMA issuer 64 keys at a time
#define ABLATE @ABLATE@
#define BH_MAJOR @BH_MAJOR@
#define ATTN_TRACE @TRACE@        // development aid: one CTA records clock stamps of its hand-offs and prints them
#ifndef INFINITY
#define INFINITY __int_as_float(0x7f800000)
#endif

// packed f32x2 helpers (two IEEE f32 operations per instruction)
__device__ __forceinline__ unsigned long long pk2(float lo, float hi) { unsigned long long r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ unsigned long long pk2u(unsigned int lo, unsigned int hi) { unsigned long long r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r; }
__device__ __forceinline__ void upk2(unsigned long long v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) { unsigned long long r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ unsigned long long sub2(unsigned long long a, unsigned long long b) { unsigned long long r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) { unsigned long long r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
// 2^x for a pair of values on the FMA pipe: x = n + f with n = round(x), f in [-1/2, 1/2];
// 2^f by a degree-4 polynomial (error below 2^-14, the result is rounded to bf16 afterwards),
// then n is added to the exponent field.  x is clamped at -126 so the exponent cannot wrap.
__device__ __forceinline__ void poly_exp2_pair(unsigned long long x2, float& out0, float& out1) {
  float x0, x1;
  upk2(x2, x0, x1);
  x2 = pk2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
  const unsigned long long magic2 = pk2(12582912.0f, 12582912.0f);
  const unsigned long long t2 = add2(x2, magic2);
  const unsigned long long f2 = sub2(x2, sub2(t2, magic2));
  unsigned long long p2 = fma2(f2, pk2(0.00961813f, 0.00961813f), pk2(0.05550411f, 0.05550411f));
  p2 = fma2(p2, f2, pk2(0.24022651f, 0.24022651f));
  p2 = fma2(p2, f2, pk2(0.69314718f, 0.69314718f));
  p2 = fma2(p2, f2, pk2(1.0f, 1.0f));
  float p0, p1, t0, t1;
  upk2(p2, p0, p1);
  upk2(t2, t0, t1);
  out0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  out1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// three-input max (one instruction on sm_100) where the compiler's PTX version has it
#if __CUDACC_VER_MAJOR__ > 12 || (__CUDACC_VER_MAJOR__ == 12 && __CUDACC_VER_MINOR__ >= 9)
__device__ __forceinline__ float max3(float a, float b, float c) { float r; asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c)); return r; }
#else
__device__ __forceinline__ float max3(float a, float b, float c) { return fmaxf(a, fmaxf(b, c)); }
#endif

__device__ __forceinline__ void tc_st32(unsigned int taddr, const unsigned int* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
               "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
               :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                  "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                  "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                  "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}

extern "C" __global__ void __launch_bounds__(384, 1)
@KERNEL@(const __grid_constant__ TensorMap map_q, const __grid_constant__ TensorMap map_k,
         const __grid_constant__ TensorMap map_v, unsigned short* __restrict__ O, int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((unsigned long long)smem_raw + 1023ull) & ~1023ull);
  // layout: Q tile 0, Q tile 1, K stages, V stages, barriers
  unsigned char* q_smem = smem;
  unsigned char* k_smem = smem + 2 * TILE_BYTES;
  unsigned char* v_smem = k_smem + KV_STAGES * TILE_BYTES;
  unsigned long long* bars = (unsigned long long*)(v_smem + KV_STAGES * TILE_BYTES);
  // bars: 0 q_full | 1..2 k_full | 3..4 k_empty | 5..6 v_full | 7..8 v_empty | 9..10 s_full | 11..12 p_full | 13..14 pv_done
  //       15..16 p_half (the first 64 keys of P are in TMEM)
  unsigned int* tmem_holder = (unsigned int*)(bars + 24);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  volatile unsigned int* turn = (volatile unsigned int*)(tmem_holder + 2);
  volatile unsigned int* zero_word = (volatile unsigned int*)(tmem_holder + 3);
  const unsigned int bar0 = smem_u32(bars);
#define BAR(i) (bar0 + 8u * (i))
#if ATTN_TRACE
  unsigned int* trace = (unsigned int*)(bars + 32);
#define TRACE_SOFTMAX @TRACE_SM@
#define TRACE_J0 8
#define TRACE_N 6
#define TR(role, j, e) if (blockIdx.x == 0 && (j) >= TRACE_J0 && (j) < TRACE_J0 + TRACE_N) trace[((role) * TRACE_N + (j) - TRACE_J0) * 8 + (e)] = (unsigned int)clock64();
#else
#define TRACE_SOFTMAX 0
#define TR(role, j, e)
#endif
  const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // work item: heaviest query pairs first
  const int n_pairs = SEQ_Q / (2 * TILE);
#if BH_MAJOR
  // the CTAs of one (batch, head) are launched together so that its K and V stay in L2
  const int pair = n_pairs - 1 - (int)(blockIdx.x % n_pairs);
  const int bh = (int)(blockIdx.x / n_pairs);
#else
  const int pair = n_pairs - 1 - (int)(blockIdx.x / BATCH);
  const int bh = (int)(blockIdx.x % BATCH);
#endif
  const int q_row0 = pair * 2 * TILE;
  // key blocks each tile attends to
#if CAUSAL
  const int n0 = q_row0 / TILE + 1, n1 = n0 + 1;
#else
  const int n0 = SEQ_K / TILE, n1 = n0;
#endif

  if (threadIdx.x == 0) {
    for (int i = 0; i < 11; ++i) mbar_init(BAR(i), (i >= 3 && i <= 4) || (i >= 7 && i <= 8) ? 2 : 1);   // the empties take one arrival per tile
    mbar_init(BAR(11), 4); mbar_init(BAR(12), 4);
    mbar_init(BAR(13), 1); mbar_init(BAR(14), 1);
    mbar_init(BAR(15), 4); mbar_init(BAR(16), 4);
    *abort_flag = 0;
    *turn = 0;
    *zero_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_holder)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned int tmem_base = *tmem_holder;
  // TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t overwrites the first 64 columns of S_t

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(BAR(0), 2 * TILE_BYTES);
      for (int t = 0; t < 2; ++t)
        for (int h = 0; h < 2; ++h)
          tma_load_3d(smem_u32(q_smem + t * TILE_BYTES + h * HALF_BYTES), &map_q, BAR(0), h * 64, q_row0 + t * TILE, bh);
      bool ok = true;
      for (int j = 0; ok && j < n1; ++j) {
        const int stage = j % KV_STAGES;
        const unsigned int ph = (unsigned int)((j / KV_STAGES) & 1);
        if (!mbar_wait(BAR(3 + stage), ph ^ 1u, abort_flag)) { ok = false; break; }
        if (ABLATE == 5 && j >= 2) mbar_arrive(BAR(1 + stage)); else {
        mbar_expect_tx(BAR(1 + stage), TILE_BYTES);
        for (int h = 0; h < 2; ++h)
          tma_load_3d(smem_u32(k_smem + stage * TILE_BYTES + h * HALF_BYTES), &map_k, BAR(1 + stage), h * 64, j * TILE, bh);
        }
        if (!mbar_wait(BAR(7 + stage), ph ^ 1u, abort_flag)) { ok = false; break; }
        if (ABLATE == 5 && j >= 2) mbar_arrive(BAR(5 + stage)); else {
        mbar_expect_tx(BAR(5 + stage), TILE_BYTES);
        for (int h = 0; h < 2; ++h)
          tma_load_3d(smem_u32(v_smem + stage * TILE_BYTES + h * HALF_BYTES), &map_v, BAR(5 + stage), h * 64, j * TILE, bh);
        }
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ---------------- MMA issuers: warp 1 serves tile 0, warp 10 tile 1 ----------------
    // One thread per tile issues that tile's MMAs.  The tensor pipe takes MMAs no faster than a
    // thread hands them over, and a thread's barrier probes, fences and commits cost it tens to
    // hundreds of cycles each; with two issuers those run while the other tile's MMAs are issued.
    // The issuers take strict turns (a counter in shared memory): tile 0's PV and next S, then
    // tile 1's, and so on.  The turns keep the two tiles half a period apart, so that one tile's
    // softmax has the special-function unit to itself while the other tile's MMAs execute; they
    // are a matter of speed only, every data dependence goes through the mbarriers.
    if (lane == 0) {
      const int t = warp == 1 ? 0 : 1;
      const int n_t = t == 0 ? n0 : n1;
      // S = Q K^T: A, B K-major, M = N = 128.  O += P V: A from TMEM, B = V with dim contiguous (N-major).
      const unsigned int idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned int)(TILE >> 3) << 17) | ((unsigned int)(TILE >> 4) << 24);
      const unsigned int idesc_o = idesc_s | (1u << 16);
      const unsigned int s_tmem = tmem_base + t * TILE, o_tmem = tmem_base + 2 * TILE + t * TILE;
      const unsigned long long q_desc = smem_desc(smem_u32(q_smem + t * TILE_BYTES), 16, 1024);
      bool ok = true;
      auto wait_kv = [&](int base, int j) {
        return mbar_wait(BAR(base + j % KV_STAGES), (unsigned int)((j / KV_STAGES) & 1), abort_flag);
      };
      auto wait_turn = [&](unsigned int want) {
        for (unsigned int i = 0; i < SPIN_LIMIT; ++i) {
          if (*turn == want) return true;
          if ((i & 255u) == 255u && *abort_flag) return false;
        }
        *abort_flag = 1;
        return false;
      };
      // descriptors advance by adding to their 14-bit address field (16-byte units)
      auto issue_s = [&](int j) {
        const unsigned long long k_desc = smem_desc(smem_u32(k_smem + (j % KV_STAGES) * TILE_BYTES), 16, 1024);
#pragma unroll
        for (int k = 0; k < HEAD_DIM / 16; ++k) {
          const unsigned long long off = (unsigned long long)(((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4);
          tc_mma_ss(s_tmem, q_desc + off, k_desc + off, idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(BAR(9 + t));
        tc_commit(BAR(3 + j % KV_STAGES));   // K stage free (one arrival per tile)
      };
      auto issue_pv_part = [&](int j, int k0) {
        const unsigned long long v_desc = smem_desc(smem_u32(v_smem + (j % KV_STAGES) * TILE_BYTES), HALF_BYTES, 1024);
#pragma unroll
        for (int k = k0; k < k0 + TILE / 32; ++k)
          tc_mma_ts(o_tmem, s_tmem + k * 8, v_desc + (unsigned long long)((k * 16 * 128) >> 4), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
      };
      // turns: 0 tile 0's first S, 1 tile 1's first S, then 2 + 2 j + t for step j of tile t
      ok = mbar_wait(BAR(0), 0, abort_flag) && wait_kv(1, 0) && wait_turn((unsigned int)t);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        *turn = (unsigned int)t + 1u;
      }
      for (int j = 0; ok && j < n_t; ++j) {
        const unsigned int ph = (unsigned int)(j & 1);
        const unsigned int my_turn = 2u + 2u * (unsigned int)j + (unsigned int)t;
        const bool more = j + 1 < n_t;
        TR(t * 3, j, 0)
        // the operands first (they are normally long in place), then P, then the turn
        if (!wait_kv(5, j) || (more && !wait_kv(1, j + 1))) { ok = false; break; }
        if (!mbar_wait(BAR((HALF_HANDOFF ? 15 : 11) + t), ph, abort_flag)) { ok = false; break; }
        TR(t * 3, j, 1)
        if (!wait_turn(my_turn)) { ok = false; break; }
        TR(t * 3, j, 2)
        tc_fence_after();
        issue_pv_part(j, 0);
        if (HALF_HANDOFF) {
          if (!mbar_wait(BAR(11 + t), ph, abort_flag)) { ok = false; break; }
          TR(t * 3, j, 3)
          tc_fence_after();
        }
        issue_pv_part(j, TILE / 32);
        tc_commit(BAR(13 + t));               // O_t holds blocks 0..j
        tc_commit(BAR(7 + j % KV_STAGES));    // V stage free (one arrival per tile)
        TR(t * 3, j, 4)
        if (more) issue_s(j + 1);
        TR(t * 3, j, 5)
        *turn = my_turn + 1u;
#if ATTN_TRACE
        if (blockIdx.x == 0 && j >= TRACE_J0 && j < TRACE_J0 + TRACE_N) {
          unsigned long long ns; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
          trace[(t * 3 * TRACE_N + j - TRACE_J0) * 8 + 7] = (unsigned int)ns;
        }
#endif
      }
      // causal programs: tile 1 has one more step, and its turn follows a turn of tile 0
      if (ok && t == 0 && n1 > n0) {
        const unsigned int my_turn = 2u + 2u * (unsigned int)n0;
        if (wait_turn(my_turn)) *turn = my_turn + 1u;
      }
    }
  } else if (warp >= 2 && warp < 10) {
    // ---------------- softmax + correction + epilogue: warps 2..5 tile 0, warps 6..9 tile 1 ----------------
    const int t = (warp - 2) >> 2;
    const unsigned int quarter = warp & 3u;
    const int row = (int)(quarter * 32 + lane);           // query row inside the tile
    const int n_t = t == 0 ? n0 : n1;
    const unsigned int lane_base = (quarter * 32u) << 16;
    const unsigned int s_addr = tmem_base + lane_base + t * TILE;
    const unsigned int o_addr = tmem_base + lane_base + 2 * TILE + t * TILE;
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int j = 0; ok && j < n_t; ++j) {
      if (((TRACE_SOFTMAX >> 0) & 1) && row == 0) { TR(1 + t, j, 0) }
      if (!mbar_wait(BAR(9 + t), (unsigned int)(j & 1), abort_flag)) { ok = false; break; }
      if (((TRACE_SOFTMAX >> 1) & 1) && row == 0) { TR(1 + t, j, 1) }
      tc_fence_after();
      const bool diagonal = CAUSAL && (j == n_t - 1);
      // the whole score row (128 columns) is read once and stays in registers for the row max
      // and for the exponentials; the four loads are in flight together
      unsigned int r0[32], r1[32], r2[32], r3[32];
      if (ABLATE == 4) {
#pragma unroll
        for (int i = 0; i < 32; ++i) { r0[i] = (unsigned int)(j * 77 + i + row) << 18; r1[i] = r0[i] + 3; r2[i] = r0[i] + 2; r3[i] = r0[i] + 1; }
      } else {
      tc_ld32(s_addr, r0);
      tc_ld32(s_addr + 32, r1);
      tc_ld32(s_addr + 64, r2);
      tc_ld32(s_addr + 96, r3);
      tc_wait_ld();
      }
      if (((TRACE_SOFTMAX >> 2) & 1) && row == 0) { TR(1 + t, j, 2) }
      // row max.  The scale is positive, so the max is taken over the raw scores and scaled once;
      // four chains of three-input max fold the 128 values.
      float m_blk;
      {
        float a = -INFINITY, b = -INFINITY, c = -INFINITY, d = -INFINITY;
        if (diagonal) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            a = fmaxf(a, i > row ? -INFINITY : __uint_as_float(r0[i]));
            b = fmaxf(b, 32 + i > row ? -INFINITY : __uint_as_float(r1[i]));
            c = fmaxf(c, 64 + i > row ? -INFINITY : __uint_as_float(r2[i]));
            d = fmaxf(d, 96 + i > row ? -INFINITY : __uint_as_float(r3[i]));
          }
        } else if (ABLATE == 2) {
          a = b = c = d = 1.0f;
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            a = max3(a, __uint_as_float(r0[i]), __uint_as_float(r0[i + 1]));
            b = max3(b, __uint_as_float(r1[i]), __uint_as_float(r1[i + 1]));
            c = max3(c, __uint_as_float(r2[i]), __uint_as_float(r2[i + 1]));
            d = max3(d, __uint_as_float(r3[i]), __uint_as_float(r3[i + 1]));
          }
        }
        m_blk = fmaxf(fmaxf(a, b), fmaxf(c, d)) * SCALE_LOG2;
      }
      if (j == 0) {
        m_run = m_blk;
      } else {
        const float m_new = fmaxf(m_run, m_blk);
        const bool need = (m_new - m_run) > RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          const float factor = need ? fast_exp2(m_run - m_new) : 1.0f;
          if (need) { m_run = m_new; l_run *= factor; }
          // O of this tile is up to date once the previous P V product has completed
          if (!mbar_wait(BAR(13 + t), (unsigned int)((j - 1) & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
          // rare path: the first score registers serve as scratch and the scores are read again
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tc_ld32(o_addr + c * 32, r0);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r0[i] = __float_as_uint(__uint_as_float(r0[i]) * factor);
            tc_st32(o_addr + c * 32, r0);
          }
          tc_wait_st();
          tc_ld32(s_addr, r0);
          tc_ld32(s_addr + 32, r1);
          tc_ld32(s_addr + 64, r2);
          tc_ld32(s_addr + 96, r3);
          tc_wait_ld();
        }
      }
      // p = 2^(scale * s - m) as packed FMAs and ex2, packed row sums, bf16 pairs written over S
      // 64 keys at a time.  A fixed share of the exponentials (POLY_SHARE of every 8 pairs of the
      // odd quarters) can run on the FMA pipe instead of the special-function unit.
      if (((TRACE_SOFTMAX >> 3) & 1) && row == 0) { TR(1 + t, j, 3) }
      const unsigned long long c2 = pk2(SCALE_LOG2, SCALE_LOG2);
      unsigned long long nm2 = pk2(-m_run, -m_run);
      unsigned long long l2a = pk2(0.0f, 0.0f), l2b = l2a;
#define EXP_QUARTER(R, COL0, OUT, AT, ACC, MASKED, POLY)                                     \
      _Pragma("unroll")                                                                      \
      for (int i = 0; i < 32; i += 2) {                                                      \
        const unsigned long long x2 = fma2(pk2u(R[i], R[i + 1]), c2, nm2);                   \
        float p0, p1;                                                                        \
        if (!(MASKED) && (POLY) && ((i >> 1) & 7) < POLY_SHARE) {                            \
          poly_exp2_pair(x2, p0, p1);                                                        \
        } else {                                                                             \
          upk2(x2, p0, p1);                                                                  \
          if (MASKED) {                                                                      \
            if ((COL0) + i > row) p0 = -INFINITY;                                            \
            if ((COL0) + i + 1 > row) p1 = -INFINITY;                                        \
          }                                                                                  \
          if (ABLATE != 1) {                                                                 \
          p0 = fast_exp2(p0);                                                                \
          p1 = fast_exp2(p1);                                                                \
          }                                                                                  \
        }                                                                                    \
        ACC = add2(ACC, pk2(p0, p1));                                                        \
        OUT[(AT) + (i >> 1)] = pack_bf16(p0, p1);                                            \
      }
#define HALF_READY()                                                                         \
      if (HALF_HANDOFF) {                                                                    \
        tc_wait_st();                                                                        \
        tc_fence_before();                                                                   \
        __syncwarp();                                                                        \
        if (lane == 0) mbar_arrive(BAR(15 + t));                                             \
        /* the second half's arithmetic takes a word read after the arrival (always zero) as an  \
           input, so that it cannot be scheduled ahead of the store and the arrival above */      \
        const unsigned int z = *zero_word;                                                   \
        nm2 = pk2u(__float_as_uint(-m_run) | z, __float_as_uint(-m_run) | z);                \
      }
      {
        unsigned int pa[32], pb[32];
        if (diagonal) {
          EXP_QUARTER(r0, 0, pa, 0, l2a, true, false)
          EXP_QUARTER(r1, 32, pa, 16, l2b, true, false)
          tc_st32(s_addr, pa);
          HALF_READY()
          EXP_QUARTER(r2, 64, pb, 0, l2a, true, false)
          EXP_QUARTER(r3, 96, pb, 16, l2b, true, false)
          tc_st32(s_addr + 32, pb);
        } else {
          EXP_QUARTER(r0, 0, pa, 0, l2a, false, false)
          EXP_QUARTER(r1, 32, pa, 16, l2b, false, true)
          if (ABLATE != 3) tc_st32(s_addr, pa); else l2a = add2(l2a, pk2u(pa[0] ^ pa[5] ^ pa[17], pa[31] ^ pa[9]));
          HALF_READY()
          if (((TRACE_SOFTMAX >> 4) & 1) && row == 0) { TR(1 + t, j, 4) }
          EXP_QUARTER(r2, 64, pb, 0, l2a, false, false)
          if (((TRACE_SOFTMAX >> 5) & 1) && row == 0) { TR(1 + t, j, 5) }
          EXP_QUARTER(r3, 96, pb, 16, l2b, false, true)
          if (ABLATE != 3) tc_st32(s_addr + 32, pb); else l2a = add2(l2a, pk2u(pb[0] ^ pb[5] ^ pb[17], pb[31] ^ pb[9]));
        }
      }
      {
        float s0, s1;
        upk2(add2(l2a, l2b), s0, s1);
        l_run += s0 + s1;
      }
      if (((TRACE_SOFTMAX >> 6) & 1) && row == 0) { TR(1 + t, j, 6) }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(11 + t));
      if (((TRACE_SOFTMAX >> 7) & 1) && row == 0) { TR(1 + t, j, 7) }
#if ATTN_TRACE
      if (!((TRACE_SOFTMAX >> 7) & 1) && lane == 0) { TR(1 + t, j, 4 + (int)quarter) }
#endif
    }
    // epilogue: O / l -> bf16 -> global
    if (ok && mbar_wait(BAR(13 + t), (unsigned int)((n_t - 1) & 1), abort_flag)) {
      tc_fence_after();
      const float inv = 1.0f / l_run;
      unsigned short* orow = O + ((long long)bh * SEQ_Q + q_row0 + t * TILE + row) * HEAD_DIM;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        unsigned int r[32];
        tc_ld32(o_addr + c * 32, r);
        tc_wait_ld();
        uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          dst[q] = make_uint4(pack_bf16(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv),
                              pack_bf16(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv),
                              pack_bf16(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv),
                              pack_bf16(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv));
        }
      }
    }
  }

  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
#if ATTN_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int role = 0; role < 4; ++role)
      for (int j = 0; j < TRACE_N; ++j) {
        const unsigned int* e = trace + (role * TRACE_N + j) * 8;
        printf("TRACE role %d j %d : %u %u %u %u %u %u %u %u\n", role, TRACE_J0 + j, e[0], e[1], e[2], e[3], e[4], e[5], e[6], e[7]);
      }
  }
#endif
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512) : "memory");
  }
}
)CUDA";

}  // namespace

void emitAttention(const AttentionOp& a, const std::string& name, Plan& plan, const ScheduleOverrides& ov) {
  if (a.head_dim != 128 || a.q_len % 256 != 0 || a.k_len % 128 != 0)
    throw PlanError("attention shape not covered by the fused kernel");
  std::string src = std::string(kConvertPrelude) + kTcPreludeShared + kAttentionTemplate;
  std::ostringstream scale;
  scale.precision(9);
  scale << std::scientific << static_cast<double>(a.scale) * 1.4426950408889634;
  replaceAll(src, "@KERNEL@", name);
  replaceAll(src, "@SEQ_Q@", std::to_string(a.q_len));
  replaceAll(src, "@SEQ_K@", std::to_string(a.k_len));
  replaceAll(src, "@BATCH@", std::to_string(a.batch));
  replaceAll(src, "@CAUSAL@", a.causal ? "1" : "0");
  replaceAll(src, "@SCALE_LOG2@", scale.str());
  // share of exponentials moved to the FMA pipe: 0/8, 2/8, 4/8 or 8/8 of the pairs of one half,
  // i.e. none, 1/8, 1/4 or 1/2 of all elements
  // measured on the causal 4096 x 128 benchmark: none 847, 1/8 832, 1/4 812, 1/2 797 TFLOP/s, so the
  // automatic choice is none (the kernel is bound by MMA/softmax hand-off latency, not by the
  // special-function unit)
  const int poly_code = ov.attention_poly & 7;
  const int poly_share = poly_code == 2 ? 2 : poly_code == 3 ? 4 : poly_code == 4 ? 8 : 0;
  replaceAll(src, "@POLY_SHARE@", std::to_string(poly_share));
  replaceAll(src, "@HALF_HANDOFF@", (ov.attention_poly & 8) ? "0" : "1");
  const bool trace = (ov.attention_poly & 16) != 0;
  replaceAll(src, "@BH_MAJOR@", (ov.attention_poly & 256) ? "0" : "1");
  replaceAll(src, "@ABLATE@", std::to_string((ov.attention_poly >> 5) & 7));
  replaceAll(src, "@TRACE@", trace ? "1" : "0");
  replaceAll(src, "@TRACE_SM@", std::to_string((ov.attention_poly >> 9) & 255));
  KernelSource ks;
  ks.name = name;
  ks.family = "attention";
  ks.source = src;
  plan.kernels.push_back(ks);

  Launch l;
  l.kernel = static_cast<int>(plan.kernels.size()) - 1;
  const long long items = (a.q_len / 256) * a.batch;
  if (items > 0x7fffffffll) throw PlanError("too many attention work items");
  l.grid[0] = static_cast<uint32_t>(items);
  l.block[0] = 384;
  l.dynamic_smem = 6 * 32768 + 1024 + 256 + (trace ? 4096 : 0);
  l.label = name;
  auto map = [&](int slot, int64_t seq) {
    KernelArg m;
    m.is_slot = false;
    m.tensor_map = true;
    m.tma.slot = slot;
    m.tma.rank = 3;
    m.tma.elem_bytes = 2;
    m.tma.swizzle = 3;
    m.tma.dims[0] = 128;
    m.tma.dims[1] = static_cast<uint64_t>(seq);
    m.tma.dims[2] = static_cast<uint64_t>(a.batch);
    m.tma.strides[0] = 128 * 2;
    m.tma.strides[1] = static_cast<uint64_t>(seq) * 128 * 2;
    m.tma.box[0] = 64;
    m.tma.box[1] = 128;
    m.tma.box[2] = 1;
    return m;
  };
  l.args.push_back(map(a.q_slot, a.q_len));
  l.args.push_back(map(a.k_slot, a.k_len));
  l.args.push_back(map(a.v_slot, a.k_len));
  KernelArg o;
  o.slot = a.o_slot;
  l.args.push_back(o);
  KernelArg st;
  st.slot = -2;
  l.args.push_back(st);
  plan.launches.push_back(l);
}

}  // namespace accy
