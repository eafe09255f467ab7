// Fused scaled-dot-product attention for sm_100a: O = softmax(scale * Q K^T [+ causal mask]) V.
//
// Replaces the reference's flash-attention lowering (src/preparation/kernelization/lowering/
// flash.zig:330-604: f32 only, head dim 64, non-causal, 32x32 tiles of scalar FMAs) and its
// library SDPA (src/kernel/library/attention.zig:389-441) with a tcgen05 kernel for bf16 or f16,
// head dim 128 or 64, optional causal mask, any number of leading batch axes:
//   * a work item is 256 consecutive queries of one (batch, head), handled as two 128-row tiles;
//     K/V blocks of 128 keys stream through a TMA ring and are shared by both tiles;
//   * the kernel is persistent: one CTA per SM takes work items from a counter in global memory
//     (in groups of 16 (batch, head) indices whose K and V stay in L2, heaviest query pairs of the
//     group first).  The TMA producer and the MMA issuers run ahead into the next item while the softmax
//     warps finish the current one, so the load latency, the pipeline fill and the epilogue of
//     one item overlap its neighbours;
//   * S = Q K^T and O += P V run on the tensor cores (tcgen05.mma, f32 accumulators in TMEM:
//     S0, S1, O0, O1 = 4 x 128 columns); P is written back over S as bf16 and read by the second
//     MMA straight from TMEM;
//   * two softmax warpgroups (one per tile, one thread per query row, so row max and row sum need
//     no shuffles) work in ping-pong with the MMA issuers: while one tile's softmax runs the
//     tensor cores serve the other tile;
//   * online softmax in f32 in the log2 domain (ex2.approx of fma(s, scale*log2e, -m)); O is only
//     rescaled when a row's running max grows by more than 2^8, so the rescale through TMEM is rare;
//   * causal programs skip key blocks above the diagonal and mask only the diagonal block;
//   * lengths need not be multiples of the tiles: loads past the end read zeros, the last key
//     block is masked, stores past the end are dropped.
// Every wait is bounded; on expiry the kernel sets the device status word and returns.
#include <algorithm>
#include <cmath>
#include <sstream>

#include "plan.hpp"

namespace accy {

extern const char* kConvertPrelude;
extern const char* kTcPreludeShared;

namespace {

void replaceAll(std::string& s, const std::string& from, const std::string& to) {
  size_t at = 0;
  while ((at = s.find(from, at)) != std::string::npos) {
    s.replace(at, from.size(), to);
    at += to.size();
  }
}

const char* kAttentionHead = R"CUDA(
#define SEQ_Q @SEQ_Q@
#define SEQ_K @SEQ_K@
#define BATCH @BATCH@
#define CAUSAL @CAUSAL@
#define HEAD_DIM @HEAD_DIM@   // 64 or 128
#define TILE 128
#define KV_STAGES 2
#define TILE_BYTES (TILE * HEAD_DIM * 2)   // one tile of 128 rows: HEAD_DIM / 64 boxes of 64 dims (16 KB each)
#define HALF_BYTES (TILE * 64 * 2)
#define N_PAIRS ((SEQ_Q + 2 * TILE - 1) / (2 * TILE))   // lengths need not be multiples of the tile: TMA
                                                        // loads read zeros past the end, TMA stores drop such rows
#define N_ITEMS (N_PAIRS * BATCH)
#define SCALE_LOG2 @SCALE_LOG2@f
#define RESCALE_THRESHOLD 8.0f
#define AB_FORMAT @AB_FORMAT@   // operand format of the MMAs: 0 = f16, 1 = bf16 (P is written in the same format)
#define PACK16 @PACK16@
#ifndef INFINITY
#define INFINITY __int_as_float(0x7f800000)
#endif

// packed f32x2 helpers (two IEEE f32 operations per instruction)
__device__ __forceinline__ unsigned long long pk2(float lo, float hi) { unsigned long long r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ unsigned long long pk2u(unsigned int lo, unsigned int hi) { unsigned long long r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r; }
__device__ __forceinline__ void upk2(unsigned long long v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) { unsigned long long r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) { unsigned long long r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
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

// TMA store of one staged tile (shared -> global), tracked by the thread's bulk-copy group
__device__ __forceinline__ void tma_store_3d(const TensorMap* map, unsigned int src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               :: "l"((unsigned long long)map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// work item -> (batch, head) index, first query row, key blocks of tile 0 and of tile 1.
// Items are ordered in groups of GROUP_HEADS (batch, head) indices; inside a group the heaviest
// query pairs of all its heads come first, then the next heaviest, and so on.  Handing out long
// items first keeps the CTAs' finishing times close together (causal items differ 16-fold in
// length at 4096 keys: per-head order left the last round 4 % short of full at 256 heads and 23 %
// at 32 heads, by a simulation of the queue), while the K and V of the heads of one or two groups
// (2 MB per head at 4096 x 128) stay in L2 for their other items.
#define GROUP_HEADS 16
__device__ __forceinline__ void decode_item(int item, int& bh, int& q_row0, int& n0, int& n1) {
  const int group = item / (GROUP_HEADS * N_PAIRS);
  const int rem = item - group * (GROUP_HEADS * N_PAIRS);
  const int left = BATCH - group * GROUP_HEADS;
  const int heads = left < GROUP_HEADS ? left : GROUP_HEADS;   // the last group may be smaller
  const int pair = N_PAIRS - 1 - rem / heads;                  // heaviest query pairs first
  bh = group * GROUP_HEADS + rem % heads;
  q_row0 = pair * 2 * TILE;
#if CAUSAL
  n0 = q_row0 / TILE + 1;
  n1 = n0 + 1;
#else
  n0 = (SEQ_K + TILE - 1) / TILE;
  n1 = n0;
#endif
}

// barriers (index into bars[]; arrivals per phase in brackets when not 1)
#define B_Q_FULL 0
#define B_Q_EMPTY 1        // [2] both tiles' last S of the item has read Q
#define B_K_FULL 2         // + stage
#define B_K_EMPTY 4        // + stage [2] one arrival per tile
#define B_V_FULL 6         // + stage
#define B_V_EMPTY 8        // + stage [2]
#define B_S_FULL 10        // + tile
#define B_P_FULL 12        // + tile [4] one arrival per softmax warp
#define B_PV_DONE 14       // + tile
#define B_P_HALF 16        // + tile [4] the first 64 keys of P are in TMEM
#define B_ITEM_FULL 18     // + slot: the next work item is published
#define B_ITEM_EMPTY 20    // + slot [10] both MMA issuers and the eight softmax warps have read it
#define N_BARS 22

extern "C" __global__ void __launch_bounds__(384, 1)
@KERNEL@(const __grid_constant__ TensorMap map_q, const __grid_constant__ TensorMap map_k,
         const __grid_constant__ TensorMap map_v, const __grid_constant__ TensorMap map_o, int* __restrict__ status,
         int* __restrict__ counters) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((unsigned long long)smem_raw + 1023ull) & ~1023ull);
  // layout: Q tile 0, Q tile 1, K stages, V stages, output staging, barriers, a few control words
  unsigned char* q_smem = smem;
  unsigned char* k_smem = smem + 2 * TILE_BYTES;
  unsigned char* v_smem = k_smem + KV_STAGES * TILE_BYTES;
  unsigned char* o_stage = v_smem + KV_STAGES * TILE_BYTES;   // 4 KB per softmax warp: 32 rows x 64 dims of O as bf16
  unsigned long long* bars = (unsigned long long*)(o_stage + 8 * 4096);
  unsigned int* tmem_holder = (unsigned int*)(bars + 24);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  volatile unsigned int* turn = (volatile unsigned int*)(tmem_holder + 2);
  volatile unsigned int* zero_word = (volatile unsigned int*)(tmem_holder + 3);
  volatile int* item_ring = (volatile int*)(tmem_holder + 4);   // two slots
  const unsigned int bar0 = smem_u32(bars);
#define BAR(i) (bar0 + 8u * (unsigned int)(i))
  const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) {
      int count = 1;
      if (i == B_Q_EMPTY || (i >= B_K_EMPTY && i < B_K_EMPTY + 2) || (i >= B_V_EMPTY && i < B_V_EMPTY + 2)) count = 2;
      if ((i >= B_P_FULL && i < B_P_FULL + 2) || (i >= B_P_HALF && i < B_P_HALF + 2)) count = 4;
      if (i >= B_ITEM_EMPTY) count = 10;
      mbar_init(BAR(i), count);
    }
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
    // ---------------- work distribution and TMA producer ----------------
    // The first item is the CTA's own index; further ones come from the counter in global memory.
    // Each item is published to the other warps through a two-slot ring; the K/V ring simply
    // continues from one item into the next, so the next item's first blocks are fetched while
    // the current item is still being computed.
    if (lane == 0) {
      int item = (int)blockIdx.x;
      unsigned int g = 0;   // K/V blocks loaded so far
      for (int it = 0;; ++it) {
        const int slot = it & 1;
        if (!mbar_wait(BAR(B_ITEM_EMPTY + slot), (unsigned int)((it >> 1) & 1) ^ 1u, abort_flag)) break;
        item_ring[slot] = item;
        mbar_arrive(BAR(B_ITEM_FULL + slot));
        if (item >= N_ITEMS) break;
        const int next = (int)gridDim.x + atomicAdd(counters, 1);
        int bh, q_row0, n0, n1;
        decode_item(item, bh, q_row0, n0, n1);
        (void)n0;
        // The item's first K/V block goes first: its stages come free a step earlier than the Q
        // tiles (which the previous item's last S still reads), so it is not held up behind Q.
        bool ok = true;
        for (int j = 0; j < n1; ++j, ++g) {
          if (j == (n1 > 1 ? 1 : 0)) {
            if (!mbar_wait(BAR(B_Q_EMPTY), (unsigned int)(it & 1) ^ 1u, abort_flag)) { ok = false; break; }
            mbar_expect_tx(BAR(B_Q_FULL), 2 * TILE_BYTES);
            for (int t = 0; t < 2; ++t)
              for (int h = 0; h < HEAD_DIM / 64; ++h)
                tma_load_3d(smem_u32(q_smem + t * TILE_BYTES + h * HALF_BYTES), &map_q, BAR(B_Q_FULL), h * 64, q_row0 + t * TILE, bh);
          }
          const unsigned int stage = g % KV_STAGES;
          const unsigned int ph = (g / KV_STAGES) & 1u;
          if (!mbar_wait(BAR(B_K_EMPTY + stage), ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(BAR(B_K_FULL + stage), TILE_BYTES);
          for (int h = 0; h < HEAD_DIM / 64; ++h)
            tma_load_3d(smem_u32(k_smem + stage * TILE_BYTES + h * HALF_BYTES), &map_k, BAR(B_K_FULL + stage), h * 64, j * TILE, bh);
          if (!mbar_wait(BAR(B_V_EMPTY + stage), ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_expect_tx(BAR(B_V_FULL + stage), TILE_BYTES);
          for (int h = 0; h < HEAD_DIM / 64; ++h)
            tma_load_3d(smem_u32(v_smem + stage * TILE_BYTES + h * HALF_BYTES), &map_v, BAR(B_V_FULL + stage), h * 64, j * TILE, bh);
        }
        if (!ok) break;
        item = next;
      }
    }
  } else if (warp == 1 || warp == 10) {
)CUDA";

const char* kAttentionIssuer = R"CUDA(
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
      // S = Q K^T: A, B K-major, M = N = 128.  O += P V: A from TMEM, B = V with dim contiguous (N-major).
      const unsigned int idesc_s = (1u << 4) | (AB_FORMAT << 7) | (AB_FORMAT << 10) | ((unsigned int)(TILE >> 3) << 17) | ((unsigned int)(TILE >> 4) << 24);
      // O += P V: M = 128, N = HEAD_DIM, B (= V) with the dims contiguous (N-major)
      const unsigned int idesc_o = (1u << 4) | (AB_FORMAT << 7) | (AB_FORMAT << 10) | (1u << 16) |
                                   ((unsigned int)(HEAD_DIM >> 3) << 17) | ((unsigned int)(TILE >> 4) << 24);
      const unsigned int s_tmem = tmem_base + t * TILE, o_tmem = tmem_base + 2 * TILE + t * TILE;
      const unsigned long long q_desc = smem_desc(smem_u32(q_smem + t * TILE_BYTES), 16, 1024);
      auto wait_turn = [&](unsigned int want) {
        for (unsigned int i = 0; i < SPIN_LIMIT; ++i) {
          if (*turn == want) return true;
          if ((i & 255u) == 255u && *abort_flag) return false;
        }
        *abort_flag = 1;
        return false;
      };
      // g counts K/V blocks over all items, in step with the producer
      auto wait_block = [&](int base, unsigned int g) {
        return mbar_wait(BAR(base + g % KV_STAGES), (g / KV_STAGES) & 1u, abort_flag);
      };
      // descriptors advance by adding to their 14-bit address field (16-byte units)
      auto issue_s_mmas = [&](unsigned int g) {
        const unsigned long long k_desc = smem_desc(smem_u32(k_smem + (g % KV_STAGES) * TILE_BYTES), 16, 1024);
#pragma unroll
        for (int k = 0; k < HEAD_DIM / 16; ++k) {
          const unsigned long long off = (unsigned long long)(((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4);
          tc_mma_ss(s_tmem, q_desc + off, k_desc + off, idesc_s, k > 0 ? 1u : 0u);
        }
      };
      auto issue_s = [&](unsigned int g, bool last_of_item) {
        issue_s_mmas(g);
        tc_commit(BAR(B_S_FULL + t));
        tc_commit(BAR(B_K_EMPTY + g % KV_STAGES));   // K stage free (one arrival per tile)
        if (last_of_item) tc_commit(BAR(B_Q_EMPTY));  // Q free (one arrival per tile)
      };
      auto issue_pv_part = [&](unsigned int g, int k0, bool first_block) {
        const unsigned long long v_desc = smem_desc(smem_u32(v_smem + (g % KV_STAGES) * TILE_BYTES), HALF_BYTES, 1024);
#pragma unroll
        for (int k = k0; k < k0 + TILE / 32; ++k)
          tc_mma_ts(o_tmem, s_tmem + k * 8, v_desc + (unsigned long long)((k * 16 * 128) >> 4), idesc_o, (!first_block || k > 0) ? 1u : 0u);
      };
      unsigned int g0 = 0;          // K/V blocks of earlier items
      unsigned int done = 0;        // blocks this tile has handled so far (parity of its barriers)
      unsigned int turn0 = 0;       // first turn of the current item
      bool ok = true;
      for (int it = 0; ok; ++it) {
        const int slot = it & 1;
        if (!mbar_wait(BAR(B_ITEM_FULL + slot), (unsigned int)((it >> 1) & 1), abort_flag)) break;
        const int item = item_ring[slot];
        mbar_arrive(BAR(B_ITEM_EMPTY + slot));
        if (item >= N_ITEMS) break;
        int bh, q_row0, n0, n1;
        decode_item(item, bh, q_row0, n0, n1);
        (void)bh; (void)q_row0;
        const int n_t = t == 0 ? n0 : n1;
        // turns of an item: 0 tile 0's first S, 1 tile 1's first S, then 2 + 2 j + t for step j of tile t
        ok = mbar_wait(BAR(B_Q_FULL), (unsigned int)(it & 1), abort_flag) && wait_block(B_K_FULL, g0) && wait_turn(turn0 + (unsigned int)t);
        if (!ok) break;
        tc_fence_after();
        issue_s(g0, n_t == 1);
        *turn = turn0 + (unsigned int)t + 1u;
        for (int j = 0; j < n_t; ++j, ++done) {
          const unsigned int ph = done & 1u;
          const unsigned int my_turn = turn0 + 2u + 2u * (unsigned int)j + (unsigned int)t;
          const unsigned int g = g0 + (unsigned int)j;
          const bool more = j + 1 < n_t;
          // the operands first (they are normally long in place), then P, then the turn
          if (!wait_block(B_V_FULL, g) || (more && !wait_block(B_K_FULL, g + 1))) { ok = false; break; }
          if (!mbar_wait(BAR(B_P_HALF + t), ph, abort_flag)) { ok = false; break; }
          if (!wait_turn(my_turn)) { ok = false; break; }
          tc_fence_after();
          issue_pv_part(g, 0, j == 0);
          if (!mbar_wait(BAR(B_P_FULL + t), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_pv_part(g, TILE / 32, j == 0);
          // The next S goes out before this step's other commits: the tile's softmax waits for
          // it, nothing waits as urgently for "O is up to date" or for the free V stage (a
          // commit covers everything issued before it, so those two now also wait for S), and
          // the other issuer gets the turn before this thread spends its ~55 cycles per commit.
          if (more) {
            issue_s_mmas(g + 1);
            tc_commit(BAR(B_S_FULL + t));
          }
          *turn = my_turn + 1u;
          tc_commit(BAR(B_PV_DONE + t));               // O_t holds blocks 0..j of the item
          tc_commit(BAR(B_V_EMPTY + g % KV_STAGES));   // V stage free (one arrival per tile)
          if (more) {
            tc_commit(BAR(B_K_EMPTY + (g + 1) % KV_STAGES));   // K stage free (one arrival per tile)
            if (j + 2 == n_t) tc_commit(BAR(B_Q_EMPTY));       // Q free (one arrival per tile)
          }
        }
        if (!ok) break;
        // causal items: tile 1 has one more block.  Tile 0 releases that block's stages on its
        // own behalf (once the block is in, i.e. the stage's previous round is over) and passes
        // the turn on.
        if (t == 0 && n1 > n0) {
          const unsigned int g = g0 + (unsigned int)n0;
          if (!wait_block(B_K_FULL, g)) break;
          mbar_arrive(BAR(B_K_EMPTY + g % KV_STAGES));
          if (!wait_block(B_V_FULL, g)) break;
          mbar_arrive(BAR(B_V_EMPTY + g % KV_STAGES));
          const unsigned int my_turn = turn0 + 2u + 2u * (unsigned int)n0;
          if (!wait_turn(my_turn)) break;
          *turn = my_turn + 1u;
        }
        g0 += (unsigned int)n1;
        turn0 += 2u + 2u * (unsigned int)n1;
      }
    }
)CUDA";

const char* kAttentionSoftmax = R"CUDA(
  } else if (warp >= 2 && warp < 10) {
    // ---------------- softmax + correction + epilogue: warps 2..5 tile 0, warps 6..9 tile 1 ----------------
    const int t = (warp - 2) >> 2;
    const unsigned int quarter = warp & 3u;
    const int row = (int)(quarter * 32 + lane);           // query row inside the tile
    const unsigned int lane_base = (quarter * 32u) << 16;
    const unsigned int s_addr = tmem_base + lane_base + t * TILE;
    const unsigned int o_addr = tmem_base + lane_base + 2 * TILE + t * TILE;
    unsigned int done = 0;   // blocks this tile has handled so far (parity of its barriers)
    bool ok = true;
    for (int it = 0; ok; ++it) {
      const int slot = it & 1;
      if (!mbar_wait(BAR(B_ITEM_FULL + slot), (unsigned int)((it >> 1) & 1), abort_flag)) break;
      const int item = item_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(B_ITEM_EMPTY + slot));
      if (item >= N_ITEMS) break;
      int bh, q_row0, n0, n1;
      decode_item(item, bh, q_row0, n0, n1);
      const int n_t = t == 0 ? n0 : n1;
      float m_run = -INFINITY, l_run = 0.0f;
      for (int j = 0; ok && j < n_t; ++j, ++done) {
        if (!mbar_wait(BAR(B_S_FULL + t), done & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // The last key block is masked: on the diagonal (causal) a row sees the keys up to its own
        // index, which also hides keys past the end; without a causal mask only a ragged key
        // length needs it, and every row sees the same SEQ_K % TILE keys of that block.
        const bool diagonal = (CAUSAL || SEQ_K % TILE != 0) && (j == n_t - 1);
        const int lim = CAUSAL ? row : SEQ_K % TILE - 1;
        // the whole score row (128 columns) is read once and stays in registers for the row max
        // and for the exponentials; the four loads are in flight together
        unsigned int r0[32], r1[32], r2[32], r3[32];
        tc_ld32(s_addr, r0);
        tc_ld32(s_addr + 32, r1);
        tc_ld32(s_addr + 64, r2);
        tc_ld32(s_addr + 96, r3);
        tc_wait_ld();
        // row max.  The scale is positive, so the max is taken over the raw scores and scaled
        // once; four chains of three-input max fold the 128 values.
        float m_blk;
        {
          float a = -INFINITY, b = -INFINITY, c = -INFINITY, d = -INFINITY;
          if (diagonal) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              a = fmaxf(a, i > lim ? -INFINITY : __uint_as_float(r0[i]));
              b = fmaxf(b, 32 + i > lim ? -INFINITY : __uint_as_float(r1[i]));
              c = fmaxf(c, 64 + i > lim ? -INFINITY : __uint_as_float(r2[i]));
              d = fmaxf(d, 96 + i > lim ? -INFINITY : __uint_as_float(r3[i]));
            }
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
            if (!mbar_wait(BAR(B_PV_DONE + t), (done - 1u) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            // rare path: the first score registers serve as scratch and the scores are read again
#pragma unroll 1
            for (int c = 0; c < HEAD_DIM / 32; ++c) {
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
        // 64 keys at a time (the first half of P V starts while the second half's exponentials run).
        const unsigned long long c2 = pk2(SCALE_LOG2, SCALE_LOG2);
        unsigned long long nm2 = pk2(-m_run, -m_run);
        unsigned long long l2a = pk2(0.0f, 0.0f), l2b = l2a;
#define EXP_QUARTER(R, COL0, OUT, AT, ACC, MASKED)                                           \
        _Pragma("unroll")                                                                    \
        for (int i = 0; i < 32; i += 2) {                                                    \
          const unsigned long long x2 = fma2(pk2u(R[i], R[i + 1]), c2, nm2);                 \
          float p0, p1;                                                                      \
          upk2(x2, p0, p1);                                                                  \
          if (MASKED) {                                                                      \
            if ((COL0) + i > lim) p0 = -INFINITY;                                            \
            if ((COL0) + i + 1 > lim) p1 = -INFINITY;                                        \
          }                                                                                  \
          p0 = fast_exp2(p0);                                                                \
          p1 = fast_exp2(p1);                                                                \
          ACC = add2(ACC, pk2(p0, p1));                                                      \
          OUT[(AT) + (i >> 1)] = PACK16(p0, p1);                                             \
        }
        // The second half's arithmetic takes a word read after the arrival (always zero) as an
        // input, so that it cannot be scheduled ahead of the first half's store and arrival.
#define HALF_READY()                                                                         \
        {                                                                                    \
          tc_wait_st();                                                                      \
          tc_fence_before();                                                                 \
          __syncwarp();                                                                      \
          if (lane == 0) mbar_arrive(BAR(B_P_HALF + t));                                     \
          const unsigned int z = *zero_word;                                                 \
          nm2 = pk2u(__float_as_uint(-m_run) | z, __float_as_uint(-m_run) | z);              \
        }
        {
          unsigned int pa[32], pb[32];
          if (diagonal) {
            EXP_QUARTER(r0, 0, pa, 0, l2a, true)
            EXP_QUARTER(r1, 32, pa, 16, l2b, true)
            tc_st32(s_addr, pa);
            HALF_READY()
            EXP_QUARTER(r2, 64, pb, 0, l2a, true)
            EXP_QUARTER(r3, 96, pb, 16, l2b, true)
            tc_st32(s_addr + 32, pb);
          } else {
            EXP_QUARTER(r0, 0, pa, 0, l2a, false)
            EXP_QUARTER(r1, 32, pa, 16, l2b, false)
            tc_st32(s_addr, pa);
            HALF_READY()
            EXP_QUARTER(r2, 64, pb, 0, l2a, false)
            EXP_QUARTER(r3, 96, pb, 16, l2b, false)
            tc_st32(s_addr + 32, pb);
          }
        }
        {
          float s0, s1;
          upk2(add2(l2a, l2b), s0, s1);
          l_run += s0 + s1;
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(B_P_FULL + t));
      }
      if (!ok) break;
      // epilogue: O / l -> bf16 -> global, once the item's last P V product has completed
      if (!mbar_wait(BAR(B_PV_DONE + t), (done - 1u) & 1u, abort_flag)) break;
      tc_fence_after();
      const float inv = 1.0f / l_run;
      // Each warp normalises its 32 rows, 64 dims at a time, into a 4 KB staging tile laid out in
      // the 128-byte swizzle (16-byte piece c of row l at piece c ^ (l % 8): the eight lanes of a
      // quarter warp hit eight different bank groups), and one lane hands the tile to the TMA
      // engine.  The rows of a thread are 256 bytes apart in global memory, so direct stores
      // would touch 32 lines per instruction; measured, the epilogue with direct stores cost the
      // benchmark 6 % (14 % for 1024-key items).
      unsigned char* stage = o_stage + (warp - 2) * 4096;
#pragma unroll 1
      for (int half = 0; half < HEAD_DIM / 64; ++half) {
        unsigned int ra[32], rb[32];
        tc_ld32(o_addr + half * 64, ra);
        tc_ld32(o_addr + half * 64 + 32, rb);
        tc_wait_ld();
        if (lane == 0) tma_store_wait_read();   // the previous store has finished reading the staging tile
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const unsigned int* r = c < 4 ? ra + c * 8 : rb + (c - 4) * 8;
          const uint4 v = make_uint4(PACK16(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv),
                                     PACK16(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv),
                                     PACK16(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv),
                                     PACK16(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv));
          *reinterpret_cast<uint4*>(stage + lane * 128 + ((c ^ (lane & 7)) << 4)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) tma_store_3d(&map_o, smem_u32(stage), half * 64, q_row0 + t * TILE + (int)quarter * 32, bh);
      }
      // the next item's first P V overwrites O: its P hand-over below comes after these loads
      tc_fence_before();
    }
  }
)CUDA";

const char* kAttentionTail = R"CUDA(
  if (warp >= 2 && warp < 10 && lane == 0) tma_store_wait_all();   // this thread's output tiles are written
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512) : "memory");
  }
  // the last CTA to leave clears the work counter for the next launch
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(counters + 1, 1) == (int)gridDim.x - 1) {
      counters[0] = 0;
      counters[1] = 0;
      __threadfence();
    }
  }
}
)CUDA";

}  // namespace

void emitAttention(const AttentionOp& a, const std::string& name, Plan& plan, const ScheduleOverrides& ov) {
  if ((a.head_dim != 128 && a.head_dim != 64) || a.q_len < 128 || a.k_len < 128)
    throw PlanError("attention shape not covered by the fused kernel");
  std::string src = std::string(kConvertPrelude) + kTcPreludeShared + kAttentionHead + kAttentionIssuer + kAttentionSoftmax + kAttentionTail;
  std::ostringstream scale;
  scale.precision(9);
  scale << std::scientific << static_cast<double>(a.scale) * 1.4426950408889634;
  replaceAll(src, "@KERNEL@", name);
  replaceAll(src, "@HEAD_DIM@", std::to_string(a.head_dim));
  replaceAll(src, "@SEQ_Q@", std::to_string(a.q_len));
  replaceAll(src, "@SEQ_K@", std::to_string(a.k_len));
  replaceAll(src, "@BATCH@", std::to_string(a.batch));
  replaceAll(src, "@CAUSAL@", a.causal ? "1" : "0");
  replaceAll(src, "@SCALE_LOG2@", scale.str());
  replaceAll(src, "@AB_FORMAT@", a.dtype == DType::f16 ? "0u" : "1u");
  replaceAll(src, "@PACK16@", a.dtype == DType::f16 ? "pack_f16" : "pack_bf16");
  KernelSource ks;
  ks.name = name;
  ks.family = "attention";
  ks.source = src;
  plan.kernels.push_back(ks);

  Launch l;
  l.kernel = static_cast<int>(plan.kernels.size()) - 1;
  const long long items = ((a.q_len + 255) / 256) * a.batch;
  if (items > 0x7fffffffll) throw PlanError("too many attention work items");
  // persistent: one CTA per SM (the kernel's shared memory allows one), fewer when there is less work
  l.grid[0] = static_cast<uint32_t>(std::min<long long>(items, ov.sm_count));
  l.block[0] = 384;
  l.dynamic_smem = 6 * 32768 + 8 * 4096 + 1024 + 256;   // Q, K, V tiles, output staging, barriers
  l.label = name;
  auto map = [&](int slot, int64_t seq) {
    KernelArg m;
    m.is_slot = false;
    m.tensor_map = true;
    m.tma.slot = slot;
    m.tma.rank = 3;
    m.tma.elem_bytes = 2;
    m.tma.swizzle = 3;
    m.tma.dims[0] = static_cast<uint64_t>(a.head_dim);
    m.tma.dims[1] = static_cast<uint64_t>(seq);
    m.tma.dims[2] = static_cast<uint64_t>(a.batch);
    m.tma.strides[0] = static_cast<uint64_t>(a.head_dim) * 2;
    m.tma.strides[1] = static_cast<uint64_t>(seq) * a.head_dim * 2;
    m.tma.box[0] = 64;
    m.tma.box[1] = 128;
    m.tma.box[2] = 1;
    return m;
  };
  l.args.push_back(map(a.q_slot, a.q_len));
  l.args.push_back(map(a.k_slot, a.k_len));
  l.args.push_back(map(a.v_slot, a.k_len));
  KernelArg o = map(a.o_slot, a.q_len);   // output tiles of 32 rows x 64 dims leave through TMA stores
  o.tma.box[1] = 32;
  l.args.push_back(o);
  KernelArg st;
  st.slot = -2;
  l.args.push_back(st);
  // work counter and exit counter: cleared at load time, left cleared by every launch
  Slot counters;
  counters.role = Slot::Scratch;
  counters.bytes = 256;
  counters.zero_init = true;
  plan.slots.push_back(counters);
  KernelArg ct;
  ct.slot = static_cast<int>(plan.slots.size()) - 1;
  l.args.push_back(ct);
  plan.launches.push_back(l);
}

}  // namespace accy
