// tcgen05 kernels for sm_100a: dense bf16 GEMM with fused epilogue, and causal attention.
//
// These replace the reference's only tensor-core path (mma.sync m16n8k8 tf32 fed by cp.async,
// src/preparation/kernelization/lowering/dot.zig:436-1119) and its SIMT flash attention
// (lowering/flash.zig:330-604) with Blackwell-native kernels:
//   * operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a ring of shared
//     memory stages guarded by mbarriers;
//   * one elected thread issues tcgen05.mma (kind::f16, bf16 inputs, f32 accumulate) with the
//     accumulator in tensor memory (TMEM); tcgen05.commit releases stages and publishes tiles;
//   * epilogue warps read the accumulator with tcgen05.ld, apply the fused elementwise epilogue
//     in f32 and store; two TMEM accumulators let the epilogue of one tile overlap the main loop
//     of the next; CTAs are persistent (one per SM) and walk tiles in an L2-friendly order.
// Every wait on an mbarrier is bounded: when the bound is hit the kernel records a code in a
// global status word, stops issuing work, releases its tensor memory and returns.
#include <cstdlib>
#include <sstream>

#include "plan.hpp"

namespace accy {

std::string emitEpilogueBody(const Epilogue& ep, std::ostringstream& o, const std::string& indent,
                             const std::string& acc, const std::string& bi, const std::string& mi,
                             const std::string& ni, const std::string& suffix);
std::string epilogueParams(const Epilogue& ep);
extern const char* kConvertPrelude;


namespace {

void replaceAll(std::string& s, const std::string& from, const std::string& to) {
  size_t at = 0;
  while ((at = s.find(from, at)) != std::string::npos) {
    s.replace(at, from.size(), to);
    at += to.size();
  }
}

// Device-side building blocks shared by the tcgen05 kernels.
const char* kTcPrelude = R"CUDA(
struct __align__(64) TensorMap { unsigned long long opaque[16]; };

__device__ __forceinline__ unsigned int smem_u32(const void* p) { return (unsigned int)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned int bar, unsigned int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned int bar, unsigned int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned int bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
// Bounded wait: gives up after SPIN_LIMIT probes (or when another thread of the CTA has given
// up), raising the CTA-wide abort flag.  Returns false on abort.
#define SPIN_LIMIT (1u << 22)
// The non-blocking test comes first: a probe of a phase that has already completed costs a few
// cycles, while mbarrier.try_wait (the potentially suspending form) was measured at 160-200 cycles
// even when it succeeds at once, which the single MMA-issuing thread cannot afford per tile.
__device__ __forceinline__ bool mbar_test(unsigned int bar, unsigned int parity) {
  unsigned int done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned int bar, unsigned int parity, volatile int* abort_flag) {
  if (mbar_test(bar, parity)) return true;
  for (unsigned int i = 0; i < SPIN_LIMIT; ++i) {
    unsigned int done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_3d(unsigned int dst, const TensorMap* map, unsigned int bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               :: "r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned int bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_ss(unsigned int d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                          unsigned int idesc, unsigned int accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_mma_ts(unsigned int d_tmem, unsigned int a_tmem, unsigned long long b_desc,
                                          unsigned int idesc, unsigned int accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(unsigned int taddr, unsigned int* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_tanh(float x) { float y; asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float fast_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ unsigned int pack_bf16(float lo, float hi) {
  unsigned int r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
}
__device__ __forceinline__ unsigned int pack_f16(float lo, float hi) {
  unsigned int r; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
}
// shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100): start address, leading
// and stride byte offsets in 16-byte units
__device__ __forceinline__ unsigned long long smem_desc(unsigned int addr, unsigned int lbo_bytes, unsigned int sbo_bytes) {
  return (unsigned long long)((addr & 0x3ffffu) >> 4) | ((unsigned long long)(lbo_bytes >> 4) << 16) |
         ((unsigned long long)(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
)CUDA";

// The GEMM kernel.  Placeholders @NAME@ are substituted per program.
const char* kGemmTemplate = R"CUDA(
#define BLOCK_M 128
#define BLOCK_N @BLOCK_N@
#define AB_FORMAT @AB_FORMAT@
#define BLOCK_K 64
#define VECTOR_STORES @VECTOR_STORES@   // rows of C start 16-byte aligned
#define STAGES @STAGES@
#define M_TOTAL @M@ll
#define N_TOTAL @N@ll
#define K_TOTAL @K@ll
#define BATCH @BATCH@ll
#define B_N_MAJOR @B_N_MAJOR@
#define A_M_MAJOR @A_M_MAJOR@
#define GROUP_M @GROUP_M@
#define A_STAGE_BYTES (BLOCK_M * BLOCK_K * 2)
#define B_STAGE_BYTES (BLOCK_N * BLOCK_K * 2)
#define STAGE_BYTES (A_STAGE_BYTES + B_STAGE_BYTES)

extern "C" __global__ void __launch_bounds__(192, 1)
@KERNEL@(const __grid_constant__ TensorMap map_a, const __grid_constant__ TensorMap map_b,
         @OUT_T@* __restrict__ C, int* __restrict__ status@EPI_PARAMS@) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // carve: stages first (1024-byte aligned for the 128-byte swizzle), then barriers
  unsigned char* smem = (unsigned char*)(((unsigned long long)smem_raw + 1023ull) & ~1023ull);
  unsigned long long* bars = (unsigned long long*)(smem + STAGES * STAGE_BYTES);
  // bars[0..STAGES) full, [STAGES..2*STAGES) empty, then tmem_full[2], tmem_empty[2]
  unsigned int* tmem_holder = (unsigned int*)(bars + 2 * STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned int full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const unsigned int tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(tfull0 + 8 * s, 1); mbar_init(tempty0 + 8 * s, 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_holder)), "r"(2 * BLOCK_N) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned int tmem_base = *tmem_holder;

  // extents need not be multiples of the tile: TMA loads read zeros past the end (zeros add nothing
  // to the sums), the epilogue clamps the indices it reads operands at and stores only inside
  const long long m_blocks = (M_TOTAL + BLOCK_M - 1) / BLOCK_M, n_blocks = (N_TOTAL + BLOCK_N - 1) / BLOCK_N,
                  k_blocks = (K_TOTAL + BLOCK_K - 1) / BLOCK_K;
  const long long tiles_per_batch = m_blocks * n_blocks;
  const long long num_tiles = tiles_per_batch * BATCH;

  // tile -> (batch, m block, n block): groups of GROUP_M row blocks are walked column by column so
  // that the CTAs running at one time share A rows and B columns in L2
  auto tile_coords = [&](long long tile, long long& b, long long& mb, long long& nb) {
    b = tile / tiles_per_batch;
    long long t = tile - b * tiles_per_batch;
    const long long group_size = (long long)GROUP_M * n_blocks;
    const long long group = t / group_size;
    const long long first_m = group * GROUP_M;
    const long long gm = (m_blocks - first_m) < GROUP_M ? (m_blocks - first_m) : GROUP_M;
    const long long in_group = t - group * group_size;
    mb = first_m + in_group % gm;
    nb = in_group / gm;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; unsigned int phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        long long b, mb, nb;
        tile_coords(tile, b, mb, nb);
        for (long long kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          const unsigned int full = full0 + 8 * stage;
          mbar_expect_tx(full, STAGE_BYTES);
          const unsigned int sa = smem_u32(smem + stage * STAGE_BYTES);
          const unsigned int sb = sa + A_STAGE_BYTES;
#if A_M_MAJOR
          // A is [k, m] with m contiguous (a transposed operand): one 64(m) x 64(k) box per 64 rows of the tile
#pragma unroll
          for (int j = 0; j < BLOCK_M / 64; ++j)
            tma_load_3d(sa + j * (64 * BLOCK_K * 2), &map_a, full, (int)(mb * BLOCK_M + j * 64), (int)(kb * BLOCK_K), (int)b);
#else
          tma_load_3d(sa, &map_a, full, (int)(kb * BLOCK_K), (int)(mb * BLOCK_M), (int)b);
#endif
#if B_N_MAJOR
          // B is [k, n] with n contiguous: one 64(n) x 64(k) box per 64 columns of the tile
#pragma unroll
          for (int j = 0; j < BLOCK_N / 64; ++j)
            tma_load_3d(sb + j * (64 * BLOCK_K * 2), &map_b, full, (int)(nb * BLOCK_N + j * 64), (int)(kb * BLOCK_K), (int)b);
#else
          // B is [n, k] with k contiguous: one 64(k) x BLOCK_N(n) box
          tma_load_3d(sb, &map_b, full, (int)(kb * BLOCK_K), (int)(nb * BLOCK_N), (int)b);
#endif
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // instruction descriptor: f32 accumulate, A and B format (0 = f16, 1 = bf16), A and B major
      // as given, N, M=128
      const unsigned int idesc = (1u << 4) | (AB_FORMAT << 7) | (AB_FORMAT << 10) | ((unsigned int)A_M_MAJOR << 15) |
                                 ((unsigned int)B_N_MAJOR << 16) |
                                 ((unsigned int)(BLOCK_N >> 3) << 17) | ((unsigned int)(BLOCK_M >> 4) << 24);
      int stage = 0; unsigned int phase = 0;
      unsigned int it = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
        const unsigned int buf = it & 1u, acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(tempty0 + 8 * buf, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const unsigned int d_tmem = tmem_base + buf * BLOCK_N;
        for (long long kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const unsigned int sa = smem_u32(smem + stage * STAGE_BYTES);
          const unsigned int sb = sa + A_STAGE_BYTES;
          // A: K-major, rows of 128 bytes, 8-row groups 1024 bytes apart
#if A_M_MAJOR
          // A: M-major, 64-row chunks 64*128 bytes apart (leading), 8-k-row groups 1024 bytes apart (stride)
          const unsigned long long a_desc = smem_desc(sa, 64 * BLOCK_K * 2, 1024);
#else
          const unsigned long long a_desc = smem_desc(sa, 16, 1024);
#endif
#if B_N_MAJOR
          // B: N-major, 64-column chunks 64*128 bytes apart (leading), 8-k-row groups 1024 bytes apart (stride)
          const unsigned long long b_desc = smem_desc(sb, 64 * BLOCK_K * 2, 1024);
#else
          const unsigned long long b_desc = smem_desc(sb, 16, 1024);
#endif
#pragma unroll
          for (int k = 0; k < BLOCK_K / 16; ++k) {
            // advance 16 k-elements: 32 bytes inside a K-major row, 16 rows of 128 bytes when N-major
#if A_M_MAJOR
            const unsigned long long a_k = a_desc + (unsigned long long)((k * 16 * 128) >> 4);
#else
            const unsigned long long a_k = a_desc + (unsigned long long)((k * 32) >> 4);
#endif
#if B_N_MAJOR
            const unsigned long long b_k = b_desc + (unsigned long long)((k * 16 * 128) >> 4);
#else
            const unsigned long long b_k = b_desc + (unsigned long long)((k * 32) >> 4);
#endif
            tc_mma_ss(d_tmem, a_k, b_k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(empty0 + 8 * stage);   // the stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(tfull0 + 8 * buf);  // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue: 4 warps, one accumulator row per thread ----------------
    const unsigned int quarter = warp & 3u;            // TMEM lanes this warp may read
    const unsigned int row_in_tile = quarter * 32 + lane;
    unsigned int it = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
      const unsigned int buf = it & 1u, acc_phase = (it >> 1) & 1u;
      long long bi, mb, nb;
      tile_coords(tile, bi, mb, nb);
      if (!mbar_wait(tfull0 + 8 * buf, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const long long mi_raw = mb * BLOCK_M + row_in_tile;
      const bool row_inside = mi_raw < M_TOTAL;
      const long long mi = row_inside ? mi_raw : M_TOTAL - 1;
      @OUT_T@* crow = C + (bi * M_TOTAL + mi) * N_TOTAL + nb * BLOCK_N;
      const unsigned int taddr = tmem_base + ((quarter * 32u) << 16) + buf * BLOCK_N;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        unsigned int r[32];
        tc_ld32(taddr + c * 32, r);
        tc_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float acc = __uint_as_float(r[j]);
          const long long ni_raw = nb * BLOCK_N + c * 32 + j;
          const long long ni = (N_TOTAL % BLOCK_N == 0 || ni_raw < N_TOTAL) ? ni_raw : N_TOTAL - 1;
          (void)ni;
@EPI_BODY@
          v[j] = @EPI_RESULT@;
        }
        const long long n_left = N_TOTAL - (nb * BLOCK_N + c * 32);   // columns of this chunk inside the matrix
        if (row_inside && n_left >= 32 && VECTOR_STORES) {
@STORE@
        } else if (row_inside && n_left > 0) {
          const int count = n_left < 32 ? (int)n_left : 32;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < count) crow[c * 32 + j] = @SCALAR_STORE@;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
    }
  }

  // ---------------- teardown ----------------
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    // let copies that are still in flight land before the shared memory goes away
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(2 * BLOCK_N) : "memory");
  }
}
)CUDA";

const char* kPairPrelude = R"CUDA(
// ---- two-CTA (cta_group::2) building blocks ----
// A pair of CTAs on the two SMs of one TPC works on one 256-row tile: each CTA stages its own 128
// rows of A and its own half of the B columns with its own (non-multicast) TMA loads, one thread
// of the even CTA issues MMAs that read both CTAs' shared memory and write both CTAs' tensor
// memory, so every B byte is loaded into shared memory once per 256 rows instead of once per 128.
__device__ __forceinline__ unsigned int cluster_rank() { unsigned int r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned int peer_smem(unsigned int local, unsigned int rank) {
  unsigned int r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrival on a barrier that may live in the other CTA of the pair (a shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(unsigned int bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(bar) : "memory");
}
// TMA load into this CTA's shared memory whose bytes are counted on a barrier of either CTA
__device__ __forceinline__ void tma_load_3d_pair(unsigned int dst, const TensorMap* map, unsigned int bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               :: "r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_mma_ss_pair(unsigned int d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                               unsigned int idesc, unsigned int accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// completion of every MMA issued so far, signalled on the barrier at this offset in both CTAs
__device__ __forceinline__ void tc_commit_pair(unsigned int bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               :: "r"(bar), "h"((unsigned short)3) : "memory");
}
)CUDA";

// The two-CTA GEMM kernel (cta_group::2).  Placeholders @NAME@ are substituted per program.
const char* kGemmPairTemplate = R"CUDA(
#define BLOCK_M 128            // rows per CTA; the pair's tile has 256
#define BLOCK_N @BLOCK_N@      // columns of the pair's tile; each CTA stages BLOCK_N / 2 of them
#define HALF_N (BLOCK_N / 2)
#define AB_FORMAT @AB_FORMAT@
#define BLOCK_K 64
#define VECTOR_STORES @VECTOR_STORES@   // rows of C start 16-byte aligned
#define STAGES @STAGES@
#define M_TOTAL @M@ll
#define N_TOTAL @N@ll
#define K_TOTAL @K@ll
#define BATCH @BATCH@ll
#define B_N_MAJOR @B_N_MAJOR@
#define A_M_MAJOR @A_M_MAJOR@
#define GROUP_M @GROUP_M@
#define A_STAGE_BYTES (BLOCK_M * BLOCK_K * 2)
#define B_STAGE_BYTES (HALF_N * BLOCK_K * 2)
#define STAGE_BYTES (A_STAGE_BYTES + B_STAGE_BYTES)

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
@KERNEL@(const __grid_constant__ TensorMap map_a, const __grid_constant__ TensorMap map_b,
         @OUT_T@* __restrict__ C, int* __restrict__ status@EPI_PARAMS@) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // carve: stages first (1024-byte aligned for the 128-byte swizzle), then barriers; the layout is
  // the same in both CTAs of the pair, which the MMA and the paired commits rely on
  unsigned char* smem = (unsigned char*)(((unsigned long long)smem_raw + 1023ull) & ~1023ull);
  unsigned long long* bars = (unsigned long long*)(smem + STAGES * STAGE_BYTES);
  // bars[0..STAGES) full (used in the even CTA), [STAGES..2*STAGES) empty, then tmem_full[2], tmem_empty[2] (even CTA)
  unsigned int* tmem_holder = (unsigned int*)(bars + 2 * STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned int rank = cluster_rank();          // 0: issues the MMAs and owns the full / tmem_empty barriers
  const unsigned int full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const unsigned int tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

  if (threadIdx.x == 0) {
    // full: one arrival (the even CTA's producer, which announces both CTAs' bytes); empty and
    // tmem_full: one paired commit; tmem_empty: the four epilogue warps of each CTA
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(tfull0 + 8 * s, 1); mbar_init(tempty0 + 8 * s, 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // each CTA allocates all of its own tensor memory (it is alone on its SM), so the two
    // accumulators sit at the same columns in both CTAs
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_holder)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();     // the other CTA's barriers are initialised before anything is signalled on them
  tc_fence_after();
  const unsigned int tmem_base = *tmem_holder;

  const long long m_blocks = (M_TOTAL + 2 * BLOCK_M - 1) / (2 * BLOCK_M), n_blocks = (N_TOTAL + BLOCK_N - 1) / BLOCK_N,
                  k_blocks = (K_TOTAL + BLOCK_K - 1) / BLOCK_K;
  const long long tiles_per_batch = m_blocks * n_blocks;
  const long long num_tiles = tiles_per_batch * BATCH;
  const long long first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;

  // tile -> (batch, m block of 256 rows, n block): groups of GROUP_M row blocks are walked column
  // by column so that the pairs running at one time share A rows and B columns in L2
  auto tile_coords = [&](long long tile, long long& b, long long& mb, long long& nb) {
    b = tile / tiles_per_batch;
    long long t = tile - b * tiles_per_batch;
    const long long group_size = (long long)GROUP_M * n_blocks;
    const long long group = t / group_size;
    const long long first_m = group * GROUP_M;
    const long long gm = (m_blocks - first_m) < GROUP_M ? (m_blocks - first_m) : GROUP_M;
    const long long in_group = t - group * group_size;
    mb = first_m + in_group % gm;
    nb = in_group / gm;
  };

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA; its own rows of A, its own half of B) ----------------
    if (lane == 0) {
      int stage = 0; unsigned int phase = 0;
      bool ok = true;
      const unsigned int leader_full0 = peer_smem(full0, 0);
      for (long long tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
        long long b, mb, nb;
        tile_coords(tile, b, mb, nb);
        const int m0 = (int)(mb * 2 * BLOCK_M + rank * BLOCK_M), n0 = (int)(nb * BLOCK_N + rank * HALF_N);
        for (long long kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * STAGE_BYTES);
          const unsigned int full = leader_full0 + 8 * stage;
          const unsigned int sa = smem_u32(smem + stage * STAGE_BYTES);
          const unsigned int sb = sa + A_STAGE_BYTES;
#if A_M_MAJOR
#pragma unroll
          for (int j = 0; j < BLOCK_M / 64; ++j)
            tma_load_3d_pair(sa + j * (64 * BLOCK_K * 2), &map_a, full, m0 + j * 64, (int)(kb * BLOCK_K), (int)b);
#else
          tma_load_3d_pair(sa, &map_a, full, (int)(kb * BLOCK_K), m0, (int)b);
#endif
#if B_N_MAJOR
#pragma unroll
          for (int j = 0; j < HALF_N / 64; ++j)
            tma_load_3d_pair(sb + j * (64 * BLOCK_K * 2), &map_b, full, n0 + j * 64, (int)(kb * BLOCK_K), (int)b);
#else
          tma_load_3d_pair(sb, &map_b, full, (int)(kb * BLOCK_K), n0, (int)b);
#endif
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one thread of the even CTA, for the pair ----------------
    if (lane == 0 && rank == 0) {
      // instruction descriptor: f32 accumulate, A and B format (0 = f16, 1 = bf16), A and B major
      // as given, N, M = 256 (the pair's rows)
      const unsigned int idesc = (1u << 4) | (AB_FORMAT << 7) | (AB_FORMAT << 10) | ((unsigned int)A_M_MAJOR << 15) |
                                 ((unsigned int)B_N_MAJOR << 16) |
                                 ((unsigned int)(BLOCK_N >> 3) << 17) | ((unsigned int)((2 * BLOCK_M) >> 4) << 24);
      int stage = 0; unsigned int phase = 0;
      unsigned int it = 0;
      bool ok = true;
      for (long long tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++it) {
        const unsigned int buf = it & 1u, acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(tempty0 + 8 * buf, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const unsigned int d_tmem = tmem_base + buf * BLOCK_N;
        for (long long kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const unsigned int sa = smem_u32(smem + stage * STAGE_BYTES);
          const unsigned int sb = sa + A_STAGE_BYTES;
#if A_M_MAJOR
          const unsigned long long a_desc = smem_desc(sa, 64 * BLOCK_K * 2, 1024);
#else
          const unsigned long long a_desc = smem_desc(sa, 16, 1024);
#endif
#if B_N_MAJOR
          const unsigned long long b_desc = smem_desc(sb, 64 * BLOCK_K * 2, 1024);
#else
          const unsigned long long b_desc = smem_desc(sb, 16, 1024);
#endif
#pragma unroll
          for (int k = 0; k < BLOCK_K / 16; ++k) {
#if A_M_MAJOR
            const unsigned long long a_k = a_desc + (unsigned long long)((k * 16 * 128) >> 4);
#else
            const unsigned long long a_k = a_desc + (unsigned long long)((k * 32) >> 4);
#endif
#if B_N_MAJOR
            const unsigned long long b_k = b_desc + (unsigned long long)((k * 16 * 128) >> 4);
#else
            const unsigned long long b_k = b_desc + (unsigned long long)((k * 32) >> 4);
#endif
            tc_mma_ss_pair(d_tmem, a_k, b_k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit_pair(empty0 + 8 * stage);   // the stage is free in both CTAs once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit_pair(tfull0 + 8 * buf);  // accumulator complete, in both CTAs
      }
    }
  } else {
    // ---------------- epilogue: 4 warps per CTA, one accumulator row per thread ----------------
    const unsigned int quarter = warp & 3u;            // TMEM lanes this warp may read
    const unsigned int row_in_tile = rank * BLOCK_M + quarter * 32 + lane;
    const unsigned int leader_tempty0 = peer_smem(tempty0, 0);
    unsigned int it = 0;
    bool ok = true;
    for (long long tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++it) {
      const unsigned int buf = it & 1u, acc_phase = (it >> 1) & 1u;
      long long bi, mb, nb;
      tile_coords(tile, bi, mb, nb);
      if (!mbar_wait(tfull0 + 8 * buf, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const long long mi_raw = mb * 2 * BLOCK_M + row_in_tile;
      const bool row_inside = mi_raw < M_TOTAL;
      const long long mi = row_inside ? mi_raw : M_TOTAL - 1;
      @OUT_T@* crow = C + (bi * M_TOTAL + mi) * N_TOTAL + nb * BLOCK_N;
      const unsigned int taddr = tmem_base + ((quarter * 32u) << 16) + buf * BLOCK_N;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        unsigned int r[32];
        tc_ld32(taddr + c * 32, r);
        tc_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float acc = __uint_as_float(r[j]);
          const long long ni_raw = nb * BLOCK_N + c * 32 + j;
          const long long ni = (N_TOTAL % BLOCK_N == 0 || ni_raw < N_TOTAL) ? ni_raw : N_TOTAL - 1;
          (void)ni;
@EPI_BODY@
          v[j] = @EPI_RESULT@;
        }
        const long long n_left = N_TOTAL - (nb * BLOCK_N + c * 32);   // columns of this chunk inside the matrix
        if (row_inside && n_left >= 32 && VECTOR_STORES) {
@STORE@
        } else if (row_inside && n_left > 0) {
          const int count = n_left < 32 ? (int)n_left : 32;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < count) crow[c * 32 + j] = @SCALAR_STORE@;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty0 + 8 * buf);
    }
  }

  // ---------------- teardown ----------------
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    // let copies that are still in flight land before the shared memory goes away
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();     // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(512) : "memory");
  }
}
)CUDA";

}  // namespace

void emitGemmTcgen05(const GemmOp& g, const std::string& name, Plan& plan, const ScheduleOverrides& ov) {
  const int block_n = (g.n % 256 == 0) ? 256 : 128;
  // Two CTAs per 256-row tile (cta_group::2) whenever the output has more than one 128-row block
  // and the GPU offers pairs of SMs; ACCY_B200_GEMM_PAIR=0 keeps every GEMM on the one-CTA kernel.
  const char* pair_env = std::getenv("ACCY_B200_GEMM_PAIR");
  const bool pair = g.m > 128 && ov.sm_count >= 2 && !(pair_env && pair_env[0] == '0');
  // shared memory per stage and CTA: 128 x 64 of A and BLOCK_N (a pair: BLOCK_N / 2) x 64 of B
  const uint32_t stage_bytes = 128 * 64 * 2 + (pair ? block_n / 2 : block_n) * 64 * 2;
  const int stages = pair ? (block_n == 256 ? 7 : 8) : (block_n == 256 ? 4 : 6);
  const bool n_major = g.b_stride_n == 1 && g.n > 1;
  const bool m_major = g.a_stride_k != 1 && g.a_stride_m == 1;
  if (g.out_dtype != DType::bf16 && g.out_dtype != DType::f16 && g.out_dtype != DType::f32)
    throw PlanError("tcgen05 GEMM output must be bf16, f16 or f32");

  std::ostringstream body;
  std::string result = emitEpilogueBody(g.epilogue, body, "          ", "acc", "bi", "mi", "ni", "");
  std::string epi = body.str();
  // bf16 programs: hardware tanh/exp approximations are inside the 2e-2 tolerance (f16 keeps tanhf)
  if (g.in_dtype == DType::bf16) replaceAll(epi, "tanhf(", "fast_tanh(");

  std::string store;
  if (g.out_dtype == DType::bf16 || g.out_dtype == DType::f16) {
    store =
        "        {\n"
        "          uint4* dst = reinterpret_cast<uint4*>(crow + c * 32);\n"
        "#pragma unroll\n"
        "          for (int q = 0; q < 4; ++q)\n"
        "            dst[q] = make_uint4(pack_bf16(v[q * 8 + 0], v[q * 8 + 1]), pack_bf16(v[q * 8 + 2], v[q * 8 + 3]),\n"
        "                                pack_bf16(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16(v[q * 8 + 6], v[q * 8 + 7]));\n"
        "        }\n";
  } else {
    store =
        "        {\n"
        "          float4* dst = reinterpret_cast<float4*>(crow + c * 32);\n"
        "#pragma unroll\n"
        "          for (int q = 0; q < 8; ++q) dst[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);\n"
        "        }\n";
  }

  std::string src = std::string(kConvertPrelude) + kTcPrelude + (pair ? std::string(kPairPrelude) + kGemmPairTemplate : std::string(kGemmTemplate));
  if (g.out_dtype == DType::f16) replaceAll(store, "pack_bf16(", "pack_f16(");
  const int out_bytes = g.out_dtype == DType::f32 ? 4 : 2;
  replaceAll(src, "@VECTOR_STORES@", (g.n * out_bytes) % 16 == 0 ? "1" : "0");
  replaceAll(src, "@SCALAR_STORE@", g.out_dtype == DType::f32 ? "v[j]" : (g.out_dtype == DType::f16 ? "f32_to_f16(v[j])" : "f32_to_bf16(v[j])"));
  replaceAll(src, "@KERNEL@", name);
  replaceAll(src, "@AB_FORMAT@", g.in_dtype == DType::f16 ? "0u" : "1u");
  replaceAll(src, "@BLOCK_N@", std::to_string(block_n));
  replaceAll(src, "@STAGES@", std::to_string(stages));
  replaceAll(src, "@M@", std::to_string(g.m));
  replaceAll(src, "@N@", std::to_string(g.n));
  replaceAll(src, "@K@", std::to_string(g.k));
  replaceAll(src, "@BATCH@", std::to_string(g.batch));
  replaceAll(src, "@B_N_MAJOR@", n_major ? "1" : "0");
  replaceAll(src, "@A_M_MAJOR@", m_major ? "1" : "0");
  replaceAll(src, "@GROUP_M@", "16");
  replaceAll(src, "@OUT_T@", storageTypeOf(g.out_dtype));
  replaceAll(src, "@EPI_PARAMS@", epilogueParams(g.epilogue));
  replaceAll(src, "@EPI_BODY@", epi);
  replaceAll(src, "@EPI_RESULT@", result);
  replaceAll(src, "@STORE@", store);

  KernelSource ks;
  ks.name = name;
  ks.family = pair ? "gemm_tcgen05_pair" : "gemm_tcgen05";
  ks.source = src;
  plan.kernels.push_back(ks);

  Launch l;
  l.kernel = static_cast<int>(plan.kernels.size()) - 1;
  const long long tiles = ((g.m + (pair ? 255 : 127)) / (pair ? 256 : 128)) * ((g.n + block_n - 1) / block_n) * g.batch;
  // persistent: one CTA per SM (a pair: one CTA pair per two SMs), fewer when there are fewer tiles
  l.grid[0] = pair ? static_cast<uint32_t>(2 * std::min<long long>(tiles, ov.sm_count / 2))
                   : static_cast<uint32_t>(std::min<long long>(tiles, ov.sm_count));
  l.block[0] = 192;
  l.dynamic_smem = stages * stage_bytes + 1024 /* alignment slack */ + 256 /* barriers */;
  l.label = name;

  KernelArg a;
  a.is_slot = false;
  a.tensor_map = true;
  a.tma.slot = g.a_slot;
  a.tma.rank = 3;
  a.tma.elem_bytes = 2;
  a.tma.swizzle = 3;
  a.tma.dims[0] = g.k;
  a.tma.dims[1] = g.m;
  a.tma.dims[2] = g.batch;
  a.tma.strides[0] = static_cast<uint64_t>(g.a_stride_m) * 2;
  a.tma.strides[1] = static_cast<uint64_t>(g.batch > 1 ? g.a_stride_b : g.m * g.a_stride_m) * 2;
  a.tma.box[0] = 64;
  a.tma.box[1] = 128;
  a.tma.box[2] = 1;
  if (m_major) {
    a.tma.dims[0] = g.m;
    a.tma.dims[1] = g.k;
    a.tma.strides[0] = static_cast<uint64_t>(g.a_stride_k) * 2;
    a.tma.strides[1] = static_cast<uint64_t>(g.batch > 1 ? g.a_stride_b : g.k * g.a_stride_k) * 2;
    a.tma.box[0] = 64;
    a.tma.box[1] = 64;
  }
  l.args.push_back(a);

  KernelArg b = a;
  b.tma.box[2] = 1;
  b.tma.slot = g.b_slot;
  if (n_major) {
    b.tma.dims[0] = g.n;
    b.tma.dims[1] = g.k;
    b.tma.strides[0] = static_cast<uint64_t>(g.b_stride_k) * 2;
    b.tma.strides[1] = static_cast<uint64_t>(g.batch > 1 ? g.b_stride_b : g.k * g.b_stride_k) * 2;
    b.tma.box[0] = 64;
    b.tma.box[1] = 64;
  } else {
    b.tma.dims[0] = g.k;
    b.tma.dims[1] = g.n;
    b.tma.strides[0] = static_cast<uint64_t>(g.b_stride_n) * 2;
    b.tma.strides[1] = static_cast<uint64_t>(g.batch > 1 ? g.b_stride_b : g.n * g.b_stride_n) * 2;
    b.tma.box[0] = 64;
    b.tma.box[1] = static_cast<uint32_t>(pair ? block_n / 2 : block_n);
  }
  b.tma.dims[2] = g.batch;
  b.tma.box[2] = 1;
  l.args.push_back(b);

  KernelArg c;
  c.slot = g.c_slot;
  l.args.push_back(c);
  KernelArg st;
  st.slot = -2;  // the session's device status word
  l.args.push_back(st);
  for (const LeafRef& leaf : g.epilogue.leaves) {
    KernelArg e;
    e.slot = leaf.slot;
    l.args.push_back(e);
  }
  plan.launches.push_back(l);
}

// the tcgen05 building blocks, shared with the attention kernel (emit_attn.cpp)
const char* kTcPreludeShared = kTcPrelude;

}  // namespace accy
