// CUDA source emission for contractions: the k-serial SIMT dot kernel (any shape, any strides,
// f32/f16/bf16) and the shared epilogue emitter.  The tcgen05 kernels live in emit_tc.cpp.
//
// The SIMT kernel restates the reference's generic dot lowering
// (src/preparation/kernelization/lowering/dot.zig:2049-2115): one thread per output element,
// k folded serially as acc = acc + a*b with separate multiply and add roundings (compiled with
// --fmad=false), 16-bit inputs widened to f32 and narrowed once at the end (:2004-2015).  It is
// the exact-order path used for f32 programs and for shapes the tensor-core tiles do not cover.
#include <cstdlib>
#include <sstream>

#include "plan.hpp"

namespace accy {

void emitGemmTcgen05(const GemmOp& g, const std::string& name, Plan& plan, const ScheduleOverrides& o);

namespace {

std::string loadConv(DType d, const std::string& raw) {
  if (d == DType::bf16) return "bf16_to_f32(" + raw + ")";
  if (d == DType::f16) return "f16_to_f32(" + raw + ")";
  return raw;
}

std::string storeConv(DType d, const std::string& v) {
  if (d == DType::bf16) return "f32_to_bf16(" + v + ")";
  if (d == DType::f16) return "f32_to_f16(" + v + ")";
  if (d == DType::i1) return "(unsigned char)(" + v + " ? 1 : 0)";
  return v;
}

}  // namespace

const char* kConvertPrelude = R"CUDA(
__device__ __forceinline__ float bf16_to_f32(unsigned short h) { return __uint_as_float(((unsigned int)h) << 16); }
__device__ __forceinline__ unsigned short f32_to_bf16(float f) { unsigned short r; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
__device__ __forceinline__ float f16_to_f32(unsigned short h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ unsigned short f32_to_f16(float f) { unsigned short r; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
)CUDA";

// Emits statements computing the epilogue for one accumulator element.  `acc` names the f32
// accumulator, (bi, mi, ni) name the element's coordinates, leaf k is pointer E<k>.  Returns the
// name of the value to store; with an empty epilogue that is `acc` itself.
std::string emitEpilogueBody(const Epilogue& ep, std::ostringstream& o, const std::string& indent,
                             const std::string& acc, const std::string& bi, const std::string& mi,
                             const std::string& ni, const std::string& suffix) {
  if (ep.nodes.empty() || ep.result < 0) return acc;
  auto nm = [&](int i) { return i == ep.acc ? acc : "e" + std::to_string(i) + suffix; };
  for (size_t i = 0; i < ep.nodes.size(); ++i) {
    const ENode& n = ep.nodes[i];
    if (static_cast<int>(i) == ep.acc) continue;
    o << indent << "const " << ctypeOf(n.dtype) << " " << nm(static_cast<int>(i)) << " = ";
    switch (n.op) {
      case ENode::Leaf: {
        const LeafRef& l = ep.leaves[n.leaf];
        std::ostringstream idx;
        idx << "(long long)" << bi << " * " << l.strides[0] << "ll + (long long)" << mi << " * " << l.strides[1]
            << "ll + (long long)" << ni << " * " << l.strides[2] << "ll";
        o << loadConv(l.dtype, "E" + std::to_string(n.leaf) + "[" + idx.str() + "]");
        break;
      }
      case ENode::Const: o << constLiteral(n); break;
      case ENode::Iota: throw PlanError("iota inside a GEMM epilogue is not supported");
      case ENode::Red: throw PlanError("reduction inside a GEMM epilogue is not supported");
      default: {
        std::string a = n.args[0] >= 0 ? nm(n.args[0]) : "", b = n.args[1] >= 0 ? nm(n.args[1]) : "",
                    c = n.args[2] >= 0 ? nm(n.args[2]) : "";
        o << elementwiseExpr(n, a, b, c, ep.nodes[n.args[n.op == ENode::Sel ? 1 : 0]].dtype);
      }
    }
    o << ";\n";
  }
  return nm(ep.result);
}

std::string epilogueParams(const Epilogue& ep) {
  std::ostringstream p;
  for (size_t k = 0; k < ep.leaves.size(); ++k)
    p << ", const " << storageTypeOf(ep.leaves[k].dtype) << "* __restrict__ E" << k;
  return p.str();
}

static void emitGemmSimt(const GemmOp& g, const std::string& name, Plan& plan) {
  std::ostringstream o;
  const char* in_t = storageTypeOf(g.in_dtype);
  const char* out_t = storageTypeOf(g.out_dtype);
  o << kConvertPrelude;
  o << "extern \"C\" __global__ void __launch_bounds__(256) " << name << "(const " << in_t
 << "* __restrict__ A, const " << storageTypeOf(g.b_dtype) << "* __restrict__ B, " << out_t << "* __restrict__ C"
    << epilogueParams(g.epilogue) << ") {\n";
  o << "  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;\n";
  o << "  if (idx >= " << g.batch * g.m * g.n << "ll) return;\n";
  o << "  const long long ni = idx % " << g.n << "ll;\n  const long long mi = (idx / " << g.n << "ll) % " << g.m
    << "ll;\n  const long long bi = idx / " << g.m * g.n << "ll;\n";
  o << "  const " << in_t << "* a = A + bi * " << g.a_stride_b << "ll + mi * " << g.a_stride_m << "ll;\n";
  o << "  const " << storageTypeOf(g.b_dtype) << "* b = B + bi * " << g.b_stride_b << "ll + ni * " << g.b_stride_n << "ll;\n";
  // integers (the reference's dot lowering takes i32 and u32, dot.zig:2211-2233) wrap around:
  // the arithmetic is done on unsigned values, whose overflow is defined
  const bool integer = g.in_dtype == DType::i32 || g.in_dtype == DType::u32;
  const char* acc_t = integer ? "unsigned int" : "float";
  o << "  " << acc_t << " acc = 0;\n";
  o << "  for (long long k = 0; k < " << g.k << "ll; ++k) {\n";
  o << "    const " << acc_t << " av = " << (integer ? "(unsigned int)" : "") << loadConv(g.in_dtype, "a[k * " + std::to_string(g.a_stride_k) + "ll]") << ";\n";
  o << "    const " << acc_t << " bv = " << (integer ? "(unsigned int)" : "") << loadConv(g.b_dtype, "b[k * " + std::to_string(g.b_stride_k) + "ll]") << ";\n";
  o << "    const " << acc_t << " prod = av * bv;\n    acc = acc + prod;\n  }\n";
  std::string result = emitEpilogueBody(g.epilogue, o, "  ", "acc", "bi", "mi", "ni", "");
  o << "  C[idx] = " << storeConv(g.out_dtype, result) << ";\n}\n";
  KernelSource ks;
  ks.name = name;
  ks.family = "gemm_simt";
  ks.source = o.str();
  ks.options.push_back("--fmad=false");
  plan.kernels.push_back(ks);
  Launch l;
  l.kernel = static_cast<int>(plan.kernels.size()) - 1;
  const long long total = g.batch * g.m * g.n;
  if ((total + 255) / 256 > 0x7fffffffll) throw PlanError("dot_general output too large for the SIMT kernel");
  l.grid[0] = static_cast<uint32_t>((total + 255) / 256);
  l.block[0] = 256;
  l.label = name;
  KernelArg a;
  a.slot = g.a_slot;
  l.args.push_back(a);
  a.slot = g.b_slot;
  l.args.push_back(a);
  a.slot = g.c_slot;
  l.args.push_back(a);
  for (const LeafRef& leaf : g.epilogue.leaves) {
    a.slot = leaf.slot;
    l.args.push_back(a);
  }
  plan.launches.push_back(l);
}

// The same arithmetic as emitGemmSimt (every output folds k serially, acc = acc + a*b with separate
// multiply and add roundings, so the results are bit-identical to it) laid out as a classic
// shared-memory SGEMM: 128 x 128 output tile per CTA of 256 threads, 16-deep k slices staged in
// shared memory (two buffers), 8 x 8 outputs per thread in two 4-wide groups 64 apart so that the
// 128-bit shared-memory reads are conflict free.  Any strides,
// any extents (guards instead of padding: a zero added past the end could turn a -0 sum into +0).
static void emitGemmSimtTiled(const GemmOp& g, const std::string& name, Plan& plan) {
  std::ostringstream o;
  const std::string in_t = storageTypeOf(g.in_dtype), b_t = storageTypeOf(g.b_dtype), out_t = storageTypeOf(g.out_dtype);
  const long long m_blocks = (g.m + 127) / 128, n_blocks = (g.n + 127) / 128;
  o << kConvertPrelude;
  o << "#define GM " << g.m << "ll\n#define GN " << g.n << "ll\n#define GK " << g.k << "ll\n";
  o << "#define A_SB " << g.a_stride_b << "ll\n#define A_SM " << g.a_stride_m << "ll\n#define A_SK " << g.a_stride_k << "ll\n";
  o << "#define B_SB " << g.b_stride_b << "ll\n#define B_SK " << g.b_stride_k << "ll\n#define B_SN " << g.b_stride_n << "ll\n";
  o << "#define M_BLOCKS " << m_blocks << "ll\n#define N_BLOCKS " << n_blocks << "ll\n";
  o << "#define LOAD_A(p) " << loadConv(g.in_dtype, "(p)") << "\n#define LOAD_B(p) " << loadConv(g.b_dtype, "(p)") << "\n";
  o << "extern \"C\" __global__ void __launch_bounds__(256, 2) " << name << "(const " << in_t << "* __restrict__ A, const "
    << b_t << "* __restrict__ B, " << out_t << "* __restrict__ C" << epilogueParams(g.epilogue) << ") {\n";
  o << R"CUDA(
  __shared__ __align__(16) float As[2][16][128];
  __shared__ __align__(16) float Bs[2][16][128];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const long long tile = blockIdx.x;
  const long long nb = tile % N_BLOCKS, mb = (tile / N_BLOCKS) % M_BLOCKS, bi = tile / (N_BLOCKS * M_BLOCKS);
  const long long m0 = mb * 128, n0 = nb * 128;
  const long long a_base = bi * A_SB, b_base = bi * B_SB;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
  // one k slice: 128 x 16 of A and 16 x 128 of B, eight elements of each per thread; the thread
  // order follows whichever index is contiguous in memory
  auto load_slice = [&](int buf, long long k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + i * 256;
      const int mm = A_SK == 1 ? e >> 4 : e & 127, kk = A_SK == 1 ? e & 15 : e >> 7;
      const long long gm = m0 + mm, gk = k0 + kk;
      As[buf][kk][mm] = (gm < GM && gk < GK) ? LOAD_A(A[a_base + gm * A_SM + gk * A_SK]) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + i * 256;
      const int nn = B_SN == 1 ? e & 127 : e >> 4, kk = B_SN == 1 ? e >> 7 : e & 15;
      const long long gn = n0 + nn, gk = k0 + kk;
      Bs[buf][kk][nn] = (gn < GN && gk < GK) ? LOAD_B(B[b_base + gk * B_SK + gn * B_SN]) : 0.0f;
    }
  };
  auto step = [&](int buf, int kk) {
    const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
    const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
    const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
    const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
    const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float prod = a[i] * b[j];   // compiled without contraction: two roundings, as the reference
        acc[i][j] = acc[i][j] + prod;
      }
  };
  const long long slices = (GK + 15) / 16;
  load_slice(0, 0);
  __syncthreads();
  for (long long s = 0; s < slices; ++s) {
    const int buf = (int)(s & 1);
    if (s + 1 < slices) load_slice(buf ^ 1, (s + 1) * 16);
    const long long left = GK - s * 16;
    if (left >= 16) {
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) step(buf, kk);
    } else {
      for (int kk = 0; kk < (int)left; ++kk) step(buf, kk);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const long long mi = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long ni = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      const float acc_v = acc[i][j];
      if (mi < GM && ni < GN) {
)CUDA";
  std::string result = emitEpilogueBody(g.epilogue, o, "        ", "acc_v", "bi", "mi", "ni", "");
  o << "        C[(bi * GM + mi) * GN + ni] = " << storeConv(g.out_dtype, result) << ";\n";
  o << "      }\n    }\n  }\n}\n";
  KernelSource ks;
  ks.name = name;
  ks.family = "gemm_simt";
  ks.source = o.str();
  ks.options.push_back("--fmad=false");
  plan.kernels.push_back(ks);
  Launch l;
  l.kernel = static_cast<int>(plan.kernels.size()) - 1;
  const long long tiles = m_blocks * n_blocks * g.batch;
  if (tiles > 0x7fffffffll) throw PlanError("dot_general output too large for the SIMT kernel");
  l.grid[0] = static_cast<uint32_t>(tiles);
  l.block[0] = 256;
  l.label = name;
  KernelArg a;
  a.slot = g.a_slot;
  l.args.push_back(a);
  a.slot = g.b_slot;
  l.args.push_back(a);
  a.slot = g.c_slot;
  l.args.push_back(a);
  for (const LeafRef& leaf : g.epilogue.leaves) {
    a.slot = leaf.slot;
    l.args.push_back(a);
  }
  plan.launches.push_back(l);
}

void emitGemm(const GemmOp& g, const std::string& name, Plan& plan, const ScheduleOverrides& o) {
  if (g.in_dtype == DType::f64) throw PlanError("f64 dot_general is not supported");
  if (g.tensor_core) emitGemmTcgen05(g, name, plan, o);
  else if (g.batch * g.m * g.n >= 4096 && g.k >= 8 && g.in_dtype != DType::i32 && g.in_dtype != DType::u32) emitGemmSimtTiled(g, name, plan);   // tiny ones: one thread per output
  else emitGemmSimt(g, name, plan);
}

}  // namespace accy
