// Execution plan for one recorded program on one B200: device slots, generated kernels and the
// ordered launch list.
//
// Plays the role of the reference's BackendArtifactPlan (src/artifact/plan.zig:177-199: slots,
// input/output slot ids, planned kernels) and of its fusion planner
// (src/preparation/fusion/pass.zig:234-292), re-decided for sm_100a:
//   * broadcasts, transposes, iotas, scalar constants and compare/select masks are folded into the
//     index math of the kernel that consumes them and never materialised
//     (cf. src/preparation/schedule/pass.zig:893-918);
//   * every elementwise op and every reduction over one set of named axes that share an iteration
//     space become ONE "row kernel" (the reference's reduction_input cluster, reduction.zig:755-879,
//     and its row pipeline, row.zig:556-668, without their op-count and column limits);
//   * a dot_general plus the elementwise ops that only it feeds becomes one GEMM with an epilogue
//     (fusion/pass.zig:1585-1699, without the 6-op chain limit);
//   * dot -> scale -> [causal mask] -> softmax -> dot becomes one attention kernel
//     (fusion/pass.zig:729-905, extended to causal masks, batch axes and bf16).
// Anything else is refused at compile time; there is no CPU fallback.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "program.hpp"

namespace accy {

// One node of a fused expression DAG, evaluated in a cluster's iteration space.
struct ENode {
  enum Op : uint8_t { Leaf, Const, Iota, Un, Bin, Cmp, Sel, Red };
  Op op = Leaf;
  uint8_t sub = 0;       // Unary / Binary / Compare / Reducer code
  DType dtype = DType::f32;
  int args[3] = {-1, -1, -1};
  uint32_t vary = 0;     // bit d set: value changes along cluster dim d
  int leaf = -1;         // Leaf: index into Cluster::leaves
  uint64_t bits = 0;     // Const: raw little-endian payload (<= 8 bytes)
  int dim = -1;          // Iota: cluster dim
  int level = 0;         // number of reductions on the longest path from the leaves
};

struct LeafRef {
  int slot = -1;                  // plan slot holding the buffer
  DType dtype = DType::f32;
  std::vector<int64_t> strides;   // element stride per cluster dim (0 = broadcast)
  uint32_t vary = 0;
};

struct ClusterOutput {
  int node = -1;
  int ref = -1;   // index into Cluster::leaves: the output buffer and its index map
};

// A fused elementwise + reduction kernel over the space [extents[0..split) | extents[split..)]:
// the leading dims index rows (kept), the trailing dims index columns (reduced).
struct Cluster {
  std::vector<int64_t> extents;
  int split = 0;
  int64_t rows = 1, cols = 1;
  std::vector<ENode> nodes;
  std::vector<LeafRef> leaves;
  std::vector<ClusterOutput> outputs;
  uint32_t rowMask() const { return split >= 32 ? 0xffffffffu : ((1u << split) - 1u); }
};

// Elementwise work applied to each accumulator element of a GEMM before it is stored: an
// expression DAG over the space [batch, m, n] whose node `acc` is the f32 accumulator.
struct Epilogue {
  std::vector<ENode> nodes;
  std::vector<LeafRef> leaves;   // strides over dims (batch, m, n)
  int acc = -1;                  // node standing for the accumulator
  int result = -1;               // node that is stored
};

struct GemmOp {
  // C[b, m, n] = sum_k A[b, m, k] * B[b, k, n]; element strides of each operand's leaf buffer
  int64_t batch = 1, m = 0, n = 0, k = 0;
  int a_slot = -1, b_slot = -1, c_slot = -1;
  int64_t a_stride_b = 0, a_stride_m = 0, a_stride_k = 0;
  int64_t b_stride_b = 0, b_stride_k = 0, b_stride_n = 0;
  DType in_dtype = DType::f32, b_dtype = DType::f32, out_dtype = DType::f32;  // storage types of A, B, C
  Epilogue epilogue;
  bool tensor_core = false;      // tcgen05 path (bf16, tile-aligned) or SIMT k-serial path
};

struct AttentionOp {
  // O[bh, q, d] = softmax_k(scale * Q[bh, q, :] . K[bh, k, :] (+ causal mask)) . V[bh, k, d]
  int64_t batch = 1, q_len = 0, k_len = 0, head_dim = 0;
  int q_slot = -1, k_slot = -1, v_slot = -1, o_slot = -1;
  float scale = 1.0f;
  bool causal = false;
  DType dtype = DType::bf16;
};

struct Slot {
  enum Role : uint8_t { Input, Output, Temp, Constant, Scratch };
  Role role = Temp;
  int io_index = -1;             // parameter index (Input) or output index (Output)
  size_t bytes = 0;
  // Element type the buffer is stored in.  Inputs, outputs and constants use the program's type;
  // a temporary holding a 16-bit-float value is stored as f32 unless a contraction reads it, so
  // intermediate results between kernels are not rounded to 16 bits.
  DType storage = DType::f32;
  uint32_t value = 0xffffffffu;  // program value the slot holds
  std::vector<uint8_t> payload;  // Constant: uploaded once at load time
  bool zero_init = false;        // Scratch: cleared once at load time (kernels that use it leave it cleared)
};

struct KernelArg {
  bool is_slot = true;
  int slot = -1;
  uint64_t scalar = 0;  // 8-byte scalar slot, as the reference's launch ABI
  int scalar_bytes = 0;
  bool tensor_map = false;       // argument is a CUtensorMap built from `tma`
  struct Tma {
    int slot = -1;
    int rank = 0;
    uint64_t dims[5] = {0, 0, 0, 0, 0};      // innermost first, in elements
    uint64_t strides[4] = {0, 0, 0, 0};      // bytes, dims 1..rank-1
    uint32_t box[5] = {1, 1, 1, 1, 1};
    int elem_bytes = 2;
    int swizzle = 0;             // 0 none, 1 32B, 2 64B, 3 128B
  } tma;
};

struct Launch {
  int kernel = -1;               // index into Plan::kernels
  uint32_t grid[3] = {1, 1, 1};
  uint32_t block[3] = {1, 1, 1};
  uint32_t dynamic_smem = 0;
  std::vector<KernelArg> args;
  std::string label;
};

struct KernelSource {
  std::string name;              // extern "C" entry point
  std::string source;            // full CUDA translation unit
  std::vector<std::string> options;  // extra compiler options (e.g. --fmad=false)
  std::string family;            // "row", "row_combine", "gemm_simt", "gemm_tcgen05", "attention"
};

// Algorithmic work of a planned program, for roofline reporting.
struct WorkEstimate {
  double bytes = 0;   // bytes that must cross HBM at least once (inputs read once + outputs written once)
  double flops = 0;   // contraction flops (2*m*n*k per dot, causal count for attention)
  double pairs = 0;   // elementwise-reduction evaluations (rows*cols summed over row kernels)
};

struct ScheduleOverrides {
  int threads_per_row = 0;       // 0 = automatic
  int vectors_per_thread = 0;
  int column_splits = 0;
  int force_simt_gemm = 0;
  int row_min_blocks = 0;
  int sm_count = 148;
};

struct Plan {
  std::vector<Slot> slots;
  std::vector<int> input_slots;   // by parameter index
  std::vector<int> output_slots;  // by output index
  std::vector<KernelSource> kernels;
  std::vector<Launch> launches;
  WorkEstimate work;
  std::string summary;            // human-readable description of the fusion decisions
};

struct PlanError : std::runtime_error {
  explicit PlanError(const std::string& what) : std::runtime_error(what) {}
};

Plan planProgram(const Program& program, const ScheduleOverrides& overrides);

// Sharding along a named axis (shard.cpp).
struct ShardInfo {
  std::string axis;
  int64_t extent = -1;          // the axis' extent in the program
  bool shardable = false;
  bool partial_sum = false;     // pieces produce partial folds of every output (combine them)
  uint32_t partial_fold = 0;    // how: 1 = add, 2 = maximum, 3 = minimum (the outputs' own reducer)
  std::vector<uint32_t> partial_outputs;
  std::string reason;           // why not, when !shardable
};
ShardInfo analyseShardAxis(const Program& program, const std::string& axis);
Program shardProgram(const Program& program, const std::string& axis, int64_t extent);

// code emission (emit_row.cpp, emit_gemm.cpp)
struct RowSchedule {
  int tpr = 32;        // threads cooperating on one row
  int rpc = 1;         // rows per CTA
  int vec = 1;         // elements per vector access along the column axis
  int vpt = 1;         // vector accesses per thread per chunk
  int64_t chunks = 1;  // chunk iterations per row (1 = the whole row lives in registers)
  int splits = 1;      // CTAs sharing one row (deterministic two-pass combine when > 1)
  int min_blocks = 0;  // resident CTAs per SM asked of the compiler (caps registers), 0 = no request
  int rpt = 1;         // rows per thread: neighbouring rows a thread folds together, sharing what does not vary along the rows
};
RowSchedule chooseRowSchedule(const Cluster& c, const ScheduleOverrides& o);
void emitRowKernels(const Cluster& c, const RowSchedule& s, const std::string& name, Plan& plan,
                    const std::string& label);
void emitGemm(const GemmOp& g, const std::string& name, Plan& plan, const ScheduleOverrides& o);
void emitAttention(const AttentionOp& a, const std::string& name, Plan& plan,
                   const ScheduleOverrides& o);
// Emits the C expression that evaluates an elementwise node from its operand expressions.
std::string elementwiseExpr(const ENode& n, const std::string& a, const std::string& b,
                            const std::string& c, DType a_dtype);
std::string constLiteral(const ENode& n);
const char* ctypeOf(DType d);   // register type used for a value of this dtype
const char* storageTypeOf(DType d);

}  // namespace accy
