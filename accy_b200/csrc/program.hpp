// Recorded tensor program: the named-axis IR that the CUDA target consumes.
//
// Mirrors the reference's recorded IR (src/tensor/program.zig:8-282): an SSA list of typed
// operations with ids dense from zero, parameters in order, and a list of output ids.  Every
// derived result type is recomputed here with the reference's Builder rules
// (src/tensor/trace/builder.zig, src/tensor/type/algebra.zig), never trusted from bytes.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace accy {

// Element types, numbered as on the wire (src/tensor/wire/format.zig:101-103) and as in
// deps/lib/compiler/gpu/abi/src/dtype.zig:38-52.
enum class DType : uint8_t { i1, i8, i16, i32, i64, u8, u16, u32, u64, f16, bf16, f32, f64, key };
constexpr uint32_t kDTypeCount = 14;
size_t dtypeSize(DType d);
const char* dtypeName(DType d);
bool dtypeIsFloat(DType d);

// Operation kinds in wire order (src/tensor/wire/format.zig:79-99).
enum class Kind : uint8_t {
  parameter, constant, unary, binary, iota, broadcast, broadcast_in_dim, reshape, transpose,
  reduce, gather, scatter_add, sparse_cross_entropy, dot_general, compare, select, custom_call,
  scan, projection
};
constexpr uint32_t kKindCount = 19;
const char* kindName(Kind k);

enum class Unary : uint8_t { neg, abs, exp, log, sqrt, tanh, sin, cos, tan };
enum class Binary : uint8_t { add, sub, mul, div, max, min, pow };
enum class Reducer : uint8_t { sum, max, min };
enum class Compare : uint8_t { lt, le, gt, ge, eq, ne };

struct Dim {
  std::string name;
  int64_t extent = 0;
};

struct Type {
  DType dtype = DType::f32;
  std::vector<Dim> dims;
  size_t rank() const { return dims.size(); }
  size_t elementCount() const;  // throws ShapeElementOverflow / InvalidDimension
  size_t byteCount() const;     // throws ShapeByteOverflow
};

// A failure named exactly as the reference's Zig error value (type/dim.zig:10-32 and the
// Builder's own), so tests read like the reference's `expectError(error.AxisExtentMismatch, …)`.
struct TensorError : std::runtime_error {
  explicit TensorError(const char* name) : std::runtime_error(name) {}
};

struct Operation {
  uint32_t id = 0;
  Type result;
  Kind kind = Kind::parameter;
  uint8_t sub = 0;                  // Unary / Binary / Reducer / Compare code
  std::vector<uint32_t> operands;   // value ids, in the reference's field order
  std::vector<int64_t> ints;        // broadcast_dims | permutation | reduce dimensions | lhs_contract
  std::vector<int64_t> rhs_contract, lhs_batch, rhs_batch;  // dot_general only
  int64_t axis = 0;                 // iota / gather / scatter_add / sparse_cross_entropy
  size_t index = 0;                 // parameter index / projection index
  std::vector<uint8_t> payload;     // constant bytes
  std::string target;               // custom_call target
  uint32_t version = 1;             // custom_call version
};

struct Program {
  std::string name;
  std::vector<Operation> ops;
  std::vector<uint32_t> parameters;
  std::vector<uint32_t> outputs;
  const Type& typeOf(uint32_t id) const { return ops[id].result; }
};

// ---- type algebra (src/tensor/type/algebra.zig) ----
long findDim(const std::vector<Dim>& dims, const std::string& name);
bool sameDims(const std::vector<Dim>& a, const std::vector<Dim>& b);
void validateDims(const std::vector<Dim>& dims);
void validateAuthoredDims(const std::vector<Dim>& dims);
void validateAuthoredName(const std::string& name);
void validateAxes(size_t rank, const std::vector<int64_t>& axes);
std::vector<Dim> unionDims(const std::vector<Dim>& lhs, const std::vector<Dim>& rhs);

struct Alignment {
  bool has_permutation = false, has_mapping = false;
  std::vector<int64_t> permutation, mapping;
};
Alignment alignment(const std::vector<Dim>& operand, const std::vector<Dim>& target);
std::vector<int64_t> axisIndices(const std::vector<Dim>& dims, const std::vector<std::string>& names);
std::vector<Dim> removeAxes(const std::vector<Dim>& dims, const std::vector<int64_t>& axes);
std::vector<Dim> permuted(const std::vector<Dim>& dims, const std::vector<int64_t>& permutation);

struct Contraction {
  std::vector<int64_t> lhs_contract, rhs_contract, lhs_batch, rhs_batch;
  std::vector<Dim> result;
};
Contraction contraction(const std::vector<Dim>& lhs, const std::vector<Dim>& rhs,
                        const std::vector<std::string>& names);
std::vector<Dim> dotGeneralDims(const std::vector<Dim>& lhs, const std::vector<Dim>& rhs,
                                const std::vector<int64_t>& lhs_contract,
                                const std::vector<int64_t>& rhs_contract,
                                const std::vector<int64_t>& lhs_batch,
                                const std::vector<int64_t>& rhs_batch);

// ---- Builder (src/tensor/trace/builder.zig:62-1047, src/tensor/trace/value.zig) ----
class Builder {
 public:
  explicit Builder(std::string name);
  // authored entry points
  uint32_t input(DType dtype, const std::vector<Dim>& dims, bool authored = true);
  uint32_t constantBytes(const Type& ty, const uint8_t* payload, size_t len);
  uint32_t fullFloat(const Type& ty, double fill);
  uint32_t iota(DType dtype, const std::vector<Dim>& dims, const std::string& axis_name);
  uint32_t unary(Unary op, uint32_t x);
  uint32_t alignedBinary(Binary op, uint32_t lhs, uint32_t rhs);
  uint32_t alignedCompare(Compare dir, uint32_t lhs, uint32_t rhs);
  uint32_t alignedSelect(uint32_t pred, uint32_t on_true, uint32_t on_false);
  uint32_t reduceNamed(uint32_t x, Reducer r, const std::vector<std::string>& names);
  uint32_t reduceWith(uint32_t x, uint32_t init, Reducer r, const std::vector<std::string>& names);
  uint32_t meanNamed(uint32_t x, const std::vector<std::string>& names);
  uint32_t contract(uint32_t lhs, uint32_t rhs, const std::vector<std::string>& names);
  uint32_t renameAxis(uint32_t x, const std::string& old_name, const std::string& new_name);
  uint32_t splitAxis(uint32_t x, const std::string& axis, const std::vector<Dim>& parts);
  uint32_t mergeAxes(uint32_t x, const std::vector<std::string>& names, const std::string& merged);
  uint32_t broadcastAxes(uint32_t x, const std::vector<Dim>& added);
  // raw entry points used by the wire decoder's replay (builder.zig:125-190 `operation`)
  uint32_t binary(Binary op, uint32_t lhs, uint32_t rhs);
  uint32_t compare(Compare dir, uint32_t lhs, uint32_t rhs);
  uint32_t select(uint32_t pred, uint32_t on_true, uint32_t on_false);
  uint32_t iotaTyped(const Type& ty, int64_t axis);
  uint32_t broadcastOp(uint32_t x, const std::vector<Dim>& result_dims);
  uint32_t broadcastTo(uint32_t x, const std::vector<Dim>& result_dims,
                       const std::vector<int64_t>& broadcast_dims);
  uint32_t reshapeTo(uint32_t x, const std::vector<Dim>& new_dims);
  uint32_t transposeBy(uint32_t x, const std::vector<int64_t>& permutation);
  uint32_t reduce(uint32_t x, uint32_t init, Reducer r, const std::vector<int64_t>& dimensions);
  uint32_t dotGeneralOp(uint32_t lhs, uint32_t rhs, const std::vector<int64_t>& lhs_contract,
                        const std::vector<int64_t>& rhs_contract,
                        const std::vector<int64_t>& lhs_batch,
                        const std::vector<int64_t>& rhs_batch);
  uint32_t alignTo(uint32_t x, const std::vector<Dim>& target);
  Program finish(const std::vector<uint32_t>& outputs);

  const Type& typeOf(uint32_t id) const;
  size_t valueCount() const { return prog_.ops.size(); }

 private:
  uint32_t emit(Operation op);
  void ensure(uint32_t id) const;
  uint32_t reducerInit(DType dtype, Reducer r);
  Program prog_;
  bool finished_ = false;
};

// ---- program transformations (src/tensor/grad.zig:19-49, src/tensor/batch.zig:14-47) ----
// Gradient of the single scalar output with respect to the parameters `wrt` (parameter indices);
// outputs = [value if keep_value,] one gradient per wrt entry.  Errors: GradientRequiresScalarOutput,
// ParameterOutOfRange, DuplicateParameter, NonDifferentiableParameter, UnsupportedDerivative.
Program gradProgram(const Program& src, const std::vector<size_t>& wrt, bool keep_value);
// Forward mode (src/tensor/autodiff.zig:725-732 `jvp`): inputs = the source's, then one tangent per
// differentiated parameter in parameter order; outputs = the source's, then their tangents.
Program jvpProgram(const Program& src, const std::vector<size_t>& wrt);
// Runs the program over a new named axis of extent axis_size.  in_axes[i] = position of the new
// axis in parameter i, or -1 for a parameter shared by all instances; every output gets the axis
// at out_axis.  An empty axis_name picks "#batch" (with a number appended while that name is
// taken).  Errors: InvalidDimension, InAxisCountMismatch, AxisOutOfRange.
Program vmapProgram(const Program& src, int64_t axis_size, const std::vector<int64_t>& in_axes, size_t out_axis,
                    const std::string& axis_name);

// ---- "ACTP" v1 wire bytes (src/tensor/wire/format.zig, encode.zig, decode.zig) ----
struct WireError : std::runtime_error {
  // name is one of BadMagic, UnsupportedVersion, UnknownTag, InvalidReference, TooManyOperands,
  // ScanTooDeep, InvalidArtifact, InvalidProgram, ScanUnsupported
  explicit WireError(const char* name) : std::runtime_error(name) {}
};
std::vector<uint8_t> encodeProgram(const Program& program);
Program decodeProgram(const uint8_t* bytes, size_t len);

}  // namespace accy
