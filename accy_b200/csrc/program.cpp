// Type algebra and the Builder mirror for recorded tensor programs.
//
// Semantics follow the reference's named-axis rules so that the same authored program records the
// same operation list, result types and error names:
//   unionDims / alignment / axisIndices / removeAxes / contraction / dotGeneralDims
//     -> src/tensor/type/algebra.zig:10-101, 320-470
//   Builder entry points -> src/tensor/trace/builder.zig:313-330, 476-485, 546-587, 743-865
#include "program.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <numeric>

namespace accy {

size_t dtypeSize(DType d) {
  switch (d) {
    case DType::i1: case DType::i8: case DType::u8: return 1;
    case DType::i16: case DType::u16: case DType::f16: case DType::bf16: return 2;
    case DType::i32: case DType::u32: case DType::f32: return 4;
    case DType::i64: case DType::u64: case DType::f64: case DType::key: return 8;
  }
  return 0;
}

const char* dtypeName(DType d) {
  static const char* names[] = {"i1", "i8", "i16", "i32", "i64", "u8", "u16",
                                "u32", "u64", "f16", "bf16", "f32", "f64", "key"};
  return names[static_cast<int>(d)];
}

bool dtypeIsFloat(DType d) {
  return d == DType::f16 || d == DType::bf16 || d == DType::f32 || d == DType::f64;
}

const char* kindName(Kind k) {
  static const char* names[] = {"parameter", "constant", "unary", "binary", "iota", "broadcast",
                                "broadcast_in_dim", "reshape", "transpose", "reduce", "gather",
                                "scatter_add", "sparse_cross_entropy", "dot_general", "compare",
                                "select", "custom_call", "scan", "projection"};
  return names[static_cast<int>(k)];
}

size_t Type::elementCount() const {
  size_t count = 1;
  for (const Dim& d : dims) {
    if (d.extent < 0) throw TensorError("InvalidDimension");
    size_t e = static_cast<size_t>(d.extent);
    if (e != 0 && count > std::numeric_limits<size_t>::max() / e)
      throw TensorError("ShapeElementOverflow");
    count *= e;
  }
  return count;
}

size_t Type::byteCount() const {
  size_t n = elementCount(), s = dtypeSize(dtype);
  if (n != 0 && s > std::numeric_limits<size_t>::max() / n) throw TensorError("ShapeByteOverflow");
  return n * s;
}

long findDim(const std::vector<Dim>& dims, const std::string& name) {
  for (size_t i = 0; i < dims.size(); ++i)
    if (dims[i].name == name) return static_cast<long>(i);
  return -1;
}

bool sameDims(const std::vector<Dim>& a, const std::vector<Dim>& b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (a[i].extent != b[i].extent || a[i].name != b[i].name) return false;
  return true;
}

void validateDims(const std::vector<Dim>& dims) {
  for (size_t i = 0; i < dims.size(); ++i) {
    if (dims[i].name.empty()) throw TensorError("AxisNameEmpty");
    if (dims[i].extent < 0) throw TensorError("InvalidDimension");
    for (size_t j = 0; j < i; ++j)
      if (dims[j].name == dims[i].name) throw TensorError("DuplicateAxis");
  }
}

void validateAuthoredName(const std::string& name) {
  if (name.empty()) throw TensorError("AxisNameEmpty");
  if (name[0] == '#') throw TensorError("AxisNameReserved");
}

void validateAuthoredDims(const std::vector<Dim>& dims) {
  validateDims(dims);
  for (const Dim& d : dims) validateAuthoredName(d.name);
}

static bool containsAxis(const std::vector<int64_t>& axes, size_t index) {
  for (int64_t a : axes)
    if (a == static_cast<int64_t>(index)) return true;
  return false;
}

// Range and duplicate check over groups of axes (src/axis/roles.zig:21-48).
static void validateAxisGroups(size_t rank, std::initializer_list<const std::vector<int64_t>*> groups) {
  std::vector<int64_t> seen;
  for (const auto* group : groups) {
    for (int64_t axis : *group) {
      if (axis < 0 || static_cast<size_t>(axis) >= rank) throw TensorError("AxisOutOfRange");
      if (std::find(seen.begin(), seen.end(), axis) != seen.end()) throw TensorError("DuplicateAxis");
      seen.push_back(axis);
    }
  }
}

void validateAxes(size_t rank, const std::vector<int64_t>& axes) { validateAxisGroups(rank, {&axes}); }

std::vector<Dim> unionDims(const std::vector<Dim>& lhs, const std::vector<Dim>& rhs) {
  std::vector<Dim> out = lhs;
  for (const Dim& d : rhs) {
    long at = findDim(lhs, d.name);
    if (at >= 0) {
      if (lhs[at].extent != d.extent) throw TensorError("AxisExtentMismatch");
    } else {
      out.push_back(d);
    }
  }
  return out;
}

Alignment alignment(const std::vector<Dim>& operand, const std::vector<Dim>& target) {
  Alignment plan;
  if (sameDims(operand, target)) return plan;
  std::vector<int64_t> positions(operand.size());
  for (size_t i = 0; i < operand.size(); ++i) {
    long at = findDim(target, operand[i].name);
    if (at < 0) throw TensorError("AxisNotFound");
    if (target[at].extent != operand[i].extent) throw TensorError("AxisExtentMismatch");
    positions[i] = at;
  }
  bool increasing = true;
  for (size_t i = 1; i < positions.size(); ++i)
    if (positions[i - 1] >= positions[i]) { increasing = false; break; }
  plan.has_mapping = true;
  if (increasing) {
    plan.mapping = positions;
    return plan;
  }
  std::vector<int64_t> order(operand.size());
  std::iota(order.begin(), order.end(), 0);
  // positions are distinct (names are unique), so any sort gives the reference's order
  std::sort(order.begin(), order.end(),
            [&](int64_t a, int64_t b) { return positions[a] < positions[b]; });
  plan.has_permutation = true;
  plan.permutation = order;
  plan.mapping.resize(operand.size());
  for (size_t i = 0; i < order.size(); ++i) plan.mapping[i] = positions[order[i]];
  return plan;
}

std::vector<int64_t> axisIndices(const std::vector<Dim>& dims, const std::vector<std::string>& names) {
  if (names.empty()) throw TensorError("AxisNotFound");
  std::vector<int64_t> indices;
  for (const std::string& name : names) {
    long at = findDim(dims, name);
    if (at < 0) throw TensorError("AxisNotFound");
    if (std::find(indices.begin(), indices.end(), at) != indices.end()) throw TensorError("DuplicateAxis");
    indices.push_back(at);
  }
  std::sort(indices.begin(), indices.end());
  return indices;
}

std::vector<Dim> removeAxes(const std::vector<Dim>& dims, const std::vector<int64_t>& axes) {
  validateAxes(dims.size(), axes);
  std::vector<Dim> out;
  for (size_t i = 0; i < dims.size(); ++i)
    if (!containsAxis(axes, i)) out.push_back(dims[i]);
  return out;
}

std::vector<Dim> permuted(const std::vector<Dim>& dims, const std::vector<int64_t>& permutation) {
  if (dims.size() != permutation.size()) throw TensorError("RankMismatch");
  validateAxes(dims.size(), permutation);
  std::vector<Dim> out;
  for (int64_t axis : permutation) out.push_back(dims[axis]);
  return out;
}

Contraction contraction(const std::vector<Dim>& lhs, const std::vector<Dim>& rhs,
                        const std::vector<std::string>& names) {
  if (names.empty()) throw TensorError("AxisNotFound");
  Contraction c;
  for (const std::string& name : names) {
    long li = findDim(lhs, name), ri = findDim(rhs, name);
    if (li < 0 || ri < 0) throw TensorError("AxisNotFound");
    if (lhs[li].extent != rhs[ri].extent) throw TensorError("AxisExtentMismatch");
    if (containsAxis(c.lhs_contract, li)) throw TensorError("DuplicateAxis");
    c.lhs_contract.push_back(li);
    c.rhs_contract.push_back(ri);
  }
  // batch axes: names shared by both sides and not contracted, in lhs order
  for (size_t i = 0; i < lhs.size(); ++i) {
    if (containsAxis(c.lhs_contract, i)) continue;
    long ri = findDim(rhs, lhs[i].name);
    if (ri < 0) continue;
    if (lhs[i].extent != rhs[ri].extent) throw TensorError("AxisExtentMismatch");
    c.lhs_batch.push_back(i);
    c.rhs_batch.push_back(ri);
  }
  for (int64_t i : c.lhs_batch) c.result.push_back(lhs[i]);
  for (size_t i = 0; i < lhs.size(); ++i)
    if (!containsAxis(c.lhs_contract, i) && !containsAxis(c.lhs_batch, i)) c.result.push_back(lhs[i]);
  for (size_t i = 0; i < rhs.size(); ++i) {
    if (containsAxis(c.rhs_contract, i) || containsAxis(c.rhs_batch, i)) continue;
    if (findDim(c.result, rhs[i].name) >= 0) throw TensorError("DuplicateAxis");
    c.result.push_back(rhs[i]);
  }
  return c;
}

std::vector<Dim> dotGeneralDims(const std::vector<Dim>& lhs, const std::vector<Dim>& rhs,
                                const std::vector<int64_t>& lhs_contract,
                                const std::vector<int64_t>& rhs_contract,
                                const std::vector<int64_t>& lhs_batch,
                                const std::vector<int64_t>& rhs_batch) {
  validateAxes(lhs.size(), lhs_contract);
  validateAxes(rhs.size(), rhs_contract);
  validateAxes(lhs.size(), lhs_batch);
  validateAxes(rhs.size(), rhs_batch);
  for (int64_t a : lhs_batch) if (containsAxis(lhs_contract, a)) throw TensorError("DuplicateAxis");
  for (int64_t a : rhs_batch) if (containsAxis(rhs_contract, a)) throw TensorError("DuplicateAxis");
  if (lhs_contract.size() != rhs_contract.size()) throw TensorError("RankMismatch");
  if (lhs_batch.size() != rhs_batch.size()) throw TensorError("RankMismatch");
  for (size_t i = 0; i < lhs_contract.size(); ++i)
    if (lhs[lhs_contract[i]].extent != rhs[rhs_contract[i]].extent) throw TensorError("AxisExtentMismatch");
  for (size_t i = 0; i < lhs_batch.size(); ++i)
    if (lhs[lhs_batch[i]].extent != rhs[rhs_batch[i]].extent) throw TensorError("AxisExtentMismatch");
  std::vector<Dim> out;
  for (int64_t a : lhs_batch) out.push_back(lhs[a]);
  for (size_t i = 0; i < lhs.size(); ++i)
    if (!containsAxis(lhs_contract, i) && !containsAxis(lhs_batch, i)) out.push_back(lhs[i]);
  for (size_t i = 0; i < rhs.size(); ++i)
    if (!containsAxis(rhs_contract, i) && !containsAxis(rhs_batch, i)) out.push_back(rhs[i]);
  for (size_t i = 0; i < out.size(); ++i)
    for (size_t j = 0; j < i; ++j)
      if (out[i].name == out[j].name) throw TensorError("DuplicateAxis");
  return out;
}

// ------------------------------------------------------------------------------------------
// Builder
// ------------------------------------------------------------------------------------------

Builder::Builder(std::string name) { prog_.name = std::move(name); }

void Builder::ensure(uint32_t id) const {
  if (finished_) throw TensorError("BuilderFinished");
  if (id >= prog_.ops.size()) throw TensorError("CrossBuilderValue");
}

const Type& Builder::typeOf(uint32_t id) const {
  if (id >= prog_.ops.size()) throw TensorError("CrossBuilderValue");
  return prog_.ops[id].result;
}

uint32_t Builder::emit(Operation op) {
  if (finished_) throw TensorError("BuilderFinished");
  validateDims(op.result.dims);
  op.id = static_cast<uint32_t>(prog_.ops.size());
  prog_.ops.push_back(std::move(op));
  return prog_.ops.back().id;
}

uint32_t Builder::input(DType dtype, const std::vector<Dim>& dims, bool authored) {
  // replayed parameters (wire decoder) skip the authored-name rule, as inputTyped does
  if (authored) validateAuthoredDims(dims);
  Operation op;
  op.kind = Kind::parameter;
  op.result = Type{dtype, dims};
  op.index = prog_.parameters.size();
  uint32_t id = emit(std::move(op));
  prog_.parameters.push_back(id);
  return id;
}

uint32_t Builder::constantBytes(const Type& ty, const uint8_t* payload, size_t len) {
  if (len != ty.byteCount()) throw TensorError("PayloadLengthMismatch");
  Operation op;
  op.kind = Kind::constant;
  op.result = ty;
  op.payload.assign(payload, payload + len);
  return emit(std::move(op));
}

static uint16_t f32ToBf16Truncate(float x) {
  // the reference's Bf16.fromF32 drops the low 16 bits (deps/lib/compiler/gpu/abi/src/dtype.zig:6-9)
  uint32_t bits;
  std::memcpy(&bits, &x, 4);
  return static_cast<uint16_t>(bits >> 16);
}

static uint16_t f32ToF16(float x) {
  // round-to-nearest-even f32 -> f16, as Zig's @floatCast does
  uint32_t b;
  std::memcpy(&b, &x, 4);
  uint32_t sign = (b >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((b >> 23) & 0xff) - 127 + 15;
  uint32_t man = b & 0x7fffffu;
  if (((b >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    uint32_t shift = static_cast<uint32_t>(14 - exp);
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

uint32_t Builder::fullFloat(const Type& ty, double fill) {
  size_t count = ty.elementCount();
  std::vector<uint8_t> bytes(count * dtypeSize(ty.dtype));
  switch (ty.dtype) {
    case DType::f16: {
      uint16_t v = f32ToF16(static_cast<float>(fill));
      for (size_t i = 0; i < count; ++i) std::memcpy(&bytes[2 * i], &v, 2);
      break;
    }
    case DType::bf16: {
      uint16_t v = f32ToBf16Truncate(static_cast<float>(fill));
      for (size_t i = 0; i < count; ++i) std::memcpy(&bytes[2 * i], &v, 2);
      break;
    }
    case DType::f32: {
      float v = static_cast<float>(fill);
      for (size_t i = 0; i < count; ++i) std::memcpy(&bytes[4 * i], &v, 4);
      break;
    }
    case DType::f64:
      for (size_t i = 0; i < count; ++i) std::memcpy(&bytes[8 * i], &fill, 8);
      break;
    default:
      throw TensorError("NonFloatDType");
  }
  Operation op;
  op.kind = Kind::constant;
  op.result = ty;
  op.payload = std::move(bytes);
  return emit(std::move(op));
}

uint32_t Builder::iotaTyped(const Type& ty, int64_t axis) {
  validateAxes(ty.dims.size(), {axis});
  Operation op;
  op.kind = Kind::iota;
  op.result = ty;
  op.axis = axis;
  return emit(std::move(op));
}

uint32_t Builder::iota(DType dtype, const std::vector<Dim>& dims, const std::string& axis_name) {
  validateAuthoredDims(dims);
  long at = findDim(dims, axis_name);
  if (at < 0) throw TensorError("AxisNotFound");
  return iotaTyped(Type{dtype, dims}, at);
}

uint32_t Builder::unary(Unary u, uint32_t x) {
  ensure(x);
  Operation op;
  op.kind = Kind::unary;
  op.sub = static_cast<uint8_t>(u);
  op.operands = {x};
  op.result = typeOf(x);
  return emit(std::move(op));
}

static void requireSameType(const Type& a, const Type& b) {
  if (a.dtype != b.dtype) throw TensorError("DTypeMismatch");
  if (!sameDims(a.dims, b.dims)) throw TensorError("ShapeMismatch");
}

uint32_t Builder::binary(Binary b, uint32_t lhs, uint32_t rhs) {
  ensure(lhs);
  ensure(rhs);
  requireSameType(typeOf(lhs), typeOf(rhs));
  Operation op;
  op.kind = Kind::binary;
  op.sub = static_cast<uint8_t>(b);
  op.operands = {lhs, rhs};
  op.result = typeOf(lhs);
  return emit(std::move(op));
}

uint32_t Builder::alignedBinary(Binary b, uint32_t lhs, uint32_t rhs) {
  ensure(lhs);
  ensure(rhs);
  if (typeOf(lhs).dtype != typeOf(rhs).dtype) throw TensorError("DTypeMismatch");
  std::vector<Dim> target = unionDims(typeOf(lhs).dims, typeOf(rhs).dims);
  uint32_t left = alignTo(lhs, target);
  uint32_t right = alignTo(rhs, target);
  return binary(b, left, right);
}

uint32_t Builder::compare(Compare dir, uint32_t lhs, uint32_t rhs) {
  ensure(lhs);
  ensure(rhs);
  requireSameType(typeOf(lhs), typeOf(rhs));
  Operation op;
  op.kind = Kind::compare;
  op.sub = static_cast<uint8_t>(dir);
  op.operands = {lhs, rhs};
  op.result = Type{DType::i1, typeOf(lhs).dims};
  return emit(std::move(op));
}

uint32_t Builder::alignedCompare(Compare dir, uint32_t lhs, uint32_t rhs) {
  ensure(lhs);
  ensure(rhs);
  if (typeOf(lhs).dtype != typeOf(rhs).dtype) throw TensorError("DTypeMismatch");
  std::vector<Dim> target = unionDims(typeOf(lhs).dims, typeOf(rhs).dims);
  uint32_t left = alignTo(lhs, target);
  uint32_t right = alignTo(rhs, target);
  return compare(dir, left, right);
}

uint32_t Builder::select(uint32_t pred, uint32_t on_true, uint32_t on_false) {
  ensure(pred);
  ensure(on_true);
  ensure(on_false);
  const Type &p = typeOf(pred), &t = typeOf(on_true), &f = typeOf(on_false);
  if (p.dtype != DType::i1) throw TensorError("DTypeMismatch");
  if (t.dtype != f.dtype) throw TensorError("DTypeMismatch");
  if (!sameDims(t.dims, f.dims)) throw TensorError("ShapeMismatch");
  if (p.rank() != 0 && !sameDims(p.dims, t.dims)) throw TensorError("ShapeMismatch");
  Operation op;
  op.kind = Kind::select;
  op.operands = {pred, on_true, on_false};
  op.result = t;
  return emit(std::move(op));
}

uint32_t Builder::alignedSelect(uint32_t pred, uint32_t on_true, uint32_t on_false) {
  ensure(pred);
  ensure(on_true);
  ensure(on_false);
  if (typeOf(on_true).dtype != typeOf(on_false).dtype) throw TensorError("DTypeMismatch");
  std::vector<Dim> target = unionDims(typeOf(on_true).dims, typeOf(on_false).dims);
  bool scalar_pred = typeOf(pred).rank() == 0;
  if (!scalar_pred) target = unionDims(target, typeOf(pred).dims);
  uint32_t t = alignTo(on_true, target);
  uint32_t f = alignTo(on_false, target);
  uint32_t p = scalar_pred ? pred : alignTo(pred, target);
  return select(p, t, f);
}

uint32_t Builder::alignTo(uint32_t x, const std::vector<Dim>& target) {
  ensure(x);
  if (sameDims(typeOf(x).dims, target)) return x;
  Alignment plan = alignment(typeOf(x).dims, target);
  uint32_t current = x;
  if (plan.has_permutation) current = transposeBy(current, plan.permutation);
  if (sameDims(typeOf(current).dims, target)) return current;
  return broadcastTo(current, target, plan.mapping);
}

uint32_t Builder::broadcastOp(uint32_t x, const std::vector<Dim>& result_dims) {
  ensure(x);
  Operation op;
  op.kind = Kind::broadcast;
  op.operands = {x};
  op.result = Type{typeOf(x).dtype, result_dims};
  for (const Dim& d : result_dims) op.ints.push_back(d.extent);
  return emit(std::move(op));
}

uint32_t Builder::broadcastTo(uint32_t x, const std::vector<Dim>& result_dims,
                              const std::vector<int64_t>& broadcast_dims) {
  ensure(x);
  const Type& in = typeOf(x);
  if (broadcast_dims.size() != in.rank()) throw TensorError("BroadcastRankMismatch");
  validateAxes(result_dims.size(), broadcast_dims);
  for (size_t i = 0; i < broadcast_dims.size(); ++i) {
    int64_t want = result_dims[broadcast_dims[i]].extent;
    if (in.dims[i].extent != 1 && in.dims[i].extent != want) throw TensorError("BroadcastDimensionMismatch");
  }
  Operation op;
  op.kind = Kind::broadcast_in_dim;
  op.operands = {x};
  op.ints = broadcast_dims;
  op.result = Type{in.dtype, result_dims};
  return emit(std::move(op));
}

uint32_t Builder::reshapeTo(uint32_t x, const std::vector<Dim>& new_dims) {
  ensure(x);
  Type result{typeOf(x).dtype, new_dims};
  validateDims(new_dims);
  if (typeOf(x).elementCount() != result.elementCount()) throw TensorError("ReshapeElementMismatch");
  Operation op;
  op.kind = Kind::reshape;
  op.operands = {x};
  for (const Dim& d : new_dims) op.ints.push_back(d.extent);
  op.result = std::move(result);
  return emit(std::move(op));
}

uint32_t Builder::transposeBy(uint32_t x, const std::vector<int64_t>& permutation) {
  ensure(x);
  Operation op;
  op.kind = Kind::transpose;
  op.operands = {x};
  op.ints = permutation;
  op.result = Type{typeOf(x).dtype, permuted(typeOf(x).dims, permutation)};
  return emit(std::move(op));
}

uint32_t Builder::reduce(uint32_t x, uint32_t init, Reducer r, const std::vector<int64_t>& dimensions) {
  ensure(x);
  ensure(init);
  if (typeOf(x).dtype != typeOf(init).dtype) throw TensorError("DTypeMismatch");
  if (typeOf(init).rank() != 0) throw TensorError("ReduceInitNotScalar");
  Operation op;
  op.kind = Kind::reduce;
  op.sub = static_cast<uint8_t>(r);
  op.operands = {x, init};
  op.ints = dimensions;
  op.result = Type{typeOf(x).dtype, removeAxes(typeOf(x).dims, dimensions)};
  return emit(std::move(op));
}

uint32_t Builder::reducerInit(DType dtype, Reducer r) {
  Type ty{dtype, {}};
  if (r == Reducer::sum) {
    std::vector<uint8_t> zero(dtypeSize(dtype), 0);
    return constantBytes(ty, zero.data(), zero.size());
  }
  bool lowest = (r == Reducer::max);
  switch (dtype) {
    case DType::f32: {
      float v = lowest ? -INFINITY : INFINITY;
      return constantBytes(ty, reinterpret_cast<uint8_t*>(&v), 4);
    }
    case DType::f64: {
      double v = lowest ? -INFINITY : INFINITY;
      return constantBytes(ty, reinterpret_cast<uint8_t*>(&v), 8);
    }
    case DType::f16: {
      uint16_t v = lowest ? 0xfc00 : 0x7c00;
      return constantBytes(ty, reinterpret_cast<uint8_t*>(&v), 2);
    }
    case DType::bf16: {
      uint16_t v = lowest ? 0xff80 : 0x7f80;
      return constantBytes(ty, reinterpret_cast<uint8_t*>(&v), 2);
    }
    case DType::i32: {
      int32_t v = lowest ? std::numeric_limits<int32_t>::min() : std::numeric_limits<int32_t>::max();
      return constantBytes(ty, reinterpret_cast<uint8_t*>(&v), 4);
    }
    case DType::i64: {
      int64_t v = lowest ? std::numeric_limits<int64_t>::min() : std::numeric_limits<int64_t>::max();
      return constantBytes(ty, reinterpret_cast<uint8_t*>(&v), 8);
    }
    default:
      throw TensorError("DTypeMismatch");
  }
}

uint32_t Builder::reduceNamed(uint32_t x, Reducer r, const std::vector<std::string>& names) {
  ensure(x);
  std::vector<int64_t> indices = axisIndices(typeOf(x).dims, names);
  uint32_t init = reducerInit(typeOf(x).dtype, r);
  return reduce(x, init, r, indices);
}

uint32_t Builder::reduceWith(uint32_t x, uint32_t init, Reducer r, const std::vector<std::string>& names) {
  ensure(x);
  return reduce(x, init, r, axisIndices(typeOf(x).dims, names));
}

uint32_t Builder::meanNamed(uint32_t x, const std::vector<std::string>& names) {
  ensure(x);
  std::vector<int64_t> indices = axisIndices(typeOf(x).dims, names);
  size_t count = 1;
  for (int64_t a : indices) {
    size_t e = static_cast<size_t>(typeOf(x).dims[a].extent);
    if (e != 0 && count > std::numeric_limits<size_t>::max() / e) throw TensorError("ShapeElementOverflow");
    count *= e;
  }
  uint32_t init = reducerInit(typeOf(x).dtype, Reducer::sum);
  uint32_t summed = reduce(x, init, Reducer::sum, indices);
  uint32_t divisor = fullFloat(Type{typeOf(x).dtype, {}}, static_cast<double>(count));
  return alignedBinary(Binary::div, summed, divisor);
}

uint32_t Builder::contract(uint32_t lhs, uint32_t rhs, const std::vector<std::string>& names) {
  ensure(lhs);
  ensure(rhs);
  if (typeOf(lhs).dtype != typeOf(rhs).dtype) throw TensorError("ContractDTypeMismatch");
  const std::vector<Dim> ld = typeOf(lhs).dims, rd = typeOf(rhs).dims;
  Contraction plan = contraction(ld, rd, names);
  const size_t nb = plan.lhs_batch.size(), nc = plan.lhs_contract.size();
  // canonical operand orders: lhs [batch.., free.., contract..], rhs [batch.., contract.., free..]
  std::vector<Dim> lhs_order, rhs_order;
  for (int64_t a : plan.lhs_batch) lhs_order.push_back(ld[a]);
  for (size_t i = 0; i < ld.size(); ++i)
    if (!containsAxis(plan.lhs_batch, i) && !containsAxis(plan.lhs_contract, i)) lhs_order.push_back(ld[i]);
  const size_t lhs_free = lhs_order.size() - nb;
  for (int64_t a : plan.lhs_contract) lhs_order.push_back(ld[a]);
  for (int64_t a : plan.rhs_batch) rhs_order.push_back(rd[a]);
  for (int64_t a : plan.rhs_contract) rhs_order.push_back(rd[a]);
  for (size_t i = 0; i < rd.size(); ++i)
    if (!containsAxis(plan.rhs_batch, i) && !containsAxis(plan.rhs_contract, i)) rhs_order.push_back(rd[i]);
  uint32_t lc = alignTo(lhs, lhs_order);
  uint32_t rc = alignTo(rhs, rhs_order);
  Operation op;
  op.kind = Kind::dot_general;
  op.operands = {lc, rc};
  for (size_t i = 0; i < nb; ++i) {
    op.lhs_batch.push_back(i);
    op.rhs_batch.push_back(i);
  }
  for (size_t i = 0; i < nc; ++i) {
    op.ints.push_back(nb + lhs_free + i);
    op.rhs_contract.push_back(nb + i);
  }
  op.result = Type{typeOf(lhs).dtype, plan.result};
  return emit(std::move(op));
}

uint32_t Builder::dotGeneralOp(uint32_t lhs, uint32_t rhs, const std::vector<int64_t>& lhs_contract,
                               const std::vector<int64_t>& rhs_contract,
                               const std::vector<int64_t>& lhs_batch,
                               const std::vector<int64_t>& rhs_batch) {
  ensure(lhs);
  ensure(rhs);
  if (typeOf(lhs).dtype != typeOf(rhs).dtype) throw TensorError("ContractDTypeMismatch");
  Operation op;
  op.kind = Kind::dot_general;
  op.operands = {lhs, rhs};
  op.ints = lhs_contract;
  op.rhs_contract = rhs_contract;
  op.lhs_batch = lhs_batch;
  op.rhs_batch = rhs_batch;
  op.result = Type{typeOf(lhs).dtype, dotGeneralDims(typeOf(lhs).dims, typeOf(rhs).dims, lhs_contract,
                                                     rhs_contract, lhs_batch, rhs_batch)};
  return emit(std::move(op));
}

uint32_t Builder::renameAxis(uint32_t x, const std::string& old_name, const std::string& new_name) {
  ensure(x);
  validateAuthoredName(new_name);
  std::vector<Dim> dims = typeOf(x).dims;
  long at = findDim(dims, old_name);
  if (at < 0) throw TensorError("AxisNotFound");
  if (findDim(dims, new_name) >= 0) throw TensorError("DuplicateAxis");
  dims[at].name = new_name;
  return reshapeTo(x, dims);
}

uint32_t Builder::splitAxis(uint32_t x, const std::string& axis, const std::vector<Dim>& parts) {
  ensure(x);
  validateAuthoredDims(parts);
  const std::vector<Dim>& dims = typeOf(x).dims;
  long at = findDim(dims, axis);
  if (at < 0) throw TensorError("AxisNotFound");
  int64_t product = 1;
  for (const Dim& p : parts) {
    if (p.extent != 0 && product > std::numeric_limits<int64_t>::max() / p.extent)
      throw TensorError("ShapeElementOverflow");
    product *= p.extent;
  }
  if (product != dims[at].extent) throw TensorError("SplitExtentMismatch");
  for (const Dim& p : parts) {
    long existing = findDim(dims, p.name);
    if (existing >= 0 && existing != at) throw TensorError("DuplicateAxis");
  }
  std::vector<Dim> out(dims.begin(), dims.begin() + at);
  out.insert(out.end(), parts.begin(), parts.end());
  out.insert(out.end(), dims.begin() + at + 1, dims.end());
  return reshapeTo(x, out);
}

uint32_t Builder::mergeAxes(uint32_t x, const std::vector<std::string>& names, const std::string& merged) {
  ensure(x);
  validateAuthoredName(merged);
  const std::vector<Dim> dims = typeOf(x).dims;
  if (names.empty()) throw TensorError("AxisNotFound");
  std::vector<size_t> picked;
  size_t block_start = dims.size();
  int64_t extent = 1;
  for (const std::string& name : names) {
    long at = findDim(dims, name);
    if (at < 0) throw TensorError("AxisNotFound");
    if (std::find(picked.begin(), picked.end(), static_cast<size_t>(at)) != picked.end())
      throw TensorError("DuplicateAxis");
    picked.push_back(at);
    block_start = std::min(block_start, static_cast<size_t>(at));
    if (dims[at].extent != 0 && extent > std::numeric_limits<int64_t>::max() / dims[at].extent)
      throw TensorError("MergeExtentOverflow");
    extent *= dims[at].extent;
  }
  long existing = findDim(dims, merged);
  if (existing >= 0 && std::find(picked.begin(), picked.end(), static_cast<size_t>(existing)) == picked.end())
    throw TensorError("DuplicateAxis");
  auto isPicked = [&](size_t i) { return std::find(picked.begin(), picked.end(), i) != picked.end(); };
  std::vector<int64_t> permutation;
  std::vector<Dim> result;
  for (size_t i = 0; i < dims.size(); ++i) {
    if (i == block_start) {
      for (size_t p : picked) permutation.push_back(p);
      result.push_back(Dim{merged, extent});
    }
    if (!isPicked(i)) {
      permutation.push_back(i);
      result.push_back(dims[i]);
    }
  }
  bool identity = true;
  for (size_t i = 0; i < permutation.size(); ++i)
    if (permutation[i] != static_cast<int64_t>(i)) identity = false;
  uint32_t current = x;
  if (!identity) current = transposeBy(current, permutation);
  return reshapeTo(current, result);
}

uint32_t Builder::broadcastAxes(uint32_t x, const std::vector<Dim>& added) {
  ensure(x);
  validateAuthoredDims(added);
  std::vector<Dim> target = typeOf(x).dims;
  for (const Dim& d : added) {
    if (findDim(target, d.name) >= 0) throw TensorError("DuplicateAxis");
  }
  target.insert(target.end(), added.begin(), added.end());
  return alignTo(x, target);
}

Program Builder::finish(const std::vector<uint32_t>& outputs) {
  if (finished_) throw TensorError("BuilderFinished");
  for (uint32_t id : outputs) ensure(id);
  prog_.outputs = outputs;
  finished_ = true;
  return prog_;
}

}  // namespace accy
