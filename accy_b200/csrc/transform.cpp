// Program-to-program transformations of a recorded tensor program: reverse-mode gradient
// (`grad`, `valueAndGrad`) and batching over a new named axis (`vmap`).
//
// Mirrors the behaviour of the reference's src/tensor/grad.zig:19-49 (one scalar output; outputs of
// the derived program are [value,] then one gradient per `wrt` entry, in `wrt` order),
// src/tensor/autodiff.zig:744-855,886-893 (the derivative of every unary / binary operation, the
// tie conventions of max / min / abs, the validation errors) and src/tensor/batch.zig:14-47,
// 128-146,943-954 (mapped input axes, `out_axis`, unmapped outputs broadcast along the new axis,
// the default axis name "#batch").  The reference reaches the gradient through linearize →
// transpose → seed; here the cotangents are propagated directly over the recorded operations,
// which yields the same arithmetic per operation with a possibly different order of the
// additions that merge several uses of one value.
#include <algorithm>
#include <optional>

#include "program.hpp"

namespace accy {

namespace {

bool contains(const std::vector<int64_t>& v, int64_t a) { return std::find(v.begin(), v.end(), a) != v.end(); }

// A value of type `ty` filled with `v`: one scalar constant broadcast to the dims (never a dense
// payload, which would put the whole array into the program bytes).
uint32_t filled(Builder& b, const Type& ty, double v) {
  uint32_t scalar = b.fullFloat(Type{ty.dtype, {}}, v);
  if (ty.rank() == 0) return scalar;
  return b.broadcastTo(scalar, ty.dims, {});
}

// Zeros of any element type (an output that carries no derivative, e.g. an integer mask).
uint32_t zerosOf(Builder& b, const Type& ty) {
  std::vector<uint8_t> payload(dtypeSize(ty.dtype), 0);
  uint32_t scalar = b.constantBytes(Type{ty.dtype, {}}, payload.data(), payload.size());
  if (ty.rank() == 0) return scalar;
  return b.broadcastTo(scalar, ty.dims, {});
}

// Same value, dims relabelled to `dims` (same extents) when the names differ.
uint32_t relabel(Builder& b, uint32_t x, const std::vector<Dim>& dims) {
  if (sameDims(b.typeOf(x).dims, dims)) return x;
  return b.reshapeTo(x, dims);
}

uint32_t replayUnchanged(Builder& b, const Operation& op, const std::vector<uint32_t>& now) {
  auto arg = [&](size_t i) { return now[op.operands[i]]; };
  switch (op.kind) {
    case Kind::parameter: return b.input(op.result.dtype, op.result.dims, /*authored=*/false);
    case Kind::constant: return b.constantBytes(op.result, op.payload.data(), op.payload.size());
    case Kind::iota: return b.iotaTyped(op.result, op.axis);
    case Kind::unary: return b.unary(static_cast<Unary>(op.sub), arg(0));
    case Kind::binary: return b.binary(static_cast<Binary>(op.sub), arg(0), arg(1));
    case Kind::compare: return b.compare(static_cast<Compare>(op.sub), arg(0), arg(1));
    case Kind::select: return b.select(arg(0), arg(1), arg(2));
    case Kind::broadcast_in_dim: return b.broadcastTo(arg(0), op.result.dims, op.ints);
    case Kind::broadcast: return b.broadcastOp(arg(0), op.result.dims);
    case Kind::reshape: return b.reshapeTo(arg(0), op.result.dims);
    case Kind::transpose: return b.transposeBy(arg(0), op.ints);
    case Kind::reduce: return b.reduce(arg(0), arg(1), static_cast<Reducer>(op.sub), op.ints);
    case Kind::dot_general:
      return b.dotGeneralOp(arg(0), arg(1), op.ints, op.rhs_contract, op.lhs_batch, op.rhs_batch);
    case Kind::custom_call: throw TensorError("CustomCallRequiresJvpContract");
    case Kind::scan:
    case Kind::projection: throw TensorError("ScanLinearizationUnsupported");
    default: throw TensorError("OperationUnsupported");
  }
}

std::vector<int64_t> keptAxes(size_t rank, const std::vector<int64_t>& reduced) {
  std::vector<int64_t> kept;
  for (size_t a = 0; a < rank; ++a)
    if (!contains(reduced, static_cast<int64_t>(a))) kept.push_back(static_cast<int64_t>(a));
  return kept;
}

std::vector<int64_t> allAxes(size_t rank) {
  std::vector<int64_t> axes(rank);
  for (size_t a = 0; a < rank; ++a) axes[a] = static_cast<int64_t>(a);
  return axes;
}

// The gradient pass.
class Reverse {
 public:
  Reverse(const Program& src, Builder& b, const std::vector<size_t>& wrt) : src_(src), b_(b) {
    now_.assign(src.ops.size(), 0);
    active_.assign(src.ops.size(), false);
    ct_.assign(src.ops.size(), std::nullopt);
    for (const Operation& op : src.ops) {
      now_[op.id] = replayUnchanged(b, op, now_);
      if (op.kind == Kind::parameter) {
        active_[op.id] = std::find(wrt.begin(), wrt.end(), op.index) != wrt.end();
      } else if (op.kind != Kind::compare && op.kind != Kind::iota && op.kind != Kind::constant) {
        size_t first = op.kind == Kind::select ? 1 : 0;  // the predicate carries no derivative
        for (size_t i = first; i < op.operands.size(); ++i) active_[op.id] = active_[op.id] || active_[op.operands[i]];
      }
    }
  }

  uint32_t primal(uint32_t id) const { return now_[id]; }

  // Cotangent of source value `id` after `run`; zeros when nothing reached it.
  uint32_t cotangent(uint32_t id) {
    if (ct_[id]) return *ct_[id];
    return filled(b_, src_.typeOf(id), 0.0);
  }

  void run(uint32_t output) {
    ct_[output] = filled(b_, src_.typeOf(output), 1.0);
    for (size_t n = src_.ops.size(); n-- > 0;) {
      const Operation& op = src_.ops[n];
      if (!ct_[op.id] || !active_[op.id]) continue;
      pull(op, *ct_[op.id]);
    }
  }

 private:
  void give(uint32_t id, uint32_t value) {
    if (!active_[id]) return;
    ct_[id] = ct_[id] ? b_.binary(Binary::add, *ct_[id], value) : value;
  }
  bool wants(uint32_t id) const { return active_[id]; }
  uint32_t bin(Binary op, uint32_t l, uint32_t r) { return b_.binary(op, l, r); }
  uint32_t neg(uint32_t x) { return b_.unary(Unary::neg, x); }

  void pull(const Operation& op, uint32_t g) {
    switch (op.kind) {
      case Kind::unary: return pullUnary(op, g);
      case Kind::binary: return pullBinary(op, g);
      case Kind::select: {
        uint32_t pred = now_[op.operands[0]];
        if (wants(op.operands[1]) || wants(op.operands[2])) {
          uint32_t zeros = filled(b_, op.result, 0.0);
          if (wants(op.operands[1])) give(op.operands[1], b_.select(pred, g, zeros));
          if (wants(op.operands[2])) give(op.operands[2], b_.select(pred, zeros, g));
        }
        return;
      }
      case Kind::broadcast_in_dim: return pullBroadcast(op, g);
      case Kind::broadcast:
        if (src_.typeOf(op.operands[0]).rank() != 0) throw TensorError("UnsupportedDerivative");
        return give(op.operands[0], sumAll(g));
      case Kind::reshape: return give(op.operands[0], b_.reshapeTo(g, src_.typeOf(op.operands[0]).dims));
      case Kind::transpose: {
        std::vector<int64_t> inverse(op.ints.size());
        for (size_t i = 0; i < op.ints.size(); ++i) inverse[op.ints[i]] = static_cast<int64_t>(i);
        return give(op.operands[0], b_.transposeBy(g, inverse));
      }
      case Kind::reduce: return pullReduce(op, g);
      case Kind::dot_general: return pullDot(op, g);
      default: return;  // parameter, constant, iota, compare: nothing upstream
    }
  }

  void pullUnary(const Operation& op, uint32_t g) {
    const uint32_t xi = op.operands[0];
    if (!dtypeIsFloat(src_.typeOf(xi).dtype)) throw TensorError("UnsupportedDerivative");
    const uint32_t x = now_[xi], y = now_[op.id];
    const Type& ty = src_.typeOf(xi);
    switch (static_cast<Unary>(op.sub)) {
      case Unary::neg: return give(xi, neg(g));
      case Unary::exp: return give(xi, bin(Binary::mul, y, g));
      case Unary::log: return give(xi, bin(Binary::div, g, x));
      case Unary::sqrt: return give(xi, bin(Binary::div, g, bin(Binary::mul, filled(b_, ty, 2.0), y)));
      case Unary::tanh: {
        uint32_t one = filled(b_, ty, 1.0);
        return give(xi, bin(Binary::mul, g, bin(Binary::sub, one, bin(Binary::mul, y, y))));
      }
      case Unary::sin: return give(xi, bin(Binary::mul, g, b_.unary(Unary::cos, x)));
      case Unary::cos: return give(xi, neg(bin(Binary::mul, g, b_.unary(Unary::sin, x))));
      case Unary::abs: {
        uint32_t non_negative = b_.compare(Compare::ge, x, filled(b_, ty, 0.0));
        return give(xi, b_.select(non_negative, g, neg(g)));
      }
      case Unary::tan: {
        uint32_t c = b_.unary(Unary::cos, x);
        return give(xi, bin(Binary::div, g, bin(Binary::mul, c, c)));
      }
    }
  }

  void pullBinary(const Operation& op, uint32_t g) {
    const uint32_t li = op.operands[0], ri = op.operands[1];
    if (!dtypeIsFloat(src_.typeOf(li).dtype)) throw TensorError("UnsupportedDerivative");
    const uint32_t l = now_[li], r = now_[ri];
    switch (static_cast<Binary>(op.sub)) {
      case Binary::add:
        give(li, g);
        give(ri, g);
        return;
      case Binary::sub:
        give(li, g);
        if (wants(ri)) give(ri, neg(g));
        return;
      case Binary::mul:
        if (wants(li)) give(li, bin(Binary::mul, g, r));
        if (wants(ri)) give(ri, bin(Binary::mul, l, g));
        return;
      case Binary::div: {
        // d(l/r) = (dl*r - l*dr) / (r*r), transposed term by term
        uint32_t q = bin(Binary::div, g, bin(Binary::mul, r, r));
        if (wants(li)) give(li, bin(Binary::mul, q, r));
        if (wants(ri)) give(ri, neg(bin(Binary::mul, l, q)));
        return;
      }
      case Binary::max:
      case Binary::min: {
        // ties go to the left operand (mask l >= r for max, l <= r for min)
        Compare dir = static_cast<Binary>(op.sub) == Binary::max ? Compare::ge : Compare::le;
        uint32_t mask = b_.compare(dir, l, r);
        uint32_t zeros = filled(b_, op.result, 0.0);
        if (wants(li)) give(li, b_.select(mask, g, zeros));
        if (wants(ri)) give(ri, b_.select(mask, zeros, g));
        return;
      }
      case Binary::pow: {
        if (wants(li)) {
          uint32_t one = filled(b_, op.result, 1.0);
          uint32_t step_down = bin(Binary::pow, l, bin(Binary::sub, r, one));
          give(li, bin(Binary::mul, bin(Binary::mul, r, step_down), g));
        }
        if (wants(ri)) {
          uint32_t scale = bin(Binary::mul, bin(Binary::pow, l, r), b_.unary(Unary::log, l));
          give(ri, bin(Binary::mul, scale, g));
        }
        return;
      }
    }
  }

  // y = broadcast_in_dim(x): x's dim i sits at y's axis ints[i]; extent-1 dims may be stretched.
  void pullBroadcast(const Operation& op, uint32_t g) {
    const uint32_t xi = op.operands[0];
    if (!wants(xi)) return;
    const Type& in = src_.typeOf(xi);
    const Type& out = op.result;
    std::vector<int64_t> summed;
    for (size_t a = 0; a < out.rank(); ++a) {
      auto at = std::find(op.ints.begin(), op.ints.end(), static_cast<int64_t>(a));
      if (at == op.ints.end()) {
        summed.push_back(static_cast<int64_t>(a));
      } else if (in.dims[at - op.ints.begin()].extent == 1 && out.dims[a].extent != 1) {
        summed.push_back(static_cast<int64_t>(a));
      }
    }
    uint32_t v = g;
    if (!summed.empty()) v = b_.reduce(g, b_.fullFloat(Type{out.dtype, {}}, 0.0), Reducer::sum, summed);
    // axes of y that survive, ascending; bring them into x's order
    std::vector<int64_t> survivors = keptAxes(out.rank(), summed);
    std::vector<int64_t> order;
    bool identity = true;
    for (size_t i = 0; i < in.rank(); ++i) {
      auto at = std::find(survivors.begin(), survivors.end(), op.ints[i]);
      if (at == survivors.end()) continue;  // a stretched extent-1 dim, restored by the reshape below
      order.push_back(at - survivors.begin());
      identity = identity && order.back() == static_cast<int64_t>(order.size() - 1);
    }
    if (!identity) v = b_.transposeBy(v, order);
    give(xi, relabel(b_, v, in.dims));
  }

  void pullReduce(const Operation& op, uint32_t g) {
    const uint32_t xi = op.operands[0], ii = op.operands[1];
    const Type& in = src_.typeOf(xi);
    if (!dtypeIsFloat(in.dtype)) throw TensorError("UnsupportedDerivative");
    const std::vector<int64_t> kept = keptAxes(in.rank(), op.ints);
    const Reducer red = static_cast<Reducer>(op.sub);
    if (red == Reducer::sum) {
      if (wants(xi)) give(xi, kept.size() == in.rank() ? g : b_.broadcastTo(g, in.dims, kept));
      if (wants(ii)) give(ii, sumAll(g));
      return;
    }
    // max / min: every element equal to the result receives the cotangent; so does the init value
    const uint32_t y = now_[op.id];
    if (wants(xi)) {
      uint32_t expanded = b_.broadcastTo(y, in.dims, kept);
      uint32_t mask = b_.compare(Compare::eq, now_[xi], expanded);
      uint32_t spread = b_.broadcastTo(g, in.dims, kept);
      give(xi, b_.select(mask, spread, filled(b_, in, 0.0)));
    }
    if (wants(ii)) {
      uint32_t init_everywhere = op.result.rank() == 0 ? now_[ii] : b_.broadcastTo(now_[ii], op.result.dims, {});
      uint32_t mask = b_.compare(Compare::eq, y, init_everywhere);
      give(ii, sumAll(b_.select(mask, g, filled(b_, op.result, 0.0))));
    }
  }

  uint32_t sumAll(uint32_t v) {
    const Type& ty = b_.typeOf(v);
    if (ty.rank() == 0) return v;
    return b_.reduce(v, b_.fullFloat(Type{ty.dtype, {}}, 0.0), Reducer::sum, allAxes(ty.rank()));
  }

  // y[batch…, lhs free…, rhs free…] = Σ_contract lhs · rhs
  void pullDot(const Operation& op, uint32_t g) {
    const uint32_t li = op.operands[0], ri = op.operands[1];
    const Type &lt = src_.typeOf(li), &rt = src_.typeOf(ri);
    if (!dtypeIsFloat(lt.dtype)) throw TensorError("UnsupportedDerivative");
    const std::vector<int64_t>&lc = op.ints, &rc = op.rhs_contract, &lb = op.lhs_batch, &rb = op.rhs_batch;
    std::vector<int64_t> lf, rf;
    for (size_t a = 0; a < lt.rank(); ++a)
      if (!contains(lc, a) && !contains(lb, a)) lf.push_back(a);
    for (size_t a = 0; a < rt.rank(); ++a)
      if (!contains(rc, a) && !contains(rb, a)) rf.push_back(a);
    const int64_t nb = static_cast<int64_t>(lb.size());
    std::vector<int64_t> g_batch(nb), g_lfree(lf.size()), g_rfree(rf.size());
    for (int64_t i = 0; i < nb; ++i) g_batch[i] = i;
    for (size_t j = 0; j < lf.size(); ++j) g_lfree[j] = nb + static_cast<int64_t>(j);
    for (size_t j = 0; j < rf.size(); ++j) g_rfree[j] = nb + static_cast<int64_t>(lf.size() + j);

    if (wants(li)) {
      // dL/dlhs = Σ_{rhs free} g · rhs  →  [batch…, lhs free…, rhs contract axes ascending]
      uint32_t v = b_.dotGeneralOp(g, now_[ri], g_rfree, rf, g_batch, rb);
      std::vector<int64_t> source_axis;  // lhs axis held by each axis of v
      for (int64_t a : lb) source_axis.push_back(a);
      for (int64_t a : lf) source_axis.push_back(a);
      std::vector<int64_t> rc_sorted = rc;
      std::sort(rc_sorted.begin(), rc_sorted.end());
      for (int64_t r : rc_sorted) source_axis.push_back(lc[std::find(rc.begin(), rc.end(), r) - rc.begin()]);
      give(li, relabel(b_, toOrder(v, source_axis), lt.dims));
    }
    if (wants(ri)) {
      // dL/drhs = Σ_{lhs free} lhs · g  →  [batch…, lhs contract axes ascending, rhs free…]
      uint32_t v = b_.dotGeneralOp(now_[li], g, lf, g_lfree, lb, g_batch);
      std::vector<int64_t> source_axis;  // rhs axis held by each axis of v
      for (int64_t a : rb) source_axis.push_back(a);
      std::vector<int64_t> lc_sorted = lc;
      std::sort(lc_sorted.begin(), lc_sorted.end());
      for (int64_t l : lc_sorted) source_axis.push_back(rc[std::find(lc.begin(), lc.end(), l) - lc.begin()]);
      for (int64_t a : rf) source_axis.push_back(a);
      give(ri, relabel(b_, toOrder(v, source_axis), rt.dims));
    }
  }

  // v's axis p holds operand axis source_axis[p]; returns v with axes in operand order.
  uint32_t toOrder(uint32_t v, const std::vector<int64_t>& source_axis) {
    std::vector<int64_t> perm(source_axis.size());
    bool identity = true;
    for (size_t p = 0; p < source_axis.size(); ++p) {
      perm[source_axis[p]] = static_cast<int64_t>(p);
      identity = identity && source_axis[p] == static_cast<int64_t>(p);
    }
    return identity ? v : b_.transposeBy(v, perm);
  }

  const Program& src_;
  Builder& b_;
  std::vector<uint32_t> now_;
  std::vector<bool> active_;
  std::vector<std::optional<uint32_t>> ct_;
};

}  // namespace

Program gradProgram(const Program& src, const std::vector<size_t>& wrt, bool keep_value) {
  if (src.outputs.size() != 1 || src.typeOf(src.outputs[0]).rank() != 0)
    throw TensorError("GradientRequiresScalarOutput");
  for (size_t i = 0; i < wrt.size(); ++i) {
    if (wrt[i] >= src.parameters.size()) throw TensorError("ParameterOutOfRange");
    for (size_t j = 0; j < i; ++j)
      if (wrt[j] == wrt[i]) throw TensorError("DuplicateParameter");
    if (!dtypeIsFloat(src.typeOf(src.parameters[wrt[i]]).dtype)) throw TensorError("NonDifferentiableParameter");
  }
  if (!dtypeIsFloat(src.typeOf(src.outputs[0]).dtype)) throw TensorError("UnsupportedDerivative");
  Builder b(src.name);
  Reverse pass(src, b, wrt);
  pass.run(src.outputs[0]);
  std::vector<uint32_t> outputs;
  if (keep_value) outputs.push_back(pass.primal(src.outputs[0]));
  for (size_t index : wrt) {
    // parameters[] is in parameter-index order
    outputs.push_back(pass.cotangent(src.parameters[index]));
  }
  return b.finish(outputs);
}

// ---------------------------------------------------------------------------------------------
// jvp: forward mode (src/tensor/autodiff.zig:86-742)
// ---------------------------------------------------------------------------------------------
namespace {

// Tangents are carried beside the primal values; a value nothing differentiable reaches has none
// (the reference records explicit zeros and prunes "structural zeros", autodiff.zig:346-352).
class Forward {
 public:
  Forward(const Program& src, Builder& b, const std::vector<size_t>& wrt) : src_(src), b_(b) {
    now_.assign(src.ops.size(), 0);
    tan_.assign(src.ops.size(), std::nullopt);
    // all primal parameters first, then one tangent parameter per differentiated parameter, in
    // parameter order (autodiff.zig:178-203)
    for (uint32_t id : src.parameters) now_[id] = replayUnchanged(b, src.ops[id], now_);
    for (uint32_t id : src.parameters) {
      const Operation& op = src.ops[id];
      if (std::find(wrt.begin(), wrt.end(), op.index) == wrt.end()) continue;
      tan_[id] = b.input(op.result.dtype, op.result.dims, /*authored=*/false);
    }
    for (const Operation& op : src.ops) {
      if (op.kind == Kind::parameter) continue;
      now_[op.id] = replayUnchanged(b, op, now_);
      push(op);
    }
  }

  uint32_t primal(uint32_t id) const { return now_[id]; }
  uint32_t tangent(uint32_t id) { return tan_[id] ? *tan_[id] : zerosOf(b_, src_.typeOf(id)); }

 private:
  using Opt = std::optional<uint32_t>;
  uint32_t bin(Binary op, uint32_t l, uint32_t r) { return b_.binary(op, l, r); }
  uint32_t neg(uint32_t x) { return b_.unary(Unary::neg, x); }
  uint32_t zerosLike(uint32_t id) { return filled(b_, src_.typeOf(id), 0.0); }
  static void needFloat(const Type& t) {
    if (!dtypeIsFloat(t.dtype)) throw TensorError("UnsupportedDerivative");
  }

  void push(const Operation& op) {
    auto t = [&](size_t i) -> Opt { return tan_[op.operands[i]]; };
    auto x = [&](size_t i) { return now_[op.operands[i]]; };
    const uint32_t y = now_[op.id];
    switch (op.kind) {
      case Kind::unary: {
        if (!t(0)) return;
        needFloat(src_.typeOf(op.operands[0]));
        const Type& ty = src_.typeOf(op.operands[0]);
        const uint32_t d = *t(0);
        switch (static_cast<Unary>(op.sub)) {
          case Unary::neg: tan_[op.id] = neg(d); return;
          case Unary::exp: tan_[op.id] = bin(Binary::mul, y, d); return;
          case Unary::log: tan_[op.id] = bin(Binary::div, d, x(0)); return;
          case Unary::sqrt: tan_[op.id] = bin(Binary::div, d, bin(Binary::mul, filled(b_, ty, 2.0), y)); return;
          case Unary::tanh:
            tan_[op.id] = bin(Binary::mul, d, bin(Binary::sub, filled(b_, ty, 1.0), bin(Binary::mul, y, y)));
            return;
          case Unary::sin: tan_[op.id] = bin(Binary::mul, d, b_.unary(Unary::cos, x(0))); return;
          case Unary::cos: tan_[op.id] = neg(bin(Binary::mul, d, b_.unary(Unary::sin, x(0)))); return;
          case Unary::abs:
            tan_[op.id] = b_.select(b_.compare(Compare::ge, x(0), filled(b_, ty, 0.0)), d, neg(d));
            return;
          case Unary::tan: {
            uint32_t c = b_.unary(Unary::cos, x(0));
            tan_[op.id] = bin(Binary::div, d, bin(Binary::mul, c, c));
            return;
          }
        }
        return;
      }
      case Kind::binary: {
        const Opt tl = t(0), tr = t(1);
        if (!tl && !tr) return;
        needFloat(src_.typeOf(op.operands[0]));
        const uint32_t l = x(0), r = x(1);
        switch (static_cast<Binary>(op.sub)) {
          case Binary::add: tan_[op.id] = tl && tr ? bin(Binary::add, *tl, *tr) : (tl ? *tl : tr.value()); return;
          case Binary::sub: tan_[op.id] = tl && tr ? bin(Binary::sub, *tl, *tr) : (tl ? *tl : neg(tr.value())); return;
          case Binary::mul: {
            Opt a = tl ? Opt(bin(Binary::mul, *tl, r)) : std::nullopt;
            Opt c = tr ? Opt(bin(Binary::mul, l, *tr)) : std::nullopt;
            tan_[op.id] = a && c ? bin(Binary::add, *a, *c) : (a ? *a : c.value());
            return;
          }
          case Binary::div: {
            Opt a = tl ? Opt(bin(Binary::mul, *tl, r)) : std::nullopt;
            Opt c = tr ? Opt(bin(Binary::mul, l, *tr)) : std::nullopt;
            uint32_t numerator = a && c ? bin(Binary::sub, *a, *c) : (a ? *a : neg(c.value()));
            tan_[op.id] = bin(Binary::div, numerator, bin(Binary::mul, r, r));
            return;
          }
          case Binary::max:
          case Binary::min: {
            Compare dir = static_cast<Binary>(op.sub) == Binary::max ? Compare::ge : Compare::le;
            uint32_t zeros = filled(b_, op.result, 0.0);
            tan_[op.id] = b_.select(b_.compare(dir, l, r), tl ? *tl : zeros, tr ? *tr : zeros);
            return;
          }
          case Binary::pow: {
            Opt base, exponent;
            if (tl) {
              uint32_t step_down = bin(Binary::pow, l, bin(Binary::sub, r, filled(b_, op.result, 1.0)));
              base = bin(Binary::mul, bin(Binary::mul, r, step_down), *tl);
            }
            if (tr) exponent = bin(Binary::mul, bin(Binary::mul, bin(Binary::pow, l, r), b_.unary(Unary::log, l)), *tr);
            tan_[op.id] = base && exponent ? bin(Binary::add, *base, *exponent) : (base ? *base : exponent.value());
            return;
          }
        }
        return;
      }
      case Kind::select: {
        const Opt tt = t(1), tf = t(2);
        if (!tt && !tf) return;
        uint32_t zeros = filled(b_, op.result, 0.0);
        tan_[op.id] = b_.select(x(0), tt ? *tt : zeros, tf ? *tf : zeros);
        return;
      }
      case Kind::broadcast_in_dim:
        if (t(0)) tan_[op.id] = b_.broadcastTo(*t(0), op.result.dims, op.ints);
        return;
      case Kind::broadcast:
        if (t(0)) tan_[op.id] = b_.broadcastOp(*t(0), op.result.dims);
        return;
      case Kind::reshape:
        if (t(0)) tan_[op.id] = b_.reshapeTo(*t(0), op.result.dims);
        return;
      case Kind::transpose:
        if (t(0)) tan_[op.id] = b_.transposeBy(*t(0), op.ints);
        return;
      case Kind::reduce: {
        const Opt tx = t(0), ti = t(1);
        if (!tx && !ti) return;
        const Type& in = src_.typeOf(op.operands[0]);
        needFloat(in);
        const Reducer red = static_cast<Reducer>(op.sub);
        const uint32_t zero = b_.fullFloat(Type{in.dtype, {}}, 0.0);
        if (red == Reducer::sum) {
          tan_[op.id] = b_.reduce(tx ? *tx : zerosLike(op.operands[0]), ti ? *ti : zero, Reducer::sum, op.ints);
          return;
        }
        const std::vector<int64_t> kept = keptAxes(in.rank(), op.ints);
        Opt from_input, from_init;
        if (tx) {
          uint32_t mask = b_.compare(Compare::eq, x(0), b_.broadcastTo(y, in.dims, kept));
          from_input = b_.reduce(b_.select(mask, *tx, zerosLike(op.operands[0])), zero, Reducer::sum, op.ints);
        }
        if (ti) {
          auto everywhere = [&](uint32_t v) { return op.result.rank() == 0 ? v : b_.broadcastTo(v, op.result.dims, {}); };
          uint32_t mask = b_.compare(Compare::eq, y, everywhere(x(1)));
          from_init = b_.select(mask, everywhere(*ti), filled(b_, op.result, 0.0));
        }
        tan_[op.id] = from_input && from_init ? bin(Binary::add, *from_input, *from_init) : (from_input ? *from_input : from_init.value());
        return;
      }
      case Kind::dot_general: {
        const Opt tl = t(0), tr = t(1);
        if (!tl && !tr) return;
        needFloat(src_.typeOf(op.operands[0]));
        Opt left = tl ? Opt(b_.dotGeneralOp(*tl, x(1), op.ints, op.rhs_contract, op.lhs_batch, op.rhs_batch)) : std::nullopt;
        Opt right = tr ? Opt(b_.dotGeneralOp(x(0), *tr, op.ints, op.rhs_contract, op.lhs_batch, op.rhs_batch)) : std::nullopt;
        tan_[op.id] = left && right ? bin(Binary::add, *left, *right) : (left ? *left : right.value());
        return;
      }
      default: return;  // constant, iota, compare: no tangent
    }
  }

  const Program& src_;
  Builder& b_;
  std::vector<uint32_t> now_;
  std::vector<Opt> tan_;
};

}  // namespace

Program jvpProgram(const Program& src, const std::vector<size_t>& wrt) {
  for (size_t i = 0; i < wrt.size(); ++i) {
    if (wrt[i] >= src.parameters.size()) throw TensorError("ParameterOutOfRange");
    for (size_t j = 0; j < i; ++j)
      if (wrt[j] == wrt[i]) throw TensorError("DuplicateParameter");
    if (!dtypeIsFloat(src.typeOf(src.parameters[wrt[i]]).dtype)) throw TensorError("NonDifferentiableParameter");
  }
  Builder b(src.name);
  Forward pass(src, b, wrt);
  std::vector<uint32_t> outputs;
  for (uint32_t id : src.outputs) outputs.push_back(pass.primal(id));
  for (uint32_t id : src.outputs) outputs.push_back(pass.tangent(id));  // zeros where nothing differentiable arrives
  return b.finish(outputs);
}

// ---------------------------------------------------------------------------------------------
// vmap
// ---------------------------------------------------------------------------------------------
namespace {

struct Batched {
  uint32_t id = 0;
  bool mapped = false;  // when set, axis 0 of the value is the new axis
};

class Vmap {
 public:
  Vmap(const Program& src, Builder& b, Dim batch, const std::vector<int64_t>& in_axes)
      : src_(src), b_(b), batch_(std::move(batch)), in_axes_(in_axes) {}

  Program run(size_t out_axis) {
    std::vector<Batched> now(src_.ops.size());
    plain_.assign(src_.ops.size(), 0);
    for (const Operation& op : src_.ops) {
      now[op.id] = step(op, now);
      plain_[op.id] = now[op.id].id;
    }
    std::vector<uint32_t> outputs;
    for (uint32_t id : src_.outputs) {
      const Type& ty = src_.typeOf(id);
      if (out_axis > ty.rank()) throw TensorError("AxisOutOfRange");
      std::vector<Dim> dims = ty.dims;
      dims.insert(dims.begin() + static_cast<long>(out_axis), batch_);
      if (now[id].mapped) {
        // move axis 0 to out_axis
        std::vector<int64_t> perm;
        for (size_t a = 0; a < dims.size(); ++a) {
          if (a == out_axis) perm.push_back(0);
          else perm.push_back(static_cast<int64_t>(a < out_axis ? a + 1 : a));
        }
        outputs.push_back(out_axis == 0 ? now[id].id : b_.transposeBy(now[id].id, perm));
      } else {
        std::vector<int64_t> mapping;
        for (size_t a = 0; a < ty.rank(); ++a) mapping.push_back(static_cast<int64_t>(a < out_axis ? a : a + 1));
        outputs.push_back(b_.broadcastTo(now[id].id, dims, mapping));
      }
    }
    return b_.finish(outputs);
  }

 private:
  std::vector<Dim> withBatch(const std::vector<Dim>& dims) const {
    std::vector<Dim> out{batch_};
    out.insert(out.end(), dims.begin(), dims.end());
    return out;
  }
  static std::vector<int64_t> shifted(const std::vector<int64_t>& axes) {
    std::vector<int64_t> out;
    for (int64_t a : axes) out.push_back(a + 1);
    return out;
  }
  // The value with the new axis in front, stretched along it when it did not depend on it.
  uint32_t lifted(const Batched& v) {
    if (v.mapped) return v.id;
    const Type& ty = b_.typeOf(v.id);
    return b_.broadcastTo(v.id, withBatch(ty.dims), shifted(allAxes(ty.rank())));
  }

  Batched step(const Operation& op, const std::vector<Batched>& now) {
    auto arg = [&](size_t i) -> const Batched& { return now[op.operands[i]]; };
    bool any = false;
    for (uint32_t id : op.operands) any = any || now[id].mapped;
    if (op.kind == Kind::parameter) return parameter(op);
    if (!any) return {replayUnchanged(b_, op, plain_), false};
    switch (op.kind) {
      case Kind::unary: return {b_.unary(static_cast<Unary>(op.sub), arg(0).id), true};
      case Kind::binary: return {b_.binary(static_cast<Binary>(op.sub), lifted(arg(0)), lifted(arg(1))), true};
      case Kind::compare: return {b_.compare(static_cast<Compare>(op.sub), lifted(arg(0)), lifted(arg(1))), true};
      case Kind::select: {
        uint32_t pred = arg(0).id;
        const bool scalar_pred = src_.typeOf(op.operands[0]).rank() == 0;
        if (arg(0).mapped && scalar_pred && op.result.rank() != 0) {
          pred = b_.broadcastTo(pred, withBatch(op.result.dims), {0});
        } else if (!arg(0).mapped && !scalar_pred) {
          pred = lifted(arg(0));
        }
        return {b_.select(pred, lifted(arg(1)), lifted(arg(2))), true};
      }
      case Kind::broadcast_in_dim: {
        std::vector<int64_t> mapping{0};
        for (int64_t a : op.ints) mapping.push_back(a + 1);
        return {b_.broadcastTo(arg(0).id, withBatch(op.result.dims), mapping), true};
      }
      case Kind::broadcast:
        // only a rank-0 operand can carry the new axis (batch.zig:698-722)
        if (src_.typeOf(op.operands[0]).rank() != 0) throw TensorError("UnsupportedBatching");
        return {b_.broadcastTo(arg(0).id, withBatch(op.result.dims), {0}), true};
      case Kind::reshape: return {b_.reshapeTo(arg(0).id, withBatch(op.result.dims)), true};
      case Kind::transpose: {
        std::vector<int64_t> perm{0};
        for (int64_t a : op.ints) perm.push_back(a + 1);
        return {b_.transposeBy(arg(0).id, perm), true};
      }
      case Kind::reduce: {
        if (arg(1).mapped) throw TensorError("BatchedReduceInitUnsupported");
        return {b_.reduce(arg(0).id, arg(1).id, static_cast<Reducer>(op.sub), shifted(op.ints)), true};
      }
      case Kind::dot_general: return dot(op, arg(0), arg(1));
      case Kind::custom_call: throw TensorError("CustomCallRequiresBatchContract");
      default: throw TensorError("OperationUnsupported");
    }
  }

  Batched parameter(const Operation& op) {
    const int64_t axis = in_axes_[op.index];
    if (axis < 0) return {b_.input(op.result.dtype, op.result.dims, /*authored=*/false), false};
    std::vector<Dim> dims = op.result.dims;
    dims.insert(dims.begin() + axis, batch_);
    uint32_t id = b_.input(op.result.dtype, dims, /*authored=*/false);
    if (axis != 0) {
      std::vector<int64_t> perm{axis};
      for (size_t a = 0; a < dims.size(); ++a)
        if (static_cast<int64_t>(a) != axis) perm.push_back(static_cast<int64_t>(a));
      id = b_.transposeBy(id, perm);
    }
    return {id, true};
  }

  Batched dot(const Operation& op, const Batched& l, const Batched& r) {
    if (l.mapped && r.mapped) {
      std::vector<int64_t> lb{0}, rb{0};
      for (int64_t a : op.lhs_batch) lb.push_back(a + 1);
      for (int64_t a : op.rhs_batch) rb.push_back(a + 1);
      return {b_.dotGeneralOp(l.id, r.id, shifted(op.ints), shifted(op.rhs_contract), lb, rb), true};
    }
    const size_t nb = op.lhs_batch.size();
    if (l.mapped) {
      // the new axis is the first free axis of lhs: it lands right after the batch axes
      uint32_t v = b_.dotGeneralOp(l.id, r.id, shifted(op.ints), op.rhs_contract, shifted(op.lhs_batch), op.rhs_batch);
      return {frontAxis(v, nb), true};
    }
    // the new axis is the first free axis of rhs: it lands after batch and lhs free axes
    const size_t lhs_free = src_.typeOf(op.operands[0]).rank() - nb - op.ints.size();
    uint32_t v = b_.dotGeneralOp(l.id, r.id, op.ints, shifted(op.rhs_contract), op.lhs_batch, shifted(op.rhs_batch));
    return {frontAxis(v, nb + lhs_free), true};
  }

  uint32_t frontAxis(uint32_t v, size_t from) {
    if (from == 0) return v;
    std::vector<int64_t> perm{static_cast<int64_t>(from)};
    for (size_t a = 0; a < b_.typeOf(v).rank(); ++a)
      if (a != from) perm.push_back(static_cast<int64_t>(a));
    return b_.transposeBy(v, perm);
  }

  const Program& src_;
  Builder& b_;
  Dim batch_;
  const std::vector<int64_t>& in_axes_;
  std::vector<uint32_t> plain_;  // new-program id of every source value, mapped or not
};

bool programHasAxis(const Program& p, const std::string& name) {
  for (const Operation& op : p.ops)
    if (findDim(op.result.dims, name) >= 0) return true;
  return false;
}

}  // namespace

Program vmapProgram(const Program& src, int64_t axis_size, const std::vector<int64_t>& in_axes, size_t out_axis,
                    const std::string& axis_name) {
  if (axis_size < 0) throw TensorError("InvalidDimension");
  if (in_axes.size() != src.parameters.size()) throw TensorError("InAxisCountMismatch");
  for (uint32_t id : src.parameters) {
    const Operation& op = src.ops[id];
    int64_t axis = in_axes[op.index];
    if (axis >= 0 && static_cast<size_t>(axis) > op.result.rank()) throw TensorError("AxisOutOfRange");
  }
  std::string name = axis_name;
  if (name.empty()) {
    name = "#batch";
    for (size_t attempt = 1; programHasAxis(src, name); ++attempt) name = "#batch" + std::to_string(attempt);
  } else {
    validateAuthoredName(name);
    if (programHasAxis(src, name)) throw TensorError("DuplicateAxis");
  }
  Builder b(src.name);
  Vmap pass(src, b, Dim{name, axis_size}, in_axes);
  return pass.run(out_axis);
}

}  // namespace accy
