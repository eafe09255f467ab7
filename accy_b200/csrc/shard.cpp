// Sharding a recorded program along a named batch-like axis.
//
// The reference runs on one device only (no collective anywhere in src/ or
// deps/lib/compiler/gpu); this is the host logic that lets one recorded program run as
// independent pieces: the same operation list re-recorded with a smaller extent for one axis.
// It is used twice: by multi-GPU runs (one rank per GPU, each rank owns a contiguous block of
// the axis) and by the host-buffer `invoke`, which streams large programs through the GPU in
// chunks so that host->device copies, kernels and device->host copies overlap.
//
// An axis can be sharded with no exchange between the pieces when no operation mixes values
// across it: it is never reduced, contracted or indexed by an iota, and every input and output
// that carries it has it as its outermost dim (so a piece is one contiguous byte range).
// When the only operation that mixes across the axis is a final sum (the output itself is
// reduce(sum) over it), the pieces produce partial sums that the caller adds up
// (`partial_sum`: one all-reduce of the per-shard outputs).
#include <algorithm>
#include <cstring>

#include "plan.hpp"

namespace accy {

namespace {

bool hasAxis(const Type& t, const std::string& axis) { return findDim(t.dims, axis) >= 0; }

std::vector<Dim> resized(const std::vector<Dim>& dims, const std::string& axis, int64_t extent) {
  std::vector<Dim> out = dims;
  for (Dim& d : out)
    if (d.name == axis) d.extent = extent;
  return out;
}

}  // namespace

ShardInfo analyseShardAxis(const Program& p, const std::string& axis) {
  ShardInfo info;
  info.axis = axis;
  std::vector<bool> is_output(p.ops.size(), false);
  for (uint32_t id : p.outputs) is_output[id] = true;
  bool carried = false;
  for (const Operation& op : p.ops) {
    if (hasAxis(op.result, axis)) carried = true;
    long at = findDim(op.result.dims, axis);
    if (at >= 0) {
      if (info.extent < 0) info.extent = op.result.dims[at].extent;
      else if (info.extent != op.result.dims[at].extent) {
        info.reason = "axis '" + axis + "' has different extents in one program";
        return info;
      }
    }
    switch (op.kind) {
      case Kind::parameter:
        if (at > 0) { info.reason = "an input carries the axis but not as its outermost dim"; return info; }
        break;
      case Kind::constant: {
        if (at < 0) break;
        size_t es = dtypeSize(op.result.dtype);
        for (size_t i = es; i < op.payload.size(); i += es)
          if (std::memcmp(&op.payload[i], &op.payload[0], es) != 0) {
            info.reason = "a non-uniform constant carries the axis";
            return info;
          }
        break;
      }
      case Kind::iota:
        if (at >= 0 && op.axis == at) { info.reason = "an iota counts along the axis"; return info; }
        break;
      case Kind::reduce: {
        const Type& in = p.typeOf(op.operands[0]);
        for (int64_t d : op.ints)
          if (in.dims[d].name == axis) {
            // allowed only as the program's final fold: the pieces' results combine with the
            // same reducer (sum: one all-reduce that adds; max / min: one that takes the extreme)
            const uint32_t fold = 1u + static_cast<uint32_t>(op.sub);
            if (static_cast<Reducer>(op.sub) == Reducer::sum) {
              // every piece folds the recorded initial value again and the all-reduce adds the
              // pieces, so a sum may be cut only when it starts from zero (a max or min may start
              // anywhere: taking the same value in twice changes nothing)
              const Operation& init = p.ops[op.operands[1]];
              bool zero = init.kind == Kind::constant;
              for (uint8_t byte : init.payload) zero = zero && byte == 0;
              if (!zero) {
                info.reason = "the axis is summed from a non-zero initial value, which every piece would add again";
                return info;
              }
            }
            if (is_output[op.id] && (info.partial_fold == 0 || info.partial_fold == fold)) {
              info.partial_fold = fold;
              info.partial_outputs.push_back(op.id);
            } else if (is_output[op.id]) {
              info.reason = "outputs fold the axis with different reducers";
              return info;
            } else {
              info.reason = "the axis is reduced inside the program";
              return info;
            }
          }
        break;
      }
      case Kind::dot_general: {
        const Type& lhs = p.typeOf(op.operands[0]);
        for (int64_t d : op.ints)
          if (lhs.dims[d].name == axis) { info.reason = "the axis is contracted"; return info; }
        break;
      }
      case Kind::reshape: {
        const Type& in = p.typeOf(op.operands[0]);
        long in_at = findDim(in.dims, axis);
        if (in_at < 0 && at < 0) break;
        // the axis must pass through untouched as the outermost dim, the rest must keep its size
        if (in_at != 0 || at != 0) { info.reason = "a reshape moves or merges the axis"; return info; }
        break;
      }
      case Kind::unary: case Kind::binary: case Kind::compare: case Kind::select:
      case Kind::broadcast_in_dim: case Kind::broadcast: case Kind::transpose:
        break;
      default:
        info.reason = std::string("operation kind not shardable: ") + kindName(op.kind);
        return info;
    }
  }
  if (!carried) { info.reason = "no value carries axis '" + axis + "'"; return info; }
  // values computed from a partial sum would need the complete sum: only outputs may be partial
  for (uint32_t part : info.partial_outputs)
    for (const Operation& op : p.ops)
      for (uint32_t a : op.operands)
        if (a == part) { info.reason = "a partial fold over the axis is used inside the program"; return info; }
  for (uint32_t id : p.outputs) {
    const Type& t = p.typeOf(id);
    long at = findDim(t.dims, axis);
    bool partial = std::find(info.partial_outputs.begin(), info.partial_outputs.end(), id) != info.partial_outputs.end();
    if (partial) continue;
    if (at != 0) {
      info.reason = at < 0 ? "an output does not carry the axis" : "an output carries the axis but not as its outermost dim";
      return info;
    }
  }
  info.shardable = true;
  info.partial_sum = !info.partial_outputs.empty();
  if (info.partial_sum && info.partial_outputs.size() != p.outputs.size()) {
    info.shardable = false;
    info.reason = "only some outputs are folds over the axis";
  }
  return info;
}

Program shardProgram(const Program& p, const std::string& axis, int64_t extent) {
  ShardInfo info = analyseShardAxis(p, axis);
  if (!info.shardable) throw PlanError("axis '" + axis + "' cannot be sharded: " + info.reason);
  if (extent <= 0 || extent > info.extent) throw PlanError("shard extent out of range");
  Builder b(p.name);
  for (const Operation& op : p.ops) {
    uint32_t made = 0;
    std::vector<Dim> dims = resized(op.result.dims, axis, extent);
    switch (op.kind) {
      case Kind::parameter:
        made = b.input(op.result.dtype, dims, /*authored=*/false);
        break;
      case Kind::constant: {
        Type t{op.result.dtype, dims};
        size_t es = dtypeSize(t.dtype), n = t.elementCount();
        std::vector<uint8_t> payload(n * es);
        if (hasAxis(op.result, axis)) {
          for (size_t i = 0; i < n; ++i) std::memcpy(&payload[i * es], op.payload.data(), es);
        } else {
          payload = op.payload;
        }
        made = b.constantBytes(t, payload.data(), payload.size());
        break;
      }
      case Kind::iota: made = b.iotaTyped(Type{op.result.dtype, dims}, op.axis); break;
      case Kind::unary: made = b.unary(static_cast<Unary>(op.sub), op.operands[0]); break;
      case Kind::binary: made = b.binary(static_cast<Binary>(op.sub), op.operands[0], op.operands[1]); break;
      case Kind::compare: made = b.compare(static_cast<Compare>(op.sub), op.operands[0], op.operands[1]); break;
      case Kind::select: made = b.select(op.operands[0], op.operands[1], op.operands[2]); break;
      case Kind::broadcast_in_dim: made = b.broadcastTo(op.operands[0], dims, op.ints); break;
      case Kind::broadcast: made = b.broadcastOp(op.operands[0], dims); break;
      case Kind::reshape: made = b.reshapeTo(op.operands[0], dims); break;
      case Kind::transpose: made = b.transposeBy(op.operands[0], op.ints); break;
      case Kind::reduce: made = b.reduce(op.operands[0], op.operands[1], static_cast<Reducer>(op.sub), op.ints); break;
      case Kind::dot_general:
        made = b.dotGeneralOp(op.operands[0], op.operands[1], op.ints, op.rhs_contract, op.lhs_batch, op.rhs_batch);
        break;
      default:
        throw PlanError("operation kind not shardable");
    }
    if (made != op.id) throw PlanError("internal: shard replay lost op numbering");
  }
  return b.finish(p.outputs);
}

}  // namespace accy
