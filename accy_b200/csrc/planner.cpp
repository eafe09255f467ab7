// Fusion planner: decides which recorded operations share a kernel.
//
// The planner works backwards from the program outputs (latest value first).  For each value
// that has to exist in device memory it builds the largest fused region that can produce it:
//   1. dot -> scale -> [causal mask] -> softmax -> dot   => one attention kernel
//      (the reference's flash matcher, src/preparation/fusion/pass.zig:729-905, here also for
//      causal masks built from iota/compare/select, leading batch axes and bf16);
//   2. dot_general + the elementwise ops only it feeds   => GEMM with epilogue
//      (fusion/pass.zig:1585-1699; the reference's 6-op single-use chain limit is lifted so a
//      tanh-GELU, which uses its input four times, still fuses);
//   3. everything elementwise plus the reductions over one set of axes => one row kernel
//      (reduction_input cluster, fusion/pass.zig:1498-1538, and row pipeline, :907-1265, without
//      the op-count, column and scalar-broadcast limits described there).
// Views (broadcast_in_dim, transpose, same-extent reshape), iota, scalar constants and masks are
// seen through: they become index arithmetic of the consuming kernel
// (src/preparation/schedule/pass.zig:893-918).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <set>
#include <sstream>

#include "plan.hpp"

namespace accy {
namespace {

bool isElementwise(Kind k) {
  return k == Kind::unary || k == Kind::binary || k == Kind::compare || k == Kind::select;
}

std::vector<int64_t> rowMajorStrides(const std::vector<Dim>& dims) {
  std::vector<int64_t> s(dims.size(), 1);
  for (long i = static_cast<long>(dims.size()) - 2; i >= 0; --i) s[i] = s[i + 1] * dims[i + 1].extent;
  return s;
}

struct Abort {};  // thrown to leave a trial build without side effects

class Planner {
 public:
  Planner(const Program& p, const ScheduleOverrides& o) : P(p), ov(o) {
    slot_of.assign(P.ops.size(), -1);
    users.resize(P.ops.size());
    for (const Operation& op : P.ops)
      for (uint32_t a : op.operands) users[a].push_back(op.id);
    is_output.assign(P.ops.size(), false);
    for (uint32_t id : P.outputs) is_output[id] = true;
    // Value numbering: an operation that repeats an earlier one (same kind, attributes, result type and
    // the same operands up to this relation) stands for it.  Inside a fused region repeated
    // subexpressions already collapse node by node; this is for values that become kernels of their
    // own, so that x.max(r) written out twice is one fold, not two.
    same_as.resize(P.ops.size());
    std::map<std::string, uint32_t> seen;
    for (const Operation& op : P.ops) {
      same_as[op.id] = op.id;
      if (op.kind == Kind::parameter) continue;
      std::string key;
      auto put = [&](int64_t x) { key.append(reinterpret_cast<const char*>(&x), sizeof(x)); };
      put(static_cast<int64_t>(op.kind)); put(op.sub); put(static_cast<int64_t>(op.result.dtype)); put(static_cast<int64_t>(op.result.rank()));
      for (const Dim& d : op.result.dims) { key += d.name; key.push_back('\0'); put(d.extent); }
      put(static_cast<int64_t>(op.operands.size()));
      for (uint32_t a : op.operands) put(same_as[a]);
      for (const std::vector<int64_t>* list : {&op.ints, &op.rhs_contract, &op.lhs_batch, &op.rhs_batch}) {
        put(static_cast<int64_t>(list->size()));
        for (int64_t x : *list) put(x);
      }
      put(op.axis); put(static_cast<int64_t>(op.index)); put(op.version);
      key += op.target; key.push_back('\0');
      key.append(reinterpret_cast<const char*>(op.payload.data()), op.payload.size());
      auto found = seen.emplace(key, op.id);
      if (!found.second) same_as[op.id] = found.first->second;
    }
  }
  std::vector<uint32_t> same_as;   // the earliest operation computing the same value
  // Values (by their same_as representative) that a first, discarded planning pass gave a region of
  // their own although they are not outputs: row statistics that a fold over another axis reads, for
  // instance.  In the second pass a region that computes such a value on its way writes it out as well,
  // so that it is not computed again from the inputs.
  std::set<uint32_t> wanted;
  std::set<uint32_t> standalone;

  Plan run() {
    plan.input_slots.resize(P.parameters.size());
    for (size_t i = 0; i < P.parameters.size(); ++i) {
      Slot s;
      s.role = Slot::Input;
      s.io_index = static_cast<int>(i);
      s.bytes = P.typeOf(P.parameters[i]).byteCount();
      s.storage = P.typeOf(P.parameters[i]).dtype;
      s.value = P.parameters[i];
      plan.slots.push_back(s);
      slot_of[P.parameters[i]] = static_cast<int>(plan.slots.size()) - 1;
      plan.input_slots[i] = slot_of[P.parameters[i]];
      plan.work.bytes += static_cast<double>(s.bytes);
    }
    // every program output gets its own slot, even when two outputs name one value
    plan.output_slots.assign(P.outputs.size(), -1);
    std::map<uint32_t, int> first_output;
    for (size_t j = 0; j < P.outputs.size(); ++j) {
      Slot s;
      s.role = Slot::Output;
      s.io_index = static_cast<int>(j);
      s.bytes = P.typeOf(P.outputs[j]).byteCount();
      s.storage = P.typeOf(P.outputs[j]).dtype;
      s.value = P.outputs[j];
      plan.slots.push_back(s);
      plan.output_slots[j] = static_cast<int>(plan.slots.size()) - 1;
      plan.work.bytes += static_cast<double>(s.bytes);
      if (!first_output.count(P.outputs[j])) first_output[P.outputs[j]] = plan.output_slots[j];
    }
    out_slot_of = first_output;
    // the largest outputs first (a region that computes a large result passes the smaller values the
    // other outputs need on its way), later operations before earlier ones among equals
    std::vector<uint32_t> roots;
    for (auto& kv : first_output) roots.push_back(kv.first);
    std::sort(roots.begin(), roots.end(), [&](uint32_t a, uint32_t b) {
      const size_t na = P.typeOf(a).elementCount(), nb = P.typeOf(b).elementCount();
      return na != nb ? na > nb : a > b;
    });
    for (uint32_t v : roots) {
      if (produced.count(v)) continue;
      if (P.typeOf(v).elementCount() == 0) {   // nothing to compute
        produced.insert(v);
        continue;
      }
      planOutputRoot(v);
    }
    // duplicate outputs and outputs that are plain inputs/constants: device-side copies
    for (size_t j = 0; j < P.outputs.size(); ++j) {
      int want = plan.output_slots[j];
      int have = out_slot_of[P.outputs[j]];
      if (want != have && plan.slots[want].bytes) copies.push_back({have, want});
    }
    for (auto& c : copies) emitCopy(c.first, c.second);
    plan.summary = summary.str();
    return std::move(plan);
  }

 private:
  const Program& P;
  ScheduleOverrides ov;
  Plan plan;
  std::vector<int> slot_of;                 // value id -> slot holding it (materialised values)
  std::vector<std::vector<uint32_t>> users;
  std::vector<bool> is_output;
  std::map<uint32_t, int> out_slot_of;      // output value -> its first output slot
  std::set<uint32_t> produced;              // output values already written by a kernel
  std::vector<std::pair<int, int>> copies;
  std::ostringstream summary;
  int kernel_counter = 0;

  std::string nextName(const char* family) {
    std::ostringstream s;
    s << "accy_" << family << "_" << kernel_counter++;
    return s.str();
  }

  int newSlot(Slot::Role role, size_t bytes, uint32_t value, DType storage) {
    Slot s;
    s.role = role;
    s.bytes = bytes;
    s.storage = storage;
    s.value = value;
    plan.slots.push_back(s);
    return static_cast<int>(plan.slots.size()) - 1;
  }

  // slot a kernel should write value v into
  int destinationSlot(uint32_t v) {
    if (is_output[v]) return out_slot_of[v];
    const Type& ty = P.typeOf(v);
    // 16-bit-float temporaries stay in f32 between kernels unless a contraction reads them
    const bool widen = (ty.dtype == DType::bf16 || ty.dtype == DType::f16) && !narrow.count(v);
    if (widen) return newSlot(Slot::Temp, ty.elementCount() * 4, v, DType::f32);
    return newSlot(Slot::Temp, ty.byteCount(), v, ty.dtype);
  }
  std::set<uint32_t> narrow;  // values that must keep their 16-bit storage (contraction operands)

  void planOutputRoot(uint32_t v) {
    const Operation& op = P.ops[v];
    if (op.kind == Kind::parameter || slot_of[v] >= 0) {
      // an output that is just an input (or already materialised for another reason)
      int src = materialize(v);
      if (src != out_slot_of[v]) copies.push_back({src, out_slot_of[v]});
      produced.insert(v);
      return;
    }
    materialize(v);
  }

  // Ensures v lives in a device buffer laid out row-major in its own dims; returns the slot.
  int materialize(uint32_t v) {
    if (slot_of[v] >= 0) return slot_of[v];
    if (same_as[v] != v && !is_output[v] && narrow.count(v) == narrow.count(same_as[v])) {
      // the same value was (or is now) computed under an earlier name: read that buffer
      const int s = materialize(same_as[v]);
      slot_of[v] = s;
      return s;
    }
    const Operation& op = P.ops[v];
    switch (op.kind) {
      case Kind::constant: {
        int s = newSlot(Slot::Constant, op.payload.size(), v, op.result.dtype);
        plan.slots[s].payload = op.payload;
        slot_of[v] = s;
        if (is_output[v]) {
          copies.push_back({s, out_slot_of[v]});
          produced.insert(v);
        }
        return s;
      }
      case Kind::reshape: {
        // a reshape of a buffer is the same bytes under other dims
        if (!is_output[v]) {
          int s = materialize(op.operands[0]);
          slot_of[v] = s;
          return s;
        }
        break;
      }
      case Kind::dot_general:
        if (tryAttention(v)) return slot_of[v];
        planGemm(v, v);
        return slot_of[v];
      default:
        break;
    }
    if (isElementwise(op.kind) && tryGemmEpilogue(v)) return slot_of[v];
    planCluster(v);
    return slot_of[v];
  }

  // ---------------------------------------------------------------------------------------
  // expression DAG construction
  // ---------------------------------------------------------------------------------------
  struct Build {
    std::vector<std::string> dim_names;
    std::vector<int64_t> extents;
    std::vector<bool> is_col;
    bool cols_fixed = false;           // a reduction has fixed which dims are columns
    std::vector<ENode> nodes;
    std::vector<LeafRef> leaves;
    std::map<std::pair<uint32_t, std::vector<int>>, int> memo;
    std::vector<std::pair<uint32_t, int>> coproduce;   // (output value, node) candidates
    uint32_t root = 0;
    uint32_t sibling = 0xffffffffu;    // an output with the root's dims that is being added to the region
    bool trial = false;                // no side effects allowed; dots become accumulator leaves
    uint32_t acc_value = 0xffffffffu;  // trial mode: the dot value standing for the accumulator
    int acc_node = -1;
    std::set<uint32_t> closure;        // computed values inlined into this region
  };

  // Nodes are pure functions of their arguments: one that repeats an earlier node (the same
  // subexpression recorded twice, e.g. x.sub(x.max(c)) written out for two uses) is that node.
  int addNode(Build& b, const ENode& n) {
    if (n.op != ENode::Leaf) {
      for (size_t i = 0; i < b.nodes.size(); ++i) {
        const ENode& e = b.nodes[i];
        if (e.op == n.op && e.sub == n.sub && e.dtype == n.dtype && e.args[0] == n.args[0] && e.args[1] == n.args[1] &&
            e.args[2] == n.args[2] && e.bits == n.bits && e.dim == n.dim && e.vary == n.vary && e.level == n.level)
          return static_cast<int>(i);
      }
    }
    b.nodes.push_back(n);
    return static_cast<int>(b.nodes.size()) - 1;
  }

  int leafNode(Build& b, int slot, const Type& ty, const std::vector<int>& map) {
    LeafRef leaf;
    leaf.slot = slot;
    leaf.dtype = plan.slots[slot].storage;
    leaf.strides.assign(b.extents.size(), 0);
    std::vector<int64_t> rm = rowMajorStrides(ty.dims);
    for (size_t i = 0; i < ty.dims.size(); ++i) {
      if (map[i] < 0 || ty.dims[i].extent == 1) continue;
      leaf.strides[map[i]] += rm[i];
      leaf.vary |= 1u << map[i];
    }
    // leaves are deduplicated so one buffer read with one index map is loaded once
    int index = -1;
    for (size_t i = 0; i < b.leaves.size(); ++i) {
      if (b.leaves[i].slot == slot && b.leaves[i].strides.size() <= leaf.strides.size()) {
        bool same = true;
        for (size_t d = 0; d < leaf.strides.size(); ++d) {
          int64_t have = d < b.leaves[i].strides.size() ? b.leaves[i].strides[d] : 0;
          if (have != leaf.strides[d]) same = false;
        }
        if (same) index = static_cast<int>(i);
      }
    }
    if (index < 0) {
      b.leaves.push_back(leaf);
      index = static_cast<int>(b.leaves.size()) - 1;
    }
    ENode n;
    n.op = ENode::Leaf;
    n.dtype = ty.dtype;
    n.leaf = index;
    n.vary = leaf.vary;
    return addNode(b, n);
  }

  static bool splatConstant(const Operation& op, uint64_t* bits) {
    size_t es = dtypeSize(op.result.dtype);
    if (es == 0 || es > 8 || op.payload.size() < es) return false;
    for (size_t i = es; i < op.payload.size(); i += es)
      if (std::memcmp(&op.payload[i], &op.payload[0], es) != 0) return false;
    *bits = 0;
    std::memcpy(bits, op.payload.data(), es);
    return true;
  }

  int clusterDimFor(Build& b, const Dim& d, const std::vector<int>& taken) {
    for (size_t i = 0; i < b.extents.size(); ++i) {
      if (b.dim_names[i] != d.name || b.extents[i] != d.extent) continue;
      if (std::find(taken.begin(), taken.end(), static_cast<int>(i)) != taken.end()) continue;
      return static_cast<int>(i);
    }
    if (b.extents.size() >= 30) throw PlanError("fused region has more than 30 axes");
    b.dim_names.push_back(d.name);
    b.extents.push_back(d.extent);
    b.is_col.push_back(false);
    return static_cast<int>(b.extents.size()) - 1;
  }

  // Builds (or finds) the node for value v seen through `map`: v's dim i is cluster dim map[i],
  // or -1 when that dim is a broadcast of extent 1.
  int buildNode(Build& b, uint32_t v, const std::vector<int>& map) {
    auto key = std::make_pair(v, map);
    auto hit = b.memo.find(key);
    if (hit != b.memo.end()) return hit->second;
    int made = buildNodeUncached(b, v, map);
    b.memo[key] = made;
    return made;
  }

  int boundaryLeaf(Build& b, uint32_t v, const std::vector<int>& map) {
    if (slot_of[v] < 0) {
      if (b.trial) throw Abort{};
      materialize(v);
    }
    return leafNode(b, slot_of[v], P.typeOf(v), map);
  }

  int buildNodeUncached(Build& b, uint32_t v, const std::vector<int>& map) {
    const Operation& op = P.ops[v];
    if (b.trial && v == b.acc_value) {
      for (size_t i = 0; i < map.size(); ++i)
        if (map[i] != static_cast<int>(i)) throw Abort{};
      if (b.acc_node < 0) {
        ENode n;
        n.op = ENode::Leaf;
        n.dtype = DType::f32;
        n.leaf = -2;  // accumulator marker
        n.vary = (1u << map.size()) - 1u;
        b.acc_node = addNode(b, n);
      }
      return b.acc_node;
    }
    if (slot_of[v] >= 0 && op.kind != Kind::constant) return leafNode(b, slot_of[v], op.result, map);
    switch (op.kind) {
      case Kind::parameter:
        return leafNode(b, slot_of[v], op.result, map);
      case Kind::constant: {
        uint64_t bits;
        if (splatConstant(op, &bits)) {
          ENode n;
          n.op = ENode::Const;
          n.dtype = op.result.dtype;
          n.bits = bits;
          return addNode(b, n);
        }
        return boundaryLeaf(b, v, map);
      }
      case Kind::iota: {
        ENode n;
        n.op = ENode::Iota;
        n.dtype = op.result.dtype;
        n.dim = map[op.axis];
        if (n.dim < 0) {
          n.op = ENode::Const;
          n.bits = 0;
        } else {
          n.vary = 1u << n.dim;
        }
        return addNode(b, n);
      }
      case Kind::unary:
      case Kind::binary:
      case Kind::compare:
      case Kind::select: {
        ENode n;
        n.op = op.kind == Kind::unary ? ENode::Un
               : op.kind == Kind::binary ? ENode::Bin
               : op.kind == Kind::compare ? ENode::Cmp : ENode::Sel;
        n.sub = op.sub;
        n.dtype = op.result.dtype;
        for (size_t i = 0; i < op.operands.size(); ++i) {
          uint32_t a = op.operands[i];
          std::vector<int> amap = P.typeOf(a).rank() == map.size() ? map : std::vector<int>{};
          n.args[i] = buildNode(b, a, amap);
          n.vary |= b.nodes[n.args[i]].vary;
          n.level = std::max(n.level, b.nodes[n.args[i]].level);
        }
        b.closure.insert(v);
        int id = -1;
        if (op.kind == Kind::binary && static_cast<Binary>(op.sub) == Binary::mul &&
            (n.dtype == DType::f32 || n.dtype == DType::f64)) {
          // x * 1 is x, bit for bit (signed zeros, infinities and NaNs included): the gradient
          // transformation multiplies by its seed of ones
          const uint64_t one = n.dtype == DType::f32 ? 0x3f800000ull : 0x3ff0000000000000ull;
          for (int side = 0; side < 2 && id < 0; ++side) {
            const ENode& k = b.nodes[n.args[side]];
            if (k.op == ENode::Const && k.dtype == n.dtype && k.bits == one && b.nodes[n.args[1 - side]].dtype == n.dtype)
              id = n.args[1 - side];
          }
        }
        if (id < 0) id = addNode(b, n);
        if ((is_output[v] || wanted.count(same_as[v])) && v != b.root && !produced.count(v)) b.coproduce.push_back({v, id});
        return id;
      }
      case Kind::broadcast_in_dim: {
        uint32_t x = op.operands[0];
        const Type& xt = P.typeOf(x);
        std::vector<int> xmap(xt.rank(), -1);
        for (size_t j = 0; j < xt.rank(); ++j) {
          int64_t target = op.result.dims[op.ints[j]].extent;
          xmap[j] = (xt.dims[j].extent == 1 && target != 1) ? -1 : map[op.ints[j]];
        }
        return buildNode(b, x, xmap);
      }
      case Kind::transpose: {
        uint32_t x = op.operands[0];
        std::vector<int> xmap(map.size(), -1);
        for (size_t i = 0; i < map.size(); ++i) xmap[op.ints[i]] = map[i];
        return buildNode(b, x, xmap);
      }
      case Kind::reshape: {
        uint32_t x = op.operands[0];
        const Type& xt = P.typeOf(x);
        bool same = xt.rank() == op.result.rank();
        for (size_t i = 0; same && i < xt.rank(); ++i)
          if (xt.dims[i].extent != op.result.dims[i].extent) same = false;
        if (same) return buildNode(b, x, map);
        if (slot_of[x] < 0) {
          if (b.trial) throw Abort{};
          materialize(x);
        }
        return leafNode(b, slot_of[x], op.result, map);
      }
      case Kind::reduce:
        return buildReduce(b, v, map);
      case Kind::dot_general:
        return boundaryLeaf(b, v, map);
      default:
        throw PlanError(std::string("operation kind not supported by the B200 target: ") + kindName(op.kind));
    }
  }

  int buildReduce(Build& b, uint32_t v, const std::vector<int>& map) {
    const Operation& op = P.ops[v];
    if (b.trial) throw Abort{};  // GEMM epilogues carry no reductions
    const Operation& init = P.ops[op.operands[1]];
    uint64_t init_bits = 0;
    if (init.kind != Kind::constant || !splatConstant(init, &init_bits))
      throw PlanError("reduce with a non-constant initial value is not supported");
    const Type& in = P.typeOf(op.operands[0]);
    // A fold over leading axes (the innermost axis of its operand is kept) whose result is used
    // further inside this region, as in a softmax or a centring over axis 0: fused, every thread
    // group would walk down a column of a row-major buffer, once per pass, 32-byte sectors for 4-byte
    // elements (measured: 0.8 TB/s).  The fold gets a kernel of its own instead (one thread per kept
    // column, neighbouring columns in neighbouring threads) and this region reads its result like
    // any other small operand, so every pass over the large operand runs along its rows.
    if (v != b.root && v != b.sibling) {
      long innermost = -1;
      for (size_t i = 0; i < in.rank(); ++i)
        if (in.dims[i].extent != 1) innermost = static_cast<long>(i);
      bool any_reduced = false, innermost_reduced = false;
      for (size_t i = 0; i < in.rank(); ++i) {
        const bool reduced = std::find(op.ints.begin(), op.ints.end(), static_cast<int64_t>(i)) != op.ints.end();
        if (reduced && in.dims[i].extent != 1) any_reduced = true;
        if (reduced && static_cast<long>(i) == innermost) innermost_reduced = true;
      }
      if (any_reduced && !innermost_reduced) return boundaryLeaf(b, v, map);
    }
    // locate column dims for the reduced axes
    std::vector<int> in_map(in.rank(), -1);
    std::vector<int> taken;
    size_t kept = 0;
    for (size_t i = 0; i < in.rank(); ++i) {
      bool reduced = std::find(op.ints.begin(), op.ints.end(), static_cast<int64_t>(i)) != op.ints.end();
      if (!reduced) {
        in_map[i] = map[kept++];
        if (in_map[i] >= 0) taken.push_back(in_map[i]);
      }
    }
    std::vector<int> col_dims;
    // a trial pass over the existing dims first, so no dims are created when the reduce turns
    // out to be incompatible with the columns this region already has
    size_t before = b.extents.size();
    for (size_t i = 0; i < in.rank(); ++i) {
      bool reduced = std::find(op.ints.begin(), op.ints.end(), static_cast<int64_t>(i)) != op.ints.end();
      if (!reduced) continue;  // a kept broadcast dim of extent 1
      int d = clusterDimFor(b, in.dims[i], taken);
      taken.push_back(d);
      in_map[i] = d;
      col_dims.push_back(d);
    }
    bool compatible = true;
    if (b.cols_fixed) {
      std::vector<int> want;
      for (size_t d = 0; d < b.is_col.size(); ++d)
        if (b.is_col[d]) want.push_back(static_cast<int>(d));
      std::vector<int> got = col_dims;
      std::sort(got.begin(), got.end());
      // dims of extent 1 do not matter
      auto strip = [&](std::vector<int>& xs) {
        xs.erase(std::remove_if(xs.begin(), xs.end(), [&](int d) { return b.extents[d] == 1; }), xs.end());
      };
      strip(want);
      strip(got);
      compatible = want == got;
    } else {
      // kept dims of this reduce must not be column dims of... nothing fixed yet: fix them now
      for (int d : col_dims) b.is_col[d] = true;
      b.cols_fixed = true;
    }
    if (!compatible) {
      // reduction over other axes: compute it in its own kernel and read the result here
      b.dim_names.resize(before);
      b.extents.resize(before);
      b.is_col.resize(before);
      return boundaryLeaf(b, v, map);
    }
    for (int d : col_dims) b.is_col[d] = true;
    ENode n;
    n.op = ENode::Red;
    n.sub = op.sub;
    n.dtype = op.result.dtype;
    n.bits = init_bits;
    n.args[0] = buildNode(b, op.operands[0], in_map);
    uint32_t col_mask = 0;
    for (int d : col_dims) col_mask |= 1u << d;
    n.vary = b.nodes[n.args[0]].vary & ~col_mask;
    n.level = b.nodes[n.args[0]].level + 1;
    b.closure.insert(v);
    int id = addNode(b, n);
    if ((is_output[v] || wanted.count(same_as[v])) && v != b.root && !produced.count(v)) b.coproduce.push_back({v, id});
    return id;
  }

  // ---------------------------------------------------------------------------------------
  // row kernels
  // ---------------------------------------------------------------------------------------
  int cluster_depth = 0;  // nesting of planCluster calls (a region materialising what it reads)

  void planCluster(uint32_t v) {
    if (!is_output[v]) standalone.insert(same_as[v]);
    Build b;
    b.root = v;
    const Type& ty = P.typeOf(v);
    std::vector<int> map(ty.rank());
    for (size_t i = 0; i < ty.rank(); ++i) {
      b.dim_names.push_back(ty.dims[i].name);
      b.extents.push_back(ty.dims[i].extent);
      b.is_col.push_back(false);
      map[i] = static_cast<int>(i);
    }
    struct Depth {
      int& d;
      explicit Depth(int& v) : d(v) { ++d; }
      ~Depth() { --d; }
    } depth(cluster_depth);
    int root_node = buildNode(b, v, map);
    // Sibling outputs with the root's own dims (e.g. a value and its slope, both sums over the
    // same axis) join this region, so inputs they share are read once (the reference's concat
    // reduction, reduction.zig:346-420, serves the same purpose).  Only a region planned for an
    // output itself takes siblings: one planned while another region is being built (a value
    // that region reads) could otherwise pull in the output that asked for it, without end.
    for (auto it = out_slot_of.rbegin(); it != out_slot_of.rend(); ++it) {
      if (cluster_depth != 1) break;
      const uint32_t u = it->first;
      if (u == v || produced.count(u) || slot_of[u] >= 0 || b.closure.count(u)) continue;
      const Operation& uop = P.ops[u];
      if (!(isElementwise(uop.kind) || uop.kind == Kind::reduce)) continue;
      if (!sameDims(uop.result.dims, ty.dims) || b.nodes.size() > 4000) continue;
      b.sibling = u;
      int node = buildNode(b, u, map);
      b.sibling = 0xffffffffu;
      bool listed = false;
      for (auto& cand : b.coproduce) listed = listed || cand.first == u;
      if (!listed) b.coproduce.push_back({u, node});
    }
    // Folds over this region's columns that another region needs (found by the first planning pass) and
    // whose operand has the root's dims join as well: the rows' shares of a loss next to the gradient
    // computed from the same rows, for instance.
    if (cluster_depth == 1 && b.cols_fixed) {
      for (uint32_t u : wanted) {
        if (u == v || produced.count(u) || slot_of[u] >= 0 || b.closure.count(u) || b.nodes.size() > 4000) continue;
        const Operation& uop = P.ops[u];
        if (uop.kind != Kind::reduce || !sameDims(P.typeOf(uop.operands[0]).dims, ty.dims)) continue;
        // it must fold exactly the column dims (those of extent 1 do not matter either way)
        bool same_axes = true;
        std::vector<int> umap;
        for (size_t d = 0; d < ty.rank(); ++d) {
          const bool folded = std::find(uop.ints.begin(), uop.ints.end(), static_cast<int64_t>(d)) != uop.ints.end();
          if (ty.dims[d].extent != 1 && folded != static_cast<bool>(b.is_col[d])) same_axes = false;
          if (!folded) umap.push_back(static_cast<int>(d));
        }
        if (!same_axes) continue;
        bool listed = false;
        for (auto& cand : b.coproduce) listed = listed || cand.first == u;
        if (listed) continue;
        b.sibling = u;
        int node = buildNode(b, u, umap);
        b.sibling = 0xffffffffu;
        if (slot_of[u] < 0 && !produced.count(u)) b.coproduce.push_back({u, node});
      }
    }
    // Without any reduction the trailing dims form the column space: enough of them to give a
    // row at least 1024 elements, so flat elementwise programs still fill the machine.
    if (!b.cols_fixed) {
      if (b.extents.empty()) {
        b.dim_names.push_back("#unit");
        b.extents.push_back(1);
        b.is_col.push_back(true);
      } else {
        int64_t cols = 1;
        for (long d = static_cast<long>(b.extents.size()) - 1; d >= 0; --d) {
          if (cols >= 1024) break;
          b.is_col[d] = true;
          cols *= b.extents[d];
        }
      }
    }
    // order dims: rows first (discovery order), then columns (discovery order)
    std::vector<int> order;
    for (size_t d = 0; d < b.extents.size(); ++d) if (!b.is_col[d]) order.push_back(static_cast<int>(d));
    int split = static_cast<int>(order.size());
    for (size_t d = 0; d < b.extents.size(); ++d) if (b.is_col[d]) order.push_back(static_cast<int>(d));
    std::vector<int> new_index(b.extents.size());
    for (size_t i = 0; i < order.size(); ++i) new_index[order[i]] = static_cast<int>(i);
    auto remask = [&](uint32_t m) {
      uint32_t out = 0;
      for (size_t d = 0; d < b.extents.size(); ++d)
        if (m & (1u << d)) out |= 1u << new_index[d];
      return out;
    };
    Cluster c;
    c.split = split;
    for (int d : order) c.extents.push_back(b.extents[d]);
    for (int i = 0; i < split; ++i) c.rows *= c.extents[i];
    for (size_t i = split; i < c.extents.size(); ++i) c.cols *= c.extents[i];
    c.nodes = b.nodes;
    for (ENode& n : c.nodes) {
      n.vary = remask(n.vary);
      if (n.op == ENode::Iota) n.dim = new_index[n.dim];
    }
    for (const LeafRef& leaf : b.leaves) {
      LeafRef l = leaf;
      l.strides.assign(order.size(), 0);
      for (size_t d = 0; d < leaf.strides.size(); ++d) l.strides[new_index[d]] = leaf.strides[d];
      l.vary = remask(leaf.vary);
      c.leaves.push_back(l);
    }
    // Outputs: the root plus every other program output computed on the way.  An output is
    // written through an index map (strides per cluster dim) like a leaf is read; it can be
    // written here only if each of its elements is produced exactly once, i.e. it spans every
    // non-unit row dim and either none or all of the non-unit column dims.
    uint32_t all_rows = 0, all_cols = 0;
    for (size_t d = 0; d < c.extents.size(); ++d) {
      if (c.extents[d] == 1) continue;
      if (static_cast<int>(d) < split) all_rows |= 1u << d; else all_cols |= 1u << d;
    }
    auto outputRef = [&](uint32_t value, int node, LeafRef* ref) {
      const Type& vt = P.typeOf(value);
      std::vector<int> vmap;
      bool found = false;
      for (auto& kv : b.memo)
        if (kv.first.first == value && kv.second == node) { vmap = kv.first.second; found = true; }
      if (!found) return false;
      ref->dtype = vt.dtype;
      ref->strides.assign(order.size(), 0);
      ref->vary = 0;
      std::vector<int64_t> rm = rowMajorStrides(vt.dims);
      for (size_t d = 0; d < vt.rank(); ++d) {
        if (vt.dims[d].extent == 1) continue;
        if (d >= vmap.size() || vmap[d] < 0) return false;
        ref->strides[new_index[vmap[d]]] += rm[d];
        ref->vary |= 1u << new_index[vmap[d]];
      }
      bool rows_ok = (ref->vary & all_rows) == all_rows;
      uint32_t cv = ref->vary & all_cols;
      return rows_ok && (cv == 0 || cv == all_cols);
    };
    std::vector<uint32_t> out_values;
    {
      LeafRef ref;
      if (!outputRef(v, root_node, &ref))
        throw PlanError("fused region writes its result more than once per element (reduction over axes the result does not span)");
      ref.slot = destinationSlot(v);
      ref.dtype = plan.slots[ref.slot].storage;
      c.leaves.push_back(ref);
      c.outputs.push_back({root_node, static_cast<int>(c.leaves.size()) - 1});
      out_values.push_back(v);
    }
    for (auto& cand : b.coproduce) {
      if (produced.count(cand.first) || slot_of[cand.first] >= 0) continue;
      if (std::find(out_values.begin(), out_values.end(), cand.first) != out_values.end()) continue;
      LeafRef ref;
      if (!outputRef(cand.first, cand.second, &ref)) continue;
      ref.slot = destinationSlot(cand.first);
      ref.dtype = plan.slots[ref.slot].storage;
      c.leaves.push_back(ref);
      c.outputs.push_back({cand.second, static_cast<int>(c.leaves.size()) - 1});
      out_values.push_back(cand.first);
    }
    RowSchedule sched = chooseRowSchedule(c, ov);
    std::string name = nextName("row");
    std::ostringstream label;
    label << name << " rows=" << c.rows << " cols=" << c.cols << " reduces=" << countReduces(c)
          << " tpr=" << sched.tpr << " rpc=" << sched.rpc << " vec=" << sched.vec << " vpt=" << sched.vpt
          << " chunks=" << sched.chunks << " splits=" << sched.splits;
    if (sched.rpt > 1) label << " rows_per_thread=" << sched.rpt;
    summary << "row kernel: " << label.str() << " outputs=" << out_values.size() << "\n";
    emitRowKernels(c, sched, name, plan, label.str());
    plan.work.pairs += static_cast<double>(c.rows) * static_cast<double>(c.cols);
    for (size_t i = 0; i < out_values.size(); ++i) {
      slot_of[out_values[i]] = c.leaves[c.outputs[i].ref].slot;
      produced.insert(out_values[i]);
    }
  }

  static int countReduces(const Cluster& c) {
    int n = 0;
    for (const ENode& e : c.nodes) if (e.op == ENode::Red) ++n;
    return n;
  }

  void emitCopy(int src, int dst) {
    // device-to-device copy as a one-leaf row kernel over bytes
    Cluster c;
    size_t bytes = plan.slots[dst].bytes;
    bool words = bytes % 4 == 0;
    int64_t count = static_cast<int64_t>(words ? bytes / 4 : bytes);
    c.extents = {count};
    c.split = 0;
    c.rows = 1;
    c.cols = count;
    LeafRef in;
    in.slot = src;
    in.dtype = words ? DType::u32 : DType::u8;
    in.strides = {1};
    in.vary = 1;
    c.leaves.push_back(in);
    ENode n;
    n.op = ENode::Leaf;
    n.dtype = in.dtype;
    n.leaf = 0;
    n.vary = 1;
    c.nodes.push_back(n);
    LeafRef out = in;
    out.slot = dst;
    c.leaves.push_back(out);
    c.outputs.push_back({0, 1});
    RowSchedule sched = chooseRowSchedule(c, ov);
    std::string name = nextName("copy");
    summary << "copy kernel: " << name << " bytes=" << bytes << "\n";
    emitRowKernels(c, sched, name, plan, name);
  }

  // ---------------------------------------------------------------------------------------
  // GEMM (+ epilogue)
  // ---------------------------------------------------------------------------------------
  struct OperandView {
    int slot = -1;
    std::vector<int64_t> strides;  // per dim of the dot operand (canonical order)
  };

  // Resolves a dot operand to a buffer and per-dim element strides, looking through transposes
  // and same-extent reshapes of a materialised value; anything computed is materialised first.
  OperandView operandView(uint32_t v) {
    const Type& ty = P.typeOf(v);
    std::vector<int> perm(ty.rank());
    for (size_t i = 0; i < perm.size(); ++i) perm[i] = static_cast<int>(i);
    uint32_t cur = v;
    while (slot_of[cur] < 0) {
      const Operation& op = P.ops[cur];
      if (op.kind == Kind::transpose) {
        // cur dim i is x dim ints[i]
        for (auto& p : perm) p = static_cast<int>(op.ints[p]);
        cur = op.operands[0];
        continue;
      }
      if (op.kind == Kind::reshape) {
        const Type& xt = P.typeOf(op.operands[0]);
        bool same = xt.rank() == op.result.rank();
        for (size_t i = 0; same && i < xt.rank(); ++i)
          if (xt.dims[i].extent != op.result.dims[i].extent) same = false;
        if (same) {
          cur = op.operands[0];
          continue;
        }
      }
      break;
    }
    OperandView view;
    if (slot_of[cur] < 0 && (P.ops[cur].kind == Kind::parameter)) throw PlanError("parameter without slot");
    if (slot_of[cur] < 0) {
      // computed operand: materialise the value itself in canonical order, in its own 16-bit type
      narrow.insert(v);
      view.slot = materialize(v);
      view.strides = rowMajorStrides(ty.dims);
      return view;
    }
    std::vector<int64_t> rm = rowMajorStrides(P.typeOf(cur).dims);
    view.slot = slot_of[cur];
    view.strides.resize(ty.rank());
    for (size_t i = 0; i < ty.rank(); ++i) view.strides[i] = rm[perm[i]];
    return view;
  }

  // collapses dims [lo, hi) with the given strides into one (extent, stride); false if the
  // group is not a single strided run
  static bool collapse(const std::vector<Dim>& dims, const std::vector<int64_t>& strides, size_t lo,
                       size_t hi, int64_t* extent, int64_t* stride) {
    *extent = 1;
    *stride = 0;
    bool first = true;
    int64_t expect = 0;
    for (long i = static_cast<long>(hi) - 1; i >= static_cast<long>(lo); --i) {
      if (dims[i].extent == 1) continue;
      if (first) {
        *stride = strides[i];
        expect = strides[i] * dims[i].extent;
        first = false;
      } else {
        if (strides[i] != expect) return false;
        expect *= dims[i].extent;
      }
      *extent *= dims[i].extent;
    }
    return true;
  }

  struct DotShape {
    size_t nb = 0, nm = 0, nk = 0, nn = 0;
  };

  DotShape canonicalDot(const Operation& op) {
    const Type& lt = P.typeOf(op.operands[0]);
    const Type& rt = P.typeOf(op.operands[1]);
    DotShape s;
    s.nb = op.lhs_batch.size();
    s.nk = op.ints.size();
    for (size_t i = 0; i < s.nb; ++i)
      if (op.lhs_batch[i] != static_cast<int64_t>(i) || op.rhs_batch[i] != static_cast<int64_t>(i))
        throw PlanError("dot_general with non-leading batch axes is not supported");
    if (lt.rank() < s.nb + s.nk || rt.rank() < s.nb + s.nk) throw PlanError("dot_general rank mismatch");
    s.nm = lt.rank() - s.nb - s.nk;
    s.nn = rt.rank() - s.nb - s.nk;
    for (size_t i = 0; i < s.nk; ++i) {
      if (op.ints[i] != static_cast<int64_t>(s.nb + s.nm + i) ||
          op.rhs_contract[i] != static_cast<int64_t>(s.nb + i))
        throw PlanError("dot_general operands are not in canonical [batch, free, contract] x [batch, contract, free] order");
    }
    return s;
  }

  void fillGemmOperands(const Operation& op, GemmOp& g) {
    DotShape s = canonicalDot(op);
    const Type& lt = P.typeOf(op.operands[0]);
    const Type& rt = P.typeOf(op.operands[1]);
    for (int attempt = 0; attempt < 2; ++attempt) {
      OperandView a = operandView(op.operands[0]);
      int64_t e;
      bool ok = collapse(lt.dims, a.strides, 0, s.nb, &g.batch, &g.a_stride_b) &&
                collapse(lt.dims, a.strides, s.nb, s.nb + s.nm, &g.m, &g.a_stride_m) &&
                collapse(lt.dims, a.strides, s.nb + s.nm, lt.rank(), &g.k, &g.a_stride_k);
      (void)e;
      if (ok) {
        g.a_slot = a.slot;
        break;
      }
      if (attempt == 1) throw PlanError("dot_general lhs layout cannot be expressed with strides");
      narrow.insert(op.operands[0]);
      materialize(op.operands[0]);
    }
    for (int attempt = 0; attempt < 2; ++attempt) {
      OperandView bview = operandView(op.operands[1]);
      int64_t bb, kk;
      bool ok = collapse(rt.dims, bview.strides, 0, s.nb, &bb, &g.b_stride_b) &&
                collapse(rt.dims, bview.strides, s.nb, s.nb + s.nk, &kk, &g.b_stride_k) &&
                collapse(rt.dims, bview.strides, s.nb + s.nk, rt.rank(), &g.n, &g.b_stride_n);
      if (ok) {
        g.b_slot = bview.slot;
        break;
      }
      if (attempt == 1) throw PlanError("dot_general rhs layout cannot be expressed with strides");
      narrow.insert(op.operands[1]);
      materialize(op.operands[1]);
    }
    g.in_dtype = plan.slots[g.a_slot].storage;
    g.b_dtype = plan.slots[g.b_slot].storage;
  }

  void planGemm(uint32_t dot, uint32_t root, Build* epilogue = nullptr, int result_node = -1) {
    const Operation& op = P.ops[dot];
    GemmOp g;
    fillGemmOperands(op, g);
    g.out_dtype = P.typeOf(root).dtype;
    const bool integer = (g.in_dtype == DType::i32 || g.in_dtype == DType::u32) && g.b_dtype == g.in_dtype && g.out_dtype == g.in_dtype;
    if (g.in_dtype != DType::f32 && g.in_dtype != DType::bf16 && g.in_dtype != DType::f16 && !integer)
      throw PlanError(std::string("dot_general element type not supported: ") + dtypeName(g.in_dtype));
    DotShape s = canonicalDot(op);
    if (epilogue) {
      // collapse leaf strides from result dims to (batch, m, n)
      const Type& rt = op.result;
      g.epilogue.nodes = epilogue->nodes;
      g.epilogue.acc = epilogue->acc_node;
      g.epilogue.result = result_node;
      for (const LeafRef& leaf : epilogue->leaves) {
        LeafRef l = leaf;
        std::vector<int64_t> st = leaf.strides;
        st.resize(rt.rank(), 0);
        int64_t e0, e1, e2, s0, s1, s2;
        // zero-stride dims are broadcast: treat them as matching any run
        auto group = [&](size_t lo, size_t hi, int64_t* e, int64_t* sres) {
          std::vector<Dim> dims;
          std::vector<int64_t> ss;
          for (size_t i = lo; i < hi; ++i) {
            dims.push_back(rt.dims[i]);
            ss.push_back(st[i]);
          }
          bool any = false, all = true;
          for (size_t i = 0; i < dims.size(); ++i) {
            if (dims[i].extent == 1) continue;
            if (ss[i] != 0) any = true; else all = false;
          }
          if (!any) { *e = 1; *sres = 0; return true; }
          if (!all) return false;
          return collapse(dims, ss, 0, dims.size(), e, sres);
        };
        if (!group(0, s.nb, &e0, &s0) || !group(s.nb, s.nb + s.nm, &e1, &s1) ||
            !group(s.nb + s.nm, rt.rank(), &e2, &s2))
          throw PlanError("epilogue operand layout not expressible");
        l.strides = {s0, s1, s2};
        g.epilogue.leaves.push_back(l);
      }
    }
    g.c_slot = destinationSlot(root);
    g.out_dtype = plan.slots[g.c_slot].storage;
    // the tensor-core kernel takes ragged extents (TMA zero fill, guarded stores); what it needs
    // is at least one full tile per dimension and 16-byte row strides for the TMA descriptors
    const bool a_ok = g.a_stride_k == 1 || (g.a_stride_m == 1 && g.a_stride_k % 8 == 0 && g.a_stride_b % 8 == 0);
    const bool aligned = g.m >= 128 && g.n >= 128 && g.k >= 64 && g.k % 8 == 0 && a_ok &&
                         ((g.b_stride_n == 1 && g.n % 8 == 0) || g.b_stride_k == 1);
    const bool half_inputs = (g.in_dtype == DType::bf16 && g.b_dtype == DType::bf16) || (g.in_dtype == DType::f16 && g.b_dtype == DType::f16);
    g.tensor_core = half_inputs && aligned && !ov.force_simt_gemm;
    std::string name = nextName(g.tensor_core ? "gemm_tc" : "gemm_simt");
    summary << "gemm: " << name << " batch=" << g.batch << " m=" << g.m << " n=" << g.n << " k=" << g.k
            << " in=" << dtypeName(g.in_dtype) << " out=" << dtypeName(g.out_dtype)
            << " epilogue_nodes=" << g.epilogue.nodes.size()
            << (g.tensor_core ? " tcgen05" : " simt") << "\n";
    emitGemm(g, name, plan, ov);
    plan.work.flops += 2.0 * static_cast<double>(g.batch) * g.m * g.n * g.k;
    slot_of[root] = g.c_slot;
    produced.insert(root);
  }

  // Tries to compute elementwise value v as the epilogue of the single dot_general that feeds it.
  bool tryGemmEpilogue(uint32_t v) {
    // find the dot: walk back through elementwise ops along same-dims operands
    std::set<uint32_t> dots;
    std::vector<uint32_t> stack = {v};
    std::set<uint32_t> seen;
    while (!stack.empty()) {
      uint32_t cur = stack.back();
      stack.pop_back();
      if (!seen.insert(cur).second) continue;
      const Operation& op = P.ops[cur];
      if (slot_of[cur] >= 0) continue;
      if (op.kind == Kind::dot_general) {
        if (sameDims(op.result.dims, P.typeOf(v).dims)) dots.insert(cur);
        continue;
      }
      if (isElementwise(op.kind) || op.kind == Kind::broadcast_in_dim)
        for (uint32_t a : op.operands) stack.push_back(a);
    }
    if (dots.size() != 1) return false;
    uint32_t dot = *dots.begin();
    // integer contractions run alone (exact wrap-around arithmetic in the SIMT kernel); what
    // follows them is an ordinary elementwise kernel
    if (P.ops[dot].result.dtype == DType::i32 || P.ops[dot].result.dtype == DType::u32) return false;
    Build b;
    b.root = v;
    b.trial = true;
    b.acc_value = dot;
    const Type& ty = P.typeOf(v);
    std::vector<int> map(ty.rank());
    for (size_t i = 0; i < ty.rank(); ++i) {
      b.dim_names.push_back(ty.dims[i].name);
      b.extents.push_back(ty.dims[i].extent);
      b.is_col.push_back(false);
      map[i] = static_cast<int>(i);
    }
    int result;
    try {
      result = buildNode(b, v, map);
    } catch (const Abort&) {
      return false;
    }
    if (b.acc_node < 0) return false;
    // every inlined value (and the dot) may only be used inside the region, except v itself
    std::set<uint32_t> region = b.closure;
    region.insert(dot);
    for (uint32_t x : region) {
      if (x == v) continue;
      if (is_output[x]) return false;
      for (uint32_t u : users[x]) {
        // uses through broadcast views that stay inside the region are fine
        if (!regionUses(region, u)) return false;
      }
    }
    try {
      planGemm(dot, v, &b, result);
    } catch (const PlanError&) {
      return false;
    }
    return true;
  }

  bool regionUses(const std::set<uint32_t>& region, uint32_t user) {
    if (region.count(user)) return true;
    const Operation& op = P.ops[user];
    if (op.kind == Kind::broadcast_in_dim || op.kind == Kind::transpose || op.kind == Kind::reshape) {
      if (is_output[user] || users[user].empty()) return false;
      for (uint32_t u : users[user])
        if (!regionUses(region, u)) return false;
      return true;
    }
    return false;
  }

  // ---------------------------------------------------------------------------------------
  // attention
  // ---------------------------------------------------------------------------------------
  uint32_t throughBroadcast(uint32_t v, std::vector<int64_t>* bd = nullptr) {
    const Operation& op = P.ops[v];
    if (op.kind != Kind::broadcast_in_dim) return v;
    if (bd) *bd = op.ints;
    return op.operands[0];
  }

  bool scalarConstant(uint32_t v, double* out) {
    v = throughBroadcast(v);
    const Operation& op = P.ops[v];
    uint64_t bits;
    if (op.kind != Kind::constant || !splatConstant(op, &bits)) return false;
    switch (op.result.dtype) {
      case DType::f32: { float f; std::memcpy(&f, &bits, 4); *out = f; return true; }
      case DType::f64: { double d; std::memcpy(&d, &bits, 8); *out = d; return true; }
      case DType::bf16: { uint32_t w = static_cast<uint32_t>(bits & 0xffff) << 16; float f; std::memcpy(&f, &w, 4); *out = f; return true; }
      case DType::f16: {
        const uint32_t h = static_cast<uint32_t>(bits & 0xffff), sign = h >> 15, ex = (h >> 10) & 31, man = h & 1023;
        double mag = ex == 0 ? std::ldexp(static_cast<double>(man), -24)
                             : (ex == 31 ? (man ? std::nan("") : INFINITY) : std::ldexp(1.0 + man / 1024.0, static_cast<int>(ex) - 15));
        *out = sign ? -mag : mag;
        return true;
      }
      default: return false;
    }
  }

  bool tryAttention(uint32_t v) {
    const Operation& pv = P.ops[v];
    if (pv.result.dtype != DType::bf16 && pv.result.dtype != DType::f16) return false;
    DotShape s2;
    try { s2 = canonicalDot(pv); } catch (const PlanError&) { return false; }
    if (s2.nm != 1 || s2.nk != 1 || s2.nn != 1) return false;
    const size_t rank = s2.nb + 2;
    std::set<uint32_t> region;
    auto take = [&](uint32_t x) { region.insert(x); return P.ops[x]; };
    // P = E / bcast(sum(E))
    const Operation& pdiv = take(pv.operands[0]);
    if (pdiv.kind != Kind::binary || pdiv.sub != static_cast<uint8_t>(Binary::div)) return false;
    uint32_t e_id = pdiv.operands[0];
    region.insert(pdiv.operands[1]);
    uint32_t sum_id = throughBroadcast(pdiv.operands[1]);
    const Operation& sum = take(sum_id);
    if (sum.kind != Kind::reduce || sum.sub != static_cast<uint8_t>(Reducer::sum) || sum.operands[0] != e_id ||
        sum.ints.size() != 1 || sum.ints[0] != static_cast<int64_t>(rank - 1))
      return false;
    {
      // the fused kernel sums from zero and takes the maximum from -inf: other recorded initial
      // values leave the pattern to the generic kernels, which fold them in
      double sum_init;
      if (!scalarConstant(sum.operands[1], &sum_init) || sum_init != 0.0) return false;
    }
    const Operation& e = take(e_id);
    if (e.kind != Kind::unary || e.sub != static_cast<uint8_t>(Unary::exp)) return false;
    const Operation& shifted = take(e.operands[0]);
    if (shifted.kind != Kind::binary || shifted.sub != static_cast<uint8_t>(Binary::sub)) return false;
    uint32_t s_id = shifted.operands[0];
    region.insert(shifted.operands[1]);
    const Operation& mx = take(throughBroadcast(shifted.operands[1]));
    if (mx.kind != Kind::reduce || mx.sub != static_cast<uint8_t>(Reducer::max) || mx.operands[0] != s_id ||
        mx.ints.size() != 1 || mx.ints[0] != static_cast<int64_t>(rank - 1))
      return false;
    {
      double max_init;
      if (!scalarConstant(mx.operands[1], &max_init) || !(max_init < -1e30)) return false;
    }
    // optional causal mask
    bool causal = false;
    uint32_t cur = s_id;
    {
      const Operation& sel = P.ops[cur];
      if (sel.kind == Kind::select) {
        region.insert(cur);
        double neg;
        if (!scalarConstant(sel.operands[2], &neg) || !(neg < -1e30)) return false;
        region.insert(sel.operands[2]);
        region.insert(sel.operands[0]);
        std::vector<int64_t> bd;
        uint32_t mask_id = throughBroadcast(sel.operands[0], &bd);
        const Operation& mask = take(mask_id);
        if (mask.kind != Kind::compare || mask.result.rank() != 2) return false;
        if (bd.size() != 2 || bd[0] != static_cast<int64_t>(rank - 2) || bd[1] != static_cast<int64_t>(rank - 1))
          return false;
        const Operation& l = take(mask.operands[0]);
        const Operation& r = take(mask.operands[1]);
        if (l.kind != Kind::iota || r.kind != Kind::iota) return false;
        Compare dir = static_cast<Compare>(mask.sub);
        bool q_ge_k = (dir == Compare::ge && l.axis == 0 && r.axis == 1) ||
                      (dir == Compare::le && l.axis == 1 && r.axis == 0);
        if (!q_ge_k) return false;
        causal = true;
        cur = sel.operands[1];
      }
    }
    // optional scale
    double scale = 1.0;
    {
      const Operation& sc = P.ops[cur];
      if (sc.kind == Kind::binary && (sc.sub == static_cast<uint8_t>(Binary::mul) || sc.sub == static_cast<uint8_t>(Binary::div))) {
        double c;
        if (scalarConstant(sc.operands[1], &c)) {
          region.insert(cur);
          region.insert(sc.operands[1]);
          scale = sc.sub == static_cast<uint8_t>(Binary::mul) ? c : 1.0 / c;
          cur = sc.operands[0];
        } else if (sc.sub == static_cast<uint8_t>(Binary::mul) && scalarConstant(sc.operands[0], &c)) {
          region.insert(cur);
          region.insert(sc.operands[0]);
          scale = c;
          cur = sc.operands[1];
        } else {
          return false;
        }
      }
    }
    const Operation& qk = take(cur);
    if (qk.kind != Kind::dot_general) return false;
    DotShape s1;
    try { s1 = canonicalDot(qk); } catch (const PlanError&) { return false; }
    if (s1.nb != s2.nb || s1.nm != 1 || s1.nk != 1 || s1.nn != 1) return false;
    // nothing inside the region may be needed elsewhere
    for (uint32_t x : region) {
      if (is_output[x]) return false;
      for (uint32_t u : users[x])
        if (u != v && !regionUses(region, u)) return false;
    }
    AttentionOp a;
    GemmOp g1, g2;
    try {
      fillGemmOperands(qk, g1);   // Q [b, q, d] . Kt [b, d, k]
      // V operand of the second dot only; its lhs is the softmax region
      const Type& vt = P.typeOf(pv.operands[1]);
      OperandView vv = operandView(pv.operands[1]);
      int64_t bb, kk;
      if (!collapse(vt.dims, vv.strides, 0, s2.nb, &bb, &g2.b_stride_b) ||
          !collapse(vt.dims, vv.strides, s2.nb, s2.nb + 1, &kk, &g2.b_stride_k) ||
          !collapse(vt.dims, vv.strides, s2.nb + 1, vt.rank(), &g2.n, &g2.b_stride_n))
        return false;
      g2.b_slot = vv.slot;
      g2.k = kk;
    } catch (const PlanError&) {
      return false;
    }
    a.batch = g1.batch;
    a.q_len = g1.m;
    a.k_len = g1.n;
    a.head_dim = g1.k;
    a.causal = causal;
    a.scale = static_cast<float>(scale);
    a.dtype = pv.result.dtype;
    // layout requirements of the fused kernel: Q, K, V, O all [batch, seq, dim] row-major
    bool layout = g1.a_stride_k == 1 && g1.a_stride_m == a.head_dim && g1.b_stride_k == 1 &&
                  g1.b_stride_n == a.head_dim && g2.b_stride_n == 1 && g2.b_stride_k == g2.n &&
                  g2.n == a.head_dim && g2.k == a.k_len &&
                  (a.batch == 1 || (g1.a_stride_b == a.q_len * a.head_dim && g1.b_stride_b == a.k_len * a.head_dim &&
                                    g2.b_stride_b == a.k_len * a.head_dim));
    bool shape = (a.head_dim == 128 || a.head_dim == 64) && a.q_len >= 128 && a.k_len >= 128 && (!causal || a.q_len == a.k_len) &&
                 scale > 0.0;
    if (!layout || !shape || ov.force_simt_gemm) return false;
    a.q_slot = g1.a_slot;
    a.k_slot = g1.b_slot;
    a.v_slot = g2.b_slot;
    a.o_slot = destinationSlot(v);
    std::string name = nextName("attention");
    summary << "attention: " << name << " batch=" << a.batch << " q=" << a.q_len << " k=" << a.k_len
            << " d=" << a.head_dim << " causal=" << (causal ? 1 : 0) << " scale=" << a.scale << "\n";
    emitAttention(a, name, plan, ov);
    double pairs = causal ? static_cast<double>(a.q_len) * (a.q_len + 1) / 2.0
                          : static_cast<double>(a.q_len) * a.k_len;
    plan.work.flops += 4.0 * a.head_dim * pairs * a.batch;
    slot_of[v] = a.o_slot;
    produced.insert(v);
    return true;
  }
};

}  // namespace

// Programs with zero-extent axes (the reference's type rules allow them, src/tensor/type/dim.zig:178
// refuses only negative extents).  A value without elements needs no kernel; the only way a value
// WITH elements can depend on one without is a reduction over an empty axis (the fold from the init
// value over nothing: the init value itself, reduction.zig:839-863) or a contraction over an empty
// axis (zeros).  Those two are re-recorded as broadcasts of a scalar; everything else is replayed
// unchanged, after which no kernel ever reads an empty value.
//
// The same pass brings every contraction to the operand order the kernels take (the reference's
// dot lowering accepts only that order, dot.zig:2117-2161; gradients of contractions produce the
// others): the operands are transposed, which costs nothing when the strides still describe them.
// A fold over the innermost axis and at least one more (the sum over rows and columns at the end of a
// loss): planned as recorded it cannot join the row kernel that computes its operand (whose rows are the
// innermost axis alone), so the operand's inputs would be read once more.  Folding the innermost axis
// first and the rest in a second, small step changes only the association of the fold, which the
// kernels' tree-shaped folds change anyway.  Innermost extents below 64 stay as recorded.
static bool foldsInTwoStages(const Program& p, const Operation& op) {
  const Type& in = p.typeOf(op.operands[0]);
  long innermost = -1;
  for (size_t i = 0; i < in.rank(); ++i)
    if (in.dims[i].extent != 1) innermost = static_cast<long>(i);
  if (innermost < 0 || in.dims[innermost].extent < 64) return false;
  bool inner_reduced = false, other_reduced = false;
  for (int64_t d : op.ints) {
    if (d == innermost) inner_reduced = true;
    else if (in.dims[d].extent != 1) other_reduced = true;
  }
  return inner_reduced && other_reduced;
}

static Program withoutEmptyFolds(const Program& p) {
  Builder b(p.name);
  std::vector<uint32_t> now(p.ops.size(), 0);
  for (const Operation& op : p.ops) {
    auto arg = [&](size_t i) { return now[op.operands[i]]; };
    const bool empty = op.result.elementCount() == 0;
    uint32_t made = 0;
    switch (op.kind) {
      case Kind::parameter: made = b.input(op.result.dtype, op.result.dims, /*authored=*/false); break;
      case Kind::constant: made = b.constantBytes(op.result, op.payload.data(), op.payload.size()); break;
      case Kind::iota: made = b.iotaTyped(op.result, op.axis); break;
      case Kind::unary: made = b.unary(static_cast<Unary>(op.sub), arg(0)); break;
      case Kind::binary: made = b.binary(static_cast<Binary>(op.sub), arg(0), arg(1)); break;
      case Kind::compare: made = b.compare(static_cast<Compare>(op.sub), arg(0), arg(1)); break;
      case Kind::select: made = b.select(arg(0), arg(1), arg(2)); break;
      case Kind::broadcast_in_dim: made = b.broadcastTo(arg(0), op.result.dims, op.ints); break;
      case Kind::broadcast:
        // a rank-0 value repeated to the result dims: the same as broadcast_in_dim with no mapped dim
        if (p.typeOf(op.operands[0]).rank() != 0) throw PlanError("broadcast of a value that is not rank 0 is not supported");
        made = b.broadcastTo(arg(0), op.result.dims, {});
        break;
      case Kind::reshape: made = b.reshapeTo(arg(0), op.result.dims); break;
      case Kind::transpose: made = b.transposeBy(arg(0), op.ints); break;
      case Kind::reduce:
        if (!empty && p.typeOf(op.operands[0]).elementCount() == 0) made = b.broadcastTo(arg(1), op.result.dims, {});
        else if (foldsInTwoStages(p, op)) {
          // innermost axis first (from the reducer's identity), then the other axes from the recorded
          // start value: the first stage can share a row kernel with whatever its operand computes
          // along that axis
          const Type& in = p.typeOf(op.operands[0]);
          long innermost = -1;
          for (size_t i = 0; i < in.rank(); ++i)
            if (in.dims[i].extent != 1) innermost = static_cast<long>(i);
          const uint32_t rows = b.reduceNamed(arg(0), static_cast<Reducer>(op.sub), {in.dims[innermost].name});
          std::vector<int64_t> rest;
          for (int64_t d : op.ints)
            if (d != innermost) rest.push_back(d > innermost ? d - 1 : d);
          made = b.reduce(rows, arg(1), static_cast<Reducer>(op.sub), rest);
        } else made = b.reduce(arg(0), arg(1), static_cast<Reducer>(op.sub), op.ints);
        break;
      case Kind::dot_general:
        if (!empty && (p.typeOf(op.operands[0]).elementCount() == 0 || p.typeOf(op.operands[1]).elementCount() == 0)) {
          std::vector<uint8_t> zero(dtypeSize(op.result.dtype), 0);
          made = b.broadcastTo(b.constantBytes(Type{op.result.dtype, {}}, zero.data(), zero.size()), op.result.dims, {});
        } else {
          // operands brought to [batch, free, contract] x [batch, contract, free] by transposes
          // (views: the contraction reads them through strides); the result dims do not change
          auto ordered = [&](uint32_t x, const std::vector<int64_t>& batch, const std::vector<int64_t>& contract,
                             bool contract_last) {
            const size_t rank = b.typeOf(x).rank();
            std::vector<int64_t> perm = batch, free_axes;
            for (size_t a = 0; a < rank; ++a) {
              const int64_t axis = static_cast<int64_t>(a);
              if (std::find(batch.begin(), batch.end(), axis) == batch.end() &&
                  std::find(contract.begin(), contract.end(), axis) == contract.end())
                free_axes.push_back(axis);
            }
            if (contract_last) perm.insert(perm.end(), free_axes.begin(), free_axes.end());
            perm.insert(perm.end(), contract.begin(), contract.end());
            if (!contract_last) perm.insert(perm.end(), free_axes.begin(), free_axes.end());
            bool identity = true;
            for (size_t a = 0; a < rank; ++a) identity = identity && perm[a] == static_cast<int64_t>(a);
            return identity ? x : b.transposeBy(x, perm);
          };
          const uint32_t lhs = ordered(arg(0), op.lhs_batch, op.ints, true);
          const uint32_t rhs = ordered(arg(1), op.rhs_batch, op.rhs_contract, false);
          const size_t nb = op.lhs_batch.size(), nk = op.ints.size();
          const size_t nm = b.typeOf(lhs).rank() - nb - nk;
          std::vector<int64_t> batch_axes, lhs_contract, rhs_contract;
          for (size_t i = 0; i < nb; ++i) batch_axes.push_back(static_cast<int64_t>(i));
          for (size_t i = 0; i < nk; ++i) {
            lhs_contract.push_back(static_cast<int64_t>(nb + nm + i));
            rhs_contract.push_back(static_cast<int64_t>(nb + i));
          }
          made = b.dotGeneralOp(lhs, rhs, lhs_contract, rhs_contract, batch_axes, batch_axes);
        }
        break;
      default:
        throw PlanError("operation kind not supported by the B200 target");
    }
    now[op.id] = made;
  }
  std::vector<uint32_t> outputs;
  for (uint32_t o : p.outputs) outputs.push_back(now[o]);
  return b.finish(outputs);
}

Plan planProgram(const Program& program, const ScheduleOverrides& overrides) {
  if (program.outputs.empty()) throw PlanError("program has no outputs");
  bool has_empty = false;
  for (const Operation& op : program.ops) {
    if (op.result.dtype == DType::key) throw PlanError("key-typed values are not supported by the B200 target");
    for (const Dim& d : op.result.dims) has_empty |= d.extent == 0;
  }
  bool reorder = false;
  for (const Operation& op : program.ops) {
    reorder |= op.kind == Kind::broadcast;
    reorder |= op.kind == Kind::reduce && foldsInTwoStages(program, op);
    if (op.kind != Kind::dot_general) continue;
    const size_t nb = op.lhs_batch.size(), nk = op.ints.size();
    const size_t nm = program.typeOf(op.operands[0]).rank() - nb - nk;
    for (size_t i = 0; i < nb; ++i)
      reorder |= op.lhs_batch[i] != static_cast<int64_t>(i) || op.rhs_batch[i] != static_cast<int64_t>(i);
    for (size_t i = 0; i < nk; ++i)
      reorder |= op.ints[i] != static_cast<int64_t>(nb + nm + i) || op.rhs_contract[i] != static_cast<int64_t>(nb + i);
  }
  auto plan_twice = [&](const Program& q) {
    std::set<uint32_t> wanted;
    {
      Planner first(q, overrides);
      first.run();
      wanted = first.standalone;
    }
    Planner planner(q, overrides);
    planner.wanted = wanted;
    return planner.run();
  };
  if (has_empty || reorder) {
    const Program rewritten = withoutEmptyFolds(program);
    return plan_twice(rewritten);
  }
  return plan_twice(program);
}

}  // namespace accy
