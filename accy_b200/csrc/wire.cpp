// "ACTP" version 1 program bytes: writer and reader.
//
// Layout (src/tensor/wire/format.zig:1-26): u32 magic "ACTP", u32 version 1, length-prefixed name,
// then the root graph = u32 operation count, the operations, u32-counted output ids.  Integers are
// little-endian, i64 values take 8 bytes, every list starts with a u32 count.  Each operation
// carries its kind code and only the fields Builder.operation needs (encode.zig:136-230); the
// reader replays every operation through the Builder so result types are always re-derived
// (decode.zig:22-30, 156-163).  A scan operation nests a body graph; this target executes no
// scans, so the reader refuses them with ScanUnsupported instead of building a nested graph.
#include <cstring>

#include "program.hpp"

namespace accy {
namespace {

constexpr uint32_t kMagic = 0x50544341u;  // "ACTP" read little-endian
constexpr uint32_t kVersion = 1;
constexpr size_t kMaxOperands = 8;            // program.zig:143
constexpr size_t kMaxCustomCallOperands = 4;  // program.zig:142

struct Writer {
  std::vector<uint8_t> out;
  void u32(uint32_t v) {
    for (int i = 0; i < 4; ++i) out.push_back(static_cast<uint8_t>(v >> (8 * i)));
  }
  void i64(int64_t v) {
    uint64_t u = static_cast<uint64_t>(v);
    for (int i = 0; i < 8; ++i) out.push_back(static_cast<uint8_t>(u >> (8 * i)));
  }
  void bytes(const void* p, size_t n) {
    if (n > 0xffffffffu) throw WireError("InvalidArtifact");
    u32(static_cast<uint32_t>(n));
    const uint8_t* b = static_cast<const uint8_t*>(p);
    out.insert(out.end(), b, b + n);
  }
  void str(const std::string& s) { bytes(s.data(), s.size()); }
  void ints(const std::vector<int64_t>& v) {
    u32(static_cast<uint32_t>(v.size()));
    for (int64_t x : v) i64(x);
  }
  void dims(const std::vector<Dim>& v) {
    u32(static_cast<uint32_t>(v.size()));
    for (const Dim& d : v) {
      str(d.name);
      i64(d.extent);
    }
  }
  void typed(const Type& t) {
    u32(static_cast<uint32_t>(t.dtype));
    dims(t.dims);
  }
};

struct Reader {
  const uint8_t* p;
  size_t len, at = 0;
  size_t remaining() const { return len - at; }
  uint32_t u32() {
    if (remaining() < 4) throw WireError("InvalidArtifact");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) v |= static_cast<uint32_t>(p[at + i]) << (8 * i);
    at += 4;
    return v;
  }
  int64_t i64() {
    if (remaining() < 8) throw WireError("InvalidArtifact");
    uint64_t v = 0;
    for (int i = 0; i < 8; ++i) v |= static_cast<uint64_t>(p[at + i]) << (8 * i);
    at += 8;
    return static_cast<int64_t>(v);
  }
  std::string str() {
    uint32_t n = u32();
    if (n > remaining()) throw WireError("InvalidArtifact");
    std::string s(reinterpret_cast<const char*>(p + at), n);
    at += n;
    return s;
  }
  std::vector<uint8_t> blob() {
    uint32_t n = u32();
    if (n > remaining()) throw WireError("InvalidArtifact");
    std::vector<uint8_t> b(p + at, p + at + n);
    at += n;
    return b;
  }
  uint32_t count(size_t min_item_bytes) {
    uint32_t n = u32();
    if (n > remaining() / min_item_bytes) throw WireError("InvalidArtifact");
    return n;
  }
  uint32_t id(size_t limit) {
    uint32_t v = u32();
    if (v >= limit) throw WireError("InvalidReference");
    return v;
  }
  std::vector<int64_t> ints() {
    uint32_t n = count(8);
    std::vector<int64_t> v(n);
    for (auto& x : v) x = i64();
    return v;
  }
  std::vector<Dim> dims() {
    uint32_t n = count(12);
    std::vector<Dim> v(n);
    for (auto& d : v) {
      d.name = str();
      d.extent = i64();
    }
    return v;
  }
  Type typed() {
    uint32_t code = u32();
    if (code >= kDTypeCount) throw WireError("UnknownTag");
    Type t;
    t.dtype = static_cast<DType>(code);
    t.dims = dims();
    return t;
  }
};

template <typename E>
E decodeCode(uint32_t code, uint32_t count) {
  if (code >= count) throw WireError("UnknownTag");
  return static_cast<E>(code);
}

}  // namespace

std::vector<uint8_t> encodeProgram(const Program& program) {
  Writer w;
  w.u32(kMagic);
  w.u32(kVersion);
  w.str(program.name);
  // graph header check (encode.zig:117-134): ids dense, parameters in parameter order
  size_t parameter_count = 0;
  for (size_t i = 0; i < program.ops.size(); ++i) {
    const Operation& op = program.ops[i];
    if (op.id != i) throw WireError("InvalidProgram");
    if (op.kind != Kind::parameter) continue;
    if (op.index != parameter_count || parameter_count >= program.parameters.size() ||
        program.parameters[parameter_count] != i)
      throw WireError("InvalidProgram");
    ++parameter_count;
  }
  if (parameter_count != program.parameters.size()) throw WireError("InvalidProgram");
  w.u32(static_cast<uint32_t>(program.ops.size()));
  for (const Operation& op : program.ops) {
    w.u32(static_cast<uint32_t>(op.kind));
    switch (op.kind) {
      case Kind::parameter:
        w.typed(op.result);
        break;
      case Kind::constant:
        w.typed(op.result);
        w.bytes(op.payload.data(), op.payload.size());
        break;
      case Kind::iota:
        w.typed(op.result);
        w.i64(op.axis);
        break;
      case Kind::custom_call:
        w.typed(op.result);
        w.str(op.target);
        w.u32(op.version);
        w.u32(static_cast<uint32_t>(op.operands.size()));
        for (uint32_t id : op.operands) w.u32(id);
        break;
      case Kind::broadcast:
      case Kind::reshape:
        w.dims(op.result.dims);
        w.u32(op.operands[0]);
        break;
      case Kind::broadcast_in_dim:
        w.dims(op.result.dims);
        w.u32(op.operands[0]);
        w.ints(op.ints);
        break;
      case Kind::unary:
        w.u32(op.sub);
        w.u32(op.operands[0]);
        break;
      case Kind::binary:
      case Kind::compare:
        w.u32(op.sub);
        w.u32(op.operands[0]);
        w.u32(op.operands[1]);
        break;
      case Kind::select:
        for (int i = 0; i < 3; ++i) w.u32(op.operands[i]);
        break;
      case Kind::projection:
        w.u32(op.operands[0]);
        w.u32(static_cast<uint32_t>(op.index));
        break;
      case Kind::transpose:
        w.u32(op.operands[0]);
        w.ints(op.ints);
        break;
      case Kind::reduce:
        w.u32(op.operands[0]);
        w.u32(op.operands[1]);
        w.u32(op.sub);
        w.ints(op.ints);
        break;
      case Kind::gather:
      case Kind::sparse_cross_entropy:
        w.u32(op.operands[0]);
        w.u32(op.operands[1]);
        w.i64(op.axis);
        break;
      case Kind::scatter_add:
        for (int i = 0; i < 3; ++i) w.u32(op.operands[i]);
        w.i64(op.axis);
        break;
      case Kind::dot_general:
        w.u32(op.operands[0]);
        w.u32(op.operands[1]);
        w.ints(op.ints);
        w.ints(op.rhs_contract);
        w.ints(op.lhs_batch);
        w.ints(op.rhs_batch);
        break;
      case Kind::scan:
        throw WireError("ScanUnsupported");
    }
  }
  w.u32(static_cast<uint32_t>(program.outputs.size()));
  for (uint32_t id : program.outputs) w.u32(id);
  return std::move(w.out);
}

Program decodeProgram(const uint8_t* bytes, size_t len) {
  Reader r{bytes, len};
  if (r.u32() != kMagic) throw WireError("BadMagic");
  if (r.u32() != kVersion) throw WireError("UnsupportedVersion");
  Builder builder(r.str());
  uint32_t op_count = r.u32();
  for (uint32_t n = 0; n < op_count; ++n) {
    Kind kind = decodeCode<Kind>(r.u32(), kKindCount);
    const size_t limit = builder.valueCount();
    uint32_t made = 0;
    switch (kind) {
      case Kind::parameter: {
        Type t = r.typed();
        made = builder.input(t.dtype, t.dims, /*authored=*/false);
        break;
      }
      case Kind::constant: {
        Type t = r.typed();
        std::vector<uint8_t> payload = r.blob();
        made = builder.constantBytes(t, payload.data(), payload.size());
        break;
      }
      case Kind::iota: {
        Type t = r.typed();
        int64_t axis = r.i64();
        made = builder.iotaTyped(t, axis);
        break;
      }
      case Kind::custom_call: {
        (void)r.typed();
        (void)r.str();
        (void)r.u32();
        uint32_t cnt = r.count(4);
        if (cnt > kMaxCustomCallOperands) throw WireError("TooManyOperands");
        for (uint32_t i = 0; i < cnt; ++i) (void)r.id(limit);
        throw WireError("CustomCallUnsupported");
      }
      case Kind::broadcast: {
        std::vector<Dim> dims = r.dims();
        made = builder.broadcastOp(r.id(limit), dims);
        break;
      }
      case Kind::broadcast_in_dim: {
        std::vector<Dim> dims = r.dims();
        uint32_t in = r.id(limit);
        made = builder.broadcastTo(in, dims, r.ints());
        break;
      }
      case Kind::reshape: {
        std::vector<Dim> dims = r.dims();
        made = builder.reshapeTo(r.id(limit), dims);
        break;
      }
      case Kind::unary: {
        Unary u = decodeCode<Unary>(r.u32(), 9);
        made = builder.unary(u, r.id(limit));
        break;
      }
      case Kind::binary: {
        Binary b = decodeCode<Binary>(r.u32(), 7);
        uint32_t lhs = r.id(limit), rhs = r.id(limit);
        made = builder.binary(b, lhs, rhs);
        break;
      }
      case Kind::compare: {
        Compare c = decodeCode<Compare>(r.u32(), 6);
        uint32_t lhs = r.id(limit), rhs = r.id(limit);
        made = builder.compare(c, lhs, rhs);
        break;
      }
      case Kind::select: {
        uint32_t p = r.id(limit), t = r.id(limit), f = r.id(limit);
        made = builder.select(p, t, f);
        break;
      }
      case Kind::transpose: {
        uint32_t in = r.id(limit);
        made = builder.transposeBy(in, r.ints());
        break;
      }
      case Kind::reduce: {
        uint32_t in = r.id(limit), init = r.id(limit);
        Reducer red = decodeCode<Reducer>(r.u32(), 3);
        made = builder.reduce(in, init, red, r.ints());
        break;
      }
      case Kind::dot_general: {
        uint32_t lhs = r.id(limit), rhs = r.id(limit);
        std::vector<int64_t> lc = r.ints(), rc = r.ints(), lb = r.ints(), rb = r.ints();
        made = builder.dotGeneralOp(lhs, rhs, lc, rc, lb, rb);
        break;
      }
      case Kind::projection:
      case Kind::gather:
      case Kind::scatter_add:
      case Kind::sparse_cross_entropy:
        throw WireError("OperationUnsupported");
      case Kind::scan:
        throw WireError("ScanUnsupported");
    }
    if (made != limit) throw WireError("InvalidProgram");
  }
  uint32_t out_count = r.count(4);
  std::vector<uint32_t> outputs(out_count);
  for (auto& id : outputs) id = r.id(builder.valueCount());
  if (r.remaining() != 0) throw WireError("InvalidArtifact");
  (void)kMaxOperands;
  return builder.finish(outputs);
}

}  // namespace accy
