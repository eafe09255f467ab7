// tcgen05 kernels (placeholder until the tensor-core emitters land).
#include "plan.hpp"

namespace accy {

bool tcgen05Ready() { return false; }

void emitGemmTcgen05(const GemmOp&, const std::string&, Plan&, const ScheduleOverrides&) {
  throw PlanError("tcgen05 GEMM emitter not available");
}

void emitAttention(const AttentionOp&, const std::string&, Plan&, const ScheduleOverrides&) {
  throw PlanError("tcgen05 attention emitter not available");
}

}  // namespace accy
