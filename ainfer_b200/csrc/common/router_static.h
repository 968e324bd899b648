// Sizes of the fixed device array behind ainfer_router_topk_static: one definition shared by
// the kernel file that owns the array and by the C entry point that checks its limit.
#pragma once

namespace ainfer {

constexpr int kRouterStaticMaxExperts = 1024;     // experts the array has room for (plus the shared-expert gate)
constexpr int kRouterStaticScratchBytes = 8192;   // logits of up to 1024 + 1 rows, then the block counter
constexpr int kRouterStaticCounterOffset = 8128;
static_assert((kRouterStaticMaxExperts + 1) * 4 <= kRouterStaticCounterOffset, "logits overlap the counter");
static_assert(kRouterStaticCounterOffset + 4 <= kRouterStaticScratchBytes, "counter outside the array");

}  // namespace ainfer
