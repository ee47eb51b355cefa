// Argument validation shared by the MoE ops of this directory: tensors in, C-ABI config and pointer table out.
#pragma once
#include <cstdint>

#include "ops/moe.h"
#include "xs_moe.h"

namespace moe_detail {

struct Checked {
    XsMoeConfig cfg{};
    XsMoeWeights w{};
};

// Throws the reference vocabulary ("dtype mismatch", "rank mismatch", "shape mismatch", "device mismatch", ...) in the
// order the reference's ops check.  local_experts >= 0: the expert tensors hold that many experts (an expert-parallel
// rank's slice) instead of all of the router's.
Checked validate(const Tensor &x, const MoEWeights &m, const MoEConfig &config, bool need_experts, std::int64_t local_experts = -1);

// non-zero C-ABI status -> std::runtime_error carrying xs_moe_last_error()
void raise_if(int rc);

} // namespace moe_detail
