// Mixture-of-experts feed-forward layer: router top-k -> token permute -> per-expert SwiGLU MLP -> weighted
// combine (+ shared expert).  It fills the slot `mlp(x, gate_up_weight, down_weight)` has in the engine's
// transformer block (reference xstar_cpp/src/ops/transformer_block.cpp:353) and follows the same op
// conventions (reference xstar_cpp/include/ops/mlp.h:51): free function, borrowed const inputs, optional
// inputs as pointers, a new owned Tensor returned by value, std::runtime_error with short messages
// ("dtype mismatch", "rank mismatch", "shape mismatch", "device mismatch") on bad arguments.
//
// This header is CUDA-free.  The device work is reached through the C ABI in include/xs_moe.h.
//
//   x                 (..., H)       bf16, leading dims collapsed to T rows
//   router_weight     (E, H)         bf16
//   router_bias       (E)            f32 or null; added to the logits for SELECTION only
//   gate_up_weight    (E, 2I, H)     rows [gate; up]; bf16, or Float8E4M3 with gate_up_scale (E, 2I/128, H/128) f32
//   down_weight       (E, H, I)      bf16, or Float8E4M3 with down_scale (E, H/128, I/128) f32
//   shared_*          (2I, H), (H, I) one always-on expert, optional
//   returns           same shape as x, bf16
//
// Numerics: router logits accumulate in ascending k in f32 (so expert choices are reproducible bit for
// bit); the k largest logit+bias win, ties to the lower expert id; weights are the softmax over the chosen
// logits; per expert silu(gate)*up in f32 with one rounding to the activation type, f32 accumulation in
// both GEMMs; out = sum over slots in ascending expert id, shared expert last, one rounding to bf16.
//
// Device::CPU inputs are rejected ("unsupported device"): the layer has no host implementation.
#pragma once
#include <cstdint>
#include <vector>

#include "tensor.h"

struct MoEConfig {
    std::int64_t top_k = 1;
};

struct MoEWeights {
    const Tensor *router_weight = nullptr;
    const Tensor *router_bias = nullptr;
    const Tensor *gate_up_weight = nullptr;
    const Tensor *gate_up_scale = nullptr;
    const Tensor *down_weight = nullptr;
    const Tensor *down_scale = nullptr;
    const Tensor *shared_gate_up_weight = nullptr;
    const Tensor *shared_gate_up_scale = nullptr;
    const Tensor *shared_down_weight = nullptr;
    const Tensor *shared_down_scale = nullptr;
};

Tensor moe(const Tensor &x, const MoEWeights &weights, const MoEConfig &config);

// The feed-forward half of a transformer block with the MoE layer in the MLP slot:
//     x + moe(rmsnorm(x, norm_weight, eps))
// which is what `add(attention_x, mlp(rmsnorm(attention_x, ln2_w, eps), gate_up_w, down_w))` computes in the
// engine's block (reference xstar_cpp/src/ops/transformer_block.cpp:353) with `mlp` replaced by `moe`.
// norm_weight (H) bf16.  Numerics follow the engine's ops one for one: rmsnorm sums the squares in f32 in
// ascending order, rounds x*inv to bf16 and then the product with the weight to bf16 (reference
// xstar_cpp/src/ops/rmsnorm.cpp:41-60); the layer output is rounded to bf16 before the residual is added in
// f32 and rounded once more (reference xstar_cpp/src/ops/add.cpp).  One normalisation kernel, and the
// residual add rides in the combine kernel: no extra pass over the activations.
Tensor moe_block(const Tensor &x, const Tensor &norm_weight, float eps, const MoEWeights &weights, const MoEConfig &config);

// Stream forms for an engine that runs its layers on a stream of its own.  The reference's ops are synchronous on the
// default stream (xstar_cpp/src/ops/mlp.cu:188-189); its roadmap row "explicit streams" (README.md:33) is what these are
// for.  moe_into / moe_block_into enqueue the layer on `stream` (nullptr = the default stream) and return without waiting;
// x, the weights, `out` (same shape as x, bf16, on the device) and `scratch` must stay alive until the stream has passed
// the call.  MoEScratch is the layer's scratch between calls: it grows to what the largest call needed (leased from the
// workspace pool, given back on destruction) and carries the device-side status word; moe_check waits for the stream and
// raises what the kernels flagged.  One scratch serves calls that do not overlap on the device (one stream, or streams that
// the caller orders).
class MoEScratch
{
public:
    MoEScratch() = default;
    ~MoEScratch();
    MoEScratch(const MoEScratch &) = delete;
    MoEScratch &operator=(const MoEScratch &) = delete;
    void *data() const { return ptr_; }
    std::size_t bytes() const { return bytes_; }
    void reserve(std::size_t bytes); // synchronises when it has to grow (the old block may still be in use)

private:
    void *ptr_ = nullptr;
    std::size_t bytes_ = 0;
    int device_ = 0;
};
void moe_into(const Tensor &x, const MoEWeights &weights, const MoEConfig &config, Tensor &out, MoEScratch &scratch, void *stream);
void moe_block_into(const Tensor &x, const Tensor &norm_weight, float eps, const MoEWeights &weights, const MoEConfig &config, Tensor &out,
                    MoEScratch &scratch, void *stream);
void moe_check(MoEScratch &scratch, void *stream);

// Routing decisions for inspection and tests: ids (T, k) ascending per row, weights (T, k),
// counts (E), offsets (E+1), perm (T*k), inv (T*k).  Host vectors; x and router tensors on the device.
struct MoERouting {
    std::vector<std::int32_t> topk_ids, counts, offsets, perm, inv;
    std::vector<float> topk_weights;
};
MoERouting moe_route(const Tensor &x, const Tensor &router_weight, const Tensor *router_bias, const MoEConfig &config);
