// The MoE layer with its experts spread over several GPUs of one box (expert parallelism): every rank holds the router,
// the always-on expert and E / world of the routed experts, takes its own batch of tokens, and the ranks exchange token
// rows so that each expert sees every token routed to it, wherever the token lives.
//
// Same op conventions as moe() (ops/moe.h; reference op style xstar_cpp/include/ops/mlp.h:51): borrowed const inputs, a new
// owned Tensor returned by value, std::runtime_error with short messages.  The reference itself is single-GPU; its
// expert all-to-all is a roadmap row (README.md:30) with no code behind it, so the interface here extends moe()'s by one
// argument, the context of the rank.
//
// One EpContext per rank: a host thread per GPU in one process (the ranks then meet in an EpGroup, which also detects a
// peer that stopped) or one process per GPU (group == nullptr; buffer addresses travel as IPC handles).  Construction is
// collective.  The context owns every device buffer of the step -- receive buffers for rows other ranks store into over
// NVLink, the return buffer, index tables, scratch -- so a step allocates nothing and never synchronises with the host:
//
//   always-on expert on a side stream | route -> permute -> all-gather of per-expert counts (NCCL) -> addresses computed
//   on the device -> dispatch kernel stores each row into its expert's owner -> barrier (one-element all-reduce) ->
//   grouped SwiGLU MLP over the local experts -> return kernel stores expert outputs into their source ranks ->
//   barrier -> weighted combine.
//
// Wire formats: bf16 experts send bf16 rows and get f32 rows back (the result is bit-identical to the single-GPU layer);
// FP8 / FP4 experts send e4m3 codes + scales (quantised once, before the trip) and get bf16 rows back.
#pragma once
#include <array>
#include <chrono>
#include <cstdint>
#include <memory>

#include "ops/moe.h"
#include "parallel/ep_group.h"
#include "tensor.h"

using EpUniqueId = std::array<std::uint8_t, 128>;
EpUniqueId ep_unique_id(); // one rank makes it, all ranks pass the same bytes to their context

struct EpShape {
    std::int64_t max_tokens = 0; // per rank and step
    std::int64_t hidden = 0, experts = 0, top_k = 0, intermediate = 0;
    DType expert_dtype = DType::BFloat16; // BFloat16 | Float8E4M3 | Float4E2M1x2 (routed experts)
    bool shared = false;                  // an always-on expert (bf16 with bf16 experts, else FP8)
};

struct EpOptions {
    // Rows this rank's receive buffers hold.  0: the worst routing (every row of every rank lands here: world * T * k).
    // Otherwise capacity_factor * T * k rows (T * k is a rank's share under balanced routing; 2 is generous); rows
    // that would not fit are dropped and flagged -- check() then throws "out-of-range index".
    double capacity_factor = 0.0;
    // Let the down GEMM's epilogue store the result rows into their source ranks (where the kernels support it: FP4 experts
    // with hidden % 256 == 0) instead of a separate return kernel after the GEMM.  Same bits either way.
    bool fused_return = true;
    // Exchange the per-expert counts and run the two barriers of a step through peer memory (xs_moe_ep_signal: one warp per
    // GPU, bounded wait) instead of NCCL's all-gather and one-element all-reduces: a third of the latency at 8 GPUs.  The
    // host check-in of the EpGroup (or, between processes, the caller's own agreement) must precede every step, since the
    // kernel waits for its peers.
    bool signal_barriers = true;
};

// rows a receive buffer holds for these sizes (the rule of EpOptions::capacity_factor), a multiple of 128
std::int64_t ep_capacity_rows(std::int64_t max_tokens, std::int64_t top_k, int world, double capacity_factor);

class EpContext
{
public:
    // Collective over all ranks.  `device`: the CUDA device of this rank (made current on the calling thread).
    EpContext(std::shared_ptr<EpGroup> group, const EpUniqueId &id, int rank, int world, int device, const EpShape &shape,
              const EpOptions &options = {});
    ~EpContext();
    EpContext(const EpContext &) = delete;
    EpContext &operator=(const EpContext &) = delete;

    int rank() const;
    int world() const;
    std::int64_t capacity_rows() const;
    bool fused_return() const; // whether steps of this context take the fused return path
    bool signal_barriers() const; // whether its counts exchange and barriers go through peer memory

    // One step, enqueued on `stream` (nullptr = the default stream), no host synchronisation after the check-in with
    // the group: x (T, H) bf16 and out (T, H) bf16 on this rank's device, T <= max_tokens.  `weights` holds the router
    // (all experts), this rank's experts [rank * E / world, (rank + 1) * E / world) and the always-on expert.
    void forward_into(const Tensor &x, const MoEWeights &weights, const MoEConfig &config, Tensor &out, void *stream);

    // Waits for `stream` and raises what the kernels flagged on the device (rows that did not fit a buffer, a bounded wait
    // that gave up) or what the communicator reports.
    void check(void *stream);

    // Leaves the group (peers waiting for this rank get "peer left") and aborts the communicator instead of the collective
    // shutdown: for a rank that stops after an error.
    void abandon() noexcept;

private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

// moe() over `ep`'s ranks: allocates the result, runs the step on the default stream, waits for it and checks the flags
// ("returns => finished", reference xstar_cpp/src/ops/mlp.cu:188-189).
Tensor moe(const Tensor &x, const MoEWeights &weights, const MoEConfig &config, EpContext *ep);
