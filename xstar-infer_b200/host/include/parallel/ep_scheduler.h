// Batch composition and rank workers for the expert-parallel layer.
//
// The engine's scheduler hands its worker a batch as concatenated sequences with cumulative lengths (cu_seqlens; reference
// serve/worker.py:27-44, serve/scheduler.py:161-260) and runs it from one thread.  With the experts spread over R GPUs
// every rank takes its own share of the batch's tokens, and the step ends when the slowest rank ends: the shares should
// hold the same number of tokens.  ep_balance_batch makes that split; EpWorkerPool is "one worker thread per rank": it owns
// one EpContext per GPU and runs a step on all of them at once.
#pragma once
#include <condition_variable>
#include <cstdint>
#include <exception>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "ops/moe_ep.h"

struct EpBatchPlan {
    std::vector<std::vector<std::int32_t>> sequences_of_rank; // indices into the batch, ascending inside a rank
    std::vector<std::int64_t> tokens_of_rank;
    std::vector<std::int32_t> rank_of_sequence;
    std::int64_t max_tokens() const;
    double imbalance() const; // max over ranks / mean over ranks (1.0 = perfectly even; 0 tokens: 1.0)
};

// Sequences are never split (a sequence's KV cache lives with one rank).  Longest sequence first, each to the rank with the
// fewest tokens so far (ties: the lower rank) -- the classic bound applies: no rank exceeds the mean by more than the longest
// sequence; a decode batch (all lengths 1) splits evenly.  Throws std::runtime_error("batch does not fit: ...") when a rank
// would exceed max_tokens_per_rank (0 = no limit), "bad cu_seqlens" for a list that does not start at 0 or decreases.
EpBatchPlan ep_balance_batch(const std::vector<std::int64_t> &cu_seqlens, int ranks, std::int64_t max_tokens_per_rank = 0);

// One thread per rank, each bound to its GPU and owning the rank's EpContext.  run() hands every thread its rank's call and
// returns when all are done; a rank that throws leaves the group (the others get "peer left" instead of waiting for it) and
// run() rethrows the first error.
class EpWorkerPool
{
public:
    EpWorkerPool(int world, std::vector<int> devices, const EpShape &shape, const EpOptions &options = {},
                 std::chrono::milliseconds timeout = std::chrono::milliseconds(30000));
    ~EpWorkerPool();
    EpWorkerPool(const EpWorkerPool &) = delete;
    EpWorkerPool &operator=(const EpWorkerPool &) = delete;

    int world() const { return world_; }

    // x[r] (T_r, H) on device r (T_r may differ between ranks, up to the shape's max_tokens), weights[r] = the router, the
    // always-on expert and rank r's experts on device r.  Returns the ranks' outputs, each on its own device.
    std::vector<Tensor> run(const std::vector<const Tensor *> &x, const std::vector<MoEWeights> &weights, const MoEConfig &config);

    // runs fn(rank, context) on every rank's thread (set-up of per-rank state, tests)
    void on_every_rank(const std::function<void(int, EpContext &)> &fn);

private:
    struct Worker;
    void dispatch(const std::function<void(int, EpContext &)> &fn);
    int world_;
    std::shared_ptr<EpGroup> group_;
    std::vector<std::unique_ptr<Worker>> workers_;
};
