#include "parallel/ep_scheduler.h"

#include <algorithm>
#include <numeric>
#include <stdexcept>
#include <string>

#include "cuda/cuda_allocator.h"

std::int64_t EpBatchPlan::max_tokens() const
{
    std::int64_t m = 0;
    for (std::int64_t t : tokens_of_rank)
        m = std::max(m, t);
    return m;
}

double EpBatchPlan::imbalance() const
{
    const std::int64_t total = std::accumulate(tokens_of_rank.begin(), tokens_of_rank.end(), std::int64_t{0});
    if (total == 0 || tokens_of_rank.empty())
        return 1.0;
    return static_cast<double>(max_tokens()) * static_cast<double>(tokens_of_rank.size()) / static_cast<double>(total);
}

EpBatchPlan ep_balance_batch(const std::vector<std::int64_t> &cu, int ranks, std::int64_t max_tokens_per_rank)
{
    if (ranks < 1)
        throw std::runtime_error("bad rank count");
    if (cu.empty() || cu[0] != 0)
        throw std::runtime_error("bad cu_seqlens");
    const std::size_t n = cu.size() - 1;
    std::vector<std::int64_t> len(n);
    for (std::size_t i = 0; i < n; i++) {
        if (cu[i + 1] < cu[i])
            throw std::runtime_error("bad cu_seqlens");
        len[i] = cu[i + 1] - cu[i];
    }
    std::vector<std::int32_t> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](std::int32_t a, std::int32_t b) { return len[a] > len[b]; });
    EpBatchPlan p;
    p.sequences_of_rank.assign(ranks, {});
    p.tokens_of_rank.assign(ranks, 0);
    p.rank_of_sequence.assign(n, 0);
    for (std::int32_t s : order) {
        int best = 0;
        for (int r = 1; r < ranks; r++)
            if (p.tokens_of_rank[r] < p.tokens_of_rank[best])
                best = r;
        p.tokens_of_rank[best] += len[s];
        p.rank_of_sequence[s] = best;
        if (max_tokens_per_rank > 0 && p.tokens_of_rank[best] > max_tokens_per_rank)
            throw std::runtime_error("batch does not fit: rank " + std::to_string(best) + " would hold " + std::to_string(p.tokens_of_rank[best]) +
                                     " tokens, capacity " + std::to_string(max_tokens_per_rank));
    }
    for (std::size_t s = 0; s < n; s++)
        p.sequences_of_rank[p.rank_of_sequence[s]].push_back(static_cast<std::int32_t>(s));
    return p;
}

// ---- workers -----------------------------------------------------------------------------------------------------
struct EpWorkerPool::Worker {
    int rank = 0, device = 0;
    std::thread thread;
    std::mutex mu;
    std::condition_variable cv;
    std::function<void(int, EpContext &)> job;
    bool has_job = false, done = false, stop = false;
    std::exception_ptr error;
    std::unique_ptr<EpContext> ctx;
};

EpWorkerPool::EpWorkerPool(int world, std::vector<int> devices, const EpShape &shape, const EpOptions &options, std::chrono::milliseconds timeout)
    : world_(world)
{
    if (world < 1 || static_cast<int>(devices.size()) != world)
        throw std::runtime_error("bad rank count");
    group_ = std::make_shared<EpGroup>(world, timeout);
    const EpUniqueId id = ep_unique_id();
    for (int r = 0; r < world; r++) {
        workers_.emplace_back(new Worker);
        workers_.back()->rank = r;
        workers_.back()->device = devices[r];
    }
    for (int r = 0; r < world; r++) {
        Worker *w = workers_[r].get();
        w->thread = std::thread([this, w, id, shape, options] {
            // the context is made on the thread that will use it: construction is collective over the ranks' threads
            try {
                cuda_set_device(w->device);
                w->ctx.reset(new EpContext(group_, id, w->rank, world_, w->device, shape, options));
            } catch (...) {
                group_->leave(w->rank);
                std::lock_guard<std::mutex> lock(w->mu);
                w->error = std::current_exception();
            }
            {
                std::lock_guard<std::mutex> lock(w->mu);
                w->done = true; // "constructed" (or failed) -- the first hand-shake with the pool
            }
            w->cv.notify_all();
            for (;;) {
                std::function<void(int, EpContext &)> job;
                {
                    std::unique_lock<std::mutex> lock(w->mu);
                    w->cv.wait(lock, [&] { return w->has_job || w->stop; });
                    if (w->stop)
                        break;
                    job = w->job;
                    w->has_job = false;
                }
                std::exception_ptr err;
                try {
                    if (!w->ctx)
                        throw std::runtime_error("rank " + std::to_string(w->rank) + " has no context");
                    job(w->rank, *w->ctx);
                } catch (...) {
                    err = std::current_exception();
                    if (w->ctx)
                        w->ctx->abandon(); // peers waiting for this rank get "peer left"
                    else
                        group_->leave(w->rank);
                }
                {
                    std::lock_guard<std::mutex> lock(w->mu);
                    w->error = err;
                    w->done = true;
                }
                w->cv.notify_all();
            }
            w->ctx.reset(); // destroyed on its own thread, with its device current
        });
    }
    std::exception_ptr first;
    for (auto &w : workers_) {
        std::unique_lock<std::mutex> lock(w->mu);
        w->cv.wait(lock, [&] { return w->done; });
        w->done = false;
        if (w->error && !first)
            first = w->error;
        w->error = nullptr;
    }
    if (first) {
        for (auto &w : workers_) {
            {
                std::lock_guard<std::mutex> lock(w->mu);
                w->stop = true;
            }
            w->cv.notify_all();
            w->thread.join();
        }
        workers_.clear();
        std::rethrow_exception(first);
    }
}

EpWorkerPool::~EpWorkerPool()
{
    for (auto &w : workers_) {
        {
            std::lock_guard<std::mutex> lock(w->mu);
            w->stop = true;
        }
        w->cv.notify_all();
        if (w->thread.joinable())
            w->thread.join();
    }
}

void EpWorkerPool::dispatch(const std::function<void(int, EpContext &)> &fn)
{
    for (auto &w : workers_) {
        {
            std::lock_guard<std::mutex> lock(w->mu);
            w->job = fn;
            w->has_job = true;
            w->done = false;
            w->error = nullptr;
        }
        w->cv.notify_all();
    }
    std::exception_ptr first;
    for (auto &w : workers_) {
        std::unique_lock<std::mutex> lock(w->mu);
        w->cv.wait(lock, [&] { return w->done; });
        if (w->error && !first)
            first = w->error;
    }
    if (first)
        std::rethrow_exception(first);
}

void EpWorkerPool::on_every_rank(const std::function<void(int, EpContext &)> &fn)
{
    dispatch(fn);
}

std::vector<Tensor> EpWorkerPool::run(const std::vector<const Tensor *> &x, const std::vector<MoEWeights> &weights, const MoEConfig &config)
{
    if (static_cast<int>(x.size()) != world_ || static_cast<int>(weights.size()) != world_)
        throw std::runtime_error("bad rank count");
    std::vector<Tensor> out(world_);
    dispatch([&](int rank, EpContext &ctx) {
        if (!x[rank])
            throw std::runtime_error("missing input");
        out[rank] = moe(*x[rank], weights[rank], config, &ctx);
    });
    return out;
}
