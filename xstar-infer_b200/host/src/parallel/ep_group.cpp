#include "parallel/ep_group.h"

EpGroup::EpGroup(int world, std::chrono::milliseconds timeout)
    : world_(world), timeout_(timeout), here_(world > 0 ? world : 0, 0), gone_(world > 0 ? world : 0, 0), signature_(world > 0 ? world : 0, 0),
      blobs_(world > 0 ? world : 0)
{
    if (world < 1)
        throw EpError("bad world size");
}

void EpGroup::fail_locked(const std::string &why)
{
    if (broken_.empty())
        broken_ = why;
    cv_.notify_all();
}

bool EpGroup::broken() const
{
    std::lock_guard<std::mutex> lock(mu_);
    return !broken_.empty();
}

void EpGroup::arrive(int rank, std::uint64_t signature)
{
    std::unique_lock<std::mutex> lock(mu_);
    if (rank < 0 || rank >= world_)
        throw EpError("bad rank");
    if (!broken_.empty())
        throw EpError("group is broken: " + broken_);
    for (int r = 0; r < world_; r++)
        if (gone_[r]) {
            fail_locked("peer left: rank " + std::to_string(r));
            throw EpError(broken_);
        }
    if (here_[rank]) {
        fail_locked("step mismatch: rank " + std::to_string(rank) + " arrived twice in one step");
        throw EpError(broken_);
    }
    here_[rank] = 1;
    signature_[rank] = signature;
    arrived_++;
    const std::uint64_t my_generation = generation_;
    if (arrived_ == world_) {
        for (int r = 0; r < world_; r++)
            if (signature_[r] != signature) {
                fail_locked("step mismatch: rank " + std::to_string(r) + " posted a different step signature than rank " +
                            std::to_string(rank));
                throw EpError(broken_);
            }
        arrived_ = 0;
        for (int r = 0; r < world_; r++)
            here_[r] = 0;
        generation_++;
        cv_.notify_all();
        return;
    }
    const bool done = cv_.wait_for(lock, timeout_, [&] { return generation_ != my_generation || !broken_.empty(); });
    if (generation_ != my_generation)
        return; // the step was released (an error recorded later belongs to a later step)
    if (!done) {
        int missing = -1;
        for (int r = 0; r < world_; r++)
            if (!here_[r]) {
                missing = r;
                break;
            }
        fail_locked("peer timeout: rank " + std::to_string(missing) + " did not arrive within " + std::to_string(timeout_.count()) + " ms");
    }
    throw EpError(broken_);
}

void EpGroup::leave(int rank) noexcept
{
    try {
        std::lock_guard<std::mutex> lock(mu_);
        if (rank >= 0 && rank < world_ && !gone_[rank]) {
            gone_[rank] = 1;
            if (arrived_ > 0) // ranks are waiting for this one right now
                fail_locked("peer left: rank " + std::to_string(rank));
        }
    } catch (...) {
    }
}

void EpGroup::post(int rank, std::vector<std::uint8_t> blob)
{
    std::lock_guard<std::mutex> lock(mu_);
    if (rank < 0 || rank >= world_)
        throw EpError("bad rank");
    blobs_[rank] = std::move(blob);
}

std::vector<std::uint8_t> EpGroup::read(int rank) const
{
    std::lock_guard<std::mutex> lock(mu_);
    if (rank < 0 || rank >= world_)
        throw EpError("bad rank");
    return blobs_[rank];
}
