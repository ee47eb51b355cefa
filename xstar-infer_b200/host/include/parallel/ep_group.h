// Host-side rendezvous of the rank threads of one process that run an expert-parallel layer together (one thread per
// GPU).  It exists for failure detection: a collective step must not be launched while a peer is missing, because a
// collective kernel that waits for a rank that never joins occupies its GPU until someone aborts it.  So every rank
// checks in here BEFORE it enqueues a step; a peer that does not check in within the time limit, that has announced
// that it left, or that checks in with a different step signature turns into a C++ exception on the ranks that did
// arrive -- on the host, with nothing of the step launched.  The check-in costs a mutex and a condition variable; it does
// not wait for the GPU.
//
// No counterpart in the reference (single GPU; its failure handling is CHECK_CUDA's exception,
// xstar_cpp/include/cuda/cuda_check.h:23-31, whose message style the errors here follow).
#pragma once
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

class EpError : public std::runtime_error
{
public:
    using std::runtime_error::runtime_error;
};

class EpGroup
{
public:
    EpGroup(int world, std::chrono::milliseconds timeout);

    int world() const { return world_; }
    std::chrono::milliseconds timeout() const { return timeout_; }

    // All `world` ranks call arrive(rank, signature) once per step; it returns on every rank when all have arrived with
    // the same signature.  Throws EpError on the waiting ranks:
    //   "peer timeout: rank R did not arrive"      a rank is late by more than the time limit
    //   "peer left: rank R"                        a rank called leave()
    //   "step mismatch: rank R ..."                signatures differ (shapes, formats or step counts disagree)
    // After an error the group stays broken: every later arrive() throws at once ("group is broken: ...").
    void arrive(int rank, std::uint64_t signature);

    // A rank that will not take part any more (its thread is unwinding) says so; never blocks.
    void leave(int rank) noexcept;

    // Small blackboard for start-up: each rank posts a blob, and after the next arrive() all ranks can read all blobs
    // (buffer addresses of ranks that live in one process travel this way).
    void post(int rank, std::vector<std::uint8_t> blob);
    std::vector<std::uint8_t> read(int rank) const;

    bool broken() const;

private:
    void fail_locked(const std::string &why);

    const int world_;
    const std::chrono::milliseconds timeout_;
    mutable std::mutex mu_;
    std::condition_variable cv_;
    std::uint64_t generation_ = 0;
    int arrived_ = 0;
    std::vector<char> here_, gone_;
    std::vector<std::uint64_t> signature_;
    std::vector<std::vector<std::uint8_t>> blobs_;
    std::string broken_;
};
