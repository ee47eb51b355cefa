// Device memory for host-side C++: raw allocation, synchronous copies, a free-memory probe and a
// workspace pool.  CUDA-free header: the functions forward to the C ABI of the kernel library
// (include/xs_moe.h), so translation units compiled by g++ never see a CUDA header -- the same layering
// as the reference's allocator wrappers (xstar_cpp/include/cuda/cuda_allocator.h:32-69), with
// "CUDA error: ..." runtime_errors on failure like CHECK_CUDA (xstar_cpp/include/cuda/cuda_check.h:23-31).
#pragma once
#include <cstddef>
#include <mutex>
#include <vector>

void *cuda_alloc(std::size_t bytes);
void cuda_free(void *ptr) noexcept;
void cuda_memcpy_h2d(void *dst, const void *src, std::size_t bytes);
void cuda_memcpy_d2h(void *dst, const void *src, std::size_t bytes);
void cuda_memcpy_d2d(void *dst, const void *src, std::size_t bytes);
std::size_t cuda_free_bytes();
int cuda_current_device();
void cuda_set_device(int device);

// Grow-only arena for per-call scratch.  The reference allocates every temporary with cudaMalloc and frees
// it when the Tensor dies (xstar_cpp/src/tensor.cpp:34-37); an MoE call needs a dozen temporaries, so the
// op leases ONE buffer from this pool and carves it up.  A lease is exclusive; returning it keeps the
// memory for the next call on the same device (blocks are keyed by the device that was current when they were
// allocated).  trim() gives everything back to the driver.
class WorkspacePool
{
public:
    struct Lease {
        void *ptr = nullptr;
        std::size_t bytes = 0;
        int device = 0; // the device the block lives on: a lease is only ever handed to a call on that device
    };
    static WorkspacePool &instance();
    Lease acquire(std::size_t bytes);
    void release(Lease lease) noexcept;
    void trim() noexcept;
    std::size_t cached_bytes() const;

private:
    mutable std::mutex mu_;
    std::vector<Lease> free_;
};

// Recycled device blocks for RESULT tensors.  The reference's ops return a fresh Tensor whose bytes come from cudaMalloc
// and go back with cudaFree (xstar_cpp/src/tensor.cpp:34-37) -- two device-wide synchronisations per call.  The MoE ops
// take their results from this cache instead: blocks are kept per device and size class (powers of two from 4 KB) and
// handed out again once their Tensor died.  A block goes back as soon as its Tensor is destroyed; with the synchronous ops
// ("returns => finished") that is always after the work that wrote it, and a caller of the stream forms must keep a result
// alive until its stream has passed the call, as with any asynchronous API.
void *cuda_alloc_cached(std::size_t bytes);
void cuda_free_cached(void *ptr) noexcept;
std::size_t cuda_cached_result_bytes();
void cuda_trim_cached() noexcept;

// RAII lease
class Workspace
{
public:
    explicit Workspace(std::size_t bytes) : lease_(WorkspacePool::instance().acquire(bytes)) {}
    ~Workspace() { WorkspacePool::instance().release(lease_); }
    Workspace(const Workspace &) = delete;
    Workspace &operator=(const Workspace &) = delete;
    void *data() const { return lease_.ptr; }
    std::size_t bytes() const { return lease_.bytes; }

private:
    WorkspacePool::Lease lease_;
};
