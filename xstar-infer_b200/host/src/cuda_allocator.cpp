#include "cuda/cuda_allocator.h"

#include <stdexcept>
#include <string>

#include "xs_moe.h"

namespace {
void raise_if(int rc)
{
    if (rc != 0)
        throw std::runtime_error(std::string(xs_moe_last_error()));
}
} // namespace

void *cuda_alloc(std::size_t bytes)
{
    void *p = nullptr;
    raise_if(xs_moe_device_alloc(&p, bytes));
    return p;
}
void cuda_free(void *ptr) noexcept
{
    if (ptr)
        xs_moe_device_free(ptr);
}
void cuda_memcpy_h2d(void *dst, const void *src, std::size_t bytes) { raise_if(xs_moe_memcpy_h2d(dst, src, bytes)); }
void cuda_memcpy_d2h(void *dst, const void *src, std::size_t bytes) { raise_if(xs_moe_memcpy_d2h(dst, src, bytes)); }
void cuda_memcpy_d2d(void *dst, const void *src, std::size_t bytes) { raise_if(xs_moe_memcpy_d2d(dst, src, bytes)); }
std::size_t cuda_free_bytes()
{
    std::size_t b = 0;
    raise_if(xs_moe_device_free_bytes(&b));
    return b;
}

int cuda_current_device()
{
    int32_t d = 0;
    raise_if(xs_moe_current_device(&d));
    return d;
}
void cuda_set_device(int device) { raise_if(xs_moe_set_device(device)); }

WorkspacePool &WorkspacePool::instance()
{
    static WorkspacePool pool;
    return pool;
}

WorkspacePool::Lease WorkspacePool::acquire(std::size_t bytes)
{
    const int dev = cuda_current_device();
    {
        std::lock_guard<std::mutex> g(mu_);
        // smallest cached block of THIS device that fits
        int best = -1;
        for (int i = 0; i < static_cast<int>(free_.size()); i++)
            if (free_[i].device == dev && free_[i].bytes >= bytes && (best < 0 || free_[i].bytes < free_[best].bytes))
                best = i;
        if (best >= 0) {
            Lease l = free_[best];
            free_.erase(free_.begin() + best);
            return l;
        }
        // nothing fits: drop this device's cached blocks so the pool does not hold stale smaller buffers
        for (std::size_t i = 0; i < free_.size();) {
            if (free_[i].device == dev) {
                cuda_free(free_[i].ptr);
                free_.erase(free_.begin() + static_cast<std::ptrdiff_t>(i));
            } else {
                i++;
            }
        }
    }
    Lease l;
    l.device = dev;
    l.bytes = (bytes + 255) / 256 * 256;
    l.ptr = cuda_alloc(l.bytes);
    raise_if(xs_moe_workspace_init(l.ptr, l.bytes, nullptr));
    raise_if(xs_moe_stream_synchronize(nullptr));
    return l;
}

void WorkspacePool::release(Lease lease) noexcept
{
    if (!lease.ptr)
        return;
    std::lock_guard<std::mutex> g(mu_);
    free_.push_back(lease);
}

void WorkspacePool::trim() noexcept
{
    std::lock_guard<std::mutex> g(mu_);
    for (auto &l : free_)
        cuda_free(l.ptr);
    free_.clear();
}

std::size_t WorkspacePool::cached_bytes() const
{
    std::lock_guard<std::mutex> g(mu_);
    std::size_t n = 0;
    for (auto &l : free_)
        n += l.bytes;
    return n;
}
