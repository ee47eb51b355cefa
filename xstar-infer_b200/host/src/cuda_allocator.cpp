#include "cuda/cuda_allocator.h"

#include <map>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>

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

namespace {
struct ResultCache {
    std::mutex mu;
    std::map<std::pair<int, std::size_t>, std::vector<void *>> free_blocks;       // (device, class bytes) -> blocks
    std::unordered_map<void *, std::pair<int, std::size_t>> live;                 // block -> (device, class bytes)
    std::size_t cached = 0;
};
ResultCache &result_cache()
{
    static ResultCache c;
    return c;
}
std::size_t size_class(std::size_t bytes)
{
    std::size_t c = 4096;
    while (c < bytes)
        c <<= 1;
    return c;
}
} // namespace

void *cuda_alloc_cached(std::size_t bytes)
{
    const int dev = cuda_current_device();
    const std::size_t cls = size_class(bytes);
    ResultCache &c = result_cache();
    {
        std::lock_guard<std::mutex> g(c.mu);
        auto it = c.free_blocks.find({dev, cls});
        if (it != c.free_blocks.end() && !it->second.empty()) {
            void *p = it->second.back();
            it->second.pop_back();
            c.cached -= cls;
            c.live[p] = {dev, cls};
            return p;
        }
    }
    void *p = cuda_alloc(cls);
    std::lock_guard<std::mutex> g(c.mu);
    c.live[p] = {dev, cls};
    return p;
}

void cuda_free_cached(void *ptr) noexcept
{
    if (!ptr)
        return;
    ResultCache &c = result_cache();
    try {
        std::lock_guard<std::mutex> g(c.mu);
        auto it = c.live.find(ptr);
        if (it == c.live.end()) {
            cuda_free(ptr); // not one of ours
            return;
        }
        c.free_blocks[it->second].push_back(ptr);
        c.cached += it->second.second;
        c.live.erase(it);
    } catch (...) {
    }
}

std::size_t cuda_cached_result_bytes()
{
    ResultCache &c = result_cache();
    std::lock_guard<std::mutex> g(c.mu);
    return c.cached;
}

void cuda_trim_cached() noexcept
{
    ResultCache &c = result_cache();
    std::lock_guard<std::mutex> g(c.mu);
    for (auto &kv : c.free_blocks)
        for (void *p : kv.second)
            cuda_free(p);
    c.free_blocks.clear();
    c.cached = 0;
}

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
