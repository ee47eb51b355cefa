#include "tensor.h"

#include <cstdlib>
#include <new>
#include <stdexcept>
#include <utility>

#include "cuda/cuda_allocator.h"

namespace {
constexpr std::size_t kHostAlign = 64;
std::size_t padded(std::size_t n)
{
    n = (n + kHostAlign - 1) / kHostAlign * kHostAlign;
    return n ? n : kHostAlign;
}
} // namespace

void Tensor::layout()
{
    strides_.assign(shape_.size(), 1);
    numel_ = 1;
    for (std::size_t i = shape_.size(); i-- > 0;) {
        if (shape_[i] < 0)
            throw std::runtime_error("negative dimension");
        strides_[i] = numel_;
        numel_ *= shape_[i];
    }
}

Tensor::Tensor() : shape_{0}
{
    layout();
}

Tensor::Tensor(Shape shape, DType dtype, Device device) : shape_(std::move(shape)), dtype_(dtype), device_(device), owner_(true)
{
    layout();
    const std::size_t n = padded(nbytes());
    if (device_ == Device::CPU)
        bytes_ = std::aligned_alloc(kHostAlign, n);
    else if (device_ == Device::CUDA)
        bytes_ = cuda_alloc(n);
    else
        throw std::runtime_error("unsupported device");
    if (!bytes_)
        throw std::bad_alloc();
}

Tensor::Tensor(const void *ptr, Shape shape, DType dtype, Device device)
    : bytes_(const_cast<void *>(ptr)), shape_(std::move(shape)), dtype_(dtype), device_(device), owner_(false)
{
    layout();
}

Tensor Tensor::result(Shape shape, DType dtype)
{
    Tensor t(nullptr, std::move(shape), dtype, Device::CUDA);
    t.bytes_ = cuda_alloc_cached(padded(t.nbytes()));
    t.owner_ = true;
    t.cached_ = true;
    return t;
}

void Tensor::drop() noexcept
{
    if (owner_ && bytes_) {
        if (device_ == Device::CPU)
            std::free(bytes_);
        else if (cached_)
            cuda_free_cached(bytes_);
        else
            cuda_free(bytes_);
    }
    bytes_ = nullptr;
}

Tensor::~Tensor()
{
    drop();
}

Tensor::Tensor(Tensor &&o) noexcept
    : bytes_(std::exchange(o.bytes_, nullptr)), shape_(std::move(o.shape_)), strides_(std::move(o.strides_)), numel_(o.numel_),
      dtype_(o.dtype_), device_(o.device_), owner_(o.owner_), cached_(o.cached_)
{
}

Tensor &Tensor::operator=(Tensor &&o) noexcept
{
    if (this != &o) {
        drop();
        bytes_ = std::exchange(o.bytes_, nullptr);
        shape_ = std::move(o.shape_);
        strides_ = std::move(o.strides_);
        numel_ = o.numel_;
        dtype_ = o.dtype_;
        device_ = o.device_;
        owner_ = o.owner_;
        cached_ = o.cached_;
    }
    return *this;
}

Tensor to_cuda(const Tensor &t)
{
    if (t.device() != Device::CPU)
        throw std::runtime_error("to_cuda: tensor is not on the CPU");
    Tensor out(t.shape(), t.dtype(), Device::CUDA);
    cuda_memcpy_h2d(out.data(), t.data(), t.nbytes());
    return out;
}

Tensor to_cpu(const Tensor &t)
{
    if (t.device() != Device::CUDA)
        throw std::runtime_error("to_cpu: tensor is not on the device");
    Tensor out(t.shape(), t.dtype(), Device::CPU);
    cuda_memcpy_d2h(out.data(), t.data(), t.nbytes());
    return out;
}
