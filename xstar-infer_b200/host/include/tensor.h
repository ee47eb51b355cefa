// Contiguous row-major buffer with a shape, an element kind and a home (host or device).
// Same contract as the engine's Tensor (reference xstar_cpp/include/tensor.h:16-98): move-only; either
// owns its bytes or borrows them; to_cuda / to_cpu are strict one-way raw copies.
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

#include "device.h"
#include "dtype.h"

class Tensor
{
public:
    using Shape = std::vector<std::int64_t>;

    // empty (shape {0}, no bytes): a slot to move a tensor into
    Tensor();
    // owning, uninitialised
    Tensor(Shape shape, DType dtype, Device device = Device::CPU);
    // borrowing view of memory that outlives this object
    Tensor(const void *ptr, Shape shape, DType dtype, Device device);
    // owning device tensor whose bytes come from, and return to, the result cache (cuda/cuda_allocator.h): what the MoE ops
    // return, so that a call costs no cudaMalloc / cudaFree once the sizes have been seen
    static Tensor result(Shape shape, DType dtype);
    ~Tensor();

    Tensor(const Tensor &) = delete;
    Tensor &operator=(const Tensor &) = delete;
    Tensor(Tensor &&other) noexcept;
    Tensor &operator=(Tensor &&other) noexcept;

    const Shape &shape() const { return shape_; }
    const Shape &strides() const { return strides_; }
    DType dtype() const { return dtype_; }
    Device device() const { return device_; }
    std::int64_t numel() const { return numel_; }
    std::size_t nbytes() const { return static_cast<std::size_t>(numel_) * dtype_size(dtype_); }
    std::int64_t dim(int i) const { return shape_[i < 0 ? shape_.size() + i : i]; }
    std::size_t rank() const { return shape_.size(); }

    void *data() { return bytes_; }
    const void *data() const { return bytes_; }
    template <typename T>
    T *data()
    {
        return static_cast<T *>(bytes_);
    }
    template <typename T>
    const T *data() const
    {
        return static_cast<const T *>(bytes_);
    }

private:
    void layout();
    void drop() noexcept;

    void *bytes_ = nullptr;
    Shape shape_;
    Shape strides_;
    std::int64_t numel_ = 1;
    DType dtype_ = DType::Float32;
    Device device_ = Device::CPU;
    bool owner_ = false;
    bool cached_ = false; // owner_ && bytes from the result cache
};

Tensor to_cuda(const Tensor &t); // throws unless t is on the CPU
Tensor to_cpu(const Tensor &t);  // throws unless t is on the device
