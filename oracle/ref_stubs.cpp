/*
 * TEST INFRASTRUCTURE ONLY.  The reference's host ops are compiled in place with g++ for their CPU
 * branches; their CUDA branches call launch functions and allocator wrappers that live in .cu files.
 * This file satisfies those symbols so the CPU-only build links.  Every stub throws: nothing here can
 * be reached by the CPU composition in ref_compose.cpp.
 *
 * Declarations come from the reference's own headers, so signatures cannot drift.
 */
#include <stdexcept>

#include "cuda/cuda_allocator.h"
#include "ops/add.h"
#include "ops/embedding.h"
#include "ops/gemm.h"
#include "ops/mlp.h"
#include "ops/rmsnorm.h"
#include "ops/softmax.h"

[[noreturn]] static void no_cuda()
{
    throw std::runtime_error("reference CPU-only build: CUDA path not available");
}

void *cuda_alloc(std::size_t) { no_cuda(); }
void cuda_free(void *) {}
void cuda_memcpy_h2d(void *, const void *, std::size_t) { no_cuda(); }
void cuda_memcpy_d2h(void *, const void *, std::size_t) { no_cuda(); }
void cuda_memcpy_d2d(void *, const void *, std::size_t) { no_cuda(); }
std::size_t cuda_free_bytes() { no_cuda(); }

void gemm_launch(void *, const void *, const void *, const void *, std::int64_t, std::int64_t, std::int64_t, bool,
                 std::int64_t, std::int64_t, std::int64_t, DType)
{
    no_cuda();
}
void gemm_silu_and_mul_launch(void *, const void *, const void *, std::int64_t, std::int64_t, std::int64_t,
                              std::int64_t, DType)
{
    no_cuda();
}
void embedding_launch(void *, const void *, const std::int64_t *, std::int64_t, std::int64_t, DType) { no_cuda(); }
void add_launch(void *, const void *, const void *, std::int64_t, DType) { no_cuda(); }
void softmax_launch(void *, const void *, std::int64_t, std::int64_t, std::int64_t, DType) { no_cuda(); }
void rmsnorm_launch(void *, const void *, const void *, std::int64_t, std::int64_t, float, DType) { no_cuda(); }
