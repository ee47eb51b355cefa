// Tensor-pipe rate probe: every CTA (one per SM) issues `iters` tcgen05.mma instructions of one shape on zeroed shared
// memory, commits, waits (bounded) and reports cycles.  It answers two questions the kernels' tile shapes depend on:
// how long one MMA of M = 128 occupies the pipe as a function of N, and what the dense FP8 / block-scaled peak of this
// part is under load.  A tuning aid, not part of the layer.
#pragma once
#include "xs_ptx.cuh"

namespace xs {

// kind: 0 = f16 (bf16 operands, K = 16), 1 = f8f6f4 (e4m3, K = 32), 2 = mxf8f6f4.block_scale (e4m3 x e2m1, K = 32)
__global__ void __launch_bounds__(64, 1)
mma_rate_kernel(int kind, int n, int iters, int chains, unsigned long long *cycles, int32_t *status)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;
    // A: 128 rows x 128 B, B: 256 rows x 128 B, scale block 1.5 KB
    for (int i = threadIdx.x; i < (128 + 256) * 128 / 16 + 96; i += blockDim.x)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    if ((threadIdx.x >> 5) == 0) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        const uint32_t sa = smem_u32(smem);
        const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sa + 128 * 128);
        const uint32_t sfs = sa + (128 + 256) * 128;
        const uint32_t sf_t = tmem_base + 2 * 256 - 16; // last 16 columns hold scales (only used when 2 * n <= 496)
        if (kind == 2) {
            tmem_cp_32x128b_x4(sf_t, make_desc_rows16(sfs));
            tmem_cp_32x128b_x4(sf_t + 4, make_desc_rows16(sfs + 512));
            tmem_cp_32x128b_x4(sf_t + 8, make_desc_rows16(sfs + 1024));
        }
        const long long t0 = clock64();
        for (int i = 0; i < iters; i++) {
            const uint32_t d = tmem_base + static_cast<uint32_t>((i % chains) * n); // `chains` independent accumulators
            const uint32_t acc = i >= chains ? 1u : 0u;
            const uint64_t ka = da + 2 * (i & 3), kb = db + 2 * (i & 3);
            if (kind == 0)
                mma_bf16(d, ka, kb, make_idesc(1, 1, 128, n), acc);
            else if (kind == 1)
                mma_f8(d, ka, kb, make_idesc(0, 0, 128, n), acc);
            else
                mma_mxf8f6f4(d, ka, kb, make_idesc_mx(0, 5, 128, n, i & 3), sf_t, sf_t + 4, acc);
        }
        const long long t_issue = clock64();
        tc_commit(&bar);
        const bool ok = mbar_wait(&bar, 0, &abort_flag);
        const long long t1 = clock64();
        if (!ok)
            atomicOr(status, 1);
        atomicAdd(&cycles[0], static_cast<unsigned long long>(t1 - t0));
        atomicAdd(&cycles[1], static_cast<unsigned long long>(t_issue - t0));
        atomicAdd(&cycles[2], 1ull);
    }
    tc_fence_before();
    __syncthreads();
    if ((threadIdx.x >> 5) == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

} // namespace xs
