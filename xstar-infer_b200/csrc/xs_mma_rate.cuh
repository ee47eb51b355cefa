// Tensor-pipe rate probe: every CTA (one per SM) issues `iters` tcgen05.mma instructions of one shape on zeroed shared
// memory, commits, waits (bounded) and reports cycles.  It answers two questions the kernels' tile shapes depend on:
// how long one MMA of M = 128 occupies the pipe as a function of N, and what the dense FP8 / block-scaled peak of this
// part is under load.  A tuning aid, not part of the layer.
#pragma once
#include "xs_ptx.cuh"

namespace xs {

// kind: 0 = f16 (bf16 operands, K = 16), 1 = f8f6f4 (e4m3, K = 32), 2 = mxf8f6f4.block_scale (e4m3 x e2m1, K = 32),
//       3 = kind 2 with three tcgen05.cp.32x128b.warpx4 scale copies before every four MMAs (one 128-deep k-block of a
//           block-scaled GEMM whose issuing thread also moves the scales from shared memory to TMEM),
//       4 / 5 = kind 1 issued the way a k-block loop with per-k-block accumulators issues it: every four MMAs start a
//           fresh accumulation in the other of two accumulators and are followed by two (4) or one (5) tcgen05.commit,
//       6 = kind 5 with the issuing thread WAITING for each group's commit before it issues the next group: cycles per
//           MMA x 4 is then the latency from issuing a k-block to seeing its completion on an mbarrier
__global__ void __launch_bounds__(64, 1)
mma_rate_kernel(int kind, int n, int iters, int chains, unsigned long long *cycles, int32_t *status)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar;
    __shared__ uint64_t side_bar[2]; // targets of the per-group commits of kinds 4 and 5; nobody waits on them
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;
    // A: 128 rows x 128 B, B: 256 rows x 128 B, scale block 1.5 KB
    for (int i = threadIdx.x; i < (128 + 256) * 128 / 16 + 96; i += blockDim.x)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init(&side_bar[0], 1);
        mbar_init(&side_bar[1], 1);
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
        const uint32_t sf_t = tmem_base + 2 * 256 - 16; // last 16 columns hold scales (block-scaled kind: chains * n <= 496)
        if (kind == 2 || kind == 3) {
            tmem_cp_32x128b_x4(sf_t, make_desc_rows16(sfs));
            tmem_cp_32x128b_x4(sf_t + 4, make_desc_rows16(sfs + 512));
            tmem_cp_32x128b_x4(sf_t + 8, make_desc_rows16(sfs + 1024));
        }
        // descriptors and accumulator columns are fixed before the clock starts; the loop body is four bare MMAs
        uint32_t idesc[4], dcol[4];
        for (int j = 0; j < 4; j++) {
            dcol[j] = tmem_base + static_cast<uint32_t>((j % chains) * n); // `chains` (1, 2 or 4) independent accumulators
            idesc[j] = kind == 0 ? make_idesc(1, 1, 128, n) : ((kind == 1 || kind >= 4) ? make_idesc(0, 0, 128, n) : make_idesc_mx(0, 5, 128, n, j));
        }
        const long long t0 = clock64();
        for (int i = 0; i < iters; i += 4) {
            if (kind == 3) {
                tmem_cp_32x128b_x4(sf_t, make_desc_rows16(sfs));
                tmem_cp_32x128b_x4(sf_t + 4, make_desc_rows16(sfs + 512));
                tmem_cp_32x128b_x4(sf_t + 8, make_desc_rows16(sfs + 1024));
            }
            if (kind >= 4) {
                const uint32_t d = tmem_base + static_cast<uint32_t>(((i >> 2) & 1) * n);
#pragma unroll
                for (int j = 0; j < 4; j++)
                    mma_f8(d, da + 2 * j, db + 2 * j, idesc[j], j ? 1u : 0u);
                tc_commit(&side_bar[0]);
                if (kind == 4)
                    tc_commit(&side_bar[1]);
                if (kind == 6 && !mbar_wait(&side_bar[0], (i >> 2) & 1, &abort_flag)) {
                    atomicOr(status, 1);
                    break;
                }
                continue;
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t acc = (i + j) >= chains ? 1u : 0u;
                if (kind == 0)
                    mma_bf16(dcol[j], da + 2 * j, db + 2 * j, idesc[j], acc);
                else if (kind == 1)
                    mma_f8(dcol[j], da + 2 * j, db + 2 * j, idesc[j], acc);
                else
                    mma_mxf8f6f4(dcol[j], da + 2 * j, db + 2 * j, idesc[j], sf_t, sf_t + 4, acc);
            }
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

// TMEM -> register read rate: `warps` warps (4, 8, 12 or 16; warp w reads the lane quarter w % 4) each read
// 32 lanes x 64 columns per iteration and wait, with the loads issued as
//   shape 0: two pairs of .32x32b.x16, a wait after each pair   shape 1: four .x16, one wait
//   shape 2: two .x32, one wait                                 shape 3: one .x64, one wait
// while (with_mma) one more warp keeps the tensor pipe busy with N = 256 e4m3 MMAs into the other half of TMEM.
// Reports the cycles of the slowest reading warp, the cycles of the MMA stream, and the CTA count.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, "
        "%45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]),
          "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]),
          "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]),
          "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr));
}

__global__ void __launch_bounds__(544, 1)
tmem_ld_rate_kernel(int shape, int warps, int iters, int with_mma, int mma_iters, unsigned long long *cycles, int32_t *status)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;
    __shared__ unsigned long long s_max;
    for (int i = threadIdx.x; i < (128 + 256) * 128 / 16; i += blockDim.x)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        s_max = 0;
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    uint32_t sink = 0;
    if (warp < warps) {
        const uint32_t t0a = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const long long t0 = clock64();
        for (int i = 0; i < iters; i++) {
            const uint32_t c = t0a + static_cast<uint32_t>((i & 3) * 64);
            if (shape == 0) {
                uint32_t a[16], b[16];
                tmem_ld16(c, a);
                tmem_ld16(c + 16, b);
                tmem_ld_wait_for(a, b);
                sink ^= a[0] ^ b[15];
                tmem_ld16(c + 32, a);
                tmem_ld16(c + 48, b);
                tmem_ld_wait_for(a, b);
                sink ^= a[1] ^ b[14];
            } else if (shape == 1) {
                uint32_t a[16], b[16], d[16], e[16];
                tmem_ld16(c, a);
                tmem_ld16(c + 16, b);
                tmem_ld16(c + 32, d);
                tmem_ld16(c + 48, e);
                tmem_ld_wait_for(a, b);
                tmem_ld_wait_for(d, e);
                sink ^= a[0] ^ b[15] ^ d[3] ^ e[7];
            } else if (shape == 2) {
                uint32_t a[32], b[32];
                tmem_ld32(c, a);
                tmem_ld32(c + 32, b);
                tmem_ld_wait();
                asm volatile("" : "+r"(a[0]), "+r"(b[31]));
                sink ^= a[0] ^ b[31];
            } else {
                uint32_t a[64];
                tmem_ld64(c, a);
                tmem_ld_wait();
                asm volatile("" : "+r"(a[0]), "+r"(a[63]));
                sink ^= a[0] ^ a[63];
            }
        }
        const long long t1 = clock64();
        if (lane == 0)
            atomicMax(&s_max, static_cast<unsigned long long>(t1 - t0));
    } else if (warp == warps && with_mma) {
        if (lane == 0) {
            const uint32_t sa = smem_u32(smem);
            const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sa + 128 * 128);
            const uint32_t idesc = make_idesc(0, 0, 128, 256);
            const uint32_t d = tmem_base + 256;
            const long long t0 = clock64();
            for (int i = 0; i < mma_iters; i += 4) {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    mma_f8(d, da + 2 * j, db + 2 * j, idesc, (i + j) ? 1u : 0u);
            }
            tc_commit(&bar);
            const bool ok = mbar_wait(&bar, 0, &abort_flag);
            const long long t1 = clock64();
            if (!ok)
                atomicOr(status, 1);
            atomicAdd(&cycles[1], static_cast<unsigned long long>(t1 - t0));
        }
    }
    if (sink == 0x9e3779b9u && lane == 0) // keeps the loaded values alive
        atomicOr(status, 0);
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        atomicAdd(&cycles[0], s_max);
        atomicAdd(&cycles[2], 1ull);
    }
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Accumulator hand-over round trip: one thread issues k-blocks of four N = 256 e4m3 MMAs alternately into two TMEM
// buffers, committing each to a "full" barrier; `resp` responder warps wait for it, (optionally) read `ld_cols` columns
// of the buffer, and arrive on the buffer's "empty" barrier, which the issuer waits for before it reuses the buffer --
// the protocol of a GEMM whose accumulator changes hands every k-block, with nothing else in the way.
// mode bit 0: responders poll with mbarrier.test_wait instead of try_wait; bit 1: the issuer does too;
// bit 2: no tcgen05 fences around the waits; bit 3: a second issuer warp takes the odd k-blocks.
__global__ void __launch_bounds__(640, 1)
handoff_rate_kernel(int resp, int iters, int mode, int ld_cols, unsigned long long *cycles, int32_t *status)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[2], empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;
    for (int i = threadIdx.x; i < (128 + 256) * 128 / 16; i += blockDim.x)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        for (int b = 0; b < 2; b++) {
            mbar_init(&full[b], 1);
            mbar_init(&empty[b], resp);
        }
        abort_flag = 0;
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const bool two_issuers = (mode & 8) != 0;
    auto wait = [&](uint64_t *bar, uint32_t parity, bool spin) { return spin ? mbar_spin_wait(bar, parity, &abort_flag) : mbar_wait(bar, parity, &abort_flag); };
    if (warp == 0 || (two_issuers && warp == 1)) {
        if (lane == 0) {
            const uint32_t sa = smem_u32(smem);
            const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sa + 128 * 128);
            const uint32_t idesc = make_idesc(0, 0, 128, 256);
            const int first = two_issuers ? warp : 0, step = two_issuers ? 2 : 1;
            bool ok = true;
            const long long t0 = clock64();
            for (int i = first; i < iters && ok; i += step) {
                const int b = i & 1;
                ok = wait(&empty[b], ((i >> 1) & 1) ^ 1, (mode & 2) != 0);
                if (!(mode & 4))
                    tc_fence_after();
#pragma unroll
                for (int j = 0; j < 4; j++)
                    mma_f8(tmem_base + b * 256, da + 2 * j, db + 2 * j, idesc, j ? 1u : 0u);
                tc_commit(&full[b]);
            }
            const long long t1 = clock64();
            if (!ok) {
                abort_flag = 1;
                atomicOr(status, 1);
            }
            if (warp == 0) {
                atomicAdd(&cycles[0], static_cast<unsigned long long>(t1 - t0));
                atomicAdd(&cycles[2], 1ull);
            }
        }
    } else if (warp >= 4 && warp < 4 + resp) {
        bool ok = true;
        uint32_t sink = 0;
        for (int i = 0; i < iters && ok; i++) {
            const int b = i & 1;
            ok = wait(&full[b], (i >> 1) & 1, (mode & 1) != 0);
            if (!(mode & 4))
                tc_fence_after();
            for (int c = 0; c < ld_cols; c += 32) {
                uint32_t x[16], y[16];
                const uint32_t t = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + b * 256 + ((warp - 4) >> 2) * 64 + c;
                tmem_ld16(t, x);
                tmem_ld16(t + 16, y);
                tmem_ld_wait_for(x, y);
                sink ^= x[0] ^ y[15];
            }
            if (!(mode & 4))
                tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&empty[b]);
        }
        if (sink == 0x9e3779b9u && lane == 0)
            atomicOr(status, 0);
        if (!ok && lane == 0) {
            abort_flag = 1;
            atomicOr(status, 1);
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

} // namespace xs
