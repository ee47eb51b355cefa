// Grouped expert GEMMs for sm_100a: tcgen05 MMA with TMEM accumulators, operands staged by TMA.
//
// The product computed per expert segment is  D[feature, token] = W_e[feature, :] . X[token, :]
// ("swap-AB"): the 128 rows of a weight tile are the MMA's M dimension and the tokens routed to the
// expert are its N dimension (16..128 per tile).  Decode-sized batches have a handful of tokens per
// expert, so the weight stream -- the bytes that bound the layer -- fills full 128-row tensor-core tiles
// whatever the token count is, and every weight byte is fetched from HBM exactly once per token tile.
//
// One persistent CTA per SM, six warps:
//   warp 0      TMA producer   (one elected lane)
//   warp 1      MMA issuer     (one elected lane) and TMEM owner
//   warps 2..5  epilogue: TMEM -> registers -> (SwiGLU) -> global, one TMEM lane quarter each
// Shared-memory stages and the two TMEM accumulator buffers are handed over through mbarriers, so the
// epilogue of one tile overlaps the weight stream of the next.
#pragma once
#include "xs_ptx.cuh"
#include <cuda_bf16.h>

namespace xs {

constexpr int kGemmThreads = 192;
constexpr int kTileM = 128;    // weight rows per tile (MMA M)
constexpr int kBlockK = 64;    // bf16 elements per 128-byte swizzled row
constexpr int kUmmaK = 16;     // K of one tcgen05.mma kind::f16

// status bits written by kernels (also used by the other kernels of the library)
constexpr int kStatusWaitTimeout = 1;
constexpr int kStatusBadIndex = 2;

// overflow-stable SiLU, the reference's form (xstar_cpp/src/ops/mlp.cpp:10-26): never exponentiates a positive argument
__device__ __forceinline__ float silu_f32(float x)
{
    float s = (x >= 0.0f) ? 1.0f / (1.0f + expf(-x)) : expf(x) / (1.0f + expf(x));
    return x * s;
}

struct GemmSmemLayout {
    int stage_bytes;
    int stages;
    int total_bytes;
};

__host__ __device__ constexpr int gemm_stage_bytes(int n_tile, bool gate_up)
{
    return (gate_up ? 2 : 1) * kTileM * kBlockK * 2 + n_tile * kBlockK * 2;
}

// tile table entry: which expert, first row of the token tile (global row in the permuted matrix)
struct TileTable {
    const int32_t *tile_expert;
    const int32_t *tile_row0;
    const int32_t *num_tiles; // device scalar
};

template <int N_TILE, bool GATE_UP>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                         const int32_t *__restrict__ offsets, TileTable tt, int w_rows_per_expert, int n_out, int K,
                         void *__restrict__ out, int32_t *__restrict__ status, int stages)
{
    constexpr int A_BYTES = kTileM * kBlockK * 2;
    constexpr int B_BYTES = N_TILE * kBlockK * 2;
    constexpr int STAGE_BYTES = (GATE_UP ? 2 : 1) * A_BYTES + B_BYTES;
    constexpr int ACC_COLS = (GATE_UP ? 2 : 1) * N_TILE;            // TMEM columns of one accumulator buffer
    constexpr int TMEM_COLS = (2 * ACC_COLS) < 32 ? 32 : 2 * ACC_COLS; // power of two >= 32 (N_TILE is a power of two)
    constexpr uint32_t IDESC = make_idesc(1, 1, kTileM, N_TILE);

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(stages) * STAGE_BYTES);
    uint64_t *full = bars;
    uint64_t *empty = bars + stages;
    uint64_t *tmem_full = bars + 2 * stages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4); // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_f_tiles = n_out / kTileM;
    const int num_tiles = *tt.num_tiles;
    const int total_work = num_tiles * n_f_tiles;
    const int num_kb = K / kBlockK;

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol_w = policy_evict_first();
            const uint64_t pol_x = policy_evict_last();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                const int tile = w / n_f_tiles;
                const int f = w - tile * n_f_tiles;
                const int e = tt.tile_expert[tile];
                const int row0 = tt.tile_row0[tile];
                const int wrow = e * w_rows_per_expert + f * kTileM;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + static_cast<size_t>(stage) * STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
                    tma_load_2d(st, &tmap_w, &full[stage], kb * kBlockK, wrow, pol_w);
                    if (GATE_UP)
                        tma_load_2d(st + A_BYTES, &tmap_w, &full[stage], kb * kBlockK, wrow + n_out, pol_w);
                    tma_load_2d(st + (GATE_UP ? 2 : 1) * A_BYTES, &tmap_x, &full[stage], kb * kBlockK, row0, pol_x);
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimeout);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
                const int buf = it & 1;
                const uint32_t use = static_cast<uint32_t>(it >> 1);
                if (!mbar_wait(&tmem_empty[buf], (use & 1) ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d0 = tmem_base + static_cast<uint32_t>(buf * ACC_COLS);
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&full[stage], phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * STAGE_BYTES);
                    const uint64_t da = make_desc_sw128(sa);
                    const uint64_t du = make_desc_sw128(sa + A_BYTES);
                    const uint64_t db = make_desc_sw128(sa + (GATE_UP ? 2 : 1) * A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < kBlockK / kUmmaK; kk++) {
                        // advancing K inside the 128-byte swizzle atom: +32 bytes = +2 in the (addr >> 4) field
                        const uint32_t acc = (kb | kk) ? 1u : 0u;
                        mma_bf16(d0, da + 2 * kk, db + 2 * kk, IDESC, acc);
                        if (GATE_UP)
                            mma_bf16(d0 + N_TILE, du + 2 * kk, db + 2 * kk, IDESC, acc);
                    }
                    tc_commit(&empty[stage]); // frees the stage once these MMAs have read it
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok)
                    tc_commit(&tmem_full[buf]);
            }
            if (!ok) {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimeout);
            }
        }
    } else {
        const int q = warp & 3; // TMEM lane quarter this warp may read
        bool ok = true;
        int it = 0;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
            const int tile = w / n_f_tiles;
            const int f = w - tile * n_f_tiles;
            const int e = tt.tile_expert[tile];
            const int row0 = tt.tile_row0[tile];
            int nvalid = offsets[e + 1] - row0;
            nvalid = nvalid < N_TILE ? nvalid : N_TILE;
            const int buf = it & 1;
            const uint32_t use = static_cast<uint32_t>(it >> 1);
            if (!mbar_wait(&tmem_full[buf], use & 1, abort_flag)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * ACC_COLS);
            const int feature = f * kTileM + q * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < N_TILE; c0 += 16) {
                if (c0 >= nvalid)
                    break;
                uint32_t g[16];
                tmem_ld16(t0 + c0, g);
                if (GATE_UP) {
                    uint32_t u[16];
                    tmem_ld16(t0 + N_TILE + c0, u);
                    tmem_ld_wait();
                    __nv_bfloat16 *act = static_cast<__nv_bfloat16 *>(out);
#pragma unroll
                    for (int c = 0; c < 16; c++)
                        if (c0 + c < nvalid) {
                            float a = silu_f32(__uint_as_float(g[c])) * __uint_as_float(u[c]);
                            act[static_cast<size_t>(row0 + c0 + c) * n_out + feature] = __float2bfloat16_rn(a);
                        }
                } else {
                    tmem_ld_wait();
                    float *y = static_cast<float *>(out);
#pragma unroll
                    for (int c = 0; c < 16; c++)
                        if (c0 + c < nvalid)
                            y[static_cast<size_t>(row0 + c0 + c) * n_out + feature] = __uint_as_float(g[c]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&tmem_empty[buf]);
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicOr(status, kStatusWaitTimeout);
        }
    }

    // Tear-down.  After an abort, give copies that may still be in flight time to land before the CTA's
    // shared memory is released.
    __syncwarp();
    if (*abort_flag)
        for (int i = 0; i < 64; i++)
            __nanosleep(4096);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// -------------------------------------------------------------------------------------------------------
// Plain CUDA-core version of the same grouped product, kept as an independent cross-check of the tensor-core
// kernel (tests run both and compare) -- one warp per (row, output feature pair), lanes stride K.
// -------------------------------------------------------------------------------------------------------
template <bool GATE_UP>
__global__ void grouped_gemm_bf16_simt_kernel(const __nv_bfloat16 *__restrict__ w, const __nv_bfloat16 *__restrict__ x,
                                              const int32_t *__restrict__ offsets, int num_experts, int w_rows_per_expert,
                                              int n_out, int K, void *__restrict__ out)
{
    const int row = blockIdx.x;
    const int total_rows = offsets[num_experts];
    if (row >= total_rows)
        return;
    // expert of this row: offsets is non-decreasing; linear scan by one thread then broadcast
    __shared__ int s_e;
    if (threadIdx.x == 0) {
        int lo = 0, hi = num_experts; // find e with offsets[e] <= row < offsets[e+1]
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (offsets[mid] <= row)
                lo = mid;
            else
                hi = mid;
        }
        s_e = lo;
    }
    __syncthreads();
    const int e = s_e;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const __nv_bfloat16 *xr = x + static_cast<size_t>(row) * K;
    const __nv_bfloat16 *we = w + static_cast<size_t>(e) * w_rows_per_expert * K;
    for (int f = blockIdx.y * nwarps + warp; f < n_out; f += gridDim.y * nwarps) {
        float g = 0.0f, u = 0.0f;
        const __nv_bfloat16 *wg = we + static_cast<size_t>(f) * K;
        const __nv_bfloat16 *wu = we + static_cast<size_t>(f + n_out) * K;
        for (int k = lane; k < K; k += 32) {
            float xv = __bfloat162float(xr[k]);
            g += xv * __bfloat162float(wg[k]);
            if (GATE_UP)
                u += xv * __bfloat162float(wu[k]);
        }
        for (int o = 16; o > 0; o >>= 1) {
            g += __shfl_xor_sync(0xffffffffu, g, o);
            u += __shfl_xor_sync(0xffffffffu, u, o);
        }
        if (lane == 0) {
            if (GATE_UP)
                static_cast<__nv_bfloat16 *>(out)[static_cast<size_t>(row) * n_out + f] = __float2bfloat16_rn(silu_f32(g) * u);
            else
                static_cast<float *>(out)[static_cast<size_t>(row) * n_out + f] = g;
        }
    }
}

} // namespace xs
