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

// SiLU for the quantised (FP8 / FP4) paths, where the result is rounded to e4m3 right away: hardware exp2-based
// exponential and reciprocal (a few ulp from the IEEE form, far below half an e4m3 step).  exp(-x) overflowing to
// +inf for very negative x gives x * 0 = -0, the right limit.
__device__ __forceinline__ float silu_fast(float x)
{
    return x * __frcp_rn(1.0f + __expf(-x));
}

// SiLU for the prefill-sized quantised kernels, whose tile tails are not overlapped with tensor work: x * sigmoid(x) =
// h + h * tanh(h) with h = x / 2 -- ONE special-function instruction (tanh.approx.f32, relative error about 2^-11) instead
// of an exponential and a reciprocal.  The result is rounded to e4m3 (3 mantissa bits) right away.
__device__ __forceinline__ float silu_tanh(float x)
{
    const float h = 0.5f * x;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
    return __fmaf_rn(h, t, h);
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
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                         const __grid_constant__ CUtensorMap tmap_x, const int32_t *__restrict__ offsets, TileTable tt, int groups,
                         int w_rows_per_expert, int n_out, int K, void *__restrict__ out, int32_t *__restrict__ status, int stages)
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
        prefetch_tmap(&tmap_w2);
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
    pdl_wait(); // everything above touches only this CTA's shared memory and TMEM

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
                // segments past `groups` belong to the always-on expert, whose weights sit behind the second map
                const CUtensorMap *tw = e < groups ? &tmap_w : &tmap_w2;
                const int wrow = (e < groups ? e * w_rows_per_expert : 0) + f * kTileM;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + static_cast<size_t>(stage) * STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
                    tma_load_2d(st, tw, &full[stage], kb * kBlockK, wrow, pol_w);
                    if (GATE_UP)
                        tma_load_2d(st + A_BYTES, tw, &full[stage], kb * kBlockK, wrow + n_out, pol_w);
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
    const int row = offsets[0] + blockIdx.x; // offsets may point into a longer table: segment 0 starts at offsets[0]
    const int total_rows = offsets[num_experts];
    if (row >= total_rows || row >= static_cast<int>(gridDim.x)) // gridDim.x = capacity of the row buffers
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

// =========================================================================================================
// FP8 (e4m3) experts with one f32 scale per 128x128 weight block and one per (token, 128 channels) of the
// activations.  The block scales are not a native tensor-core format, so each 128-deep k-block is accumulated
// on its own in TMEM (4 x tcgen05.mma kind::f8f6f4, K = 32 each), handed to the epilogue warps, and promoted
// into f32 registers as  acc += partial * (s_token * s_weight)  -- the same association the CPU restatement
// uses.  Two TMEM buffers let the tensor core work on k-block i+1 while k-block i is promoted.
//
// Because a weight tile is 128 rows and scale blocks are 128 rows, the weight scale of a (tile, k-block) is a
// single scalar; the token scale varies per accumulator column.
//
// gate/up: act = silu(gate) * up in f32 is quantised again for the down GEMM: the 128 features of a tile are
// exactly one 1x128 quantisation group of a token, so amax is a reduction over the tile's 128 TMEM lanes.
// =========================================================================================================
#include <cuda_fp8.h>

namespace xs {

constexpr int kBlockK8 = 128; // e4m3 elements per 128-byte swizzled row
constexpr int kUmmaK8 = 32;

__device__ __forceinline__ uint8_t f32_to_e4m3(float v)
{
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

struct Fp8Scales {
    const float *w_scale;   // (groups * w_rows_per_expert / 128, K / 128)
    const float *w_scale2;  // same for the always-on expert (segments >= groups): (w_rows_per_expert / 128, K / 128)
    const float *x_scale;   // (rows, K / 128)
    float *act_scale;       // GATE_UP only: (rows, n_out / 128) written by the epilogue
    int max_rows;           // rows of x_scale (reads past the last segment are clamped to it)
};

template <int N_TILE, bool GATE_UP>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                        const __grid_constant__ CUtensorMap tmap_x, const int32_t *__restrict__ offsets, TileTable tt, Fp8Scales sc,
                        int groups, int w_rows_per_expert, int n_out, int K, void *__restrict__ out, int32_t *__restrict__ status,
                        int stages)
{
    constexpr int A_BYTES = kTileM * kBlockK8;
    constexpr int B_BYTES = N_TILE * kBlockK8;
    constexpr int STAGE_BYTES = (GATE_UP ? 2 : 1) * A_BYTES + B_BYTES;
    constexpr int ACC_COLS = (GATE_UP ? 2 : 1) * N_TILE;
    // k-block accumulators in flight: enough that the tensor core keeps consuming stages while the epilogue warps
    // finish a tile (quantise / store) -- as many as fit in the 512 TMEM columns, at most 8
    constexpr int NBUF = (512 / ACC_COLS) < 8 ? (512 / ACC_COLS) : 8;
    constexpr int TMEM_COLS = NBUF * ACC_COLS; // a power of two >= 32 for every instantiation (16..64 tokens)
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS >= 32 && TMEM_COLS <= 512, "TMEM allocation must be a power of two");
    constexpr uint32_t IDESC = make_idesc(0, 0, kTileM, N_TILE); // e4m3 x e4m3 -> f32

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(stages) * STAGE_BYTES);
    uint64_t *full = bars;
    uint64_t *empty = bars + stages;
    uint64_t *tmem_full = bars + 2 * stages;
    uint64_t *tmem_empty = tmem_full + NBUF;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + NBUF);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    uint64_t *xbar = tmem_empty + NBUF + 1;                     // amax exchange among the four epilogue warps
    float *amax_x = reinterpret_cast<float *>(bars) + 128;      // [2 buffers][4 warps][N_TILE], 512 bytes after the barriers

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    unsigned long long *prof = reinterpret_cast<unsigned long long *>(status + 16); // role profile, see xs_moe_debug_counters
    const long long t_start = prof_clock();
    long long w0 = 0, w1 = 0;
    // no early pdl_launch_dependents() here: the next kernel's blocks would sit beside this one's CTAs for its whole run
    // (measured: 7 us slower at 256 tokens); they are let in as this kernel's CTAs exit

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < NBUF; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4);
        }
        mbar_init(xbar, 4);
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_w2);
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
    pdl_wait(); // everything above touches only this CTA's shared memory and TMEM

    const int n_f_tiles = n_out / kTileM;
    const int num_tiles = *tt.num_tiles;
    const int total_work = num_tiles * n_f_tiles;
    const int num_kb = K / kBlockK8;

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
                // segments past `groups` belong to the always-on expert, whose weights sit behind the second map
                const CUtensorMap *tw = e < groups ? &tmap_w : &tmap_w2;
                const int wrow = (e < groups ? e * w_rows_per_expert : 0) + f * kTileM;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_t(&empty[stage], phase ^ 1, abort_flag, w0)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + static_cast<size_t>(stage) * STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
                    tma_load_2d(st, tw, &full[stage], kb * kBlockK8, wrow, pol_w);
                    if (GATE_UP)
                        tma_load_2d(st + A_BYTES, tw, &full[stage], kb * kBlockK8, wrow + n_out, pol_w);
                    tma_load_2d(st + (GATE_UP ? 2 : 1) * A_BYTES, &tmap_x, &full[stage], kb * kBlockK8, row0, pol_x);
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
            prof_add(prof, 0, w0);
            prof_add(prof, 6, prof_clock() - t_start);
            prof_add(prof, 7, 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            uint32_t g_kb = 0; // k-blocks issued so far, across tiles: selects the TMEM buffer
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                for (int kb = 0; kb < num_kb; kb++, g_kb++) {
                    const int buf = g_kb % NBUF;
                    if (!mbar_wait_t(&full[stage], phase, abort_flag, w0) ||
                        !mbar_wait_t(&tmem_empty[buf], ((g_kb / NBUF) & 1) ^ 1, abort_flag, w1)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d0 = tmem_base + static_cast<uint32_t>(buf * ACC_COLS);
                    const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * STAGE_BYTES);
                    const uint64_t da = make_desc_sw128(sa);
                    const uint64_t du = make_desc_sw128(sa + A_BYTES);
                    const uint64_t db = make_desc_sw128(sa + (GATE_UP ? 2 : 1) * A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < kBlockK8 / kUmmaK8; kk++) {
                        mma_f8(d0, da + 2 * kk, db + 2 * kk, IDESC, kk ? 1u : 0u);
                        if (GATE_UP)
                            mma_f8(d0 + N_TILE, du + 2 * kk, db + 2 * kk, IDESC, kk ? 1u : 0u);
                    }
                    tc_commit(&empty[stage]);
                    tc_commit(&tmem_full[buf]);
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
            prof_add(prof, 1, w0);
            prof_add(prof, 3, w1);
        }
    } else {
        const int q = warp & 3;
        const int ew = warp - 2; // 0..3, index into the amax exchange
        bool ok = true;
        uint32_t g_kb = 0;
        uint32_t it = 0;
        const int kbs = K / kBlockK8; // scale columns per row
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
            const int tile = w / n_f_tiles;
            const int f = w - tile * n_f_tiles;
            const int e = tt.tile_expert[tile];
            const int row0 = tt.tile_row0[tile];
            int nvalid = offsets[e + 1] - row0;
            nvalid = nvalid < N_TILE ? nvalid : N_TILE;
            const int feature = f * kTileM + q * 32 + lane;
            const float *ws_g = (e < groups ? sc.w_scale + static_cast<size_t>(e) * (w_rows_per_expert / kTileM) * kbs : sc.w_scale2) +
                                static_cast<size_t>(f) * kbs;
            const float *ws_u = ws_g + static_cast<size_t>(n_out / kTileM) * kbs;
            float acc_g[N_TILE];
            float acc_u[GATE_UP ? N_TILE : 1];
#pragma unroll
            for (int c = 0; c < N_TILE; c++) {
                acc_g[c] = 0.0f;
                if constexpr (GATE_UP)
                    acc_u[c] = 0.0f;
            }
            for (int kb = 0; kb < num_kb; kb++, g_kb++) {
                const int buf = g_kb % NBUF;
                // scales of this k-block first: their latency overlaps the wait for the tensor core
                const float swg = __ldg(ws_g + kb);
                const float swu = GATE_UP ? __ldg(ws_u + kb) : 0.0f;
                float sxw_g[N_TILE], sxw_u[GATE_UP ? N_TILE : 1];
#pragma unroll
                for (int c = 0; c < N_TILE; c++) {
                    const float sx = __ldg(sc.x_scale + static_cast<size_t>(row0 + (c < nvalid ? c : 0)) * kbs + kb);
                    sxw_g[c] = __fmul_rn(sx, swg);
                    if constexpr (GATE_UP)
                        sxw_u[c] = __fmul_rn(sx, swu);
                }
                if (!mbar_wait_t(&tmem_full[buf], (g_kb / NBUF) & 1, abort_flag, w0)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * ACC_COLS);
                if constexpr (N_TILE == 16) {
                    // whole k-block in one round trip; the TMEM buffer is handed back before the arithmetic
                    uint32_t g[16], u[16];
                    tmem_ld16(t0, g);
                    if constexpr (GATE_UP)
                        tmem_ld16(t0 + N_TILE, u);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&tmem_empty[buf]);
#pragma unroll
                    for (int c = 0; c < 16; c++) {
                        acc_g[c] = __fadd_rn(acc_g[c], __fmul_rn(__uint_as_float(g[c]), sxw_g[c]));
                        if constexpr (GATE_UP)
                            acc_u[c] = __fadd_rn(acc_u[c], __fmul_rn(__uint_as_float(u[c]), sxw_u[c]));
                    }
                } else {
#pragma unroll
                    for (int c0 = 0; c0 < N_TILE; c0 += 16) {
                        if (c0 < nvalid) {
                            uint32_t g[16];
                            tmem_ld16(t0 + c0, g);
                            uint32_t u[16];
                            if constexpr (GATE_UP)
                                tmem_ld16(t0 + N_TILE + c0, u);
                            tmem_ld_wait();
#pragma unroll
                            for (int c = 0; c < 16; c++) {
                                const int col = c0 + c;
                                acc_g[col] = __fadd_rn(acc_g[col], __fmul_rn(__uint_as_float(g[c]), sxw_g[col]));
                                if constexpr (GATE_UP)
                                    acc_u[col] = __fadd_rn(acc_u[col], __fmul_rn(__uint_as_float(u[c]), sxw_u[col]));
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&tmem_empty[buf]);
                }
            }
            if (!ok)
                break;
            if constexpr (GATE_UP) {
                // act = silu(g) * u, then 1x128 quantisation over the tile's 128 features (lanes of all 4 epilogue warps)
                // The exchange buffer alternates between tiles: a warp can only write buffer (it+2)&1 after passing the
                // exchange barrier of tile it+1, which every warp reaches after it has finished reading buffer it&1.
                uint8_t *actq = static_cast<uint8_t *>(out);
                float *ax = amax_x + (it & 1) * 4 * N_TILE;
#pragma unroll
                for (int c = 0; c < N_TILE; c++) {
                    const float a = silu_fast(acc_g[c]) * acc_u[c];
                    acc_g[c] = a;
                    float m = fabsf(a);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1)
                        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                    if (lane == 0)
                        ax[ew * N_TILE + c] = m;
                }
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(xbar); // release: this warp's amax values are visible to the waiters
                if (!mbar_wait(xbar, it & 1, abort_flag)) {
                    ok = false;
                    break;
                }
#pragma unroll
                for (int c = 0; c < N_TILE; c++) {
                    if (c < nvalid) {
                        const float m = fmaxf(fmaxf(ax[c], ax[N_TILE + c]), fmaxf(ax[2 * N_TILE + c], ax[3 * N_TILE + c]));
                        const float s = __fdiv_rn(fmaxf(m, 1e-10f), 448.0f);
                        actq[static_cast<size_t>(row0 + c) * n_out + feature] = f32_to_e4m3(__fdiv_rn(acc_g[c], s));
                        if (ew == 0 && lane == 0)
                            sc.act_scale[static_cast<size_t>(row0 + c) * (n_out / kTileM) + f] = s;
                    }
                }
            } else {
                float *y = static_cast<float *>(out);
#pragma unroll
                for (int c = 0; c < N_TILE; c++)
                    if (c < nvalid)
                        y[static_cast<size_t>(row0 + c) * n_out + feature] = acc_g[c];
            }
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicOr(status, kStatusWaitTimeout);
        }
        if (warp == 2 && lane == 0)
            prof_add(prof, 5, w0);
    }

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

// x (rows, cols) bf16 -> e4m3 codes + one f32 scale per (row, 128 columns): s = max(amax, 1e-10) / 448,
// q = e4m3_rne_sat(x / s).  One warp per 128-column group; IEEE division on both steps so the codes equal
// the CPU restatement bit for bit.
__global__ void __launch_bounds__(256)
quantize_rows_fp8_kernel(const __nv_bfloat16 *__restrict__ x, uint8_t *__restrict__ q, float *__restrict__ scale, int rows, int cols)
{
    const int groups = cols / 128;
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    if (gw >= rows * groups)
        return;
    const int r = gw / groups, g = gw - r * groups;
    const __nv_bfloat16 *p = x + static_cast<size_t>(r) * cols + g * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    float v[4];
    v[0] = __uint_as_float(raw.x << 16);
    v[1] = __uint_as_float(raw.x & 0xffff0000u);
    v[2] = __uint_as_float(raw.y << 16);
    v[3] = __uint_as_float(raw.y & 0xffff0000u);
    float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float s = __fdiv_rn(fmaxf(m, 1e-10f), 448.0f);
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; i++)
        packed |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(v[i], s))) << (8 * i);
    *reinterpret_cast<uint32_t *>(q + static_cast<size_t>(r) * cols + g * 128 + lane * 4) = packed;
    if (lane == 0)
        scale[static_cast<size_t>(r) * groups + g] = s;
}

} // namespace xs
