// Prefill-sized grouped GEMM for FP8 (e4m3, 128x128 block scales) experts.
//
// With a hundred or more tokens per expert the decode kernel's shape (128 weight rows x <= 64 tokens per MMA) leaves
// the tensor core mostly idle: a tcgen05.mma with M = 128 occupies the pipe for about as long whatever N is, so the
// work per instruction has to be as large as the instruction allows.  Here the TOKENS are the M dimension (128 per
// tile) and 256 weight rows are the N dimension of one MMA: for gate/up the 128 gate rows and the 128 up rows of one
// feature block sit side by side in shared memory and form a single N = 256 operand; for down, 256 consecutive output
// rows.  D[token, column] lives in TMEM as 128 lanes x 256 columns, double-buffered (all 512 columns).
//
// Block scales: each 128-deep k-block is accumulated on its own and promoted by the epilogue warps,
//     acc += partial * (s_token[kb] * s_weight_block[kb]),
// with one scalar token scale per TMEM lane and one scalar weight scale per 128 columns.  The promotion is bound by the
// latency of the TMEM reads, so FOUR epilogue warpgroups (16 warps, 4 per scheduler) share the 256 columns, 64
// accumulator registers per thread: for gate/up each takes 32 gate + the matching 32 up columns so that SwiGLU needs no
// exchange; only the 1x128 amax of the re-quantised activations crosses the warpgroups.
//
// Warps: 0 TMA producer | 1 MMA issuer, TMEM owner | 2..17 epilogue (group = (warp - 2) / 4, lane quarter = warp % 4).
#pragma once
#include "xs_grouped_gemm.cuh"

#ifndef XS_PF8_SPIN
#define XS_PF8_SPIN 0
#endif
#ifndef XS_PF8_FMA2
#define XS_PF8_FMA2 0
#endif
#ifndef XS_PF8_DEBUG
#define XS_PF8_DEBUG 0
#endif

namespace xs {

// d0 += a0 * s, d1 += a1 * s as one packed instruction (two independent IEEE fused multiply-adds)
__device__ __forceinline__ void ffma2(float &d0, float &d1, float a0, float a1, float s)
{
    asm("{\n\t"
        ".reg .b64 ra, rb, rc;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %4};\n\t"
        "mov.b64 rc, {%0, %1};\n\t"
        "fma.rn.f32x2 rc, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rc;\n\t"
        "}\n"
        : "+f"(d0), "+f"(d1)
        : "f"(a0), "f"(a1), "f"(s));
}

constexpr int kPfGroups = 4;                     // epilogue warpgroups sharing the 256 columns
constexpr int kPfThreads = 64 + kPfGroups * 128;
constexpr int kPfTokens = 128;  // MMA M
constexpr int kPfCols = 256;    // MMA N
constexpr int kPfStageBytes = (kPfTokens + kPfCols) * kBlockK8; // 48 KB
constexpr int kPfTailBytes = 512 + 2 * kPfGroups * 128 * 4; // barriers + amax exchange (2 tile parities x groups x 128 floats)

template <bool GATE_UP>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                        const __grid_constant__ CUtensorMap tmap_x, const int32_t *__restrict__ offsets, TileTable tt, Fp8Scales sc,
                        int groups, int w_rows_per_expert, int n_out, int K, void *__restrict__ out, int32_t *__restrict__ status,
                        int stages)
{
    constexpr int X_BYTES = kPfTokens * kBlockK8;
    constexpr int W_HALF = 128 * kBlockK8;
    constexpr int NBUF = 2;
    constexpr int TMEM_COLS = 512;
    constexpr uint32_t IDESC = make_idesc(0, 0, kPfTokens, kPfCols);
    constexpr int N_PER_TILE = GATE_UP ? 128 : 256; // output features covered by one work item

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(stages) * kPfStageBytes);
    uint64_t *full = bars;
    uint64_t *empty = bars + stages;
    uint64_t *tmem_full = bars + 2 * stages;
    uint64_t *tmem_empty = tmem_full + NBUF;
    uint64_t *xbar = tmem_empty + NBUF;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(xbar + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    float *amax_x = reinterpret_cast<float *>(bars) + 128; // [2 tile parities][groups][128 rows]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // role profile (see xs_moe_debug_counters): cycles each role spent blocked, summed over CTAs
    unsigned long long *prof = reinterpret_cast<unsigned long long *>(status + 16);
    const long long t_start = prof_clock();
    long long w0 = 0, w1 = 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < NBUF; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4 * kPfGroups); // one arrival per epilogue warp
        }
        mbar_init(xbar, 4 * kPfGroups);
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

    const int n_n_tiles = n_out / N_PER_TILE;
    const int num_tiles = *tt.num_tiles;
    const int total_work = num_tiles * n_n_tiles;
    const int num_kb = K / kBlockK8;

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol_w = policy_evict_last(); // weights are re-read by the other token tiles of the expert
            const uint64_t pol_x = policy_evict_last();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                const int tile = w / n_n_tiles;
                const int nt = w - tile * n_n_tiles;
                const int e = tt.tile_expert[tile];
                const int row0 = tt.tile_row0[tile];
                const CUtensorMap *tw = e < groups ? &tmap_w : &tmap_w2;
                const int wbase = (e < groups ? e * w_rows_per_expert : 0) + nt * N_PER_TILE;
                const int wrow2 = GATE_UP ? wbase + n_out : wbase + 128; // up block of the same features | next 128 rows
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_t(&empty[stage], phase ^ 1, abort_flag, w0)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + static_cast<size_t>(stage) * kPfStageBytes;
#if XS_PF8_DEBUG == 6
                    (void)st; (void)tw; (void)wbase; (void)wrow2; (void)row0; (void)pol_x; (void)pol_w;
                    mbar_arrive(&full[stage]);
#elif XS_PF8_DEBUG == 7
                    (void)tw; (void)wbase; (void)wrow2; (void)pol_w;
                    mbar_arrive_expect_tx(&full[stage], X_BYTES);
                    tma_load_2d(st, &tmap_x, &full[stage], kb * kBlockK8, row0, pol_x);
#else
                    mbar_arrive_expect_tx(&full[stage], kPfStageBytes);
                    tma_load_2d(st, &tmap_x, &full[stage], kb * kBlockK8, row0, pol_x);
                    tma_load_2d(st + X_BYTES, tw, &full[stage], kb * kBlockK8, wbase, pol_w);
                    tma_load_2d(st + X_BYTES + W_HALF, tw, &full[stage], kb * kBlockK8, wrow2, pol_w);
#endif
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
            uint32_t g_kb = 0;
            long long w_issue = 0; // role profile: cycles spent issuing (descriptors, four MMAs, two commits)
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                for (int kb = 0; kb < num_kb; kb++, g_kb++) {
                    const int buf = g_kb & 1;
#if XS_PF8_SPIN
                    if (!mbar_wait_t(&full[stage], phase, abort_flag, w0) ||
                        !mbar_spin_wait_t(&tmem_empty[buf], ((g_kb >> 1) & 1) ^ 1, abort_flag, w1)) {
#else
                    if (!mbar_wait_t(&full[stage], phase, abort_flag, w0) ||
                        !mbar_wait_t(&tmem_empty[buf], ((g_kb >> 1) & 1) ^ 1, abort_flag, w1)) {
#endif
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const long long t_issue = prof_clock();
                    const uint32_t d0 = tmem_base + static_cast<uint32_t>(buf * kPfCols);
                    const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * kPfStageBytes);
                    const uint64_t dx = make_desc_sw128(sa);
                    const uint64_t dw = make_desc_sw128(sa + X_BYTES); // 256 rows: the two 128-row boxes are contiguous
#pragma unroll
                    for (int kk = 0; kk < kBlockK8 / kUmmaK8; kk++)
                        mma_f8(d0, dx + 2 * kk, dw + 2 * kk, IDESC, kk ? 1u : 0u);
                    tc_commit(&empty[stage]);
                    tc_commit(&tmem_full[buf]);
                    w_issue += prof_clock() - t_issue;
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
            prof_add(prof, 9, w_issue);
        }
    } else {
#include "xs_prefill_fp8_epilogue.inl"
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

} // namespace xs
