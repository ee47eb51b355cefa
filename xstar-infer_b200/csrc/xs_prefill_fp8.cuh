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
// with one scalar token scale per TMEM lane and one scalar weight scale per 128 columns.  FOUR epilogue warpgroups (16
// warps, 4 per scheduler) share the 256 columns, 64 accumulator registers per thread: for gate/up each takes 32 gate +
// the matching 32 up columns so that SwiGLU needs no exchange; only the 1x128 amax of the re-quantised activations
// crosses the warpgroups.
//
// Because the accumulator changes hands once per k-block (four MMAs), what the issuing thread does BETWEEN k-blocks is on
// the tensor pipe's critical path: a thread that issues tcgen05.mma is held until the pipe takes the instruction, so it
// cannot run ahead, and its commits, barrier waits and descriptor set-up for the next k-block leave the pipe idle every
// time.  Measured with the hand-over probe (xs_moe_probe_handoff: this protocol and nothing else): one issuing thread
// 810-880 cycles per k-block, TWO warps issuing alternate k-blocks (each owns one of the two accumulator buffers) 510-580,
// the rate of the four MMAs themselves.  So two warps issue.
//
// What bounds the kernel after that (gate/up launch of the 8192-token layer, 2048 k-blocks per CTA; each line removes one
// thing from the kernel and times it): protocol + MMAs alone 0.77 ms; + the promotion FMAs 0.94; + the operand loads
// 1.18 without / 1.31 with the FMAs (48 KB per k-block per SM: 12 TB/s out of L2, the floor of this tile shape); + the
// per-tile tail (SwiGLU, re-quantisation, stores; the accumulator registers are busy, so the next tile's k-loop stops
// after two k-blocks) 1.78 ms.
//
// Warps: 0 TMA producer | 1, 2 MMA issuers (1 owns TMEM) | 3 idle | 4..19 epilogue (group = (warp - 4) / 4, lane quarter =
// warp % 4).  Warps 0..3 hand most of their registers to the epilogue warpgroups (setmaxnreg), whose 64 accumulators + TMEM
// staging registers per thread do not fit the even share of 20 warps.
#pragma once
#include "xs_grouped_gemm.cuh"


namespace xs {

constexpr int kPfGroups = 4;                     // epilogue warpgroups sharing the 256 columns
constexpr int kPfIssuers = 2;                     // MMA issuer warps, k-blocks taken round-robin (== accumulator buffers)
constexpr int kPfEpiWarp0 = 4;                   // first epilogue warp: warps 0..3 form the light warpgroup (3 idles)
constexpr int kPfThreads = 32 * kPfEpiWarp0 + kPfGroups * 128;
constexpr int kPfTokens = 128;  // MMA M
constexpr int kPfCols = 256;    // MMA N
constexpr int kPfStageBytes = (kPfTokens + kPfCols) * kBlockK8; // 48 KB
constexpr int kPfTailBytes = 512 + 2 * kPfGroups * 128 * 4; // barriers + amax exchange (2 tile parities x groups x 128 floats)

template <bool GATE_UP>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                        const __grid_constant__ CUtensorMap tmap_x, const int32_t *__restrict__ offsets, TileTable tt, Fp8Scales sc,
                        int groups, int w_rows_per_expert, int n_out, int K, void *__restrict__ out, int32_t *__restrict__ status,
                        int stages, int y_bf16)
{
    constexpr int X_BYTES = kPfTokens * kBlockK8;
    constexpr int W_HALF = 128 * kBlockK8;
    constexpr int NBUF = kPfIssuers; // issuer m fills buffer m
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
    pdl_wait(); // everything above touches only this CTA's shared memory and TMEM

    const int n_n_tiles = n_out / N_PER_TILE;
    const int num_tiles = *tt.num_tiles;
    const int total_work = num_tiles * n_n_tiles;
    const int num_kb = K / kBlockK8;

    if (warp < kPfEpiWarp0)
        reg_dealloc<40>();
    else
        reg_alloc<104>();
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
                    mbar_arrive_expect_tx(&full[stage], kPfStageBytes);
                    tma_load_2d(st, &tmap_x, &full[stage], kb * kBlockK8, row0, pol_x);
                    tma_load_2d(st + X_BYTES, tw, &full[stage], kb * kBlockK8, wbase, pol_w);
                    tma_load_2d(st + X_BYTES + W_HALF, tw, &full[stage], kb * kBlockK8, wrow2, pol_w);
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
    } else if (warp <= kPfIssuers) {
        if (lane == 0) {
            const uint32_t me = static_cast<uint32_t>(warp - 1); // this issuer's k-blocks: g_kb % kPfIssuers == me
            // k-blocks of this CTA, over all its work items
            const uint32_t n_items = static_cast<int>(blockIdx.x) < total_work
                                         ? static_cast<uint32_t>((total_work - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1)
                                         : 0u;
            const uint32_t n_kb = n_items * static_cast<uint32_t>(num_kb);
            bool ok = true;
            long long w_issue = 0; // role profile: cycles spent issuing (descriptors, four MMAs, two commits)
            for (uint32_t g_kb = me; g_kb < n_kb; g_kb += kPfIssuers) {
                const uint32_t stage = g_kb % static_cast<uint32_t>(stages);
                const uint32_t phase = (g_kb / static_cast<uint32_t>(stages)) & 1u;
                const uint32_t use = g_kb / kPfIssuers; // how often this issuer's buffer has been filled before
                if (!mbar_wait_t(&full[stage], phase, abort_flag, w0) || !mbar_wait_t(&tmem_empty[me], (use & 1u) ^ 1u, abort_flag, w1)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const long long t_issue = prof_clock();
                const uint32_t d0 = tmem_base + me * kPfCols;
                const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * kPfStageBytes);
                const uint64_t dx = make_desc_sw128(sa);
                const uint64_t dw = make_desc_sw128(sa + X_BYTES); // 256 rows: the two 128-row boxes are contiguous
#pragma unroll
                for (int kk = 0; kk < kBlockK8 / kUmmaK8; kk++)
                    mma_f8(d0, dx + 2 * kk, dw + 2 * kk, IDESC, kk ? 1u : 0u);
                tc_commit(&empty[stage]);
                tc_commit(&tmem_full[me]);
                w_issue += prof_clock() - t_issue;
            }
            if (!ok) {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimeout);
            }
            if (me == 0) {
                prof_add(prof, 1, w0);
                prof_add(prof, 3, w1);
                prof_add(prof, 9, w_issue);
            }
        }
    } else if (warp >= kPfEpiWarp0) {
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
