// Prefill-sized grouped GEMM for FP4 (e2m1 + e8m0/32) experts with MX-FP8 activations.
//
// Same tile shape as the FP8 prefill kernel -- 128 TOKENS as the MMA's M, 256 weight rows (gate block + up block, or
// 256 output rows of the down matrix) as its N -- but the scales are applied by the tensor core
// (tcgen05.mma kind::mxf8f6f4.block_scale), so the whole K accumulates in TMEM and the epilogue runs once per tile.
// TMEM: 256 accumulator columns + a ring of scale slots (4 columns for the 128 token rows, 8 for the 256 weight
// rows); the accumulator is single-buffered, the epilogue of a tile (about a tenth of its main loop) is not overlapped.
//
// Warps: 0 TMA producer | 1 MMA issuer (+ tcgen05.cp of the scales), TMEM owner | 2..5 and 7..10 epilogue (two warps per
// TMEM lane quarter, each taking half of the columns) | 6 and 11 scale loaders (alternate k-blocks).
#pragma once
#include "xs_grouped_gemm_fp4.cuh"
#include "xs_prefill_fp8.cuh"

namespace xs {

constexpr int kPf4Loaders = 2;                      // scale-loader warps: 6, 11, 12, ...
constexpr int kPf4Threads = 352 + 32 * (kPf4Loaders - 1);
constexpr int kPf4SfBytesPerStage = 1536; // tokens | weight rows 0..127 | weight rows 128..255
constexpr int kPf4SfSlots = 8;            // shared-memory ring of scale blocks (barriers of its own)
constexpr int kPf4TailBytes = 512 + kPf4SfSlots * kPf4SfBytesPerStage;

template <bool GATE_UP>
__global__ void __launch_bounds__(kPf4Threads, 1)
prefill_gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const int32_t *__restrict__ offsets, TileTable tt, MxScales sc, int w_rows_per_expert, int n_out, int K,
                        void *__restrict__ out, int32_t *__restrict__ status, int stages)
{
    constexpr int X_BYTES = kPfTokens * kBlockK8;
    constexpr int W_HALF = 128 * kBlockK8;               // shared-memory footprint (one code per byte)
    constexpr int TX_BYTES = X_BYTES + 2 * (W_HALF / 2); // the copy engine counts the packed weight bytes
    constexpr int SF_COLS = 12;                          // 4 (tokens) + 8 (weight rows)
    constexpr int TMEM_COLS = 512;
    constexpr int N_PER_TILE = GATE_UP ? 128 : 256;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(stages) * kPfStageBytes);
    uint64_t *full = bars;
    uint64_t *empty = bars + stages;
    uint64_t *sf_full = bars + 2 * stages;  // scale slots: a ring of kPf4SfSlots of its own, not tied to the operand stages
    uint64_t *sf_empty = sf_full + kPf4SfSlots;
    uint64_t *tmem_full = sf_empty + kPf4SfSlots;
    uint64_t *tmem_empty = tmem_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    uint8_t *sf_smem = reinterpret_cast<uint8_t *>(bars) + 512;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    unsigned long long *prof = reinterpret_cast<unsigned long long *>(status + 16);
    const long long t_start = prof_clock();
    long long w0 = 0, w1 = 0, w2 = 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < kPf4SfSlots; s++) {
            mbar_init(&sf_full[s], 1);
            mbar_init(&sf_empty[s], 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, 8);
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
    const uint32_t sf_base = tmem_base + kPfCols;

    const int n_n_tiles = n_out / N_PER_TILE;
    const int num_tiles = *tt.num_tiles;
    const int total_work = num_tiles * n_n_tiles;
    const int num_kb = K / kBlockK8;
    const int kbs = K / 32;

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol = policy_evict_last();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                const int tile = w / n_n_tiles;
                const int nt = w - tile * n_n_tiles;
                const int e = tt.tile_expert[tile];
                const int row0 = tt.tile_row0[tile];
                const int wbase = e * w_rows_per_expert + nt * N_PER_TILE;
                const int wrow2 = GATE_UP ? wbase + n_out : wbase + 128;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_t(&empty[stage], phase ^ 1, abort_flag, w0)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + static_cast<size_t>(stage) * kPfStageBytes;
                    mbar_arrive_expect_tx(&full[stage], TX_BYTES);
                    tma_load_2d(st, &tmap_x, &full[stage], kb * kBlockK8, row0, pol);
                    tma_load_2d(st + X_BYTES, &tmap_w, &full[stage], kb * kBlockK8, wbase, pol);
                    tma_load_2d(st + X_BYTES + W_HALF, &tmap_w, &full[stage], kb * kBlockK8, wrow2, pol);
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
            uint32_t it = 0, n = 0; // n: k-blocks issued so far; its scales sit in slot n % kPf4SfSlots
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
                if (!mbar_wait_t(tmem_empty, (it & 1) ^ 1, abort_flag, w2)) { // previous tile drained by the epilogue
                    ok = false;
                    break;
                }
                tc_fence_after();
                for (int kb = 0; kb < num_kb; kb++, n++) {
                    const uint32_t slot = n % kPf4SfSlots;
                    if (!mbar_wait_t(&full[stage], phase, abort_flag, w0) ||
                        !mbar_wait_t(&sf_full[slot], (n / kPf4SfSlots) & 1u, abort_flag, w1)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * kPfStageBytes);
                    const uint64_t dx = make_desc_sw128(sa);
                    const uint64_t dw = make_desc_sw128(sa + X_BYTES);
                    const uint32_t sfx = sf_base + static_cast<uint32_t>(stage * SF_COLS);
                    const uint32_t sfw = sfx + 4;
                    const uint32_t sfs = smem_u32(sf_smem + static_cast<size_t>(slot) * kPf4SfBytesPerStage);
                    tmem_cp_32x128b_x4(sfx, make_desc_rows16(sfs));
                    tmem_cp_32x128b_x4(sfw, make_desc_rows16(sfs + 512));
                    tmem_cp_32x128b_x4(sfw + 4, make_desc_rows16(sfs + 1024));
#pragma unroll
                    for (int kk = 0; kk < kBlockK8 / kUmmaK8; kk++) {
                        const uint32_t idesc = make_idesc_mx(0, 5, kPfTokens, kPfCols, kk); // A = e4m3 tokens, B = e2m1 weights
                        mma_mxf8f6f4(tmem_base, dx + 2 * kk, dw + 2 * kk, idesc, sfx, sfw, (kb | kk) ? 1u : 0u);
                    }
                    tc_commit(&empty[stage]);
                    tc_commit(&sf_empty[slot]);
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok)
                    tc_commit(tmem_full);
            }
            if (!ok) {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimeout);
            }
            prof_add(prof, 1, w0);
            prof_add(prof, 2, w1);
            prof_add(prof, 3, w2);
        }
    } else if (warp == 6 || warp >= 11) {
#include "xs_prefill_fp4_scales.inl"
    } else {
#include "xs_prefill_fp4_epilogue.inl"
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
