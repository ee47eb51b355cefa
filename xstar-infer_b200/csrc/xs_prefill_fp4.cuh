// Prefill-sized grouped GEMM for FP4 (e2m1 + e8m0/32) experts with MX-FP8 activations.
//
// Same tile shape as the FP8 prefill kernel -- 128 TOKENS as the MMA's M, 256 weight rows (gate block + up block, or
// 256 output rows of the down matrix) as its N -- but the scales are applied by the tensor core
// (tcgen05.mma kind::mxf8f6f4.block_scale), so the whole K accumulates in TMEM and the epilogue runs once per tile.
// TMEM: 256 accumulator columns + a ring of scale slots (4 columns for the 128 token rows, 8 for the 256 weight
// rows); the accumulator is single-buffered, the epilogue of a tile (about a tenth of its main loop) is not overlapped.
//
// The kernel also serves decode-sized batches (a handful of tokens per expert): there the token box of the TMA load is
// 32 rows instead of 128 (tile_rows), the other rows of the MMA's M are whatever the shared-memory stage held before, and
// their accumulator lanes are never read.  An N = 256 block-scaled MMA consumes 4 KB of packed weights, twice what the
// weights-as-M orientation feeds one (whose MMAs do not get cheaper below N = 128), which is what decode -- bound by the
// weight stream -- needs.
//
// Scales: the e8m0 bytes of a k-block's 128 token rows and 256 weight rows must sit in shared memory as three 512-byte
// blocks (lane i: rows i, 32+i, 64+i, 96+i) for tcgen05.cp.  Where the shapes allow (K a multiple of 512, 16-byte aligned
// scale matrices) the TMA producer fetches the scales of FOUR k-blocks at a time -- a 16-byte x 128-row box per operand
// block, three boxes per group -- into a small raw ring, and one warp re-orders each group into four scale slots with
// 12 shared-memory reads and 12 writes.  (Fetching them with per-lane global loads made the loader warps the kernel's
// bottleneck: every lane of such a load touches its own sector.)  Other shapes keep the per-lane loader.
//
// Warps: 0 TMA producer | 1 MMA issuer (+ tcgen05.cp of the scales), TMEM owner | 2..5 and 7..10 epilogue (two warps per
// TMEM lane quarter, each taking half of the columns) | 6 scale warp.
#pragma once
#include "xs_grouped_gemm_fp4.cuh"
#include "xs_prefill_fp8.cuh"

namespace xs {

constexpr int kPf4Loaders = 1;                      // scale-loader warps: 6, 11, 12, ...
constexpr int kPf4Threads = 352 + 32 * (kPf4Loaders - 1);
constexpr int kPf4SfBytesPerStage = 1536; // tokens | weight rows 0..127 | weight rows 128..255
constexpr int kPf4SfSlots = 6;            // scale blocks in shared memory: one per operand stage (at most 6 stages)
constexpr int kPf4RawSlots = 2;           // raw ring: scales of four k-blocks as the TMA delivers them (3 x 128 rows x 16 bytes)
constexpr int kPf4RawBytes = 3 * 128 * 16;
constexpr int kPf4TailBytes = 512 + kPf4SfSlots * kPf4SfBytesPerStage + kPf4RawSlots * kPf4RawBytes;

template <bool GATE_UP>
__global__ void __launch_bounds__(kPf4Threads, 1)
prefill_gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const __grid_constant__ CUtensorMap tmap_ws, const __grid_constant__ CUtensorMap tmap_xs,
                        const int32_t *__restrict__ offsets, TileTable tt, MxScales sc, int w_rows_per_expert, int n_out, int K,
                        void *__restrict__ out, int32_t *__restrict__ status, int stages, int tile_rows, int sf_tma, EpReturnArgs ret)
{
    constexpr int X_BYTES = kPfTokens * kBlockK8;
    constexpr int W_HALF = 128 * kBlockK8;               // shared-memory footprint (one code per byte)
    // the copy engine counts the packed weight bytes; the token box is tile_rows (32 or 128) rows of 128 bytes
    const uint32_t tx_bytes = static_cast<uint32_t>(tile_rows) * kBlockK8 + 2 * (W_HALF / 2);
    constexpr int SF_COLS = 12;                          // 4 (tokens) + 8 (weight rows)
    constexpr int TMEM_COLS = 512;
    constexpr int N_PER_TILE = GATE_UP ? 128 : 256;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(stages) * kPfStageBytes);
    uint64_t *full = bars;
    uint64_t *empty = bars + stages;
    uint64_t *tmem_full = bars + 2 * stages;
    uint64_t *tmem_empty = tmem_full + 1;
    uint64_t *raw_full = tmem_empty + 1;
    uint64_t *raw_empty = raw_full + kPf4RawSlots;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(raw_empty + kPf4RawSlots);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    uint8_t *sf_smem = reinterpret_cast<uint8_t *>(bars) + 512;
    uint8_t *raw_smem = sf_smem + kPf4SfSlots * kPf4SfBytesPerStage; // 128-byte aligned: a TMA destination

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // role profile (profile builds only): counters 0..7 for the gate/up instantiation, 8..15 for the down one
    unsigned long long *prof = reinterpret_cast<unsigned long long *>(status + 16) + (GATE_UP ? 0 : 8);
    const long long t_start = prof_clock();
    long long w0 = 0, w1 = 0, w2 = 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 2); // the producer's expect-tx arrival and the scale warp's
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < kPf4RawSlots; s++) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&raw_empty[s], 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, 8);
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_x);
        if (sf_tma) {
            prefetch_tmap(&tmap_ws);
            prefetch_tmap(&tmap_xs);
        }
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
            uint32_t phase = 0, group = 0; // group: groups of four k-blocks whose scales were requested so far
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                const int tile = w / n_n_tiles;
                const int nt = w - tile * n_n_tiles;
                const int e = tt.tile_expert[tile];
                const int row0 = tt.tile_row0[tile];
                const int wbase = e * w_rows_per_expert + nt * N_PER_TILE;
                const int wrow2 = GATE_UP ? wbase + n_out : wbase + 128;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (sf_tma && (kb & 3) == 0) {
                        // scales of k-blocks kb..kb+3: 16 bytes per row, rows of the token tile and of the two weight blocks
                        const uint32_t rs = group % kPf4RawSlots;
                        if (!mbar_wait_t(&raw_empty[rs], ((group / kPf4RawSlots) & 1u) ^ 1u, abort_flag, w0)) {
                            ok = false;
                            break;
                        }
                        uint8_t *raw = raw_smem + rs * kPf4RawBytes;
                        mbar_arrive_expect_tx(&raw_full[rs], kPf4RawBytes);
                        tma_load_2d(raw, &tmap_xs, &raw_full[rs], kb * 4, row0, pol);
                        tma_load_2d(raw + 2048, &tmap_ws, &raw_full[rs], kb * 4, wbase, pol);
                        tma_load_2d(raw + 4096, &tmap_ws, &raw_full[rs], kb * 4, wrow2, pol);
                        group++;
                    }
                    if (!mbar_wait_t(&empty[stage], phase ^ 1, abort_flag, w0)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + static_cast<size_t>(stage) * kPfStageBytes;
                    mbar_arrive_expect_tx(&full[stage], tx_bytes);
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
            uint32_t it = 0;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
                if (!mbar_wait_t(tmem_empty, (it & 1) ^ 1, abort_flag, w2)) { // previous tile drained by the epilogue
                    ok = false;
                    break;
                }
                tc_fence_after();
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_t(&full[stage], phase, abort_flag, w0)) { // operands landed and scale block written
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * kPfStageBytes);
                    const uint64_t dx = make_desc_sw128(sa);
                    const uint64_t dw = make_desc_sw128(sa + X_BYTES);
                    const uint32_t sfx = sf_base + static_cast<uint32_t>(stage * SF_COLS);
                    const uint32_t sfw = sfx + 4;
                    const uint32_t sfs = smem_u32(sf_smem + static_cast<size_t>(stage) * kPf4SfBytesPerStage);
                    tmem_cp_32x128b_x4(sfx, make_desc_rows16(sfs));
                    tmem_cp_32x128b_x4(sfw, make_desc_rows16(sfs + 512));
                    tmem_cp_32x128b_x4(sfw + 4, make_desc_rows16(sfs + 1024));
#pragma unroll
                    for (int kk = 0; kk < kBlockK8 / kUmmaK8; kk++) {
                        const uint32_t idesc = make_idesc_mx(0, 5, kPfTokens, kPfCols, kk); // A = e4m3 tokens, B = e2m1 weights
                        mma_mxf8f6f4(tmem_base, dx + 2 * kk, dw + 2 * kk, idesc, sfx, sfw, (kb | kk) ? 1u : 0u);
                    }
                    tc_commit(&empty[stage]); // frees the operand stage and its scale block
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
