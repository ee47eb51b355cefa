// FP4 (e2m1) experts with one e8m0 scale per 32 elements of K, activations as MX-FP8 (e4m3 codes with one e8m0
// scale per 32 channels).  Both scale kinds are what the tensor core's block-scaled MMA applies itself
// (tcgen05.mma kind::mxf8f6f4.block_scale): the k-loop accumulates the whole K in TMEM, like the bf16 kernel,
// and no promotion pass is needed.
//
// Weights stay packed (two codes per byte) in HBM -- the bytes that bound decode -- and are expanded to one
// code per byte by the TMA unit on the way into shared memory (tensor map type 16U4_ALIGN16B), which is the
// shared-memory form the f8f6f4 MMA kinds read.
//
// Scale factors live in TMEM.  For an MMA of K = 32 each operand row has one scale byte; a 32-bit TMEM column
// carries the bytes of FOUR consecutive 32-blocks (the instruction descriptor's scale id picks the byte), and
// row r of the operand sits in lane r % 32, column r / 32, replicated in all four lane quarters.  One scale warp
// fetches them from global memory (one 32-bit load per row, issued a few k-blocks ahead) into a 512-byte block
// per operand tile in shared memory -- lane i writes the 16 bytes {rows i, 32+i, 64+i, 96+i} -- and the MMA
// thread moves each block into TMEM with tcgen05.cp (32x128b, replicated x4) right before the MMAs that use it,
// so no thread ever waits for a TMEM store.
//
// Warps: 0 TMA producer | 1 MMA issuer, TMEM owner | 2..5 epilogue | 6 scale loader.
#pragma once
#include "xs_grouped_gemm.cuh"

namespace xs {

constexpr int kFp4Threads = 224;
constexpr int kFp4SfBytesPerStage = 1536; // three 512-byte scale blocks: gate rows, up rows, tokens

struct MxScales {
    const uint8_t *w_scale; // (groups * w_rows_per_expert, K / 32) e8m0
    const uint8_t *x_scale; // (rows, K / 32) e8m0
    uint8_t *act_scale;     // GATE_UP only: (rows, n_out / 32) written by the epilogue
    int max_rows;           // rows of x_scale (for clamping reads past the last segment)
};

// Expert-parallel return trip folded into the down GEMM's epilogue: with peer_back set, output row g of local expert el
// -- the j-th row that source rank s sent for that expert -- is rounded to bf16 and stored straight into row
// src_offsets[s][e] + j of rank s's return buffer (plain peer stores over NVLink), instead of going to y as f32 for a
// separate return kernel to pick up.  all_counts (ranks, experts), src_offsets (ranks, experts): the tables of ep_plan.
struct EpReturnArgs {
    uint8_t *const *peer_back = nullptr; // `ranks` pointers (this rank's own buffer included); null: store f32 rows to y
    const int32_t *all_counts = nullptr;
    const int32_t *src_offsets = nullptr;
    int experts = 0, ranks = 1, me = 0, back_capacity = 0;
    int y_bf16 = 0; // no peers: store the rows to `out` as bf16 instead of f32 (the layer's own combine reads them)
};

// smallest e8m0 exponent whose power of two is >= v (v > 0, normal)
__device__ __forceinline__ uint32_t e8m0_ceil(float v)
{
    const uint32_t b = __float_as_uint(v);
    uint32_t e = (b >> 23) & 0xffu;
    if (b & 0x7fffffu)
        e += 1;
    return e > 254u ? 254u : e;
}

template <int N_TILE, bool GATE_UP>
__global__ void __launch_bounds__(kFp4Threads, 1)
grouped_gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const int32_t *__restrict__ offsets, TileTable tt, MxScales sc, int w_rows_per_expert, int n_out, int K,
                        void *__restrict__ out, int32_t *__restrict__ status, int stages)
{
    constexpr int A_BYTES = kTileM * kBlockK8;   // one code per byte in shared memory
    constexpr int B_BYTES = N_TILE * kBlockK8;
    constexpr int STAGE_BYTES = (GATE_UP ? 2 : 1) * A_BYTES + B_BYTES;
    // the copy engine reports the PACKED bytes it fetched for a 4-bit tile (half of the shared-memory footprint)
    constexpr int TX_BYTES = (GATE_UP ? 2 : 1) * (A_BYTES / 2) + B_BYTES;
    constexpr int ACC_COLS = (GATE_UP ? 2 : 1) * N_TILE;
    constexpr int SF_W_COLS = GATE_UP ? 8 : 4;   // 4 columns = 128 rows of one weight tile
    constexpr int SF_X_COLS = 4;                 // tokens n -> lane n % 32, column n / 32 (N_TILE <= 128)
    constexpr int SF_COLS = SF_W_COLS + SF_X_COLS;
    constexpr int kMaxStages = 8;
    constexpr int NEED = 2 * ACC_COLS + kMaxStages * SF_COLS;
    constexpr int TMEM_COLS = NEED <= 128 ? 128 : (NEED <= 256 ? 256 : 512);
    static_assert(NEED <= 512, "token tile too wide for the TMEM budget");

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(stages) * STAGE_BYTES);
    uint64_t *full = bars;
    uint64_t *empty = bars + stages;
    uint64_t *sf_full = bars + 2 * stages;
    uint64_t *tmem_full = bars + 3 * stages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    uint8_t *sf_smem = reinterpret_cast<uint8_t *>(bars) + 512; // [stages][kFp4SfBytesPerStage], 16-byte aligned

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // role profile: cycles each role spent blocked, summed over CTAs into eight 64-bit counters behind the status word
    unsigned long long *prof = reinterpret_cast<unsigned long long *>(status + 16);
    const long long t_start = prof_clock();
    long long w0 = 0, w1 = 0, w2 = 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
            mbar_init(&sf_full[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4);
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
    pdl_wait(); // everything above touches only this CTA's shared memory and TMEM
    const uint32_t sf_base = tmem_base + 2 * ACC_COLS;

    const int n_f_tiles = n_out / kTileM;
    const int num_tiles = *tt.num_tiles;
    const int total_work = num_tiles * n_f_tiles;
    const int num_kb = K / kBlockK8;
    const int kbs = K / 32; // scale bytes per row

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
                    if (!mbar_wait_t(&empty[stage], phase ^ 1, abort_flag, w0)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + static_cast<size_t>(stage) * STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[stage], TX_BYTES);
                    tma_load_2d(st, &tmap_w, &full[stage], kb * kBlockK8, wrow, pol_w);
                    if (GATE_UP)
                        tma_load_2d(st + A_BYTES, &tmap_w, &full[stage], kb * kBlockK8, wrow + n_out, pol_w);
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
            int it = 0;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
                const int buf = it & 1;
                const uint32_t use = static_cast<uint32_t>(it >> 1);
                if (!mbar_wait_t(&tmem_empty[buf], (use & 1) ^ 1, abort_flag, w2)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d0 = tmem_base + static_cast<uint32_t>(buf * ACC_COLS);
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_t(&full[stage], phase, abort_flag, w0) || !mbar_wait_t(&sf_full[stage], phase, abort_flag, w1)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * STAGE_BYTES);
                    const uint64_t da = make_desc_sw128(sa);
                    const uint64_t du = make_desc_sw128(sa + A_BYTES);
                    const uint64_t db = make_desc_sw128(sa + (GATE_UP ? 2 : 1) * A_BYTES);
                    const uint32_t sfw = sf_base + static_cast<uint32_t>(stage * SF_COLS);
                    const uint32_t sfx = sfw + SF_W_COLS;
                    const uint32_t sfs = smem_u32(sf_smem + static_cast<size_t>(stage) * kFp4SfBytesPerStage);
                    tmem_cp_32x128b_x4(sfw, make_desc_rows16(sfs));
                    if (GATE_UP)
                        tmem_cp_32x128b_x4(sfw + 4, make_desc_rows16(sfs + 512));
                    tmem_cp_32x128b_x4(sfx, make_desc_rows16(sfs + 1024));
#pragma unroll
                    for (int kk = 0; kk < kBlockK8 / kUmmaK8; kk++) {
                        const uint32_t idesc = make_idesc_mx(5, 0, kTileM, N_TILE, kk); // A = e2m1, B = e4m3, scale byte kk
                        const uint32_t acc = (kb | kk) ? 1u : 0u;
                        mma_mxf8f6f4(d0, da + 2 * kk, db + 2 * kk, idesc, sfw, sfx, acc);
                        if (GATE_UP)
                            mma_mxf8f6f4(d0 + N_TILE, du + 2 * kk, db + 2 * kk, idesc, sfw + 4, sfx, acc);
                    }
                    tc_commit(&empty[stage]); // frees the shared-memory stage and its scale slot
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
            prof_add(prof, 1, w0);
            prof_add(prof, 2, w1);
            prof_add(prof, 3, w2);
        }
    } else if (warp == 6) {
        // Scale loader.  The global loads run kSfAhead k-blocks ahead of the shared-memory stores (a register ring),
        // so their latency is off the per-stage critical path.
        constexpr int kSfAhead = 3;
        struct Cursor {
            int w, kb, row0;
            size_t wrow;
            bool valid;
        };
        auto locate = [&](Cursor &c) {
            c.valid = c.w < total_work;
            if (c.valid) {
                const int tile = c.w / n_f_tiles;
                const int f = c.w - tile * n_f_tiles;
                c.row0 = tt.tile_row0[tile];
                c.wrow = static_cast<size_t>(tt.tile_expert[tile]) * w_rows_per_expert + f * kTileM;
            }
        };
        auto advance = [&](Cursor &c) {
            if (++c.kb == num_kb) {
                c.kb = 0;
                c.w += gridDim.x;
                locate(c);
            }
        };
        auto fetch = [&](const Cursor &c, uint32_t (&r)[SF_COLS]) {
            if (!c.valid)
                return;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                r[i] = __ldg(reinterpret_cast<const uint32_t *>(sc.w_scale + (c.wrow + i * 32 + lane) * kbs + c.kb * 4));
                if constexpr (GATE_UP)
                    r[4 + i] = __ldg(reinterpret_cast<const uint32_t *>(sc.w_scale + (c.wrow + n_out + i * 32 + lane) * kbs + c.kb * 4));
            }
#pragma unroll
            for (int i = 0; i < SF_X_COLS; i++) {
                int row = c.row0 + i * 32 + lane;
                row = row < sc.max_rows ? row : sc.max_rows - 1;
                r[SF_W_COLS + i] =
                    (i * 32 < N_TILE) ? __ldg(reinterpret_cast<const uint32_t *>(sc.x_scale + static_cast<size_t>(row) * kbs + c.kb * 4)) : 0u;
            }
        };
        uint32_t ring[kSfAhead + 1][SF_COLS];
        Cursor ld{static_cast<int>(blockIdx.x), 0, 0, 0, false}, stc = ld;
        locate(ld);
        locate(stc);
#pragma unroll
        for (int j = 0; j < kSfAhead; j++) {
            fetch(ld, ring[j]);
            advance(ld);
        }
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        while (stc.valid && ok) {
#pragma unroll
            for (int j = 0; j <= kSfAhead; j++) {
                if (!stc.valid)
                    break;
                fetch(ld, ring[(j + kSfAhead) % (kSfAhead + 1)]);
                advance(ld);
                if (!mbar_wait_t(&empty[stage], phase ^ 1, abort_flag, w0)) {
                    ok = false;
                    break;
                }
                const uint32_t (&r)[SF_COLS] = ring[j];
                uint8_t *blk = sf_smem + static_cast<size_t>(stage) * kFp4SfBytesPerStage + lane * 16;
                *reinterpret_cast<uint4 *>(blk) = make_uint4(r[0], r[1], r[2], r[3]);
                if constexpr (GATE_UP)
                    *reinterpret_cast<uint4 *>(blk + 512) = make_uint4(r[4], r[5], r[6], r[7]);
                *reinterpret_cast<uint4 *>(blk + 1024) = make_uint4(r[SF_W_COLS], r[SF_W_COLS + 1], r[SF_W_COLS + 2], r[SF_W_COLS + 3]);
                fence_proxy_async_smem(); // the tensor-core copy engine reads these bytes through the async proxy
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&sf_full[stage]);
                if (++stage == stages) {
                    stage = 0;
                    phase ^= 1;
                }
                advance(stc);
            }
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicOr(status, kStatusWaitTimeout);
        }
        if (warp == 6 && lane == 0)
            prof_add(prof, 4, w0);
    } else {
        const int q = warp & 3;
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
            if (!mbar_wait_t(&tmem_full[buf], use & 1, abort_flag, w0)) {
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
                if constexpr (GATE_UP) {
                    uint32_t u[16];
                    tmem_ld16(t0 + N_TILE + c0, u);
                    tmem_ld_wait();
                    uint8_t *actq = static_cast<uint8_t *>(out);
#pragma unroll
                    for (int c = 0; c < 16; c++) {
                        // the 32 features of this warp are one MX group of the token: amax by shuffles
                        const float a = silu_fast(__uint_as_float(g[c])) * __uint_as_float(u[c]);
                        float m = fabsf(a);
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1)
                            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                        const uint32_t se = e8m0_ceil(__fdiv_rn(fmaxf(m, 1e-30f), 448.0f));
                        const float inv = __uint_as_float((254u - se) << 23); // 2^(127 - se), exact
                        if (c0 + c < nvalid) {
                            actq[static_cast<size_t>(row0 + c0 + c) * n_out + feature] = f32_to_e4m3(__fmul_rn(a, inv));
                            if (lane == 0)
                                sc.act_scale[static_cast<size_t>(row0 + c0 + c) * (n_out / 32) + f * 4 + q] = static_cast<uint8_t>(se);
                        }
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

// x (rows, cols) bf16 -> MX-FP8: e4m3 codes + one e8m0 scale per (row, 32 columns):
// s = smallest power of two >= max(amax, 1e-30) / 448, code = e4m3_rne_sat(x / s) (exact scaling by a power of two).
// Optionally scatters: row r of the input goes to rows dst[r*nd .. r*nd+nd) of the output (nd = 1, dst = NULL: in place order).
__global__ void __launch_bounds__(256)
quantize_rows_mxfp8_kernel(const __nv_bfloat16 *__restrict__ x, const int32_t *__restrict__ dst, int nd, uint8_t *__restrict__ q,
                           uint8_t *__restrict__ scale, int rows, int cols)
{
    const int r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (r >= rows)
        return;
    const int groups = cols / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // one warp handles 4 groups (128 columns) per step: 8 lanes x 4 elements per group
    for (int c0 = warp * 128; c0 < cols; c0 += (blockDim.x >> 5) * 128) {
        const uint2 raw = *reinterpret_cast<const uint2 *>(x + static_cast<size_t>(r) * cols + c0 + lane * 4);
        float v[4];
        v[0] = __uint_as_float(raw.x << 16);
        v[1] = __uint_as_float(raw.x & 0xffff0000u);
        v[2] = __uint_as_float(raw.y << 16);
        v[3] = __uint_as_float(raw.y & 0xffff0000u);
        float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1)
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o)); // within groups of 8 lanes
        const uint32_t se = e8m0_ceil(__fdiv_rn(fmaxf(m, 1e-30f), 448.0f));
        const float inv = __uint_as_float((254u - se) << 23);
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 4; i++)
            packed |= static_cast<uint32_t>(f32_to_e4m3(__fmul_rn(v[i], inv))) << (8 * i);
        for (int d = 0; d < nd; d++) {
            const size_t orow = dst ? static_cast<size_t>(dst[static_cast<size_t>(r) * nd + d]) : static_cast<size_t>(r);
            *reinterpret_cast<uint32_t *>(q + orow * cols + c0 + lane * 4) = packed;
            if ((lane & 7) == 0)
                scale[orow * groups + (c0 >> 5) + (lane >> 3)] = static_cast<uint8_t>(se);
        }
    }
}

} // namespace xs
