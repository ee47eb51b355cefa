// Epilogue of prefill_gemm_fp4_kernel (warps 2..5 = half 0, warps 7..10 = half 1; included inside the kernel body).
// Thread = token row r = q*32 + lane of the tile and one half of the output columns, walked 16 at a time.
{
    const int q = warp & 3;
    const int half = warp > 6 ? 1 : 0;
    const int r = q * 32 + lane;
    bool ok = true;
    uint32_t it = 0;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
        const int tile = w / n_n_tiles;
        const int nt = w - tile * n_n_tiles;
        const int e = tt.tile_expert[tile];
        const int row0 = tt.tile_row0[tile];
        int nvalid = offsets[e + 1] - row0;
        nvalid = nvalid < kPfTokens ? nvalid : kPfTokens;
        const bool valid = r < nvalid;
        if (!mbar_wait_t(tmem_full, it & 1, abort_flag, w0)) {
            ok = false;
            break;
        }
        tc_fence_after();
        const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        if (q * 32 >= nvalid) {
            // no valid token in this warp's lane quarter (decode-sized segments): nothing to read or store
        } else if constexpr (GATE_UP) {
            // features nt*128 + [0,128): gate in columns [0,128), up in [128,256); MX groups of 32 features = 2 chunks
            uint8_t *arow = static_cast<uint8_t *>(out) + static_cast<size_t>(row0 + r) * n_out + nt * 128;
            uint8_t *srow = sc.act_scale + static_cast<size_t>(row0 + r) * (n_out / 32) + nt * 4;
#pragma unroll 1
            for (int grp = 2 * half; grp < 2 * half + 2; grp++) {
                float a[32];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t pg[16], pu[16];
                    tmem_ld16(t0 + grp * 32 + h * 16, pg);
                    tmem_ld16(t0 + 128 + grp * 32 + h * 16, pu);
                    tmem_ld_wait_for(pg, pu);
#pragma unroll
                    for (int c = 0; c < 16; c++)
                        a[h * 16 + c] = silu_fast(__uint_as_float(pg[c])) * __uint_as_float(pu[c]);
                }
                float m = 0.0f;
#pragma unroll
                for (int c = 0; c < 32; c++)
                    m = fmaxf(m, fabsf(a[c]));
                const uint32_t se = e8m0_ceil(__fdiv_rn(fmaxf(m, 1e-30f), 448.0f));
                const float inv = __uint_as_float((254u - se) << 23);
                if (valid) {
#pragma unroll
                    for (int v = 0; v < 2; v++) {
                        uint32_t pk[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            pk[j] = 0;
#pragma unroll
                            for (int b = 0; b < 4; b++)
                                pk[j] |= static_cast<uint32_t>(f32_to_e4m3(__fmul_rn(a[v * 16 + j * 4 + b], inv))) << (8 * b);
                        }
                        *reinterpret_cast<uint4 *>(arow + grp * 32 + v * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                    srow[grp] = static_cast<uint8_t>(se);
                }
            }
        } else {
            float *yrow = static_cast<float *>(out) + static_cast<size_t>(row0 + r) * n_out + nt * 256;
#pragma unroll 1
            for (int c0 = 128 * half; c0 < 128 * half + 128; c0 += 32) {
                uint32_t pa[16], pb[16];
                tmem_ld16(t0 + c0, pa);
                tmem_ld16(t0 + c0 + 16, pb);
                tmem_ld_wait_for(pa, pb);
                if (valid) {
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        *reinterpret_cast<uint4 *>(yrow + c0 + v * 4) = make_uint4(pa[v * 4], pa[v * 4 + 1], pa[v * 4 + 2], pa[v * 4 + 3]);
                        *reinterpret_cast<uint4 *>(yrow + c0 + 16 + v * 4) = make_uint4(pb[v * 4], pb[v * 4 + 1], pb[v * 4 + 2], pb[v * 4 + 3]);
                    }
                }
            }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
            mbar_arrive(tmem_empty);
    }
    if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
    if (warp == 2 && lane == 0)
        atomicAdd(&prof[5], static_cast<unsigned long long>(w0));
}
