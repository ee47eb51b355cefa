// Epilogue of prefill_gemm_fp8_kernel (included inside the kernel body; warps 2..9).
// Group g = 0/1, TMEM lane quarter q: this thread owns token row r = q*32 + lane of the tile and 128 of its 256 columns.
{
    const int g = (warp - 2) >> 2;
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int kbs = K / kBlockK8;
    bool ok = true;
    uint32_t g_kb = 0, it = 0;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
        const int tile = w / n_n_tiles;
        const int nt = w - tile * n_n_tiles;
        const int e = tt.tile_expert[tile];
        const int row0 = tt.tile_row0[tile];
        int nvalid = offsets[e + 1] - row0;
        nvalid = nvalid < kPfTokens ? nvalid : kPfTokens;
        const bool valid = r < nvalid;
        const float *xs_row = sc.x_scale + static_cast<size_t>(row0 + (valid ? r : 0)) * kbs;
        const float *wbase = e < groups ? sc.w_scale + static_cast<size_t>(e) * (w_rows_per_expert / 128) * kbs : sc.w_scale2;
        const float *ws_a = wbase + static_cast<size_t>(GATE_UP ? nt : nt * 2 + g) * kbs;
        const float *ws_b = GATE_UP ? wbase + static_cast<size_t>(n_out / 128 + nt) * kbs : ws_a;
        // columns of this thread: gate/up -> gate [64g, 64g+64) and up [128+64g, 128+64g+64); down -> [128g, 128g+128)
        const uint32_t col_a = GATE_UP ? 64u * g : 128u * g;
        const uint32_t col_b = GATE_UP ? 128u + 64u * g : 128u * g + 64u;
        float acc[128];
#pragma unroll
        for (int c = 0; c < 128; c++)
            acc[c] = 0.0f;
        for (int kb = 0; kb < num_kb; kb++, g_kb++) {
            const int buf = g_kb & 1;
            const float sx = __ldg(xs_row + kb);
            const float sa = __fmul_rn(sx, __ldg(ws_a + kb));
            const float sb = __fmul_rn(sx, __ldg(ws_b + kb));
            if (!mbar_wait_t(&tmem_full[buf], (g_kb >> 1) & 1, abort_flag, w0)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * kPfCols);
            // four rounds of 2 x 16 columns; the loads of round i+1 are in flight while round i is accumulated
            uint32_t pa[2][16], pb[2][16];
            tmem_ld16(t0 + col_a, pa[0]);
            tmem_ld16(t0 + col_b, pb[0]);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                tmem_ld_wait_for(pa[i & 1], pb[i & 1]);
                if (i < 3) {
                    tmem_ld16(t0 + col_a + (i + 1) * 16, pa[(i + 1) & 1]);
                    tmem_ld16(t0 + col_b + (i + 1) * 16, pb[(i + 1) & 1]);
                }
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    acc[i * 16 + c] = __fmaf_rn(__uint_as_float(pa[i & 1][c]), sa, acc[i * 16 + c]);
                    acc[64 + i * 16 + c] = __fmaf_rn(__uint_as_float(pb[i & 1][c]), sb, acc[64 + i * 16 + c]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&tmem_empty[buf]);
        }
        if (!ok)
            break;
        if constexpr (GATE_UP) {
            // act = silu(gate) * up for this thread's 64 features; the 1x128 group spans both warpgroups
            float m = 0.0f;
#pragma unroll
            for (int c = 0; c < 64; c++) {
                acc[c] = silu_fast(acc[c]) * acc[64 + c];
                m = fmaxf(m, fabsf(acc[c]));
            }
            float *ax = amax_x + (it & 1) * 256;
            ax[g * 128 + r] = m;
            __syncwarp();
            if (lane == 0)
                mbar_arrive(xbar);
            if (!mbar_wait(xbar, it & 1, abort_flag)) {
                ok = false;
                break;
            }
            m = fmaxf(ax[r], ax[128 + r]);
            const float s = __fdiv_rn(fmaxf(m, 1e-10f), 448.0f);
            if (valid) {
                uint8_t *dst = static_cast<uint8_t *>(out) + static_cast<size_t>(row0 + r) * n_out + nt * 128 + 64 * g;
#pragma unroll
                for (int v = 0; v < 4; v++) {
                    uint32_t pk[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        pk[j] = 0;
#pragma unroll
                        for (int b = 0; b < 4; b++)
                            pk[j] |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(acc[v * 16 + j * 4 + b], s))) << (8 * b);
                    }
                    *reinterpret_cast<uint4 *>(dst + v * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
                if (g == 0)
                    sc.act_scale[static_cast<size_t>(row0 + r) * (n_out / 128) + nt] = s;
            }
        } else {
            if (valid) {
                float *dst = static_cast<float *>(out) + static_cast<size_t>(row0 + r) * n_out + nt * 256 + 128 * g;
#pragma unroll
                for (int v = 0; v < 32; v++)
                    *reinterpret_cast<float4 *>(dst + v * 4) = make_float4(acc[v * 4], acc[v * 4 + 1], acc[v * 4 + 2], acc[v * 4 + 3]);
            }
        }
    }
    if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
    if (warp == 2 && lane == 0)
        atomicAdd(&prof[5], static_cast<unsigned long long>(w0));
}
