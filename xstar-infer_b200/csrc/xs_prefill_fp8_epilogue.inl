// Epilogue of prefill_gemm_fp8_kernel (included inside the kernel body; warps 2..17).
// Group g = 0..3, TMEM lane quarter q: this thread owns token row r = q*32 + lane of the tile and 64 of its 256 columns.
{
    constexpr int CPT = 256 / kPfGroups; // columns per thread (64)
    constexpr int HALF = CPT / 2;        // gate/up: 32 gate + 32 up columns
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
        // gate/up: gate block nt and up block nt; down: the 128-column block this group's columns fall into
        const float *ws_a = wbase + static_cast<size_t>(GATE_UP ? nt : nt * 2 + (g * CPT) / 128) * kbs;
        const float *ws_b = GATE_UP ? wbase + static_cast<size_t>(n_out / 128 + nt) * kbs : ws_a;
        // columns of this thread: gate/up -> gate [32g, 32g+32) and up [128+32g, 128+32g+32); down -> [64g, 64g+64)
        const uint32_t col_a = GATE_UP ? static_cast<uint32_t>(HALF * g) : static_cast<uint32_t>(CPT * g);
        const uint32_t col_b = GATE_UP ? 128u + static_cast<uint32_t>(HALF * g) : static_cast<uint32_t>(CPT * g + HALF);
        float acc[CPT];
#pragma unroll
        for (int c = 0; c < CPT; c++)
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
#pragma unroll
            for (int i = 0; i < HALF / 16; i++) {
                uint32_t pa[16], pb[16];
                tmem_ld16(t0 + col_a + i * 16, pa);
                tmem_ld16(t0 + col_b + i * 16, pb);
                tmem_ld_wait_for(pa, pb);
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    acc[i * 16 + c] = __fmaf_rn(__uint_as_float(pa[c]), sa, acc[i * 16 + c]);
                    acc[HALF + i * 16 + c] = __fmaf_rn(__uint_as_float(pb[c]), sb, acc[HALF + i * 16 + c]);
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
            // act = silu(gate) * up for this thread's 32 features; the 1x128 group spans the four warpgroups
            float m = 0.0f;
#pragma unroll
            for (int c = 0; c < HALF; c++) {
                acc[c] = silu_fast(acc[c]) * acc[HALF + c];
                m = fmaxf(m, fabsf(acc[c]));
            }
            float *ax = amax_x + (it & 1) * (kPfGroups * 128);
            ax[g * 128 + r] = m;
            __syncwarp();
            if (lane == 0)
                mbar_arrive(xbar);
            if (!mbar_wait(xbar, it & 1, abort_flag)) {
                ok = false;
                break;
            }
#pragma unroll
            for (int j = 0; j < kPfGroups; j++)
                m = fmaxf(m, ax[j * 128 + r]);
            const float s = __fdiv_rn(fmaxf(m, 1e-10f), 448.0f);
            if (valid) {
                uint8_t *dst = static_cast<uint8_t *>(out) + static_cast<size_t>(row0 + r) * n_out + nt * 128 + HALF * g;
#pragma unroll
                for (int v = 0; v < HALF / 16; v++) {
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
                float *dst = static_cast<float *>(out) + static_cast<size_t>(row0 + r) * n_out + nt * 256 + CPT * g;
#pragma unroll
                for (int v = 0; v < CPT / 4; v++)
                    *reinterpret_cast<float4 *>(dst + v * 4) = make_float4(acc[v * 4], acc[v * 4 + 1], acc[v * 4 + 2], acc[v * 4 + 3]);
            }
        }
    }
    if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
    if (warp == 2 && lane == 0)
        prof_add(prof, 5, w0);
}
