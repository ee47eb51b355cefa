// Epilogue of prefill_gemm_fp8_kernel (included inside the kernel body; warps kPfEpiWarp0 .. kPfEpiWarp0 + 15).
// Group g = 0..3, TMEM lane quarter q: this thread owns token row r = q*32 + lane of the tile and 64 of its 256 columns.
{
    constexpr int CPT = 256 / kPfGroups; // columns per thread (64)
    constexpr int HALF = CPT / 2;        // gate/up: 32 gate + 32 up columns
    const int g = (warp - kPfEpiWarp0) >> 2;
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int kbs = K / kBlockK8;
    bool ok = true;
    uint32_t g_kb = 0, it = 0;
    long long w_body = 0, w_tail = 0, w_x = 0; // role profile: cycles in the promotion bodies / per-tile tails / amax exchange waits
    // scale rows of a work item: gate/up -> gate block nt and up block nt; down -> the 128-column block this group's columns
    // fall into (twice)
    auto weight_scale_rows = [&](int e_, int nt_, const float *&a, const float *&b) {
        const float *wbase = e_ < groups ? sc.w_scale + static_cast<size_t>(e_) * (w_rows_per_expert / 128) * kbs : sc.w_scale2;
        a = wbase + static_cast<size_t>(GATE_UP ? nt_ : nt_ * 2 + (g * CPT) / 128) * kbs;
        b = GATE_UP ? wbase + static_cast<size_t>(n_out / 128 + nt_) * kbs : a;
    };
    // Token scales four k-blocks per 16-byte load and weight scales one k-block per lane (see below) need scale rows that
    // are 16-byte multiples and at most 32 k-blocks; other shapes take one k-block at a time.
    const bool wide = (kbs & 3) == 0 && num_kb <= 32 && (reinterpret_cast<uintptr_t>(sc.x_scale) & 15) == 0;
    // The tile-table entry of the NEXT work item and its weight scales are fetched while the current one is processed, so
    // that a work item starts with one memory latency in front of it instead of three dependent ones.
    auto scale_row = [&](int row0_) {
        const int row = row0_ + r;
        return sc.x_scale + static_cast<size_t>(row < sc.max_rows ? row : sc.max_rows - 1) * kbs;
    };
    int e_cur = 0, row0_cur = 0;
    float wa_cur = 0.0f, wb_cur = 0.0f;
    float4 cx = make_float4(0.0f, 0.0f, 0.0f, 0.0f); // token scales of the coming four k-blocks (wide path)
    if (static_cast<int>(blockIdx.x) < total_work) {
        const int tile0 = blockIdx.x / n_n_tiles;
        e_cur = tt.tile_expert[tile0];
        row0_cur = tt.tile_row0[tile0];
        if (wide && lane < num_kb) {
            const float *a, *b;
            weight_scale_rows(e_cur, blockIdx.x - tile0 * n_n_tiles, a, b);
            wa_cur = __ldg(a + lane);
            wb_cur = __ldg(b + lane);
        }
        if (wide)
            cx = ldg_f4_pinned(scale_row(row0_cur));
    }
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, it++) {
        const int tile = w / n_n_tiles;
        const int nt = w - tile * n_n_tiles;
        const int e = e_cur;
        const int row0 = row0_cur;
        const int w_next = w + gridDim.x;
        const int tile_next = w_next / n_n_tiles;
        int e_next = 0, row0_next = 0;
        if (w_next < total_work) {
            e_next = __ldg(tt.tile_expert + tile_next);
            row0_next = __ldg(tt.tile_row0 + tile_next);
        }
        int nvalid = offsets[e + 1] - row0;
        nvalid = nvalid < kPfTokens ? nvalid : kPfTokens;
        const bool valid = r < nvalid;
        // rows past the segment's end read some other row's scales (their results are never stored); the clamp keeps the
        // read inside the array, and the address does not wait for the segment's length
        const float *xs_row = scale_row(row0);
        const float *ws_a, *ws_b;
        weight_scale_rows(e, nt, ws_a, ws_b);
        // columns of this thread: gate/up -> gate [32g, 32g+32) and up [128+32g, 128+32g+32); down -> [64g, 64g+64)
        const uint32_t col_a = GATE_UP ? static_cast<uint32_t>(HALF * g) : static_cast<uint32_t>(CPT * g);
        const uint32_t col_b = GATE_UP ? 128u + static_cast<uint32_t>(HALF * g) : static_cast<uint32_t>(CPT * g + HALF);
        float acc[CPT];
#pragma unroll
        for (int c = 0; c < CPT; c++)
            acc[c] = 0.0f;
        // One k-block: wait for its partial product in TMEM, promote it into the register accumulators with the block's
        // combined scales, hand the TMEM buffer back.
        auto promote = [&](float sa, float sb) -> bool {
            const uint32_t buf = g_kb % kPfIssuers;
            if (!mbar_wait_t(&tmem_full[buf], (g_kb / kPfIssuers) & 1u, abort_flag, w0))
                return false;
            tc_fence_after();
            const long long t_body = prof_clock();
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kPfCols;
            // sixteen columns at a time: the register budget leaves room for one staging block beside the 64 accumulators
#pragma unroll
            for (int i = 0; i < CPT / 16; i++) {
                uint32_t p[16];
                const bool second = i >= HALF / 16; // gate/up: the up columns; down: the upper half of the 64 columns
                tmem_ld16(t0 + (second ? col_b + (i - HALF / 16) * 16 : col_a + i * 16), p);
                tmem_ld_wait_16(p);
                const float sc_ = second ? sb : sa;
#pragma unroll
                for (int c = 0; c < 16; c++)
                    acc[i * 16 + c] = __fmaf_rn(__uint_as_float(p[c]), sc_, acc[i * 16 + c]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&tmem_empty[buf]);
            w_body += prof_clock() - t_body;
            g_kb++;
            return true;
        };
        // The scales of a k-block (one per token row, one per 128-column weight block) come from global memory.  Fetched
        // where they are used, their latency -- the same for all sixteen warps, which leave the accumulator barrier together
        // -- is paid once per k-block and the tensor pipe waits for it.  So:
        //   * token scales: the four scales of a row for four consecutive k-blocks are 16 contiguous bytes; they are
        //     fetched one such group ahead, so a group's registers are first read four k-blocks after its loads;
        //   * weight scales (the same for every thread of a warp): lane l holds the scales of k-block l -- one coalesced
        //     load per scale row and work item, issued during the previous work item -- and every k-block takes its pair
        //     by a warp shuffle.
        float wa_next = 0.0f, wb_next = 0.0f;
        if (wide) {
            for (int kb = 0; kb < num_kb && ok; kb += 4) {
                // pinned: the compiler would otherwise sink this load to its first use (it costs four live registers),
                // and the use would then wait out the whole memory latency once per group.  The last group of a work item
                // fetches the first group of the next one.
                float4 nx = cx;
                if (kb + 4 < num_kb)
                    nx = ldg_f4_pinned(xs_row + kb + 4);
                else if (w_next < total_work)
                    nx = ldg_f4_pinned(scale_row(row0_next));
                const float sx[4] = {cx.x, cx.y, cx.z, cx.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float a = __shfl_sync(0xffffffffu, wa_cur, kb + j), b = __shfl_sync(0xffffffffu, wb_cur, kb + j);
                    ok = ok && promote(__fmul_rn(sx[j], a), __fmul_rn(sx[j], b));
                }
                cx = nx;
                if (kb == 0 && w_next < total_work && lane < num_kb) { // the next work item's table entry has arrived by now
                    const float *a, *b;
                    weight_scale_rows(e_next, w_next - tile_next * n_n_tiles, a, b);
                    wa_next = __ldg(a + lane);
                    wb_next = __ldg(b + lane);
                }
            }
        } else {
            for (int kb = 0; kb < num_kb && ok; kb++) {
                const float sx = __ldg(xs_row + kb);
                ok = promote(__fmul_rn(sx, __ldg(ws_a + kb)), __fmul_rn(sx, __ldg(ws_b + kb)));
            }
        }
        e_cur = e_next;
        row0_cur = row0_next;
        wa_cur = wa_next;
        wb_cur = wb_next;
        if (!ok)
            break;
        const long long t_tail = prof_clock();
        if constexpr (GATE_UP) {
            // act = silu(gate) * up for this thread's 32 features; the 1x128 group spans the four warpgroups
            float m = 0.0f;
#pragma unroll
            for (int c = 0; c < HALF; c++) {
                acc[c] = silu_tanh(acc[c]) * acc[HALF + c];
                m = fmaxf(m, fabsf(acc[c]));
            }
            float *ax = amax_x + (it & 1) * (kPfGroups * 128);
            ax[g * 128 + r] = m;
            __syncwarp();
            if (lane == 0)
                mbar_arrive(xbar);
            if (!mbar_wait_t(xbar, it & 1, abort_flag, w_x)) {
                ok = false;
                break;
            }
#pragma unroll
            for (int j = 0; j < kPfGroups; j++)
                m = fmaxf(m, ax[j * 128 + r]);
            // s = max(amax, 1e-10) / 448 is what the down GEMM multiplies back; the codes are acc * (1 / s) with the
            // reciprocal taken once per row (against a division per element: at most one f32 ulp before the e4m3 rounding)
            const float mm = fmaxf(m, 1e-10f);
            const float s = __fdiv_rn(mm, 448.0f);
            const float rs = __fdiv_rn(448.0f, mm);
            if (valid) {
                uint8_t *dst = static_cast<uint8_t *>(out) + static_cast<size_t>(row0 + r) * n_out + nt * 128 + HALF * g;
#pragma unroll
                for (int v = 0; v < HALF / 16; v++) {
                    uint32_t pk[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int c = v * 16 + j * 4;
                        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(acc[c], rs), __fmul_rn(acc[c + 1], rs)), __NV_SATFINITE, __NV_E4M3);
                        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(acc[c + 2], rs), __fmul_rn(acc[c + 3], rs)), __NV_SATFINITE, __NV_E4M3);
                        pk[j] = lo | (hi << 16);
                    }
                    *reinterpret_cast<uint4 *>(dst + v * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
                if (g == 0)
                    sc.act_scale[static_cast<size_t>(row0 + r) * (n_out / 128) + nt] = s;
            }
        } else {
            // This thread holds 64 consecutive f32 columns of ONE row, so a plain 16-byte store per lane would touch 32
            // rows per instruction (32 separate lines for the store path to walk).  The four lanes of a quad first
            // transpose 4 x 4 blocks of 16-byte chunks among themselves: afterwards lane q of quad a holds chunks q, q + 4,
            // q + 8, q + 12 of each of the quad's four rows, and one store instruction writes 64 contiguous bytes per quad,
            // 8 rows instead of 32.
            const int qd = lane & 3;
            const int rq = q * 32 + (lane & ~3); // first row of the quad within the tile
            if (y_bf16) {
                // the layer's own combine reads these rows: bf16 halves the store and the read (the quantised formats'
                // tolerance allows the extra rounding, as on the expert-parallel wire).  64 columns = 8 chunks of 8.
#pragma unroll
                for (int m = 0; m < 2; m++) {
                    uint4 b[4];
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        uint32_t pk[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[(4 * m + v) * 8 + 2 * u], acc[(4 * m + v) * 8 + 2 * u + 1]);
                            pk[u] = *reinterpret_cast<const uint32_t *>(&h2);
                        }
                        b[v] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                    quad_transpose_chunks(b, qd); // b[i] = chunk 4 m + qd (8 columns) of row rq + i
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        if (rq + i < nvalid) {
                            __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(out) + static_cast<size_t>(row0 + rq + i) * n_out + nt * 256 + CPT * g;
                            *reinterpret_cast<uint4 *>(dst + (4 * m + qd) * 8) = b[i];
                        }
                }
            } else {
            float4 ch[16];
#pragma unroll
            for (int v = 0; v < 16; v++)
                ch[v] = make_float4(acc[v * 4], acc[v * 4 + 1], acc[v * 4 + 2], acc[v * 4 + 3]);
#pragma unroll
            for (int m = 0; m < 4; m++) {
                uint4 b[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    b[j] = make_uint4(__float_as_uint(ch[4 * m + j].x), __float_as_uint(ch[4 * m + j].y), __float_as_uint(ch[4 * m + j].z),
                                      __float_as_uint(ch[4 * m + j].w));
                quad_transpose_chunks(b, qd); // b[i] = chunk 4 m + qd of row rq + i
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (rq + i < nvalid) {
                        float *dst = static_cast<float *>(out) + static_cast<size_t>(row0 + rq + i) * n_out + nt * 256 + CPT * g;
                        *reinterpret_cast<uint4 *>(dst + (4 * m + qd) * 4) = b[i];
                    }
            }
            }
        }
        w_tail += prof_clock() - t_tail;
    }
    if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
    if (warp == kPfEpiWarp0 && lane == 0) {
        prof_add(prof, 5, w0);
        prof_add(prof, 2, w_body);
        prof_add(prof, 4, w_tail - w_x); // the tail's own work
        prof_add(prof, 8, w_x);
    }
}
