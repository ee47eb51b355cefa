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
        nvalid = nvalid < tile_rows ? nvalid : tile_rows;
        const bool valid = r < nvalid;
        if (!mbar_wait_t(tmem_full, it & 1, abort_flag, w0)) {
            ok = false;
            break;
        }
        tc_fence_after();
        const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        // The raw accumulators leave TMEM first and the accumulator is handed back to the MMA thread BEFORE SwiGLU, the
        // quantisation and the global stores, which then overlap the next tile's main loop.
        const bool active = q * 32 < nvalid; // no valid token in this warp's lane quarter: nothing to read or store
        if constexpr (GATE_UP) {
            // features nt*128 + [0,128): gate in columns [0,128), up in [128,256); this thread: groups 2*half, 2*half + 1
            uint32_t pg[2][2][16], pu[2][2][16]; // raw gate / up accumulators of this thread's two groups
            if (active) {
#pragma unroll
                for (int g = 0; g < 2; g++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        tmem_ld16(t0 + (2 * half + g) * 32 + h * 16, pg[g][h]);
                        tmem_ld16(t0 + 128 + (2 * half + g) * 32 + h * 16, pu[g][h]);
                    }
#pragma unroll
                for (int g = 0; g < 2; g++)
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        tmem_ld_wait_for(pg[g][h], pu[g][h]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(tmem_empty);
            float a[2][32];
            if (active) {
#pragma unroll
                for (int g = 0; g < 2; g++)
#pragma unroll
                    for (int h = 0; h < 2; h++)
#pragma unroll
                        for (int c = 0; c < 16; c++)
                            a[g][h * 16 + c] = silu_tanh(__uint_as_float(pg[g][h][c])) * __uint_as_float(pu[g][h][c]);
            }
            if (active) {
                uint8_t *arow = static_cast<uint8_t *>(out) + static_cast<size_t>(row0 + r) * n_out + nt * 128;
                uint8_t *srow = sc.act_scale + static_cast<size_t>(row0 + r) * (n_out / 32) + nt * 4;
#pragma unroll
                for (int g = 0; g < 2; g++) {
                    const int grp = 2 * half + g; // one MX group of 32 features
                    float m = 0.0f;
#pragma unroll
                    for (int c = 0; c < 32; c++)
                        m = fmaxf(m, fabsf(a[g][c]));
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
                                    pk[j] |= static_cast<uint32_t>(f32_to_e4m3(__fmul_rn(a[g][v * 16 + j * 4 + b], inv))) << (8 * b);
                            }
                            *reinterpret_cast<uint4 *>(arow + grp * 32 + v * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        }
                        srow[grp] = static_cast<uint8_t>(se);
                    }
                }
            }
        } else {
            uint32_t y[8][16]; // this thread's 128 columns
            if (active) {
#pragma unroll
                for (int i = 0; i < 8; i++)
                    tmem_ld16(t0 + 128 * half + i * 16, y[i]);
#pragma unroll
                for (int i = 0; i < 4; i++)
                    tmem_ld_wait_for(y[2 * i], y[2 * i + 1]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(tmem_empty);
            // (all lanes of an active warp take part in the quad transposes; rows past the segment are not stored)
            if (active && ret.peer_back == nullptr && !ret.y_bf16) {
                const int qd = lane & 3;
                const int rq = q * 32 + (lane & ~3); // first row of the quad within the tile
                float *ybase = static_cast<float *>(out) + static_cast<size_t>(row0 + rq) * n_out + nt * 256 + 128 * half;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    uint4 b[4];
#pragma unroll
                    for (int v = 0; v < 4; v++)
                        b[v] = make_uint4(y[i][v * 4], y[i][v * 4 + 1], y[i][v * 4 + 2], y[i][v * 4 + 3]);
                    quad_transpose_chunks(b, qd); // b[r] = chunk qd of columns [16 i, 16 i + 16) of row rq + r
#pragma unroll
                    for (int r = 0; r < 4; r++)
                        if (rq + r < nvalid)
                            *reinterpret_cast<uint4 *>(ybase + static_cast<size_t>(r) * n_out + i * 16 + qd * 4) = b[r];
                }
            } else if (active) {
                // bf16 rows.  Expert-parallel return: this thread's row is the j-th row source rank s sent for this expert; it
                // goes to row src_offsets[s][e] + j of that rank's return buffer.  Without peers: to its own row of `out`.
                uint8_t *dst = nullptr;
                if (valid && ret.peer_back == nullptr) {
                    dst = static_cast<uint8_t *>(out) + (static_cast<size_t>(row0 + r) * n_out + nt * 256 + 128 * half) * 2; // local bf16 rows
                } else if (valid) {
                    const int El = ret.experts / ret.ranks;
                    const int eg = ret.me * El + e;
                    int j = row0 + r - offsets[e];
                    int s = 0;
                    while (s < ret.ranks - 1 && j >= ret.all_counts[s * ret.experts + eg]) {
                        j -= ret.all_counts[s * ret.experts + eg];
                        s++;
                    }
                    const int drow = ret.src_offsets[s * ret.experts + eg] + j;
                    if (drow >= 0 && drow < ret.back_capacity)
                        dst = ret.peer_back[s] + (static_cast<size_t>(drow) * n_out + nt * 256 + 128 * half) * 2;
                    else
                        atomicOr(status, kStatusBadIndex);
                }
                const int qd = lane & 3;
                const unsigned long long mine = reinterpret_cast<unsigned long long>(dst);
                unsigned long long qdst[4]; // destinations of the four rows of this lane's quad
#pragma unroll
                for (int rr = 0; rr < 4; rr++)
                    qdst[rr] = __shfl_sync(0xffffffffu, mine, (lane & ~3) + rr);
                // 128 f32 columns -> 64 bf16 pairs = 16 chunks of 16 bytes (8 columns each); quads transpose four chunks at a
                // time, so each store instruction writes 64 contiguous bytes per row
#pragma unroll
                for (int m = 0; m < 4; m++) {
                    uint4 b[4];
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        const uint32_t *src = &y[(4 * m + v) >> 1][((4 * m + v) & 1) * 8];
                        uint32_t pk[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(src[2 * u]), __uint_as_float(src[2 * u + 1]));
                            pk[u] = *reinterpret_cast<const uint32_t *>(&h2);
                        }
                        b[v] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                    quad_transpose_chunks(b, qd); // b[rr] = chunk 4 m + qd (8 columns) of row rq + rr
#pragma unroll
                    for (int rr = 0; rr < 4; rr++)
                        if (qdst[rr])
                            *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(qdst[rr]) + (4 * m + qd) * 16) = b[rr];
                }
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
