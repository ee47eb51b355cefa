// Scale loaders of prefill_gemm_fp4_kernel (warps 6 and 11; included inside the kernel body).
// Per k-block: three 512-byte blocks -- e8m0 scales of the 128 token rows, of weight rows 0..127 and of weight rows
// 128..255 of the tile -- lane i writing the 16 bytes {rows i, 32+i, 64+i, 96+i}.  Global loads run kSfAhead of the
// warp's k-blocks ahead of the shared-memory stores.  The kPf4Loaders warps take k-blocks round-robin of the CTA's sequence (one
// warp alone was the kernel's bottleneck: it never once waited for a free slot while the MMA thread waited for scales).
{
    constexpr int kSfAhead = 3;
    const int loader = warp == 6 ? 0 : warp - 10; // warps 6, 11, 12, ...
    struct Cursor {
        int w, kb, row0;
        size_t wrow, wrow2;
        bool valid;
    };
    auto locate = [&](Cursor &c) {
        c.valid = c.w < total_work;
        if (c.valid) {
            const int tile = c.w / n_n_tiles;
            const int nt = c.w - tile * n_n_tiles;
            c.row0 = tt.tile_row0[tile];
            c.wrow = static_cast<size_t>(tt.tile_expert[tile]) * w_rows_per_expert + nt * N_PER_TILE;
            c.wrow2 = GATE_UP ? c.wrow + n_out : c.wrow + 128;
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
            int row = c.row0 + i * 32 + lane;
            row = row < sc.max_rows ? row : sc.max_rows - 1;
            r[i] = __ldg(reinterpret_cast<const uint32_t *>(sc.x_scale + static_cast<size_t>(row) * kbs + c.kb * 4));
            r[4 + i] = __ldg(reinterpret_cast<const uint32_t *>(sc.w_scale + (c.wrow + i * 32 + lane) * kbs + c.kb * 4));
            r[8 + i] = __ldg(reinterpret_cast<const uint32_t *>(sc.w_scale + (c.wrow2 + i * 32 + lane) * kbs + c.kb * 4));
        }
    };
    uint32_t ring[kSfAhead + 1][SF_COLS];
    Cursor ld{static_cast<int>(blockIdx.x), 0, 0, 0, 0, false}, stc = ld;
    locate(ld);
    locate(stc);
    uint32_t seq = loader; // index of this warp's next k-block in the CTA's sequence: slot = seq % stages
    for (int i = 0; i < loader && ld.valid; i++) {
        advance(ld);
        advance(stc);
    }
#pragma unroll
    for (int j = 0; j < kSfAhead; j++) {
        fetch(ld, ring[j]);
#pragma unroll
        for (int i = 0; i < kPf4Loaders; i++)
            if (ld.valid)
                advance(ld);
    }
    bool ok = true;
    while (stc.valid && ok) {
#pragma unroll
        for (int j = 0; j <= kSfAhead; j++) {
            if (!stc.valid)
                break;
            fetch(ld, ring[(j + kSfAhead) % (kSfAhead + 1)]);
#pragma unroll
            for (int i = 0; i < kPf4Loaders; i++)
                if (ld.valid)
                    advance(ld);
            const int stage = static_cast<int>(seq % static_cast<uint32_t>(stages));
            const uint32_t phase = (seq / static_cast<uint32_t>(stages)) & 1u;
            if (!mbar_wait_t(&empty[stage], phase ^ 1, abort_flag, w0)) {
                ok = false;
                break;
            }
            const uint32_t (&r)[SF_COLS] = ring[j];
            uint8_t *blk = sf_smem + static_cast<size_t>(stage) * kPf4SfBytesPerStage + lane * 16;
            *reinterpret_cast<uint4 *>(blk) = make_uint4(r[0], r[1], r[2], r[3]);
            *reinterpret_cast<uint4 *>(blk + 512) = make_uint4(r[4], r[5], r[6], r[7]);
            *reinterpret_cast<uint4 *>(blk + 1024) = make_uint4(r[8], r[9], r[10], r[11]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&sf_full[stage]);
            seq += kPf4Loaders;
#pragma unroll
            for (int i = 0; i < kPf4Loaders; i++)
                if (stc.valid)
                    advance(stc);
        }
    }
    if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
    if (lane == 0 && loader == 0)
        atomicAdd(&prof[4], static_cast<unsigned long long>(w0));
}
