// Scale warp(s) of prefill_gemm_fp4_kernel (warp 6, and 11.. when kPf4Loaders > 1; included inside the kernel body).
// Per k-block: three 512-byte blocks -- e8m0 scales of the 128 token rows, of weight rows 0..127 and of weight rows
// 128..255 of the tile -- lane i writing the 16 bytes {rows i, 32+i, 64+i, 96+i}.  The scale block of a k-block travels with
// its operand stage: slot = stage, the warp waits for empty[stage] like the TMA producer and is the second arrival on
// full[stage], so the MMA thread has one barrier to wait for and one commit per k-block.
// sf_tma: the TMA producer has put the scales of a group of four k-blocks into a raw slot as three row-major
// (128 rows x 16 bytes) boxes; this warp re-orders them.  Otherwise (K not a multiple of 512, unaligned scale matrices) the
// warp fetches the scales itself, one 32-bit load per row and k-block, a few k-blocks ahead (a row's scales of one k-block
// are 128 or 64 bytes away from the next row's, so every lane of such a load touches its own sector: slow, and kept for
// the shapes the TMA path cannot take).
{
    const int loader = warp == 6 ? 0 : warp - 10; // warps 6, 11, 12, ...
    const uint32_t nst = static_cast<uint32_t>(stages);
    if (sf_tma) {
        const int gpt = num_kb >> 2; // groups of four k-blocks per work item
        auto word = [](const uint4 &v, int j) { return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w)); };
        uint32_t group = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
            for (int g = 0; g < gpt && ok; g++, group++) {
                const uint32_t rs = group % kPf4RawSlots;
                if (!mbar_wait_t(&raw_full[rs], (group / kPf4RawSlots) & 1u, abort_flag, w0)) {
                    ok = false;
                    break;
                }
                const uint8_t *raw = raw_smem + rs * kPf4RawBytes;
                uint4 v[SF_COLS];
#pragma unroll
                for (int b = 0; b < 3; b++)
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        v[b * 4 + c] = *reinterpret_cast<const uint4 *>(raw + b * 2048 + (c * 32 + lane) * 16);
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&raw_empty[rs]); // the raw slot is in registers: the producer may refill it
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t seq = group * 4u + static_cast<uint32_t>(j);
                    const uint32_t slot = seq % nst;
                    if (!mbar_wait_t(&empty[slot], ((seq / nst) & 1u) ^ 1u, abort_flag, w0)) {
                        ok = false;
                        break;
                    }
                    uint8_t *blk = sf_smem + static_cast<size_t>(slot) * kPf4SfBytesPerStage + lane * 16;
                    *reinterpret_cast<uint4 *>(blk) = make_uint4(word(v[0], j), word(v[1], j), word(v[2], j), word(v[3], j));
                    *reinterpret_cast<uint4 *>(blk + 512) = make_uint4(word(v[4], j), word(v[5], j), word(v[6], j), word(v[7], j));
                    *reinterpret_cast<uint4 *>(blk + 1024) = make_uint4(word(v[8], j), word(v[9], j), word(v[10], j), word(v[11], j));
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&full[slot]);
                }
            }
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicOr(status, kStatusWaitTimeout);
        }
        if (lane == 0 && loader == 0)
            prof_add(prof, 4, w0);
    } else {
    constexpr int kSfAhead = 3;
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
    uint32_t ring[kSfAhead][SF_COLS];
    Cursor ld{static_cast<int>(blockIdx.x), 0, 0, 0, 0, false}, stc = ld;
    locate(ld);
    locate(stc);
    uint32_t seq = loader; // index of this warp's next k-block in the CTA's sequence
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
        for (int j = 0; j < kSfAhead; j++) {
            if (!stc.valid)
                break;
            const uint32_t slot = seq % nst;
            if (!mbar_wait_t(&empty[slot], ((seq / nst) & 1u) ^ 1u, abort_flag, w0)) {
                ok = false;
                break;
            }
            const uint32_t (&r)[SF_COLS] = ring[j];
            uint8_t *blk = sf_smem + static_cast<size_t>(slot) * kPf4SfBytesPerStage + lane * 16;
            *reinterpret_cast<uint4 *>(blk) = make_uint4(r[0], r[1], r[2], r[3]);
            *reinterpret_cast<uint4 *>(blk + 512) = make_uint4(r[4], r[5], r[6], r[7]);
            *reinterpret_cast<uint4 *>(blk + 1024) = make_uint4(r[8], r[9], r[10], r[11]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&full[slot]);
            seq += kPf4Loaders;
#pragma unroll
            for (int i = 0; i < kPf4Loaders; i++)
                if (stc.valid)
                    advance(stc);
            // Refill the slot just consumed AFTER its stores: a register read waits on a scoreboard it may share with the
            // newest loads, so a fetch issued before the stores would put its whole latency in front of them.
            fetch(ld, ring[j]);
#pragma unroll
            for (int i = 0; i < kPf4Loaders; i++)
                if (ld.valid)
                    advance(ld);
        }
    }
    if (!ok && lane == 0) {
        *abort_flag = 1;
        atomicOr(status, kStatusWaitTimeout);
    }
    if (lane == 0 && loader == 0)
        prof_add(prof, 4, w0);
    }
}
