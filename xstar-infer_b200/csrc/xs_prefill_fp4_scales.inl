// Scale loaders of prefill_gemm_fp4_kernel (warps 6 and 11; included inside the kernel body).
// Per k-block: three 512-byte blocks -- e8m0 scales of the 128 token rows, of weight rows 0..127 and of weight rows
// 128..255 of the tile -- lane i writing the 16 bytes {rows i, 32+i, 64+i, 96+i}.  The kPf4Loaders warps take k-blocks
// round-robin of the CTA's sequence (one warp alone was the kernel's bottleneck).
// A row's scales of one k-block are 4 bytes, 128 or 64 bytes away from the next row's: every lane of a load touches its
// own 32-byte sector, and it is the number of such requests that bounds a loader (measured: 1200 cycles to issue the 12
// loads of a k-block, 1300 more until their data could be stored).  So where the shapes allow (K a multiple of 512) a
// loader fetches 16 bytes per row -- FOUR k-blocks -- per request and keeps them in registers (wide path); the loaders
// take such groups round-robin.  The scale blocks go through a ring of kPf4SfSlots shared-memory slots with barriers of its
// own (sf_full / sf_empty, the latter arrived by tcgen05.commit): slot n % kPf4SfSlots for the n-th k-block of the CTA, so a
// slot is always written by the same loader and its consecutive uses are exactly one barrier phase apart.
{
    const int loader = warp == 6 ? 0 : warp - 10; // warps 6, 11, 12, ...
    static_assert(kPf4SfSlots % (4 * kPf4Loaders) == 0, "every scale slot belongs to one loader, in both paths");
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(sc.x_scale) | reinterpret_cast<uintptr_t>(sc.w_scale)) & 15) == 0;
    if ((kbs & 15) == 0 && (num_kb & 3) == 0 && aligned16) {
        const int gpt = num_kb >> 2; // groups of four k-blocks per work item
        struct Group {
            int g, row0;
            size_t wrow, wrow2;
            bool valid;
        };
        auto locate_group = [&](uint32_t q, Group &c) { // q: index of the group in this CTA's sequence
            const int it = static_cast<int>(q / static_cast<uint32_t>(gpt));
            const int w = static_cast<int>(blockIdx.x) + it * static_cast<int>(gridDim.x);
            c.g = static_cast<int>(q % static_cast<uint32_t>(gpt));
            c.valid = w < total_work;
            if (c.valid) {
                const int tile = w / n_n_tiles;
                const int nt = w - tile * n_n_tiles;
                c.row0 = tt.tile_row0[tile];
                c.wrow = static_cast<size_t>(tt.tile_expert[tile]) * w_rows_per_expert + nt * N_PER_TILE;
                c.wrow2 = GATE_UP ? c.wrow + n_out : c.wrow + 128;
            }
        };
        auto fetch_group = [&](const Group &c, uint4 (&r)[SF_COLS]) {
            if (!c.valid)
                return;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int row = c.row0 + i * 32 + lane;
                row = row < sc.max_rows ? row : sc.max_rows - 1;
                r[i] = __ldg(reinterpret_cast<const uint4 *>(sc.x_scale + static_cast<size_t>(row) * kbs + c.g * 16));
                r[4 + i] = __ldg(reinterpret_cast<const uint4 *>(sc.w_scale + (c.wrow + i * 32 + lane) * kbs + c.g * 16));
                r[8 + i] = __ldg(reinterpret_cast<const uint4 *>(sc.w_scale + (c.wrow2 + i * 32 + lane) * kbs + c.g * 16));
            }
        };
        auto word = [](const uint4 &v, int j) { return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w)); };
        uint4 cur[SF_COLS], nxt[SF_COLS];
        Group gc, gn;
        uint32_t q = static_cast<uint32_t>(loader); // the loaders take groups round-robin
        locate_group(q, gc);
        fetch_group(gc, cur);
        bool ok = true;
        while (gc.valid && ok) {
            locate_group(q + kPf4Loaders, gn);
            fetch_group(gn, nxt); // this loader's next group: 4 * kPf4Loaders k-blocks ahead
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t seq = q * 4u + static_cast<uint32_t>(j); // num_kb = 4 * gpt: the sequence number of the k-block
                const uint32_t slot = seq % kPf4SfSlots;                 // 4 | kPf4SfSlots: a slot always belongs to one loader
                if (!mbar_wait_t(&sf_empty[slot], ((seq / kPf4SfSlots) & 1u) ^ 1u, abort_flag, w0)) {
                    ok = false;
                    break;
                }
                uint8_t *blk = sf_smem + static_cast<size_t>(slot) * kPf4SfBytesPerStage + lane * 16;
                *reinterpret_cast<uint4 *>(blk) = make_uint4(word(cur[0], j), word(cur[1], j), word(cur[2], j), word(cur[3], j));
                *reinterpret_cast<uint4 *>(blk + 512) = make_uint4(word(cur[4], j), word(cur[5], j), word(cur[6], j), word(cur[7], j));
                *reinterpret_cast<uint4 *>(blk + 1024) = make_uint4(word(cur[8], j), word(cur[9], j), word(cur[10], j), word(cur[11], j));
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&sf_full[slot]);
            }
#pragma unroll
            for (int i = 0; i < SF_COLS; i++)
                cur[i] = nxt[i];
            gc = gn;
            q += kPf4Loaders;
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
            const uint32_t slot = seq % kPf4SfSlots; // kPf4Loaders | kPf4SfSlots: a slot always belongs to one loader
            if (!mbar_wait_t(&sf_empty[slot], ((seq / kPf4SfSlots) & 1u) ^ 1u, abort_flag, w0)) {
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
                mbar_arrive(&sf_full[slot]);
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
