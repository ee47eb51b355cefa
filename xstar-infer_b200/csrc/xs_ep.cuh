// Expert parallelism over peer memory: the dispatch and return trips of the MoE layer as kernels that store rows
// straight into the buffers of the rank that needs them (NVLink peer stores), instead of pack -> all-to-all -> unpack.
//
// Every rank knows the (R, E) matrix of per-rank, per-expert row counts (one small all-gather).  From it every address
// follows on the device, with no host synchronisation:
//   * rank d keeps the rows it receives GROUPED by local expert, inside an expert ordered by source rank, then by the
//     source's own row order:   row(d; e, s, j) = offsets_local_d[e mod El] + sum_{s' < s} counts[s'][e] + j
//   * the result of that row goes back to the source's row  offsets_s[e] + j  (its permuted row index)
// The dispatch, return and plan kernels never wait for another GPU: completion of the stores is established between kernels
// by a barrier on the stream -- a collective of the caller's, or ep_signal_kernel below, the one kernel of this file that
// does wait for peers, with a bounded wait.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace xs {

// One block, blockDim.x >= E (E <= 1024).  From all_counts (R, E):
//   dest_base[e]       first row, in the owner's grouped buffer, of MY rows of expert e
//   offsets_local[El+1] segment offsets of the experts I own (my grouped buffer)
//   src_offsets[s][e]  exclusive prefix over experts of counts[s][.]  (rank s's own permuted row offsets)
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int32_t *__restrict__ all_counts, int R, int E, int me, int32_t *__restrict__ dest_base,
               int32_t *__restrict__ offsets_local, int32_t *__restrict__ src_offsets)
{
    __shared__ int col_sum[1024];  // rows of expert e over all sources
    const int El = E / R;
    const int e = threadIdx.x;
    int tot = 0, before_me = 0;
    if (e < E)
        for (int s = 0; s < R; s++) {
            const int c = all_counts[s * E + e];
            if (s < me)
                before_me += c;
            tot += c;
        }
    col_sum[threadIdx.x] = e < E ? tot : 0;
    __syncthreads();
    if (e < E) {
        // exclusive prefix of col_sum inside the owner's block of El experts (El <= 1024: a short serial loop)
        const int first = (e / El) * El;
        int off = 0;
        for (int k = first; k < e; k++)
            off += col_sum[k];
        dest_base[e] = off + before_me;
        if (e / El == me) {
            offsets_local[e - first] = off;
            if (e - first == El - 1)
                offsets_local[El] = off + tot;
        }
    }
    // per-source exclusive prefix over experts: thread s handles one source
    if (threadIdx.x < R) {
        int run = 0;
        for (int k = 0; k < E; k++) {
            src_offsets[threadIdx.x * E + k] = run;
            run += all_counts[threadIdx.x * E + k];
        }
    }
}

// Barrier between the ranks of one box over peer memory, optionally carrying every rank's per-expert counts (the layer's
// all-gather): one warp per GPU.  Each rank keeps a launch counter (`epoch`, in its own memory: it advances by itself, so the
// kernel can be replayed inside a CUDA graph) and a row of R flags that its peers write.
//   1. (counts != null) lane-strided copy of my E counts into row `me` of every rank's all_counts (my own included);
//   2. __threadfence_system: these stores, and all stores of the kernels before this one on the stream (the rows a dispatch
//      or return kernel put into the peers' buffers), are ordered before
//   3. flag[me] = epoch, stored into every peer's flag row;
//   4. lanes 0..R-1 poll my own flag row until flags[r] >= epoch for every r, then fence again: what the peers wrote before
//      their flag is visible to the kernels that follow on this stream.
// ">=": a peer that is already one barrier ahead has passed this one.  The wait is bounded (about two seconds of polling with
// back-off); when it runs out the kernel sets the wait-timeout bit of the status word and returns, and the
// host raises -- a rank must only call this after the ranks agreed on the host that all of them will (the host check-in).
// Never run two ranks' signal kernels on ONE GPU (virtual ranks): they would wait for each other across launches.
__global__ void __launch_bounds__(32)
ep_signal_kernel(const int32_t *__restrict__ counts, int E, int32_t *const *__restrict__ peer_all_counts, int32_t *const *__restrict__ peer_flags,
                 volatile int32_t *my_flags, int32_t *epoch_counter, int R, int me, int32_t *status)
{
    const int lane = threadIdx.x;
    int epoch = 0;
    if (lane == 0) {
        epoch = *epoch_counter + 1;
        *epoch_counter = epoch;
    }
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
    if (counts)
        for (int r = 0; r < R; r++)
            for (int e = lane; e < E; e += 32)
                peer_all_counts[r][me * E + e] = counts[e];
    __threadfence_system();
    __syncwarp();
    __threadfence_system(); // cumulative: the other lanes' stores, ordered before the barrier above, come before my flag store
    if (lane < R)
        *reinterpret_cast<volatile int32_t *>(peer_flags[lane] + me) = epoch;
    bool ok = true;
    if (lane < R) {
        unsigned spins = 0;
        while (my_flags[lane] - epoch < 0) { // wrap-safe comparison
            if (++spins > (1u << 24)) {
                ok = false;
                break;
            }
            if (spins > 64)
                __nanosleep(spins > 4096 ? 128 : 32);
        }
    }
    __threadfence_system();
    if (!ok)
        atomicOr(status, 1);
}

// FMT: 0 = bf16 rows, 1 = e4m3 codes + f32 scale per 128, 2 = e4m3 codes + e8m0 scale per 32 (MX-FP8).
// One block per token: the row is (quantised once and) stored into the grouped buffer of the owner of each of its k
// experts.  peer_rows[d] / peer_scales[d] are rank d's buffers as seen from this GPU.
template <int FMT>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16 *__restrict__ x, const int32_t *__restrict__ topk_ids, const int32_t *__restrict__ inv,
                   const int32_t *__restrict__ my_offsets, const int32_t *__restrict__ dest_base, uint8_t *const *__restrict__ peer_rows,
                   uint8_t *const *__restrict__ peer_scales, int T, int H, int K, int E, int R, int capacity, int32_t *status)
{
    const int t = blockIdx.x;
    if (t >= T)
        return;
    __shared__ uint8_t *s_rows[32];
    __shared__ uint8_t *s_scales[32];
    const int El = E / R;
    const int row_bytes = FMT == 0 ? H * 2 : H;
    const int scale_bytes = FMT == 1 ? (H / 128) * 4 : (FMT == 2 ? H / 32 : 0);
    if (threadIdx.x < K) {
        const int e = topk_ids[static_cast<size_t>(t) * K + threadIdx.x];
        const int i = inv[static_cast<size_t>(t) * K + threadIdx.x]; // my permuted row
        const bool e_ok = e >= 0 && e < E;
        const int row = e_ok ? dest_base[e] + (i - my_offsets[e]) : -1;
        const int d = e_ok ? e / El : 0;
        if (row < 0 || row >= capacity) {
            atomicOr(status, 2);
            s_rows[threadIdx.x] = nullptr;
            s_scales[threadIdx.x] = nullptr;
        } else {
            s_rows[threadIdx.x] = peer_rows[d] + static_cast<size_t>(row) * row_bytes;
            s_scales[threadIdx.x] = scale_bytes ? peer_scales[d] + static_cast<size_t>(row) * scale_bytes : nullptr;
        }
    }
    __syncthreads();
    if constexpr (FMT == 0) {
        const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(t) * H);
        for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
            const uint4 v = src[c];
            for (int j = 0; j < K; j++)
                if (s_rows[j])
                    reinterpret_cast<uint4 *>(s_rows[j])[c] = v;
        }
    } else {
        // 16 elements per lane: a lane's codes are one 16-byte store and a warp writes 512 contiguous bytes of a destination
        // row per instruction (remote rows travel over NVLink, where 4-byte-per-lane stores -- 128 bytes per instruction -- cost
        // about half of the link's rate).  Same arithmetic as the single-GPU scatter, element for element.
        constexpr int G = FMT == 1 ? 128 : 32;      // quantisation group
        constexpr int LPG = G / 16;                 // lanes per group
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int c0 = warp * 512; c0 < H; c0 += (blockDim.x >> 5) * 512) {
            const int col = c0 + lane * 16;
            const bool in = col < H; // H is a multiple of the group size, so a group is inside or outside as a whole
            uint4 raw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
            if (in) {
                const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(t) * H + col);
                raw[0] = src[0];
                raw[1] = src[1];
            }
            const uint32_t w32[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
            float v[16];
            float m = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                v[2 * i] = __uint_as_float(w32[i] << 16);
                v[2 * i + 1] = __uint_as_float(w32[i] & 0xffff0000u);
                m = fmaxf(m, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
            }
#pragma unroll
            for (int o = LPG / 2; o > 0; o >>= 1)
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            uint32_t pk[4] = {0, 0, 0, 0};
            float s_f32 = 0.0f;
            uint32_t s_e8 = 0;
            if constexpr (FMT == 1) {
                s_f32 = __fdiv_rn(fmaxf(m, 1e-10f), 448.0f);
#pragma unroll
                for (int i = 0; i < 16; i++)
                    pk[i >> 2] |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fdiv_rn(v[i], s_f32), __NV_SATFINITE, __NV_E4M3)) << (8 * (i & 3));
            } else {
                const uint32_t b = __float_as_uint(__fdiv_rn(fmaxf(m, 1e-30f), 448.0f));
                s_e8 = (b >> 23) & 0xffu;
                if (b & 0x7fffffu)
                    s_e8 += 1;
                s_e8 = s_e8 > 254u ? 254u : s_e8;
                const float inv_s = __uint_as_float((254u - s_e8) << 23);
#pragma unroll
                for (int i = 0; i < 16; i++)
                    pk[i >> 2] |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fmul_rn(v[i], inv_s), __NV_SATFINITE, __NV_E4M3)) << (8 * (i & 3));
            }
            if (!in)
                continue;
            for (int j = 0; j < K; j++) {
                if (!s_rows[j])
                    continue;
                *reinterpret_cast<uint4 *>(s_rows[j] + col) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                if ((lane % LPG) == 0) {
                    if constexpr (FMT == 1)
                        reinterpret_cast<float *>(s_scales[j])[col / 128] = s_f32;
                    else
                        s_scales[j][col >> 5] = static_cast<uint8_t>(s_e8);
                }
            }
        }
    }
}

// Results back to their sources: grouped row g of local expert el came from source s as its j-th row of that expert and
// returns to row src_offsets[s][e] + j of rank s's return buffer (f32, or rounded to bf16 on the way: WIRE_BF16).
template <bool WIRE_BF16>
__global__ void __launch_bounds__(256)
ep_return_kernel(const float *__restrict__ y, const int32_t *__restrict__ all_counts, const int32_t *__restrict__ offsets_local,
                 const int32_t *__restrict__ src_offsets, uint8_t *const *__restrict__ peer_back, int H, int E, int R, int me,
                 int y_capacity, int back_capacity, int32_t *status)
{
    const int El = E / R;
    int total = offsets_local[El];
    if (total > y_capacity) { // never read past the rows y holds; the shortfall is reported
        total = y_capacity;
        if (blockIdx.x == 0 && threadIdx.x == 0)
            atomicOr(status, 2);
    }
    __shared__ int s_dst_rank, s_dst_row;
    for (int g = blockIdx.x; g < total; g += gridDim.x) {
        if (threadIdx.x == 0) {
            int lo = 0, hi = El; // expert with offsets_local[lo] <= g < offsets_local[lo+1]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (offsets_local[mid] <= g)
                    lo = mid;
                else
                    hi = mid;
            }
            const int e = me * El + lo;
            int j = g - offsets_local[lo];
            int s = 0;
            while (s < R - 1 && j >= all_counts[s * E + e]) {
                j -= all_counts[s * E + e];
                s++;
            }
            const int row = src_offsets[s * E + e] + j;
            if (row < 0 || row >= back_capacity) {
                atomicOr(status, 2);
                s_dst_rank = -1;
            } else {
                s_dst_rank = s;
                s_dst_row = row;
            }
        }
        __syncthreads();
        if (s_dst_rank >= 0) {
            const float *src = y + static_cast<size_t>(g) * H;
            if constexpr (WIRE_BF16) {
                __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(peer_back[s_dst_rank]) + static_cast<size_t>(s_dst_row) * H;
                for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
                    const float4 a = *reinterpret_cast<const float4 *>(src + c), b = *reinterpret_cast<const float4 *>(src + c + 4);
                    __nv_bfloat162 o[4] = {__floats2bfloat162_rn(a.x, a.y), __floats2bfloat162_rn(a.z, a.w),
                                           __floats2bfloat162_rn(b.x, b.y), __floats2bfloat162_rn(b.z, b.w)};
                    *reinterpret_cast<uint4 *>(dst + c) = *reinterpret_cast<uint4 *>(o);
                }
            } else {
                float *dst = reinterpret_cast<float *>(peer_back[s_dst_rank]) + static_cast<size_t>(s_dst_row) * H;
                for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4)
                    *reinterpret_cast<float4 *>(dst + c) = *reinterpret_cast<const float4 *>(src + c);
            }
        }
        __syncthreads();
    }
}

} // namespace xs
