// Deterministic token permutation (rows sorted by expert, then token), tile tables for the grouped GEMMs,
// the row gather, and the weighted combine.  No order-dependent atomics: membership bitmaps are built with
// atomicOr (whose result does not depend on arrival order) and ranks are popcounts over them.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "xs_route.cuh"

namespace xs {

constexpr int kChunkTokens = 256; // tokens per block in the counting / ranking kernels
constexpr int kChunkWords = kChunkTokens / 32;

// bits[e][w]: bit (t & 31) of word (t >> 5) is set iff local token t of this chunk selected expert e.
__device__ __forceinline__ void build_bits(uint32_t *bits, const int32_t *__restrict__ topk_ids, int T, int E, int K, int chunk,
                                           int32_t *status)
{
    for (int i = threadIdx.x; i < E * kChunkWords; i += blockDim.x)
        bits[i] = 0u;
    __syncthreads();
    const int tl = threadIdx.x;
    const int t = chunk * kChunkTokens + tl;
    if (t < T) {
        for (int j = 0; j < K; j++) {
            const int e = topk_ids[static_cast<size_t>(t) * K + j];
            if (e < 0 || e >= E) {
                atomicOr(status, 2);
                continue;
            }
            atomicOr(&bits[e * kChunkWords + (tl >> 5)], 1u << (tl & 31));
        }
    }
    __syncthreads();
}

// grid = chunks, block = kChunkTokens, dynamic smem = E * kChunkWords * 4
__global__ void __launch_bounds__(kChunkTokens)
permute_count_kernel(const int32_t *__restrict__ topk_ids, int32_t *__restrict__ chunk_counts, int T, int E, int K,
                     int32_t *status)
{
    extern __shared__ uint32_t bits[];
    build_bits(bits, topk_ids, T, E, K, blockIdx.x, status);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
#pragma unroll
        for (int w = 0; w < kChunkWords; w++)
            c += __popc(bits[e * kChunkWords + w]);
        chunk_counts[static_cast<size_t>(blockIdx.x) * E + e] = c;
    }
}

// block-wide exclusive scan of one int per thread (blockDim.x <= 1024); returns the exclusive prefix and
// leaves the grand total in *total_smem
__device__ __forceinline__ int block_exclusive_scan(int v, int *warp_sums, int *total_smem)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o)
            inc += n;
    }
    if (lane == 31)
        warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int s = (lane < (blockDim.x + 31) / 32) ? warp_sums[lane] : 0;
        int sinc = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, sinc, o);
            if (lane >= o)
                sinc += n;
        }
        warp_sums[lane] = sinc - s; // exclusive
        if (lane == 31)
            *total_smem = sinc;
    }
    __syncthreads();
    const int res = warp_sums[warp] + inc - v;
    __syncthreads();
    return res;
}

// one block, blockDim.x >= E (rounded up to a warp multiple).  counts, offsets (exclusive scan), and the
// first row of every (chunk, expert) group.
__global__ void __launch_bounds__(1024)
permute_scan_kernel(const int32_t *__restrict__ chunk_counts, int32_t *__restrict__ counts, int32_t *__restrict__ offsets,
                    int32_t *__restrict__ chunk_base, int num_chunks, int E, int extra_rows)
{
    __shared__ int warp_sums[32];
    __shared__ int total;
    const int e = threadIdx.x;
    int c = 0;
    if (e < E)
        for (int ch = 0; ch < num_chunks; ch++)
            c += chunk_counts[static_cast<size_t>(ch) * E + e];
    const int off = block_exclusive_scan(c, warp_sums, &total);
    if (e < E) {
        counts[e] = c;
        offsets[e] = off;
        int b = off;
        for (int ch = 0; ch < num_chunks; ch++) {
            chunk_base[static_cast<size_t>(ch) * E + e] = b;
            b += chunk_counts[static_cast<size_t>(ch) * E + e];
        }
    }
    if (threadIdx.x == 0) {
        offsets[E] = total;
        if (extra_rows >= 0) // rows of the always-on expert follow the routed rows: segment E
            offsets[E + 1] = total + extra_rows;
    }
}

// one block, blockDim.x >= E.  Token tiles of n_tile rows per expert segment, in expert order.
// `offsets` may come from a caller: every entry is clamped into [0, max_rows] (and made non-decreasing) before use, and
// the clamped copy, E + 1 entries, is what the GEMM kernels read, so that no tile and no epilogue store can reach a row
// at or beyond the capacity of the row buffers.  A clamp that changed anything raises the bad-index status bit.
__global__ void __launch_bounds__(1024)
tile_table_kernel(const int32_t *__restrict__ offsets, int E, int n_tile, int max_tiles, int max_rows, int32_t *__restrict__ offsets_clamped,
                  int32_t *__restrict__ tile_expert, int32_t *__restrict__ tile_row0, int32_t *__restrict__ num_tiles, int32_t *status)
{
    __shared__ int warp_sums[32];
    __shared__ int total;
    const int e = threadIdx.x;
    int rows = 0, start = 0;
    if (e < E) {
        const int a = offsets[e], b = offsets[e + 1];
        start = a < 0 ? 0 : (a > max_rows ? max_rows : a);
        int end = b < 0 ? 0 : (b > max_rows ? max_rows : b);
        if (end < start)
            end = start;
        if (start != a || end != b)
            atomicOr(status, 2);
        rows = end - start;
        offsets_clamped[e] = start;
        if (e == E - 1)
            offsets_clamped[E] = end;
    }
    const int nt = (rows + n_tile - 1) / n_tile;
    const int first = block_exclusive_scan(nt, warp_sums, &total);
    for (int i = 0; i < nt; i++) {
        if (first + i >= max_tiles) {
            atomicOr(status, 2);
            break;
        }
        tile_expert[first + i] = e;
        tile_row0[first + i] = start + i * n_tile;
    }
    if (threadIdx.x == 0)
        *num_tiles = total < max_tiles ? total : max_tiles;
}

// grid = chunks, block = kChunkTokens.  row = first row of (chunk, expert) + number of earlier tokens of the
// chunk that chose the same expert.
__global__ void __launch_bounds__(kChunkTokens)
permute_fill_kernel(const int32_t *__restrict__ topk_ids, const int32_t *__restrict__ chunk_base, int32_t *__restrict__ perm,
                    int32_t *__restrict__ inv, int T, int E, int K, int32_t *status)
{
    extern __shared__ uint32_t bits[];
    build_bits(bits, topk_ids, T, E, K, blockIdx.x, status);
    const int tl = threadIdx.x;
    const int t = blockIdx.x * kChunkTokens + tl;
    if (t >= T)
        return;
    for (int j = 0; j < K; j++) {
        const int e = topk_ids[static_cast<size_t>(t) * K + j];
        if (e < 0 || e >= E)
            continue;
        const uint32_t *b = bits + e * kChunkWords;
        int rank = __popc(b[tl >> 5] & ((1u << (tl & 31)) - 1u));
        for (int w = 0; w < (tl >> 5); w++)
            rank += __popc(b[w]);
        const int row = chunk_base[static_cast<size_t>(blockIdx.x) * E + e] + rank;
        perm[row] = t * K + j;
        inv[static_cast<size_t>(t) * K + j] = row;
    }
}


// Decode-sized batches (T <= 256, one chunk): permutation and the GEMM tile table in ONE launch.
// One block of 256 threads: thread = token for the membership bitmaps / ranks, then a block scan over the experts.
// Produces exactly what permute_count/scan/fill + tile_table_kernel produce.
__global__ void __launch_bounds__(kChunkTokens)
permute_small_kernel(const int32_t *__restrict__ topk_ids, int32_t *__restrict__ counts, int32_t *__restrict__ offsets,
                     int32_t *__restrict__ perm, int32_t *__restrict__ inv, int T, int E, int K, int extra_rows, int n_tile,
                     int max_tiles, int32_t *__restrict__ tile_expert, int32_t *__restrict__ tile_row0, int32_t *__restrict__ num_tiles,
                     int32_t *status)
{
    extern __shared__ uint32_t bits[]; // E * kChunkWords words, then E ints of offsets
    int *s_off = reinterpret_cast<int *>(bits + E * kChunkWords);
    __shared__ int warp_sums[32];
    __shared__ int total;
    pdl_launch_dependents();
    pdl_wait();
    build_bits(bits, topk_ids, T, E, K, 0, status);
    // counts and offsets: experts in passes of blockDim.x, carrying the running total
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += kChunkTokens) {
        const int e = e0 + threadIdx.x;
        int c = 0;
        if (e < E) {
#pragma unroll
            for (int w = 0; w < kChunkWords; w++)
                c += __popc(bits[e * kChunkWords + w]);
        }
        const int off = carry + block_exclusive_scan(c, warp_sums, &total);
        if (e < E) {
            counts[e] = c;
            offsets[e] = off;
            s_off[e] = off;
        }
        carry += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        offsets[E] = carry;
        if (extra_rows >= 0)
            offsets[E + 1] = carry + extra_rows;
    }
    // ranks
    const int t = threadIdx.x;
    if (t < T) {
        for (int j = 0; j < K; j++) {
            const int e = topk_ids[static_cast<size_t>(t) * K + j];
            if (e < 0 || e >= E)
                continue;
            const uint32_t *b = bits + e * kChunkWords;
            int rank = __popc(b[t >> 5] & ((1u << (t & 31)) - 1u));
            for (int w = 0; w < (t >> 5); w++)
                rank += __popc(b[w]);
            const int row = s_off[e] + rank;
            perm[row] = t * K + j;
            inv[static_cast<size_t>(t) * K + j] = row;
        }
    }
    // tile table over E (+1 when the always-on expert's rows follow) segments
    if (tile_expert) {
        const int segs = E + (extra_rows >= 0 ? 1 : 0);
        int tcarry = 0;
        for (int e0 = 0; e0 < segs; e0 += kChunkTokens) {
            const int e = e0 + threadIdx.x;
            int rows = 0, start = 0;
            if (e < E) {
                start = s_off[e];
                rows = (e + 1 < E ? s_off[e + 1] : carry) - start;
            } else if (e == E && e < segs) {
                start = carry;
                rows = extra_rows;
            }
            const int nt = (rows + n_tile - 1) / n_tile;
            const int first = tcarry + block_exclusive_scan(nt, warp_sums, &total);
            for (int i = 0; i < nt; i++) {
                if (first + i >= max_tiles) {
                    atomicOr(status, 2);
                    break;
                }
                tile_expert[first + i] = e;
                tile_row0[first + i] = start + i * n_tile;
            }
            tcarry += total;
            __syncthreads();
        }
        if (threadIdx.x == 0)
            *num_tiles = tcarry < max_tiles ? tcarry : max_tiles;
    }
}

// One block per token: the row of x goes to its k routed rows (inv) and, when there is an always-on expert, to
// row n_routed + t.  bf16 rows are copied in 16-byte pieces; for FP8 experts the row is quantised on the way
// (1x128 groups, as quantize_rows_fp8_kernel) and codes and scales are written to every destination, so x is
// read once instead of k+1 times and no intermediate copy of the quantised x exists.
template <bool FP8>
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const __nv_bfloat16 *__restrict__ x, const int32_t *__restrict__ inv, uint8_t *__restrict__ rows_out,
                    float *__restrict__ row_scales, int T, int H, int K, int n_routed, int with_shared)
{
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (t >= T)
        return;
    __shared__ int dst[33];
    const int nd = K + (with_shared ? 1 : 0);
    if (threadIdx.x < K)
        dst[threadIdx.x] = inv[static_cast<size_t>(t) * K + threadIdx.x];
    if (threadIdx.x == 0 && with_shared)
        dst[K] = n_routed + t;
    __syncthreads();
    if constexpr (!FP8) {
        const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(t) * H);
        for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
            const uint4 v = src[i];
            for (int d = 0; d < nd; d++)
                reinterpret_cast<uint4 *>(rows_out + static_cast<size_t>(dst[d]) * H * 2)[i] = v;
        }
    } else {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int groups = H / 128;
        for (int g = warp; g < groups; g += blockDim.x / 32) {
            const uint2 raw = *reinterpret_cast<const uint2 *>(x + static_cast<size_t>(t) * H + g * 128 + lane * 4);
            float v[4];
            v[0] = __uint_as_float(raw.x << 16);
            v[1] = __uint_as_float(raw.x & 0xffff0000u);
            v[2] = __uint_as_float(raw.y << 16);
            v[3] = __uint_as_float(raw.y & 0xffff0000u);
            float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const float s = __fdiv_rn(fmaxf(m, 1e-10f), 448.0f);
            uint32_t packed = 0;
#pragma unroll
            for (int i = 0; i < 4; i++)
                packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fdiv_rn(v[i], s), __NV_SATFINITE, __NV_E4M3)) << (8 * i);
            for (int d = 0; d < nd; d++) {
                *reinterpret_cast<uint32_t *>(rows_out + static_cast<size_t>(dst[d]) * H + g * 128 + lane * 4) = packed;
                if (lane == 0)
                    row_scales[static_cast<size_t>(dst[d]) * groups + g] = s;
            }
        }
    }
}

// rows_out[row] = x[perm[row] / K] for row < n_routed;  rows_out[n_routed + t] = x[t] for the shared expert.
// 16-byte copies; row_bytes % 16 == 0.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint8_t *__restrict__ x, const int32_t *__restrict__ perm, uint8_t *__restrict__ rows_out, int n_routed,
                   int n_total, int K, int row_bytes)
{
    const int row = blockIdx.x;
    if (row >= n_total)
        return;
    const int t = row < n_routed ? perm[row] / K : row - n_routed;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(t) * row_bytes);
    uint4 *dst = reinterpret_cast<uint4 *>(rows_out + static_cast<size_t>(row) * row_bytes);
    for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x)
        dst[i] = src[i];
}

// same for rows that are a multiple of 4 bytes only (short scale rows)
__global__ void __launch_bounds__(64)
gather_rows4_kernel(const uint32_t *__restrict__ x, const int32_t *__restrict__ perm, uint32_t *__restrict__ rows_out, int n_routed,
                    int n_total, int K, int row_words)
{
    const int row = blockIdx.x;
    if (row >= n_total)
        return;
    const int t = row < n_routed ? perm[row] / K : row - n_routed;
    for (int i = threadIdx.x; i < row_words; i += blockDim.x)
        rows_out[static_cast<size_t>(row) * row_words + i] = x[static_cast<size_t>(t) * row_words + i];
}

// out[t,h] = bf16( sum_j w[t,j] * y[inv[t,j], h]  (+ shared[t,h]) ), slot order, shared last; separate
// multiply and add (no contraction) so the sum is the same sequence of IEEE operations as the CPU's.
// Eight outputs per thread: 16-byte loads, one 16-byte store.  YB16: y rows are bf16 (expert-parallel return rows of
// the quantised formats travel as bf16); the always-on expert's rows stay f32.
__device__ __forceinline__ void load8(const float *p, float (&v)[8])
{
    const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8])
{
    const uint4 r = *reinterpret_cast<const uint4 *>(p);
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
    v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xffff0000u);
    v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xffff0000u);
}

// residual (T, H) bf16 or null: the block's skip connection, added the way the engine's `add` op adds two bf16 tensors
// (xstar_cpp/src/ops/add.cpp:27-49 in the reference): the layer's result is rounded to bf16 first, then
// out = bf16(float(residual) + float(result)).
template <typename YT, typename ST>
__global__ void __launch_bounds__(128)
combine_kernel(const YT *__restrict__ y, const int32_t *__restrict__ inv, const float *__restrict__ topk_w,
               const ST *__restrict__ shared, __nv_bfloat16 *__restrict__ out, int T, int H, int K,
               const __nv_bfloat16 *__restrict__ residual = nullptr)
{
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (t >= T)
        return;
    __shared__ int s_row[32];
    __shared__ float s_w[32];
    if (threadIdx.x < K) {
        s_row[threadIdx.x] = inv[static_cast<size_t>(t) * K + threadIdx.x];
        s_w[threadIdx.x] = topk_w[static_cast<size_t>(t) * K + threadIdx.x];
    }
    __syncthreads();
    for (int h0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8; h0 < H; h0 += gridDim.y * blockDim.x * 8) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            acc[i] = 0.0f;
        for (int j = 0; j < K; j++) {
            float v[8];
            load8(y + static_cast<size_t>(s_row[j]) * H + h0, v);
            const float w = s_w[j];
#pragma unroll
            for (int i = 0; i < 8; i++)
                acc[i] = __fadd_rn(acc[i], __fmul_rn(w, v[i]));
        }
        if (shared) {
            float v[8];
            load8(shared + static_cast<size_t>(t) * H + h0, v);
#pragma unroll
            for (int i = 0; i < 8; i++)
                acc[i] = __fadd_rn(acc[i], v[i]);
        }
        __nv_bfloat162 o[4];
#pragma unroll
        for (int i = 0; i < 4; i++)
            o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        if (residual) {
            const uint4 rr = *reinterpret_cast<const uint4 *>(residual + static_cast<size_t>(t) * H + h0);
            const uint32_t rw4[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 m = __bfloat1622float2(o[i]);
                o[i] = __floats2bfloat162_rn(__fadd_rn(__uint_as_float(rw4[i] << 16), m.x),
                                             __fadd_rn(__uint_as_float(rw4[i] & 0xffff0000u), m.y));
            }
        }
        *reinterpret_cast<uint4 *>(out + static_cast<size_t>(t) * H + h0) = *reinterpret_cast<uint4 *>(o);
    }
}

// RMS norm of bf16 rows with the reference's arithmetic (xstar_cpp/src/ops/rmsnorm.cpp:52-72): the sum of squares is
// accumulated in f32 in ASCENDING column order (so the result equals the CPU op bit for bit, and the router that reads it
// makes the same expert choices), inv = 1 / sqrt(sum / H + eps) with IEEE square root and division, and
// out[j] = bf16(bf16(x[j] * inv) * w[j]).
// One block per 32 rows: 256-column chunks are staged in shared memory by all threads (coalesced), then ONE thread per row
// walks its row's chunk in order; the write pass is done by all threads again.
constexpr int kRnRows = 32, kRnChunk = 256, kRnThreads = 256, kRnStride = kRnChunk + 8;
__global__ void __launch_bounds__(kRnThreads)
rmsnorm_rows_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ w, __nv_bfloat16 *__restrict__ out, int rows,
                    int H, float eps)
{
    __shared__ __align__(16) __nv_bfloat16 tile[kRnRows][kRnStride];
    __shared__ float s_inv[kRnRows];
    const int r0 = blockIdx.x * kRnRows;
    const int nr = rows - r0 < kRnRows ? rows - r0 : kRnRows;
    float sum = 0.0f;
    for (int c0 = 0; c0 < H; c0 += kRnChunk) {
        const int cw = H - c0 < kRnChunk ? H - c0 : kRnChunk; // a multiple of 8
        __syncthreads();
        for (int p = threadIdx.x; p < nr * (cw / 8); p += kRnThreads) {
            const int r = p / (cw / 8), c = (p - r * (cw / 8)) * 8;
            *reinterpret_cast<uint4 *>(&tile[r][c]) = __ldg(reinterpret_cast<const uint4 *>(x + static_cast<size_t>(r0 + r) * H + c0 + c));
        }
        __syncthreads();
        if (threadIdx.x < nr) {
            const uint4 *p = reinterpret_cast<const uint4 *>(&tile[threadIdx.x][0]);
            for (int i = 0; i < cw / 8; i++) {
                const uint4 v = p[i];
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float a = __uint_as_float(u[j] << 16), b = __uint_as_float(u[j] & 0xffff0000u);
                    sum = __fadd_rn(sum, __fmul_rn(a, a));
                    sum = __fadd_rn(sum, __fmul_rn(b, b));
                }
            }
        }
    }
    if (threadIdx.x < nr)
        s_inv[threadIdx.x] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, static_cast<float>(H)), eps)));
    __syncthreads();
    for (int p = threadIdx.x; p < nr * (H / 8); p += kRnThreads) {
        const int r = p / (H / 8), c = (p - r * (H / 8)) * 8;
        const float inv = s_inv[r];
        const uint4 xv = __ldg(reinterpret_cast<const uint4 *>(x + static_cast<size_t>(r0 + r) * H + c));
        const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(w + c));
        const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w}, wu[4] = {wv.x, wv.y, wv.z, wv.w};
        __nv_bfloat162 o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __nv_bfloat162 n = __floats2bfloat162_rn(__fmul_rn(__uint_as_float(xu[j] << 16), inv),
                                                           __fmul_rn(__uint_as_float(xu[j] & 0xffff0000u), inv));
            const float2 nf = __bfloat1622float2(n);
            o[j] = __floats2bfloat162_rn(__fmul_rn(nf.x, __uint_as_float(wu[j] << 16)), __fmul_rn(nf.y, __uint_as_float(wu[j] & 0xffff0000u)));
        }
        *reinterpret_cast<uint4 *>(out + static_cast<size_t>(r0 + r) * H + c) = *reinterpret_cast<uint4 *>(o);
    }
}

// dst[r] = bf16(src[index[r]]) for f32 rows of `cols` columns (cols % 8 == 0): gather and round in one pass
__global__ void __launch_bounds__(256)
gather_rows_f32_to_bf16_kernel(const float *__restrict__ src, const int32_t *__restrict__ index, __nv_bfloat16 *__restrict__ dst,
                               int n_rows, int cols)
{
    const int row = blockIdx.x;
    if (row >= n_rows)
        return;
    const float *s = src + static_cast<size_t>(index[row]) * cols;
    __nv_bfloat16 *d = dst + static_cast<size_t>(row) * cols;
    for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
        float v[8];
        load8(s + c, v);
        __nv_bfloat162 o[4];
#pragma unroll
        for (int i = 0; i < 4; i++)
            o[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(d + c) = *reinterpret_cast<uint4 *>(o);
    }
}

} // namespace xs
