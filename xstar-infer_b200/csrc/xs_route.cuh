// Router: logits = x . router_w^T with each output accumulated in ascending k in f32 (so that the logits
// equal, bit for bit, a sequential CPU loop and near-ties cannot flip an expert choice), then per-token
// selection of the k largest keys with warp-shuffle reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace xs {

// Large batches: (16 * TPT) tokens x 128 experts per block, TPT x 8 outputs per thread (TPT = 4, or 2 when the batch is
// too small to fill the SMs with 64-token tiles).  Operands are widened to f32 while they are staged in shared memory,
// so the inner loop is (TPT + 8) 16-byte shared loads per 32 * TPT FMAs and no conversions; k chunks of 32 are
// double-buffered.  Same contract: every accumulator sees k = 0, 1, 2, ... in order.
constexpr int kRbExperts = 128, kRbK = 32, kRbThreads = 256, kRbStride = kRbK + 4;
template <int TPT>
constexpr int rb_smem_bytes()
{
    return 2 * (16 * TPT + kRbExperts) * kRbStride * 4;
}
template <int TPT>
__global__ void __launch_bounds__(kRbThreads, 2)
router_logits_big_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ rw, float *__restrict__ logits,
                         int T, int H, int E)
{
    constexpr int TOK = 16 * TPT;
    constexpr int PIECES = (TOK + kRbExperts) * 4; // 16-byte pieces (8 bf16) per k chunk
    constexpr int PPT = (PIECES + kRbThreads - 1) / kRbThreads;
    extern __shared__ __align__(16) float rb_smem[];
    float (*xs)[TOK][kRbStride] = reinterpret_cast<float (*)[TOK][kRbStride]>(rb_smem);
    float (*ws)[kRbExperts][kRbStride] = reinterpret_cast<float (*)[kRbExperts][kRbStride]>(rb_smem + 2 * TOK * kRbStride);
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int t0 = blockIdx.y * TOK, e0 = blockIdx.x * kRbExperts;
    uint4 stage_regs[PPT];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < PPT; i++) {
            const int p = tid + i * kRbThreads;
            const int r = p >> 2, c = (p & 3) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (p < PIECES) {
                if (r < TOK) {
                    if (t0 + r < T)
                        v = __ldg(reinterpret_cast<const uint4 *>(x + static_cast<size_t>(t0 + r) * H + k0 + c));
                } else if (e0 + r - TOK < E) {
                    v = __ldg(reinterpret_cast<const uint4 *>(rw + static_cast<size_t>(e0 + r - TOK) * H + k0 + c));
                }
            }
            stage_regs[i] = v;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < PPT; i++) {
            const int p = tid + i * kRbThreads;
            if (p >= PIECES)
                continue;
            const int r = p >> 2, c = (p & 3) * 8;
            const uint4 v = stage_regs[i];
            float *dst = r < TOK ? &xs[buf][r][c] : &ws[buf][r - TOK][c];
            *reinterpret_cast<float4 *>(dst) = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                                                            __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
            *reinterpret_cast<float4 *>(dst + 4) = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                                                                __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
        }
    };
    float acc[TPT][8];
#pragma unroll
    for (int i = 0; i < TPT; i++)
#pragma unroll
        for (int j = 0; j < 8; j++)
            acc[i][j] = 0.0f;
    fetch(0);
    stash(0);
    __syncthreads();
    const int chunks = H / kRbK;
    for (int ch = 0; ch < chunks; ch++) {
        const int buf = ch & 1;
        if (ch + 1 < chunks)
            fetch((ch + 1) * kRbK);
#pragma unroll
        for (int k = 0; k < kRbK; k += 4) {
            float4 xv[TPT], wv[8];
#pragma unroll
            for (int i = 0; i < TPT; i++)
                xv[i] = *reinterpret_cast<const float4 *>(&xs[buf][ty + 16 * i][k]);
#pragma unroll
            for (int j = 0; j < 8; j++)
                wv[j] = *reinterpret_cast<const float4 *>(&ws[buf][tx + 16 * j][k]);
#pragma unroll
            for (int i = 0; i < TPT; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float a = acc[i][j];
                    a = __fmaf_rn(xv[i].x, wv[j].x, a);
                    a = __fmaf_rn(xv[i].y, wv[j].y, a);
                    a = __fmaf_rn(xv[i].z, wv[j].z, a);
                    a = __fmaf_rn(xv[i].w, wv[j].w, a);
                    acc[i][j] = a;
                }
        }
        if (ch + 1 < chunks)
            stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TPT; i++) {
        const int t = t0 + ty + 16 * i;
        if (t >= T)
            continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int e = e0 + tx + 16 * j;
            if (e < E)
                logits[static_cast<size_t>(t) * E + e] = acc[i][j];
        }
    }
}

// The same tile with the f32 FMAs issued two at a time (fma.rn.f32x2: two independent IEEE FMAs per instruction, so
// every accumulator still sees k = 0, 1, 2, ... one rounding per step).  For that the operands sit k-major in shared
// memory -- sm[k][token columns | expert columns] -- so that one 16-byte read yields four neighbouring experts (two
// packed operands) at one k; a thread owns TPT consecutive tokens and experts {4 tx .. 4 tx + 3, 64 + 4 tx .. 64 + 4 tx + 3}.
// Per k and thread: 3 shared reads, 4 * TPT packed FMAs.  The transposing stores of the staging step are conflict-free
// because consecutive lanes stage consecutive rows.
__device__ __forceinline__ void fma2(float2 &acc, const float2 a, const float2 b)
{
    unsigned long long &c = reinterpret_cast<unsigned long long &>(acc);
    asm("fma.rn.f32x2 %0, %1, %2, %0;"
        : "+l"(c)
        : "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(b)));
}

template <int TPT>
constexpr int rp_smem_bytes()
{
    return 2 * kRbK * (16 * TPT + kRbExperts) * 4;
}
template <int TPT>
__global__ void __launch_bounds__(kRbThreads, 2)
router_logits_pair_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ rw, float *__restrict__ logits,
                          int T, int H, int E)
{
    constexpr int TOK = 16 * TPT;
    constexpr int ROWS = TOK + kRbExperts;
    constexpr int PIECES = ROWS * 4; // 16-byte pieces (8 bf16 along k) per k chunk of 32
    constexpr int PPT = (PIECES + kRbThreads - 1) / kRbThreads;
    extern __shared__ __align__(16) float rp_smem[];
    float (*sm)[kRbK][ROWS] = reinterpret_cast<float (*)[kRbK][ROWS]>(rp_smem);
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int t0 = blockIdx.y * TOK, e0 = blockIdx.x * kRbExperts;
    uint4 stage_regs[PPT];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < PPT; i++) {
            const int p = tid + i * kRbThreads;
            const int r = p % ROWS, c = (p / ROWS) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (p < PIECES) {
                if (r < TOK) {
                    if (t0 + r < T)
                        v = __ldg(reinterpret_cast<const uint4 *>(x + static_cast<size_t>(t0 + r) * H + k0 + c));
                } else if (e0 + r - TOK < E) {
                    v = __ldg(reinterpret_cast<const uint4 *>(rw + static_cast<size_t>(e0 + r - TOK) * H + k0 + c));
                }
            }
            stage_regs[i] = v;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < PPT; i++) {
            const int p = tid + i * kRbThreads;
            if (p >= PIECES)
                continue;
            const int r = p % ROWS, c = (p / ROWS) * 8;
            const uint4 v = stage_regs[i];
            sm[buf][c + 0][r] = __uint_as_float(v.x << 16);
            sm[buf][c + 1][r] = __uint_as_float(v.x & 0xffff0000u);
            sm[buf][c + 2][r] = __uint_as_float(v.y << 16);
            sm[buf][c + 3][r] = __uint_as_float(v.y & 0xffff0000u);
            sm[buf][c + 4][r] = __uint_as_float(v.z << 16);
            sm[buf][c + 5][r] = __uint_as_float(v.z & 0xffff0000u);
            sm[buf][c + 6][r] = __uint_as_float(v.w << 16);
            sm[buf][c + 7][r] = __uint_as_float(v.w & 0xffff0000u);
        }
    };
    float2 acc[TPT][4];
#pragma unroll
    for (int i = 0; i < TPT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            acc[i][j] = make_float2(0.0f, 0.0f);
    fetch(0);
    stash(0);
    __syncthreads();
    const int chunks = H / kRbK;
    for (int ch = 0; ch < chunks; ch++) {
        const int buf = ch & 1;
        if (ch + 1 < chunks)
            fetch((ch + 1) * kRbK);
#pragma unroll 8
        for (int k = 0; k < kRbK; k++) {
            float xv[TPT];
            if constexpr (TPT == 4) {
                const float4 v = *reinterpret_cast<const float4 *>(&sm[buf][k][ty * 4]);
                xv[0] = v.x, xv[1] = v.y, xv[2] = v.z, xv[3] = v.w;
            } else {
                const float2 v = *reinterpret_cast<const float2 *>(&sm[buf][k][ty * 2]);
                xv[0] = v.x, xv[1] = v.y;
            }
            const float4 wa = *reinterpret_cast<const float4 *>(&sm[buf][k][TOK + tx * 4]);
            const float4 wb = *reinterpret_cast<const float4 *>(&sm[buf][k][TOK + 64 + tx * 4]);
            const float2 w0 = make_float2(wa.x, wa.y), w1 = make_float2(wa.z, wa.w);
            const float2 w2 = make_float2(wb.x, wb.y), w3 = make_float2(wb.z, wb.w);
#pragma unroll
            for (int i = 0; i < TPT; i++) {
                const float2 xx = make_float2(xv[i], xv[i]);
                fma2(acc[i][0], xx, w0);
                fma2(acc[i][1], xx, w1);
                fma2(acc[i][2], xx, w2);
                fma2(acc[i][3], xx, w3);
            }
        }
        if (ch + 1 < chunks)
            stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TPT; i++) {
        const int t = t0 + ty * TPT + i;
        if (t >= T)
            continue;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int e = e0 + 64 * h + tx * 4;
            float *dst = logits + static_cast<size_t>(t) * E + e;
            const float2 a = acc[i][2 * h], b = acc[i][2 * h + 1];
            if (e + 3 < E && (E & 3) == 0) {
                *reinterpret_cast<float4 *>(dst) = make_float4(a.x, a.y, b.x, b.y);
            } else {
                const float v[4] = {a.x, a.y, b.x, b.y};
                for (int j = 0; j < 4; j++)
                    if (e + j < E)
                        dst[j] = v[j];
            }
        }
    }
}

// Decode-sized batches.  Block = 8 experts x 32 tokens, one output per thread (warp = one expert, lanes = tokens),
// so a batch of 128 tokens x 256 experts spreads over 128 SMs.  Operands arrive through an 8-stage cp.async
// pipeline of 128-wide k chunks; inside a chunk each thread walks k upwards, 8 elements per 16-byte shared-memory
// read (the router row is a warp-wide broadcast, the token rows are padded to stay bank-conflict free).
// One accumulator per thread, touched once per k in ascending order: the contract's summation order -- which makes the
// H dependent FMAs the floor of this kernel; the pipeline is eight chunks deep because at decode sizes the kernel is
// otherwise bound by the latency of fetching its operands.
constexpr int kRdExperts = 8, kRdTokens = 32, kRdK = 128, kRdStages = 8, kRdThreads = 256;
constexpr int kRdXStride = kRdK + 8; // bf16 elements; 272-byte rows: 16-byte aligned and conflict-free for 16-byte reads
constexpr int kRdSmemBytes = kRdStages * (kRdExperts * kRdK + kRdTokens * kRdXStride) * 2;

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool valid)
{
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    const int sz = valid ? 16 : 0; // 0 source bytes => the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}

__global__ void __launch_bounds__(kRdThreads)
router_logits_decode_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ rw, float *__restrict__ logits,
                            int T, int H, int E)
{
    extern __shared__ __align__(16) uint8_t rd_smem[]; // kRdSmemBytes
    __nv_bfloat16 (*ws)[kRdExperts][kRdK] = reinterpret_cast<__nv_bfloat16 (*)[kRdExperts][kRdK]>(rd_smem);
    __nv_bfloat16 (*xsm)[kRdTokens][kRdXStride] =
        reinterpret_cast<__nv_bfloat16 (*)[kRdTokens][kRdXStride]>(rd_smem + kRdStages * kRdExperts * kRdK * 2);
    const int tid = threadIdx.x;
    const int el = tid >> 5, tl = tid & 31;
    const int e0 = blockIdx.x * kRdExperts, t0 = blockIdx.y * kRdTokens;
    const int chunks = H / kRdK;

    auto issue = [&](int chunk, int stage) {
        const int k0 = chunk * kRdK;
        // 16-byte pieces: 8 experts x 16 + 32 tokens x 16 = 640
        for (int p = tid; p < (kRdExperts + kRdTokens) * (kRdK / 8); p += kRdThreads) {
            const int r = p / (kRdK / 8), c = (p - r * (kRdK / 8)) * 8;
            if (r < kRdExperts) {
                const int e = e0 + r;
                const bool ok = e < E;
                cp_async16(&ws[stage][r][c], rw + static_cast<size_t>(ok ? e : 0) * H + k0 + c, ok);
            } else {
                const int t = t0 + r - kRdExperts;
                const bool ok = t < T;
                cp_async16(&xsm[stage][r - kRdExperts][c], x + static_cast<size_t>(ok ? t : 0) * H + k0 + c, ok);
            }
        }
    };

#pragma unroll
    for (int s = 0; s < kRdStages - 1; s++) {
        if (s < chunks)
            issue(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc = 0.0f;
    for (int ch = 0; ch < chunks; ch++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kRdStages - 2) : "memory");
        __syncthreads(); // chunk ch has landed for every thread; everyone has finished chunk ch-1
        const int nxt = ch + kRdStages - 1;
        if (nxt < chunks)
            issue(nxt, nxt % kRdStages);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int st = ch % kRdStages;
        const uint4 *wp = reinterpret_cast<const uint4 *>(&ws[st][el][0]);
        const uint4 *xp = reinterpret_cast<const uint4 *>(&xsm[st][tl][0]);
#pragma unroll 4
        for (int i = 0; i < kRdK / 8; i++) {
            const uint4 w = wp[i], v = xp[i];
            acc = __fmaf_rn(__uint_as_float(v.x << 16), __uint_as_float(w.x << 16), acc);
            acc = __fmaf_rn(__uint_as_float(v.x & 0xffff0000u), __uint_as_float(w.x & 0xffff0000u), acc);
            acc = __fmaf_rn(__uint_as_float(v.y << 16), __uint_as_float(w.y << 16), acc);
            acc = __fmaf_rn(__uint_as_float(v.y & 0xffff0000u), __uint_as_float(w.y & 0xffff0000u), acc);
            acc = __fmaf_rn(__uint_as_float(v.z << 16), __uint_as_float(w.z << 16), acc);
            acc = __fmaf_rn(__uint_as_float(v.z & 0xffff0000u), __uint_as_float(w.z & 0xffff0000u), acc);
            acc = __fmaf_rn(__uint_as_float(v.w << 16), __uint_as_float(w.w << 16), acc);
            acc = __fmaf_rn(__uint_as_float(v.w & 0xffff0000u), __uint_as_float(w.w & 0xffff0000u), acc);
        }
    }
    const int e = e0 + el, t = t0 + tl;
    if (e < E && t < T)
        logits[static_cast<size_t>(t) * E + e] = acc;
}

// One warp per token.  Lane l holds experts l, l+32, l+64, ...  (NPL per lane).
// Selection: K rounds of "largest key, ties to the lower expert id" by butterfly shuffles.
// Output slots are in ascending expert id.  Weights: softmax over the selected unbiased logits,
// max-shifted, summed in slot order.
template <int NPL>
__device__ __forceinline__ void topk_warp(const float *__restrict__ logits, const float *__restrict__ bias,
                                          int32_t *__restrict__ topk_ids, float *__restrict__ topk_w, int warp, int lane, int E, int K)
{
    const float *l = logits + static_cast<size_t>(warp) * E;
    float key[NPL], lg[NPL];
    uint32_t selected = 0; // bit i: expert lane + 32*i chosen
#pragma unroll
    for (int i = 0; i < NPL; i++) {
        const int e = lane + 32 * i;
        if (e < E) {
            lg[i] = l[e];
            key[i] = bias ? __fadd_rn(lg[i], bias[e]) : lg[i];
        } else {
            lg[i] = 0.0f;
            key[i] = 0.0f;
            selected |= 1u << i; // never eligible
        }
    }
    const uint32_t never = selected;
    for (int r = 0; r < K; r++) {
        // local best among the not yet selected
        float bk = 0.0f;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < NPL; i++) {
            const int e = lane + 32 * i;
            const bool free_ = !((selected >> i) & 1u);
            if (free_ && (be == 0x7fffffff || key[i] > bk)) { // ascending e within the lane: strict > keeps the lower id
                bk = key[i];
                be = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ok = __shfl_xor_sync(0xffffffffu, bk, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            const bool take = (oe != 0x7fffffff) && (be == 0x7fffffff || ok > bk || (ok == bk && oe < be));
            if (take) {
                bk = ok;
                be = oe;
            }
        }
        if (be != 0x7fffffff && (be & 31) == lane)
            selected |= 1u << (be >> 5);
    }
    const uint32_t chosen = selected & ~never;
    // ascending expert id = ascending i, then ascending lane
    int base = 0;
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NPL; i++) {
        const bool c = (chosen >> i) & 1u;
        const uint32_t mask = __ballot_sync(0xffffffffu, c);
        if (c) {
            const int slot = base + __popc(mask & ((1u << lane) - 1u));
            topk_ids[static_cast<size_t>(warp) * K + slot] = lane + 32 * i;
            topk_w[static_cast<size_t>(warp) * K + slot] = lg[i]; // raw logit for now
            m = fmaxf(m, lg[i]);
        }
        base += __popc(mask);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncwarp();
    // slot-ordered softmax; K <= 32: lane j owns slot j
    float ex = 0.0f;
    if (lane < K)
        ex = expf(topk_w[static_cast<size_t>(warp) * K + lane] - m);
    float sum = 0.0f;
    for (int j = 0; j < K; j++)
        sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, ex, j));
    if (lane < K)
        topk_w[static_cast<size_t>(warp) * K + lane] = __fdiv_rn(ex, sum);
}

template <int NPL>
__global__ void __launch_bounds__(128)
topk_kernel(const float *__restrict__ logits, const float *__restrict__ bias, int32_t *__restrict__ topk_ids,
            float *__restrict__ topk_w, int T, int E, int K)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= T)
        return;
    topk_warp<NPL>(logits, bias, topk_ids, topk_w, warp, lane, E, K);
}

} // namespace xs
