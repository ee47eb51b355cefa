// Router for large batches: tensor-core FILTER, exact REFINE.
//
// The contract of the router is order-exact: every logit is the f32 result of accumulating x[k] * w[k] in ascending k,
// because the expert choice of a token hangs on comparisons between logits and a reordered sum can flip a near-tie.
// Computing all T x E logits that way on the CUDA cores is the slowest stage of a prefill-sized layer (chains of H dependent
// FMAs).  But only the logits near a token's k / k+1 boundary decide anything, and only the k selected ones are used
// afterwards (softmax weights).  So:
//   1. router_logits_tc_kernel: approximate logits for everything with tcgen05 MMAs (bf16 operands, f32 accumulation in
//      TMEM) -- microseconds;
//   2. router_candidates_kernel, one warp per token: from the approximate keys and an error bound `delta` find the
//      experts that are selected for certain, those that are out for certain, and the ambiguous rest;
//      router_exact_rows_kernel recomputes EXACTLY (ascending k, one lane per expert) the logits of the
//      approximately-selected and of the ambiguous experts, and overwrites them in the logits row.  Everything the selection can touch is then exact: an expert left approximate has
//      key < a_k - 2 delta, hence a true key below the true k-th key, and can neither be chosen nor tie;
//   3. the ordinary selection kernel (topk_kernel) runs on that row and gives the exact ids and weights.
//
// Error bound.  Products of two bf16 numbers are exact in f32; what differs from the sequential sum is the accumulation.
// Assumed of the tensor core: one K = 16 MMA step (sixteen exact products added to the accumulator) loses at most 2^-22 of
// the sum of the magnitudes involved, so over H / 16 steps
//     |approx - exact| <= (H / 16) * 2^-22 * S + gamma_H * S,      S = sum_k |x_k w_k| <= ||x||_2 ||w||_2,
// where the second term is the sequential sum's own rounding (gamma_H = H 2^-24 / (1 - H 2^-24)).
// delta = router_delta_coeff(H) * ||x_t||_2 * max_e ||w_e||_2, the coefficient being 1.6 times the sum of the two terms and
// both norms rounded up (the Cauchy-Schwarz step alone leaves a factor of about 1.6 at the benchmark's distributions; errors
// observed are two orders of magnitude below delta).  The assumption is checked where it can be: every recomputed logit is
// compared with its approximation, and a token with a deviation above delta, with a non-finite value, or with more than 32
// candidates, is recomputed exactly in full.
#pragma once
#include "xs_grouped_gemm.cuh"
#include "xs_route.cuh"

namespace xs {

constexpr int kRtThreads = 192;  // warp 0 TMA producer | 1 MMA issuer, TMEM owner | 2..5 epilogue
constexpr int kRtTokens = 128;   // MMA M
constexpr int kRtMaxN = 128;     // MMA N: experts per tile, a multiple of 16 (128: two expert tiles at 256 experts keep 128 SMs busy at 8192 tokens)

__host__ __device__ constexpr int rt_stage_bytes(int n)
{
    return (kRtTokens + n) * kBlockK * 2;
}

// logits[t, e0 + c] ~= x[t, :] . router_w[e0 + c, :] for one tile of 128 tokens x n experts (n a multiple of 16, <= kRtMaxN).
// grid = (token tiles, expert tiles, k splits).  Rows past T / E are zero-filled by the TMA unit and not stored.  With
// gridDim.z > 1 every CTA takes 1 / gridDim.z of the hidden dimension and ADDS its partial sums (red.global.add.f32 into
// logits the launcher zeroed): a small batch has few tiles, and one CTA walking all of H alone takes as long as a whole
// wave of them.  The order of those additions is not fixed, and need not be: these logits are the approximate ones, and
// the few extra roundings are inside the error bound (router_delta_coeff).
__global__ void __launch_bounds__(kRtThreads, 1)
router_logits_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, float *__restrict__ logits,
                        int T, int H, int E, int n, int32_t *__restrict__ status, int stages)
{
    constexpr int X_BYTES = kRtTokens * kBlockK * 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int stage_bytes = rt_stage_bytes(n);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(stages) * stage_bytes);
    uint64_t *full = bars;
    uint64_t *empty = bars + stages;
    uint64_t *done = bars + 2 * stages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(done + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(done, 1);
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_x);
        prefetch_tmap(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kRtMaxN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int t0 = blockIdx.x * kRtTokens, e0 = blockIdx.y * kRtMaxN;
    const int num_kb = H / kBlockK / static_cast<int>(gridDim.z); // the launcher picks a split that divides H / kBlockK
    const int kb0 = static_cast<int>(blockIdx.z) * num_kb;
    const bool add = gridDim.z > 1;

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol = policy_evict_last(); // both operands are re-read by other CTAs
            bool ok = true;
            for (int kb = 0; kb < num_kb; kb++) {
                const int stage = kb % stages;
                if (!mbar_wait(&empty[stage], ((kb / stages) & 1) ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                uint8_t *st = smem + static_cast<size_t>(stage) * stage_bytes;
                mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(stage_bytes));
                tma_load_2d(st, &tmap_x, &full[stage], (kb0 + kb) * kBlockK, t0, pol);
                tma_load_2d(st + X_BYTES, &tmap_w, &full[stage], (kb0 + kb) * kBlockK, e0, pol);
            }
            if (!ok) {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimeout);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(1, 1, kRtTokens, static_cast<uint32_t>(n));
            bool ok = true;
            for (int kb = 0; kb < num_kb; kb++) {
                const int stage = kb % stages;
                if (!mbar_wait(&full[stage], (kb / stages) & 1, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + static_cast<size_t>(stage) * stage_bytes);
                const uint64_t dx = make_desc_sw128(sa), dw = make_desc_sw128(sa + X_BYTES);
#pragma unroll
                for (int kk = 0; kk < kBlockK / kUmmaK; kk++)
                    mma_bf16(tmem_base, dx + 2 * kk, dw + 2 * kk, idesc, (kb | kk) ? 1u : 0u);
                tc_commit(&empty[stage]);
            }
            if (ok)
                tc_commit(done);
            else {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimeout);
            }
        }
    } else {
        const int q = warp & 3;
        const int t = t0 + q * 32 + lane;
        if (mbar_wait(done, 0, abort_flag)) {
            tc_fence_after();
            const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
            for (int c0 = 0; c0 < n; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(ta + c0, v);
                tmem_ld_wait_16(v);
                if (t < T) {
                    float *row = logits + static_cast<size_t>(t) * E + e0 + c0;
                    if (add) {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (e0 + c0 + j < E)
                                atomicAdd(row + j, __uint_as_float(v[j])); // result unused: compiles to a reduction
                    } else if (e0 + c0 + 16 <= E && (E & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            *reinterpret_cast<uint4 *>(row + 4 * j) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (e0 + c0 + j < E)
                                row[j] = __uint_as_float(v[j]);
                    }
                }
            }
            tc_fence_before();
        } else if (lane == 0) {
            *abort_flag = 1;
            atomicOr(status, kStatusWaitTimeout);
        }
    }

    __syncwarp();
    if (*abort_flag)
        for (int i = 0; i < 64; i++)
            __nanosleep(4096);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kRtMaxN);
    }
}

// max over experts of ||router_w[e, :]||_2, rounded up a little: one warp per expert, atomic max on the float's bits
// (non-negative floats order like integers; a NaN row yields a NaN bit pattern above every number, which then sends
// every token to the full exact path).  *out must be zero on entry.
__global__ void __launch_bounds__(256)
router_wnorm_kernel(const __nv_bfloat16 *__restrict__ rw, int E, int H, float *__restrict__ out)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * (blockDim.x >> 5) + warp;
    if (e >= E)
        return;
    const __nv_bfloat16 *r = rw + static_cast<size_t>(e) * H;
    float s = 0.0f;
    for (int k = lane * 8; k < H; k += 256) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(r + k));
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float a = __uint_as_float(w4[j] << 16), b = __uint_as_float(w4[j] & 0xffff0000u);
            s = fmaf(a, a, fmaf(b, b, s));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0)
        atomicMax(reinterpret_cast<int *>(out), __float_as_int(sqrtf(s) * 1.001f));
}

// delta = coeff * ||x|| * max ||w||: (H / 16) * 2^-22 for the tensor core's accumulation (+ 8 * 2^-22, far more than the
// up to kRtMaxSplits - 1 extra roundings of a split hidden dimension lose) plus H * 2^-24 * 1.01 (>= gamma_H for H < 2^17)
// for the sequential sum's own rounding, times 1.6.
constexpr int kRtMaxSplits = 4;
__host__ __device__ inline float router_delta_coeff(int H)
{
    return 1.6f * (static_cast<float>(H / 16 + 8) * 2.384185791015625e-07f + static_cast<float>(H) * 5.9604644775390625e-08f * 1.01f);
}

constexpr int kRcWarps = 4;      // tokens per block of the candidates kernel
constexpr int kRcFull = 33;      // candidate count that means "recompute every expert of this token"

// One warp per token.  From the approximate logits row: the experts whose exact logit the selection needs -- the K
// approximately-selected ones (their logits feed the softmax) and, unless the K-th and (K+1)-th keys are more than
// 2 delta apart, every expert whose key is within 2 delta of the K-th.  Writes up to 32 expert ids, their count (kRcFull if
// there are more, or if anything is not finite) and delta.  Lane l holds experts l, l + 32, ... (NPL per lane).
template <int NPL>
__global__ void __launch_bounds__(kRcWarps * 32)
router_candidates_kernel(const __nv_bfloat16 *__restrict__ x, const float *__restrict__ bias, const float *__restrict__ logits,
                         const float *__restrict__ wnorm_max, int32_t *__restrict__ cand, int32_t *__restrict__ cand_meta, int T, int H,
                         int E, int K, float coeff)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * kRcWarps + warp;
    if (t >= T)
        return;
    // ||x_t||^2 (any summation order: it only feeds a bound, and is rounded up)
    float ss = 0.0f;
    {
        const uint4 *xg = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(t) * H);
        for (int i = lane; i < H / 8; i += 32) {
            const uint4 v = __ldg(xg + i);
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float a = __uint_as_float(w4[j] << 16), b = __uint_as_float(w4[j] & 0xffff0000u);
                ss = fmaf(a, a, fmaf(b, b, ss));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    const float delta = coeff * (sqrtf(ss) * 1.001f) * __ldg(wnorm_max);
    const float *row = logits + static_cast<size_t>(t) * E;
    float key[NPL];
    uint32_t dead = 0; // bit i: slot i holds no expert
    bool finite = delta == delta && delta < 3.0e38f;
#pragma unroll
    for (int i = 0; i < NPL; i++) {
        const int e = lane + 32 * i;
        if (e < E) {
            const float a = row[e];
            key[i] = bias ? __fadd_rn(a, bias[e]) : a;
            finite = finite && fabsf(key[i]) < 3.0e38f; // false for NaN and +-Inf
        } else {
            key[i] = -INFINITY;
            dead |= 1u << i;
        }
    }
    int n = kRcFull;
    if (__all_sync(0xffffffffu, finite)) {
        // the K largest approximate keys (ties to the lower id), then the (K+1)-th
        uint32_t selected = dead;
        float a_k = INFINITY, a_k1 = -INFINITY;
        for (int r = 0; r <= K; r++) {
            float bk = -INFINITY;
            int be = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < NPL; i++) {
                const bool free_ = !((selected >> i) & 1u);
                if (free_ && (be == 0x7fffffff || key[i] > bk)) {
                    bk = key[i];
                    be = lane + 32 * i;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ok_ = __shfl_xor_sync(0xffffffffu, bk, o);
                const int oe = __shfl_xor_sync(0xffffffffu, be, o);
                if (oe != 0x7fffffff && (be == 0x7fffffff || ok_ > bk || (ok_ == bk && oe < be))) {
                    bk = ok_;
                    be = oe;
                }
            }
            if (be == 0x7fffffff)
                break; // fewer than K + 1 experts: no boundary beyond the last one
            if (r < K) {
                a_k = bk;
                if ((be & 31) == lane)
                    selected |= 1u << (be >> 5);
            } else {
                a_k1 = bk;
            }
        }
        uint32_t want = selected & ~dead; // the selected experts' logits feed the softmax: always exact
        // (the small second term covers the rounding of logit + bias on both sides)
        if (!(a_k - a_k1 > 2.0f * delta + 4.8e-7f * fabsf(a_k))) {
            // not separated: everything that is not out for certain is a candidate
            const float lo = a_k - 2.0f * delta - 4.8e-7f * fabsf(a_k);
#pragma unroll
            for (int i = 0; i < NPL; i++)
                if (!((dead >> i) & 1u) && key[i] >= lo)
                    want |= 1u << i;
        }
        n = 0;
#pragma unroll
        for (int i = 0; i < NPL; i++)
            n += __popc(__ballot_sync(0xffffffffu, (want >> i) & 1u));
        if (n > 32)
            n = kRcFull;
        else {
            int base = 0;
#pragma unroll
            for (int i = 0; i < NPL; i++) {
                const bool c = (want >> i) & 1u;
                const uint32_t mask = __ballot_sync(0xffffffffu, c);
                if (c)
                    cand[static_cast<size_t>(t) * 32 + base + __popc(mask & ((1u << lane) - 1u))] = lane + 32 * i;
                base += __popc(mask);
            }
        }
    }
    if (lane == 0) {
        cand_meta[2 * t] = n;
        cand_meta[2 * t + 1] = __float_as_int(delta);
    }
}

// Exact logits of a token's candidate experts: one WARP per block and token, lane = candidate, kReRows candidates per pass
// (a token has its K selected experts and seldom more than one or two ambiguous ones).  The chain of H dependent FMAs per
// output sets the time (about 10 us at H = 4096), so the kernel only has to keep it fed, and with thousands of such warps
// in flight a load takes a couple of thousand cycles to come back: the candidates' router rows arrive by bulk async copies
// (cp.async.bulk, one 256-byte piece per row and 128-wide k chunk, issued by the row's own lane, completion counted on the
// stage's mbarrier) through a ring of kReStages chunks -- few rows per pass is what makes that depth affordable in shared
// memory; 272-byte rows are conflict-free for 16-byte reads.  The token row's chunk travels the same way and is widened to
// f32 once by the whole warp.  Every accumulator sees k = 0, 1, 2, ... in order.  A token whose count is kRcFull, or one of
// whose exact logits is further than delta from its approximation, gets all E logits recomputed.
constexpr int kReK = 128, kReStages = 10, kReRows = 8, kReWStride = kReK + 8;
constexpr int kReStageBytes = (kReRows * kReWStride + kReK) * 2;
constexpr int kReSmemBytes = kReStages * kReStageBytes + 2 * kReK * 4 + kReStages * 8 + 16;

__device__ __forceinline__ void bulk_copy_g2s(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__global__ void __launch_bounds__(32)
router_exact_rows_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ rw, float *__restrict__ logits,
                         const int32_t *__restrict__ cand, const int32_t *__restrict__ cand_meta, int T, int H, int E,
                         unsigned long long *__restrict__ counters, int32_t *__restrict__ status)
{
    extern __shared__ __align__(16) uint8_t re_smem[];
    float (*xf)[kReK] = reinterpret_cast<float (*)[kReK]>(re_smem + kReStages * kReStageBytes);
    uint64_t *full = reinterpret_cast<uint64_t *>(re_smem + kReStages * kReStageBytes + 2 * kReK * 4);
    volatile uint32_t *abort_flag = reinterpret_cast<uint32_t *>(full + kReStages);
    const int lane = threadIdx.x;
    const int t = blockIdx.x;
    if (t >= T)
        return;
    if (lane == 0) {
        for (int s = 0; s < kReStages; s++)
            mbar_init(&full[s], 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncwarp();
    const int n_cand = cand_meta[2 * t];
    const float delta = __int_as_float(cand_meta[2 * t + 1]);
    const int chunks = H / kReK;
    float *row = logits + static_cast<size_t>(t) * E;
    const __nv_bfloat16 *xrow = x + static_cast<size_t>(t) * H;
    uint32_t g = 0; // chunks consumed so far, over all passes: chunk g lives in stage g % kReStages, phase (g / kReStages) & 1
    bool ok = true;

    // one pass: exact logit of expert `e` for every lane < rows (rows <= kReRows); returns this lane's
    auto pass = [&](int rows, int e) -> float {
        const __nv_bfloat16 *wrow = rw + static_cast<size_t>(lane < rows ? e : 0) * H;
        auto issue = [&](int ch, uint32_t gi) { // called by the whole warp, after every lane is done with the stage's old content
            const uint32_t st = gi % kReStages;
            uint8_t *sb = re_smem + st * kReStageBytes;
            if (lane == 0)
                mbar_arrive_expect_tx(&full[st], static_cast<uint32_t>(rows + 1) * kReK * 2);
            __syncwarp();
            if (lane < rows)
                bulk_copy_g2s(sb + lane * kReWStride * 2, wrow + ch * kReK, kReK * 2, &full[st]);
            else if (lane == kReRows)
                bulk_copy_g2s(sb + kReRows * kReWStride * 2, xrow + ch * kReK, kReK * 2, &full[st]);
        };
        const int pre = chunks < kReStages - 1 ? chunks : kReStages - 1;
        for (int c = 0; c < pre; c++)
            issue(c, g + c);
        float acc = 0.0f;
        for (int ch = 0; ch < chunks && ok; ch++, g++) {
            const uint32_t st = g % kReStages;
            if (!mbar_wait(&full[st], (g / kReStages) & 1u, abort_flag)) {
                ok = false;
                break;
            }
            const uint8_t *sb = re_smem + st * kReStageBytes;
            { // 128 token elements -> f32, four per lane
                const uint2 v = *reinterpret_cast<const uint2 *>(sb + kReRows * kReWStride * 2 + lane * 8);
                *reinterpret_cast<float4 *>(&xf[ch & 1][lane * 4]) =
                    make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                                __uint_as_float(v.y & 0xffff0000u));
            }
            __syncwarp(); // xf[ch & 1] is complete; every lane has finished chunk ch - 1, whose stage is refilled now
            if (ch + kReStages - 1 < chunks)
                issue(ch + kReStages - 1, g + kReStages - 1);
            if (lane < rows) {
                const uint4 *wp = reinterpret_cast<const uint4 *>(sb + lane * kReWStride * 2);
#pragma unroll 4
                for (int i = 0; i < kReK / 8; i++) {
                    const uint4 w = wp[i];
                    const float4 a = *reinterpret_cast<const float4 *>(&xf[ch & 1][i * 8]);
                    const float4 b = *reinterpret_cast<const float4 *>(&xf[ch & 1][i * 8 + 4]);
                    acc = __fmaf_rn(a.x, __uint_as_float(w.x << 16), acc);
                    acc = __fmaf_rn(a.y, __uint_as_float(w.x & 0xffff0000u), acc);
                    acc = __fmaf_rn(a.z, __uint_as_float(w.y << 16), acc);
                    acc = __fmaf_rn(a.w, __uint_as_float(w.y & 0xffff0000u), acc);
                    acc = __fmaf_rn(b.x, __uint_as_float(w.z << 16), acc);
                    acc = __fmaf_rn(b.y, __uint_as_float(w.z & 0xffff0000u), acc);
                    acc = __fmaf_rn(b.z, __uint_as_float(w.w << 16), acc);
                    acc = __fmaf_rn(b.w, __uint_as_float(w.w & 0xffff0000u), acc);
                }
            }
        }
        __syncwarp(); // every lane is done with the last chunks: the stages may be refilled by the next pass
        return acc;
    };

    bool full_token = n_cand > 32;
    if (!full_token) {
        bool bad = false;
        for (int c0 = 0; c0 < n_cand && ok; c0 += kReRows) {
            const int rows = n_cand - c0 < kReRows ? n_cand - c0 : kReRows;
            const int e = lane < rows ? cand[static_cast<size_t>(t) * 32 + c0 + lane] : 0;
            const float exact = pass(rows, e);
            if (lane < rows && ok) {
                bad = bad || !(fabsf(exact - row[e]) <= delta); // the assumed bound does not hold here (or a NaN turned up)
                row[e] = exact;
            }
        }
        full_token = __any_sync(0xffffffffu, bad);
        if (!full_token && counters && lane == 0)
            atomicAdd(&counters[1], static_cast<unsigned long long>(n_cand));
    }
    if (full_token) {
        for (int e0 = 0; e0 < E && ok; e0 += kReRows) {
            const int rows = E - e0 < kReRows ? E - e0 : kReRows;
            const float exact = pass(rows, e0 + lane);
            if (lane < rows && ok)
                row[e0 + lane] = exact;
        }
        if (counters && lane == 0) {
            atomicAdd(&counters[0], 1ull);
            atomicAdd(&counters[1], static_cast<unsigned long long>(E));
        }
    }
    if (!ok) {
        if (lane == 0)
            atomicOr(status, kStatusWaitTimeout);
        for (int i = 0; i < 64; i++) // copies that may still be in flight land before the block's shared memory is released
            __nanosleep(4096);
    }
}

// The same recomputation for up to 256 experts, organised by k-slices instead of by token: a block owns 64 tokens and gives
// every (token, candidate) pair of theirs a THREAD, whose accumulator lives in a register while the block walks the
// hidden dimension in slices of 64: per slice the whole router matrix slice (E x 64 bf16) and the 64 token rows' slice are
// brought into shared memory once, by coalesced cp.async copies, and shared by all the block's chains.  The router
// matrix is then read once per BLOCK (64 tokens) rather than once per pair, in full lines -- per-pair gathers of 128-byte
// pieces, thousands of warps deep, return at about 2 TB/s and left the per-token kernel above at four times the time of its
// FMA chains.  Every accumulator still sees k = 0, 1, 2, ... in order.
constexpr int kRxTokens = 64, kRxThreads = 512, kRxK = 64, kRxStages = 4, kRxStride = kRxK + 8, kRxMaxExperts = 256;
constexpr int kRxStageBytes = (kRxMaxExperts + kRxTokens) * kRxStride * 2;
constexpr int kRxSmemBytes = kRxStages * kRxStageBytes + (kRxTokens + 1) * 4 * 2 + kRxTokens * 4 + (2 * kRxThreads + 16 * 8 + 24 + 2 * kRxMaxExperts + 4) * 4;

__global__ void __launch_bounds__(kRxThreads)
router_exact_slices_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ rw, float *__restrict__ logits,
                           const int32_t *__restrict__ cand, const int32_t *__restrict__ cand_meta, int T, int H, int E,
                           unsigned long long *__restrict__ counters, int tokens_per_block)
{
    // tokens_per_block <= kRxTokens: smaller batches give each block fewer tokens so that the grid still covers the SMs (a
    // block's time is set by walking H once, whatever its token count)
    extern __shared__ __align__(16) uint8_t rx_smem[];
    int *s_off = reinterpret_cast<int *>(rx_smem + kRxStages * kRxStageBytes); // [kRxTokens + 1] exclusive prefix of chain counts
    int *s_cnt = s_off + kRxTokens + 1;                                        // [kRxTokens + 1] candidates per token (E = all)
    int *s_bad = s_cnt + kRxTokens + 1;                                        // [kRxTokens] token needs the full recomputation
    int *s_chain = s_bad + kRxTokens; // [kRxThreads] thread slot -> token << 16 | expert, -1: idle
    int *s_spill = s_chain + kRxThreads; // [kRxThreads] chains whose bucket was full
    int *s_wcnt = s_spill + kRxThreads;  // [16 warps][8 buckets] counts, then exclusive prefixes
    int *s_bcnt = s_wcnt + 16 * 8;       // [8] chains per bucket, [8] prefix of idle slots, [1] spilled chains
    int *s_slot = s_bcnt + 24;           // [kRxMaxExperts] expert -> row of the stage that holds its router row, -1: not staged
    int *s_rows = s_slot + kRxMaxExperts; // [kRxMaxExperts] row of the stage -> expert
    int *s_nrows = s_rows + kRxMaxExperts; // rows staged per slice
    const int tid = threadIdx.x;
    const int t0 = blockIdx.x * tokens_per_block;
    const int nt = T - t0 < tokens_per_block ? T - t0 : tokens_per_block;
    const int slices = H / kRxK;

    auto issue = [&](int sl, int st) {
        const int k0 = sl * kRxK;
        __nv_bfloat16 *wst = reinterpret_cast<__nv_bfloat16 *>(rx_smem + st * kRxStageBytes);
        __nv_bfloat16 *xst = wst + kRxMaxExperts * kRxStride;
        const int nrows = *s_nrows;
        for (int p = tid; p < nrows * 8; p += kRxThreads) { // staged router rows x 8 pieces of 8 bf16
            const int r = p >> 3, c = (p & 7) * 8;
            cp_async16(wst + r * kRxStride + c, rw + static_cast<size_t>(s_rows[r]) * H + k0 + c, true);
        }
        for (int p = tid; p < nt * 8; p += kRxThreads) {
            const int r = p >> 3, c = (p & 7) * 8;
            cp_async16(xst + r * kRxStride + c, x + static_cast<size_t>(t0 + r) * H + k0 + c, true);
        }
    };

    // phase 0: the candidates of every token (all experts for a token marked kRcFull); phase 1: all experts of the tokens
    // one of whose recomputed logits was further than delta from its approximation
    for (int phase = 0; phase < 2; phase++) {
        __syncthreads();
        if (tid < nt) {
            if (phase == 0) {
                const int n = cand_meta[2 * (t0 + tid)];
                s_cnt[tid] = n > 32 ? E : n;
                s_bad[tid] = 0;
            } else {
                s_cnt[tid] = s_bad[tid] ? E : 0;
            }
        }
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int i = 0; i < nt; i++) {
                s_off[i] = run;
                run += s_cnt[i];
            }
            s_off[nt] = run;
        }
        __syncthreads();
        const int chains = s_off[nt];
        for (int base = 0; base < chains; base += kRxThreads) {
            const int c = base + tid;
            bool live = c < chains;
            int tl = 0, e = 0;
            if (live) {
                int lo = 0, hi = nt; // token with s_off[lo] <= c < s_off[lo + 1]
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (s_off[mid] <= c)
                        lo = mid;
                    else
                        hi = mid;
                }
                tl = lo;
                const int j = c - s_off[tl];
                e = (s_cnt[tl] == E && (phase == 1 || cand_meta[2 * (t0 + tl)] > 32)) ? j : cand[static_cast<size_t>(t0 + tl) * 32 + j];
            }
            // Router rows to stage: a block with few chains touches few experts, and what bounds it is what an SM can take in
            // (about 25 bytes per cycle: 53 us for the whole 2 MB matrix), so one round of chains stages only the rows
            // its chains read, compacted; more rounds, or a token that needs its whole row, stage every row.
            if (tid < kRxMaxExperts)
                s_slot[tid] = -1;
            __syncthreads();
            if (chains <= kRxThreads && live)
                s_slot[e] = 0; // needed (same value from every writer)
            __syncthreads();
            if (tid < 32) {
                int run = 0;
                for (int i = 0; i < kRxMaxExperts / 32; i++) {
                    const int ex = i * 32 + tid;
                    const bool need = ex < E && (chains > kRxThreads || s_slot[ex] == 0);
                    const unsigned m = __ballot_sync(0xffffffffu, need);
                    if (need) {
                        const int sl = run + __popc(m & ((1u << tid) - 1u));
                        s_slot[ex] = sl;
                        s_rows[sl] = ex;
                    }
                    run += __popc(m);
                }
                if (tid == 0)
                    *s_nrows = run;
            }
            __syncthreads();
            if (live)
                e |= s_slot[e] << 8; // bits 8..: the row of the stage
            if (chains <= kRxThreads) {
                // One round: re-deal the chains so that the 8 lanes of a quarter warp hold 8 different values of
                // (staged row mod 8).  A 16-byte read of a staged router row lands in the bank group 4 * row mod 32, so a quarter
                // warp of arbitrary rows needs 2 to 3 passes over shared memory per read and one of distinct residues
                // needs one; the token rows follow (rows 4 * token mod 32; buckets keep token order, so a quarter warp sees
                // neighbouring tokens).  Stable counting sort by residue: bucket b fills slots b, 8 + b, 16 + b, ...; what
                // overflows a bucket takes the slots that emptier buckets leave idle.  Which thread runs a chain changes
                // nothing in its result.
                const int wid = tid >> 5, ln = tid & 31;
                if (tid < 16 * 8)
                    s_wcnt[tid] = 0;
                if (tid == 0)
                    s_bcnt[16] = 0;
                s_chain[tid] = -1;
                __syncthreads();
                const int b = live ? ((e >> 8) & 7) : 8;
                const unsigned peers = __match_any_sync(0xffffffffu, b);
                const int rank = __popc(peers & ((1u << ln) - 1u));
                if (live && rank == 0)
                    s_wcnt[wid * 8 + b] = __popc(peers);
                __syncthreads();
                if (tid < 8) {
                    int run = 0;
                    for (int w = 0; w < 16; w++) {
                        const int n = s_wcnt[w * 8 + tid];
                        s_wcnt[w * 8 + tid] = run;
                        run += n;
                    }
                    s_bcnt[tid] = run;
                }
                __syncthreads();
                const int packed = (tl << 16) | e; // token, row of the stage, expert
                if (live) {
                    const int pos = s_wcnt[wid * 8 + b] + rank;
                    if (pos < kRxThreads / 8)
                        s_chain[pos * 8 + b] = packed;
                    else
                        s_spill[atomicAdd(&s_bcnt[16], 1)] = packed;
                }
                if (tid == 0) {
                    int run = 0;
                    for (int i = 0; i < 8; i++) {
                        s_bcnt[8 + i] = run;
                        const int used = s_bcnt[i] < kRxThreads / 8 ? s_bcnt[i] : kRxThreads / 8;
                        run += kRxThreads / 8 - used;
                    }
                }
                __syncthreads();
                if (tid < s_bcnt[16]) {
                    int bb = 7;
                    while (bb > 0 && s_bcnt[8 + bb] > tid)
                        bb--;
                    const int used = s_bcnt[bb] < kRxThreads / 8 ? s_bcnt[bb] : kRxThreads / 8;
                    s_chain[(used + tid - s_bcnt[8 + bb]) * 8 + bb] = s_spill[tid];
                }
                __syncthreads();
                const int mine = s_chain[tid];
                live = mine >= 0;
                tl = live ? mine >> 16 : 0;
                e = live ? mine & 0xffff : 0;
            }
            float acc = 0.0f;
            __syncthreads(); // the stages of the previous round are no longer read
#pragma unroll
            for (int s = 0; s < kRxStages - 1; s++) {
                if (s < slices)
                    issue(s, s);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            for (int sl = 0; sl < slices; sl++) {
                asm volatile("cp.async.wait_group %0;" ::"n"(kRxStages - 2) : "memory"); // this thread's pieces of slice sl have landed
                __syncthreads(); // ... and everyone's; everyone has finished slice sl - 1, whose stage is refilled now
                const int nxt = sl + kRxStages - 1;
                if (nxt < slices)
                    issue(nxt, nxt % kRxStages);
                asm volatile("cp.async.commit_group;" ::: "memory");
                if (live) {
                    const __nv_bfloat16 *wst = reinterpret_cast<const __nv_bfloat16 *>(rx_smem + (sl % kRxStages) * kRxStageBytes);
                    const uint4 *wp = reinterpret_cast<const uint4 *>(wst + (e >> 8) * kRxStride);
                    const uint4 *xp = reinterpret_cast<const uint4 *>(wst + (kRxMaxExperts + tl) * kRxStride);
#pragma unroll
                    for (int i = 0; i < kRxK / 8; i++) {
                        const uint4 w = wp[i], a = xp[i];
                        acc = __fmaf_rn(__uint_as_float(a.x << 16), __uint_as_float(w.x << 16), acc);
                        acc = __fmaf_rn(__uint_as_float(a.x & 0xffff0000u), __uint_as_float(w.x & 0xffff0000u), acc);
                        acc = __fmaf_rn(__uint_as_float(a.y << 16), __uint_as_float(w.y << 16), acc);
                        acc = __fmaf_rn(__uint_as_float(a.y & 0xffff0000u), __uint_as_float(w.y & 0xffff0000u), acc);
                        acc = __fmaf_rn(__uint_as_float(a.z << 16), __uint_as_float(w.z << 16), acc);
                        acc = __fmaf_rn(__uint_as_float(a.z & 0xffff0000u), __uint_as_float(w.z & 0xffff0000u), acc);
                        acc = __fmaf_rn(__uint_as_float(a.w << 16), __uint_as_float(w.w << 16), acc);
                        acc = __fmaf_rn(__uint_as_float(a.w & 0xffff0000u), __uint_as_float(w.w & 0xffff0000u), acc);
                    }
                }
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            if (live) {
                float *cell = logits + static_cast<size_t>(t0 + tl) * E + (e & 0xff);
                if (phase == 0 && s_cnt[tl] != E) {
                    const float delta = __int_as_float(cand_meta[2 * (t0 + tl) + 1]);
                    if (!(fabsf(acc - *cell) <= delta)) // the assumed bound does not hold here (or a NaN turned up)
                        s_bad[tl] = 1;
                }
                *cell = acc;
            }
        }
        if (counters && tid == 0 && chains)
            atomicAdd(&counters[1], static_cast<unsigned long long>(chains));
    }
    __syncthreads();
    if (counters && tid < nt && (s_bad[tid] || cand_meta[2 * (t0 + tid)] > 32))
        atomicAdd(&counters[0], 1ull);
}

} // namespace xs
