// Router: logits = x . router_w^T with each output accumulated in ascending k in f32 (so that the logits
// equal, bit for bit, a sequential CPU loop and near-ties cannot flip an expert choice), then per-token
// selection of the k largest keys with warp-shuffle reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "xs_ptx.cuh"

namespace xs {

// Large batches: (16 * TPT) tokens x 128 experts per block, TPT x 8 outputs per thread (launched with TPT = 4: 64-token
// tiles, once there are enough of them to fill the SMs; smaller batches take router_logits_mid_kernel below).  Operands are
// widened to f32 while they are staged in shared memory, so the inner loop is (TPT + 8) 16-byte shared loads per 32 * TPT
// FMAs and no conversions; k chunks of 32 are double-buffered.  Same contract: every accumulator sees k = 0, 1, 2, ... in order.
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

// Decode-sized batches.  Block = 8 experts x 32 tokens, one output per thread (warp = one expert, lanes = tokens),
// so a batch of 128 tokens x 256 experts spreads over 128 SMs.  Operands arrive through an 8-stage cp.async
// pipeline of 128-wide k chunks; inside a chunk each thread walks k upwards, 8 elements per 16-byte shared-memory
// read (the router row is a warp-wide broadcast, the token rows are padded to stay bank-conflict free).
// One accumulator per thread, touched once per k in ascending order: the contract's summation order -- which makes the
// H dependent FMAs the floor of this kernel; the pipeline is eight chunks deep because at decode sizes the kernel is
// otherwise bound by the latency of fetching its operands.  (A version with feeder warps that widen the operands to f32 once
// per block, as the small-batch kernel below does, was no faster here: 256 chain threads reading their token's f32 operand
// are bound by shared-memory wavefronts, 40 per 4 k and SM against the 19 cycles the chains need.)
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
    pdl_launch_dependents();
    pdl_wait();

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

// Medium batches (too few 64-token tiles to fill the SMs): 32 tokens x 128 experts per block, 2 x 8 outputs per thread.
// With that small a register tile the f32-staged kernel above is bound by shared-memory wavefronts (profile: shared pipe
// at 76 % of peak, FMA pipe at 36 %), so here the operands stay bf16 in shared memory -- a 16-byte read carries 8 k
// instead of 4 -- and are widened in registers, one ALU operation each on a pipe that is otherwise idle.  (With the 4 x 8
// tile the extra instructions cost more than the wavefronts saved, which is why both kernels exist.)  Same contract: every
// accumulator sees k = 0, 1, 2, ... in order.
constexpr int kRmStride = kRbK + 8; // bf16 elements; 80-byte rows: conflict-free 16-byte reads
template <int TPT>
constexpr int rm_smem_bytes()
{
    return 2 * (16 * TPT + kRbExperts) * kRmStride * 2;
}
__device__ __forceinline__ float bf16_at(const uint4 &v, int k) // element k (0..7) of eight packed bf16, widened
{
    const uint32_t w = k < 2 ? v.x : (k < 4 ? v.y : (k < 6 ? v.z : v.w));
    return (k & 1) ? __uint_as_float(w & 0xffff0000u) : __uint_as_float(w << 16);
}
template <int TPT>
__global__ void __launch_bounds__(kRbThreads, 2)
router_logits_mid_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ rw, float *__restrict__ logits,
                         int T, int H, int E)
{
    constexpr int TOK = 16 * TPT;
    constexpr int PIECES = (TOK + kRbExperts) * 4; // 16-byte pieces (8 bf16) per k chunk
    constexpr int PPT = (PIECES + kRbThreads - 1) / kRbThreads;
    extern __shared__ __align__(16) uint16_t rm_smem[];
    uint16_t (*xs)[TOK][kRmStride] = reinterpret_cast<uint16_t (*)[TOK][kRmStride]>(rm_smem);
    uint16_t (*ws)[kRbExperts][kRmStride] = reinterpret_cast<uint16_t (*)[kRbExperts][kRmStride]>(rm_smem + 2 * TOK * kRmStride);
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
            uint16_t *dst = r < TOK ? &xs[buf][r][c] : &ws[buf][r - TOK][c];
            *reinterpret_cast<uint4 *>(dst) = stage_regs[i];
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
        for (int k = 0; k < kRbK; k += 8) {
            uint4 xv[TPT], wv[8];
#pragma unroll
            for (int i = 0; i < TPT; i++)
                xv[i] = *reinterpret_cast<const uint4 *>(&xs[buf][ty + 16 * i][k]);
#pragma unroll
            for (int j = 0; j < 8; j++)
                wv[j] = *reinterpret_cast<const uint4 *>(&ws[buf][tx + 16 * j][k]);
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                float xf[TPT], wf[8];
#pragma unroll
                for (int i = 0; i < TPT; i++)
                    xf[i] = bf16_at(xv[i], kk);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    wf[j] = bf16_at(wv[j], kk);
#pragma unroll
                for (int i = 0; i < TPT; i++)
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        acc[i][j] = __fmaf_rn(xf[i], wf[j], acc[i][j]);
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

// The smallest batches (a few tokens per SM at most): the floor of the router is the chain of H dependent FMAs of one
// output (about 10 us at H = 4096), so the kernel is built to keep that chain fed and to put nothing else into the warp that
// runs it.  A warp issues in program order: every instruction that shares a warp with the chain -- widening bf16 to f32,
// address arithmetic, the copies' issue -- takes an issue slot the chain's next FMA then waits behind (a single-warp version
// of this kernel executed 4 instructions per k and spent 3 cycles on each).  So a block is FOUR warps for 32 experts x one
// token:
//   warps 1..3, the feeders: each thread issues the cp.async copies of its own 16-byte pieces of the router rows (4 stages
//     of 128-wide k chunks) and of the token row, and widens exactly those pieces to f32 in shared memory once they have
//     landed (so a thread only ever waits for its own copies), one chunk ahead of the chain (one feeder warp alone took
//     longer per chunk than the chain does).  Measured at one token: 18 us with the top-k (the chain alone takes 11); staging
//     the pieces in registers instead of shared memory, 256-wide chunks, more feeder warps and deeper copy pipelines were
//     each measured and changed nothing;
//   warp 0, the chain: lane = expert; per 4 k one 16-byte read of its own f32 row, one broadcast read of the token's, 4 FMAs.
// All four meet once per chunk at a named barrier.  Same contract: every accumulator sees k = 0, 1, 2, ... in order.
constexpr int kRsK = 128, kRsStages = 4, kRsWStride = kRsK + 8; // bf16 elements; 272-byte rows are conflict-free for 16-byte reads
constexpr int kRsFStride = kRsK + 4;                            // f32 elements; 528-byte rows: conflict-free 16-byte reads per quarter warp
constexpr int kRsThreads = 128, kRsFeeders = kRsThreads - 32;
constexpr int rs_smem_bytes()
{
    return kRsStages * (32 * kRsWStride + kRsK) * 2 + 2 * (32 * kRsFStride + kRsK) * 4;
}
__global__ void __launch_bounds__(kRsThreads)
router_logits_small_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ rw, float *__restrict__ logits,
                           int T, int H, int E)
{
    extern __shared__ __align__(16) uint8_t rs_smem[];
    __nv_bfloat16 (*wsm)[32][kRsWStride] = reinterpret_cast<__nv_bfloat16 (*)[32][kRsWStride]>(rs_smem);
    __nv_bfloat16 (*xsm)[kRsK] = reinterpret_cast<__nv_bfloat16 (*)[kRsK]>(rs_smem + kRsStages * 32 * kRsWStride * 2);
    float *fbase = reinterpret_cast<float *>(rs_smem + kRsStages * (32 * kRsWStride + kRsK) * 2);
    auto wf = [&](int buf) { return fbase + buf * (32 * kRsFStride + kRsK); };                  // [32][kRsFStride]
    auto xf = [&](int buf) { return fbase + buf * (32 * kRsFStride + kRsK) + 32 * kRsFStride; }; // [kRsK]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = blockIdx.x * 32, t = blockIdx.y;
    const int chunks = H / kRsK;
    pdl_launch_dependents();
    pdl_wait();
    auto meet = [] { asm volatile("bar.sync 1, %0;" ::"n"(kRsThreads) : "memory"); };
    auto widen8 = [](const uint4 &v, float *d) {
        *reinterpret_cast<float4 *>(d) = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                                                    __uint_as_float(v.y & 0xffff0000u));
        *reinterpret_cast<float4 *>(d + 4) = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                                                        __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
    };

    if (warp >= 1) {
        const int fid = threadIdx.x - 32; // 0 .. kRsFeeders - 1
        constexpr int kPieces = 32 * (kRsK / 8), kIters = (kPieces + kRsFeeders - 1) / kRsFeeders;
        auto issue = [&](int ch, int st) {
            const int k0 = ch * kRsK;
#pragma unroll
            for (int i = 0; i < kIters; i++) { // 32 router rows x 16 pieces of 8 bf16
                const int p = fid + kRsFeeders * i;
                if (p < kPieces) {
                    const int r = p >> 4, c = (p & 15) * 8;
                    const bool ok = e0 + r < E;
                    cp_async16(&wsm[st][r][c], rw + static_cast<size_t>(ok ? e0 + r : 0) * H + k0 + c, ok);
                }
            }
            if (fid < kRsK / 8)
                cp_async16(&xsm[st][fid * 8], x + static_cast<size_t>(t) * H + k0 + fid * 8, true);
        };
        auto widen = [&](int st, int buf) { // this thread's own pieces of the landed chunk: bf16 -> f32
            // every read before the first write: the compiler cannot prove that the f32 buffer and the bf16 stage are apart,
            // and would otherwise run read -> widen -> write one piece after the other, a shared-memory round trip each
            float *w = wf(buf);
            uint4 v[kIters], vx = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int i = 0; i < kIters; i++) {
                const int p = fid + kRsFeeders * i;
                v[i] = make_uint4(0, 0, 0, 0);
                if (p < kPieces)
                    v[i] = *reinterpret_cast<const uint4 *>(&wsm[st][p >> 4][(p & 15) * 8]);
            }
            if (fid < kRsK / 8)
                vx = *reinterpret_cast<const uint4 *>(&xsm[st][fid * 8]);
#pragma unroll
            for (int i = 0; i < kIters; i++) {
                const int p = fid + kRsFeeders * i;
                if (p < kPieces)
                    widen8(v[i], w + (p >> 4) * kRsFStride + (p & 15) * 8);
            }
            if (fid < kRsK / 8)
                widen8(vx, xf(buf) + fid * 8);
        };
#pragma unroll
        for (int sidx = 0; sidx < kRsStages - 1; sidx++) {
            if (sidx < chunks)
                issue(sidx, sidx);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        for (int ch = 0; ch < chunks; ch++) {
            asm volatile("cp.async.wait_group %0;" ::"n"(kRsStages - 2) : "memory"); // this thread's pieces of chunk ch have landed
            widen(ch % kRsStages, ch & 1);
            const int nxt = ch + kRsStages - 1; // the pieces just read out are this thread's own: refill them
            if (nxt < chunks)
                issue(nxt, nxt % kRsStages);
            asm volatile("cp.async.commit_group;" ::: "memory");
            // hand chunk ch over; the chain finished chunk ch - 1 by then, so buffer (ch + 1) & 1 is free for the next chunk
            meet();
        }
    } else {
        float acc = 0.0f;
        for (int ch = 0; ch < chunks; ch++) {
            meet(); // chunk ch is widened
            const float4 *wp = reinterpret_cast<const float4 *>(wf(ch & 1) + lane * kRsFStride);
            const float4 *xp = reinterpret_cast<const float4 *>(xf(ch & 1));
            // a window of 8 reads stays in flight ahead of the FMAs, so the chain does not wait for shared memory inside a chunk
            float4 wq[8], xq[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                wq[i] = wp[i];
                xq[i] = xp[i];
            }
#pragma unroll
            for (int i = 0; i < kRsK / 4; i++) {
                const float4 w = wq[i & 7], a = xq[i & 7];
                if (i + 8 < kRsK / 4) {
                    wq[i & 7] = wp[i + 8];
                    xq[i & 7] = xp[i + 8];
                }
                acc = __fmaf_rn(a.x, w.x, acc);
                acc = __fmaf_rn(a.y, w.y, acc);
                acc = __fmaf_rn(a.z, w.z, acc);
                acc = __fmaf_rn(a.w, w.w, acc);
            }
        }
        const int e = e0 + lane;
        if (e < E)
            logits[static_cast<size_t>(t) * E + e] = acc;
    }
}

// One warp per token.  Lane l holds experts l, l+32, l+64, ...  (NPL per lane).
// Selection: K rounds of "largest key, ties to the lower expert id" by butterfly shuffles; a NaN key counts as -inf.
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
            const float kv = bias ? __fadd_rn(lg[i], bias[e]) : lg[i];
            key[i] = (kv != kv) ? -INFINITY : kv; // a NaN key orders as -inf, so every lane sees one total order
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
        const int slot = base + __popc(mask & ((1u << lane) - 1u));
        if (c && slot < K) {
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
    pdl_launch_dependents();
    pdl_wait();
    if (warp >= T)
        return;
    topk_warp<NPL>(logits, bias, topk_ids, topk_w, warp, lane, E, K);
}

} // namespace xs
