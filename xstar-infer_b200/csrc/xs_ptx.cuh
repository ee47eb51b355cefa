// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA, TMEM), fences.
// Every wait in this file is bounded: a wait that gives up returns false and the caller raises the
// kernel's status word instead of spinning forever.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace xs {

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Polls fast first, then backs off with nanosleep.  `abort_flag` (shared memory) lets one
// role that gave up release all the others.  Returns false on time-out or abort.
constexpr uint32_t kFastPolls = 2048;
constexpr uint32_t kSlowPolls = 1u << 21; // x >=64 ns  => gives up after roughly a quarter of a second
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag)
{
    for (uint32_t i = 0; i < kFastPolls; i++)
        if (mbar_try_wait(bar, parity))
            return true;
    for (uint32_t i = 0; i < kSlowPolls; i++) {
        if (mbar_try_wait(bar, parity))
            return true;
        if (*abort_flag)
            return false;
        __nanosleep(64);
    }
    return false;
}

// Non-suspending variant for waits on the critical path of a two-stage hand-over (accumulator buffers): polls with
// mbarrier.test_wait, which never parks the thread, so the waiter resumes within a poll of the phase completing.  Bounded
// like mbar_wait (about a quarter of a second of polling).
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_spin_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag)
{
    for (uint32_t i = 0; i < (1u << 24); i++) {
        if (mbar_test_wait(bar, parity))
            return true;
        if ((i & 1023u) == 1023u && *abort_flag)
            return false;
    }
    return false;
}

// Role profiling (who waits for whom inside a warp-specialised kernel) is a tuning aid compiled in only with
// -DXS_ROLE_PROFILE=1: cycle counters summed into the eight 64-bit words behind the workspace status word.  In the
// default build the helpers below reduce to the plain bounded wait and to nothing.
#ifndef XS_ROLE_PROFILE
#define XS_ROLE_PROFILE 0
#endif
__device__ __forceinline__ long long prof_clock()
{
#if XS_ROLE_PROFILE
    return clock64();
#else
    return 0;
#endif
}
__device__ __forceinline__ void prof_add(unsigned long long *prof, int slot, long long v)
{
#if XS_ROLE_PROFILE
    atomicAdd(&prof[slot], static_cast<unsigned long long>(v));
#else
    (void)prof;
    (void)slot;
    (void)v;
#endif
}
// The bounded wait, adding the cycles spent blocked to `acc` when role profiling is compiled in.
__device__ __forceinline__ bool mbar_wait_t(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, long long &acc)
{
#if XS_ROLE_PROFILE
    // the whole wait is timed, first poll included: mbarrier.try_wait may itself suspend the thread until the phase
    // completes, so a wait that its first poll satisfies can still have been a long one
    const long long t0 = clock64();
    const bool ok = mbar_wait(bar, parity, abort_flag);
    acc += clock64() - t0;
    return ok;
#else
    (void)acc;
    return mbar_wait(bar, parity, abort_flag);
#endif
}

// Register budget of the calling warpgroup (four consecutive warps, all of which must execute the same instruction):
// the light roles of a warp-specialised kernel give registers back so that the register-hungry ones can take them.
template <int N>
__device__ __forceinline__ void reg_dealloc()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_alloc()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// ---- TMA ----------------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with the programmatic-serialisation attribute may be scheduled while
// the kernel before it in the stream is still running: pdl_wait() returns once that kernel has completed and its writes
// are visible, so everything before it (barrier setup, TMEM allocation, tensor-map prefetch) overlaps the predecessor's
// tail, and nothing before it may read or write global memory that another kernel of the stream produces or reads.  Every
// thread of a kernel launched that way calls pdl_wait() on every path, so that "kernel k completed" implies "kernel k - 1
// completed".  pdl_launch_dependents() lets the next kernel be scheduled as soon as every CTA of this one has called it.
// Both are no-ops in a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// 2-D tiled load, global -> this CTA's shared memory, completion on an mbarrier.  c0 is the innermost
// coordinate and c0 * element_size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *m, uint64_t *bar, int32_t c0, int32_t c1,
                                            uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "l"(policy)
        : "memory");
}

// 16-byte read-only global load that stays where it is written: a volatile asm is not moved across the other volatile
// asms of a loop body (barrier waits, TMEM loads), so a load placed one iteration ahead of its use is ISSUED there.
__device__ __forceinline__ float4 ldg_f4_pinned(const float *p)
{
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldg_f32_pinned(const float *p)
{
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ int ldg_s32_pinned(const int32_t *p)
{
    int v;
    asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// ---- tcgen05 ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// arrive on an mbarrier once all previously issued MMAs of this thread have completed
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes wide and stored with the
// 128-byte swizzle (what a TMA box of 128 bytes x rows with SWIZZLE_128B produces).  Groups of 8 rows are
// 1024 bytes apart.  Bits: [0,14) start>>4, [16,30) leading offset>>4 (unused for swizzled K-major, 1),
// [32,46) stride offset>>4 = 64, [46,48) version = 1, [61,64) layout = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor, dense, f32 accumulate, both operands K-major.
// fmt: kind::f16 -> 0 = f16, 1 = bf16; kind::f8f6f4 -> 0 = e4m3, 1 = e5m2, 5 = e2m1.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n)
{
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// TMEM -> registers: 32 lanes (this warp's quarter) x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
// Wait for outstanding tcgen05.ld and tie the wait to the destination registers, so that no use of them can be
// scheduled ahead of it (the loads are asynchronous: their registers are valid only after the wait).
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&a)[16], uint32_t (&b)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]), "+r"(a[9]),
                   "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]), "+r"(b[0]), "+r"(b[1]), "+r"(b[2]),
                   "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]), "+r"(b[8]), "+r"(b[9]), "+r"(b[10]), "+r"(b[11]),
                   "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15])
                 :
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_16(uint32_t (&a)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]), "+r"(a[9]),
                   "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15])
                 :
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

} // namespace xs

namespace xs {

// Instruction descriptor for block-scaled MMA (kind::mxf8f6f4, one ue8m0 scale per 32 elements of K):
// bits [4,6) B scale id, [7,10) A format, [10,13) B format, [17,23) N>>3, [23] scale format (1 = ue8m0),
// [24,29) M>>4, [29,31) A scale id.  A scale id selects which byte of the 32-bit TMEM scale column is used.
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n, uint32_t sf_id)
{
    return (sf_id << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (sf_id << 29);
}

__device__ __forceinline__ void mma_mxf8f6f4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t tmem_sfa,
                                             uint32_t tmem_sfb, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// Shared-memory descriptor of an unswizzled block of 16-byte rows stored back to back (row r at r * 16): groups of
// 8 rows are 128 bytes apart.  Used as the source of tcgen05.cp.
__device__ __forceinline__ uint64_t make_desc_rows16(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(16 >> 4) << 16;  // leading offset (unused: one 16-byte column)
    d |= static_cast<uint64_t>(128 >> 4) << 32; // stride between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}
// shared memory -> TMEM: 32 rows x 128 bits land in lanes 0..31 of FOUR consecutive columns and are replicated into
// all four lane quarters.  Ordered with the tcgen05.mma instructions the same thread issues afterwards.
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// make generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05 reads of shared memory)
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 4 x 4 transpose of 16-byte chunks among the four lanes of a quad (lanes 4a..4a+3): on entry b[j] is chunk j of this
// lane's row, on exit b[i] is chunk (lane & 3) of the row of lane 4a + i.  A thread that holds consecutive columns of ONE
// row would store 16 bytes per lane to 32 different rows per instruction; after the transpose a quad writes 64 contiguous
// bytes of one row, 8 rows per instruction.
__device__ __forceinline__ void quad_transpose_chunks(uint4 (&b)[4], int qd)
{
    auto shfl4 = [](const uint4 &v, int m) {
        return make_uint4(__shfl_xor_sync(0xffffffffu, v.x, m), __shfl_xor_sync(0xffffffffu, v.y, m),
                          __shfl_xor_sync(0xffffffffu, v.z, m), __shfl_xor_sync(0xffffffffu, v.w, m));
    };
    {
        // lanes l and l ^ 1 swap the off-diagonal elements of each 2 x 2 block
        const bool odd = qd & 1;
        const uint4 s0 = shfl4(odd ? b[0] : b[1], 1), s1 = shfl4(odd ? b[2] : b[3], 1);
        if (odd) {
            b[0] = s0;
            b[2] = s1;
        } else {
            b[1] = s0;
            b[3] = s1;
        }
    }
    {
        // lanes l and l ^ 2 swap the off-diagonal 2 x 2 blocks
        const bool hi = qd & 2;
        const uint4 s0 = shfl4(hi ? b[0] : b[2], 2), s1 = shfl4(hi ? b[1] : b[3], 2);
        if (hi) {
            b[0] = s0;
            b[1] = s1;
        } else {
            b[2] = s0;
            b[3] = s1;
        }
    }
}

} // namespace xs
