// C ABI of the MoE forward path (declared in include/xs_moe.h): argument checks, workspace planning,
// tensor-map construction and kernel launches.  No exception leaves this file; every failure becomes a
// negative status plus a thread-local message.
#include "xs_moe.h"
#include "xs_moe_tuning.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <utility>
#include <type_traits>
#include <vector>
#include <string>

#include "xs_grouped_gemm.cuh"
#include "xs_grouped_gemm_fp4.cuh"
#include "xs_prefill_fp8.cuh"
#include "xs_prefill_fp4.cuh"
#include "xs_mma_rate.cuh"
#include "xs_permute.cuh"
#include "xs_route.cuh"
#include "xs_route_tc.cuh"
#include "xs_ep.cuh"

namespace {

thread_local std::string g_last_error;

// kernels this library has enqueued since the process started (captured launches count once, at capture)
std::atomic<unsigned long long> g_launches{0};
inline void note_launch()
{
    g_launches.fetch_add(1, std::memory_order_relaxed);
}

// Launch with the programmatic-serialisation attribute (see pdl_wait in xs_ptx.cuh): only for kernels whose every thread
// calls xs::pdl_wait() before its first access to global memory that other kernels of the stream write or read.
// XS_MOE_PDL=0 in the environment turns the attribute off (the kernels then start after their predecessor, as usual).
inline bool pdl_enabled()
{
    static const bool on = [] {
        const char *e = getenv("XS_MOE_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

int fail(int status, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return status;
}

#define XS_CUDA(call)                                                                                       \
    do {                                                                                                    \
        cudaError_t err__ = (call);                                                                         \
        if (err__ != cudaSuccess)                                                                           \
            return fail(XS_MOE_ERR_CUDA, "CUDA error: %s (%s) at %s:%d", cudaGetErrorString(err__), #call, \
                        __FILE__, __LINE__);                                                                \
    } while (0)

inline size_t align_up(size_t v, size_t a)
{
    return (v + a - 1) / a * a;
}

// ---- driver entry point for tensor maps (no link-time dependency on libcuda) ---------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Encoded maps are kept: a layer call describes the same weight matrices (and, with a reused workspace, the same
// activation buffers) every time, and an encode costs about a microsecond of host time -- a tenth of a decode step's launch
// budget when a call needs eight of them.  The key is everything the encoding depends on, so a cached map is exactly the map
// a fresh encode would give.  Small, linear, thread-safe; the oldest entry is replaced when it is full.
struct TmapKey {
    uintptr_t base;
    uint64_t d0, d1, s0;
    uint32_t b0, b1;
    int32_t dt, swizzle, l2;
    bool operator==(const TmapKey &o) const
    {
        return base == o.base && d0 == o.d0 && d1 == o.d1 && s0 == o.s0 && b0 == o.b0 && b1 == o.b1 && dt == o.dt && swizzle == o.swizzle &&
               l2 == o.l2;
    }
};
CUresult encode_2d_cached(EncodeTiledFn fn, CUtensorMap *m, CUtensorMapDataType dt, const void *base, const cuuint64_t *dims,
                          const cuuint64_t *strides, const cuuint32_t *box, CUtensorMapSwizzle swz, CUtensorMapL2promotion l2)
{
    constexpr int kEntries = 128;
    struct Entry {
        TmapKey key;
        CUtensorMap map;
    };
    static std::mutex mu;
    static std::vector<Entry> table;
    static size_t next = 0;
    const TmapKey key{reinterpret_cast<uintptr_t>(base), dims[0], dims[1], strides[0], box[0], box[1], static_cast<int32_t>(dt),
                      static_cast<int32_t>(swz), static_cast<int32_t>(l2)};
    {
        std::lock_guard<std::mutex> lock(mu);
        for (const Entry &e : table)
            if (e.key == key) {
                *m = e.map;
                return CUDA_SUCCESS;
            }
    }
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, l2,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        std::lock_guard<std::mutex> lock(mu);
        if (table.size() < kEntries) {
            table.push_back(Entry{key, *m});
        } else {
            table[next] = Entry{key, *m};
            next = (next + 1) % kEntries;
        }
    }
    return r;
}

// 2-D row-major matrix (rows, cols) of `elem_bytes`-wide elements; box = (box_cols, box_rows); 128-byte swizzle.
int make_tmap_2d(CUtensorMap *m, CUtensorMapDataType dt, int elem_bytes, const void *base, uint64_t rows, uint64_t cols,
                 uint32_t box_rows, uint32_t box_cols)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn)
        return fail(XS_MOE_ERR_CUDA, "CUDA error: cuTensorMapEncodeTiled entry point not available");
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (cols * elem_bytes) % 16 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "tensor map operand must be 16-byte aligned with a 16-byte multiple row pitch");
    if (box_cols * elem_bytes != 128)
        return fail(XS_MOE_ERR_INVALID_ARG, "internal: swizzled box must be 128 bytes wide");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * static_cast<uint64_t>(elem_bytes)};
    cuuint32_t box[2] = {box_cols, box_rows};
    CUresult r = encode_2d_cached(fn, m, dt, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (r != CUDA_SUCCESS)
        return fail(XS_MOE_ERR_CUDA, "CUDA error: cuTensorMapEncodeTiled failed with code %d (rows=%llu cols=%llu)", (int)r,
                    (unsigned long long)rows, (unsigned long long)cols);
    return 0;
}

// 2-D row-major byte matrix (rows, row_bytes) read in boxes of (box_bytes, box_rows) WITHOUT swizzle: rows of the box land
// back to back in shared memory.
int make_tmap_bytes(CUtensorMap *m, const void *base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, uint32_t box_bytes)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn)
        return fail(XS_MOE_ERR_CUDA, "CUDA error: cuTensorMapEncodeTiled entry point not available");
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || row_bytes % 16 != 0 || box_bytes % 16 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "tensor map operand must be 16-byte aligned with a 16-byte multiple row pitch");
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_bytes, box_rows};
    CUresult r = encode_2d_cached(fn, m, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_NONE);
    if (r != CUDA_SUCCESS)
        return fail(XS_MOE_ERR_CUDA, "CUDA error: cuTensorMapEncodeTiled failed with code %d (rows=%llu row bytes=%llu)", (int)r,
                    (unsigned long long)rows, (unsigned long long)row_bytes);
    return 0;
}

struct DeviceInfo {
    int ok = 0;
    int sms = 0;
    int max_smem = 0;
};

int device_info(DeviceInfo *out)
{
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    static DeviceInfo cache[64];
    if (dev < 64 && cache[dev].ok) {
        *out = cache[dev];
        return 0;
    }
    int major = 0, sms = 0, smem = 0;
    XS_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    XS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    XS_CUDA(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    if (major != 10)
        return fail(XS_MOE_ERR_DEVICE, "this library holds sm_100a kernels only; device %d has compute capability %d.x", dev, major);
    DeviceInfo d;
    d.ok = 1;
    d.sms = sms;
    d.max_smem = smem;
    if (dev < 64)
        cache[dev] = d;
    *out = d;
    return 0;
}

// ---- configuration checks ------------------------------------------------------------------------------
int check_cfg(const XsMoeConfig *c)
{
    if (!c)
        return fail(XS_MOE_ERR_INVALID_ARG, "config is null");
    if (c->num_tokens < 0 || c->hidden <= 0 || c->num_experts <= 0 || c->intermediate <= 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: non-positive dimension");
    if (c->top_k <= 0 || c->top_k > c->num_experts || c->top_k > 32)
        return fail(XS_MOE_ERR_INVALID_ARG, "top_k out of range");
    if (c->num_experts > 1024)
        return fail(XS_MOE_ERR_UNSUPPORTED, "expert count mismatch: at most 1024 routed experts");
    if (c->num_shared < 0 || c->num_shared > 1)
        return fail(XS_MOE_ERR_INVALID_ARG, "num_shared must be 0 or 1");
    if (c->hidden % 128 != 0 || c->intermediate % 128 != 0)
        return fail(XS_MOE_ERR_UNSUPPORTED, "shape mismatch: hidden and intermediate must be multiples of 128");
    if (c->local_expert_begin < 0 || c->local_expert_count <= 0 ||
        c->local_expert_begin + c->local_expert_count > c->num_experts)
        return fail(XS_MOE_ERR_INVALID_ARG, "expert count mismatch: local expert range outside [0, num_experts)");
    if (c->routed_format != XS_MOE_BF16 && c->routed_format != XS_MOE_FP8_BLOCK128 && c->routed_format != XS_MOE_FP4_MX32)
        return fail(XS_MOE_ERR_UNSUPPORTED, "unsupported dtype: routed experts must be bf16, FP8 e4m3 (128x128 scales) or FP4 e2m1 (e8m0/32)");
    if (c->num_shared) {
        const int want = c->routed_format == XS_MOE_FP4_MX32 ? XS_MOE_FP8_BLOCK128 : c->routed_format;
        if (c->shared_format != want)
            return fail(XS_MOE_ERR_UNSUPPORTED, "unsupported dtype: the shared expert must be bf16 next to bf16 experts and FP8 e4m3 "
                                                "(128x128 scales) next to FP8 or FP4 experts");
    }
    if (c->gemm_impl != 0 && c->gemm_impl != 1)
        return fail(XS_MOE_ERR_INVALID_ARG, "gemm_impl must be 0 or 1");
    if (c->gemm_impl == 1 && c->routed_format != XS_MOE_BF16)
        return fail(XS_MOE_ERR_UNSUPPORTED, "unsupported dtype: the CUDA-core cross-check kernels are bf16 only");
    for (int i = 0; i < 5; i++)
        if (c->reserved[i] != 0)
            return fail(XS_MOE_ERR_INVALID_ARG, "reserved fields must be zero");
    return 0;
}

// Rows per token tile.  bf16: 16..128 tokens as the N of a 128-weight-row MMA.  FP8/FP4: up to 64 in that shape (the
// FP8 epilogue keeps one f32 accumulator per token column in registers); FP8 batches with many tokens per expert use
// the prefill kernel instead, whose tiles are 128 tokens as the M of an N = 256 MMA (needs hidden % 256 == 0).
int pick_n_tile(long rows, int groups, int fmt, int hidden)
{
    const long avg = groups > 0 ? (rows + groups - 1) / groups : rows;
    // FP4: the tokens-as-M kernel at every batch size (an N = 256 block-scaled MMA consumes twice the packed weight bytes of
    // a weights-as-M one); 32-row token boxes while experts see a handful of tokens, 128-row ones beyond
    if (fmt == XS_MOE_FP4_MX32 && hidden % 256 == 0)
        return avg <= 20 ? 32 : 128;
    if (avg <= 8)
        return 16;
    if (avg <= 20)
        return 32;
    // FP8 / FP4 with more than ~20 tokens per expert: the tokens-as-M kernels win (measured: at 48 tokens per expert the
    // FP8 layer takes 0.9 ms there against 2.1 ms in the 64-token decode shape)
    if ((fmt == XS_MOE_FP8_BLOCK128 || fmt == XS_MOE_FP4_MX32) && hidden % 256 == 0)
        return 128;
    if (avg <= 48 || fmt != XS_MOE_BF16)
        return 64;
    return 128;
}

// ---- workspace plans -----------------------------------------------------------------------------------
// Scratch of one grouped MLP over `max_rows` rows in `segments` expert segments (the routed experts and, when the
// always-on expert is merged into the same launches, one more segment for its rows).
struct GroupedPlan {
    int n_tile = 0, max_tiles = 0;
    size_t off_tile_expert = 0, off_tile_row0 = 0, off_num_tiles = 0, off_offsets = 0, off_act = 0, off_act_scale = 0, bytes = 0;
};

GroupedPlan plan_grouped(int max_rows, int routed_rows, int routed_groups, int segments, int I, int fmt, int H)
{
    GroupedPlan p;
    p.n_tile = pick_n_tile(routed_rows, routed_groups, fmt, H);
    p.max_tiles = max_rows / p.n_tile + segments + 1;
    size_t o = 0;
    p.off_tile_expert = o; o = align_up(o + sizeof(int32_t) * p.max_tiles, 256);
    p.off_tile_row0 = o;   o = align_up(o + sizeof(int32_t) * p.max_tiles, 256);
    p.off_num_tiles = o;   o = align_up(o + sizeof(int32_t), 256);
    p.off_offsets = o;     o = align_up(o + sizeof(int32_t) * (segments + 1), 256); // segment offsets clamped to max_rows
    p.off_act = o;         o = align_up(o + static_cast<size_t>(max_rows) * I * (fmt == XS_MOE_BF16 ? 2 : 1), 256);
    p.off_act_scale = o;   o = align_up(o + (fmt == XS_MOE_BF16 ? 0 : static_cast<size_t>(max_rows) * (I / 128) * 4), 256); // FP4: I/32 bytes
    p.bytes = o;
    return p;
}

constexpr size_t kStatusBytes = 256;
constexpr int kRouterFilterTokens = 256; // larger batches may take the tensor-core filter + exact refine router

struct ForwardPlan {
    int chunks = 0;
    size_t off_logits = 0, off_cand = 0, off_cand_meta = 0, off_ids = 0, off_w = 0, off_counts = 0, off_offsets = 0, off_perm = 0, off_inv = 0;
    size_t off_chunk_counts = 0, off_chunk_base = 0, off_rows = 0, off_rows_scale = 0, off_y = 0, off_grouped = 0;
    size_t off_sh_rows = 0, off_sh_scale = 0, off_sh_offsets = 0, off_sh_grouped = 0; // FP4: the FP8 always-on expert runs on its own
    GroupedPlan grouped, sh_grouped;
    size_t bytes = 0;
};

ForwardPlan plan_forward(const XsMoeConfig *c)
{
    ForwardPlan p;
    const size_t T = c->num_tokens, H = c->hidden, E = c->num_experts, K = c->top_k, I = c->intermediate, S = c->num_shared;
    p.chunks = static_cast<int>((T + xs::kChunkTokens - 1) / xs::kChunkTokens);
    if (p.chunks == 0)
        p.chunks = 1;
    size_t o = kStatusBytes;
    auto take = [&](size_t bytes) {
        size_t at = o;
        o = align_up(o + bytes, 256);
        return at;
    };
    const bool fp8 = c->routed_format == XS_MOE_FP8_BLOCK128, fp4 = c->routed_format == XS_MOE_FP4_MX32;
    const size_t Sm = fp4 ? 0 : S; // rows of the always-on expert merged behind the routed rows
    p.off_logits = take(T * E * 4);
    p.off_cand = take(T > kRouterFilterTokens ? T * 32 * 4 : 0);      // filter + refine router: experts to recompute exactly
    p.off_cand_meta = take(T > kRouterFilterTokens ? T * 2 * 4 : 0);  // ... their count and the token's error bound
    p.off_ids = take(T * K * 4);
    p.off_w = take(T * K * 4);
    p.off_counts = take(E * 4);
    p.off_offsets = take((E + 2) * 4);
    p.off_perm = take(T * K * 4);
    p.off_inv = take(T * K * 4);
    p.off_chunk_counts = take(static_cast<size_t>(p.chunks) * E * 4);
    p.off_chunk_base = take(static_cast<size_t>(p.chunks) * E * 4);
    p.off_rows = take((T * K + Sm * T) * H * (fp8 || fp4 ? 1 : 2));
    p.off_rows_scale = take(fp8 ? (T * K + Sm * T) * (H / 128) * 4 : (fp4 ? T * K * (H / 32) : 0));
    p.off_y = take((T * K + S * T) * H * 4);
    p.grouped = plan_grouped(static_cast<int>(T * K + Sm * T), static_cast<int>(T * K), static_cast<int>(E), static_cast<int>(E + Sm),
                             static_cast<int>(I), c->routed_format, static_cast<int>(H));
    p.off_grouped = take(p.grouped.bytes);
    if (fp4 && S) {
        p.off_sh_rows = take(T * H);
        p.off_sh_scale = take(T * (H / 128) * 4);
        p.off_sh_offsets = take(8);
        p.sh_grouped = plan_grouped(static_cast<int>(T), static_cast<int>(T), 1, 1, static_cast<int>(I), XS_MOE_FP8_BLOCK128,
                                    static_cast<int>(H));
        p.off_sh_grouped = take(p.sh_grouped.bytes);
    }
    p.bytes = o;
    return p;
}

int check_workspace(const void *ws, size_t have, size_t need)
{
    if (!ws)
        return fail(XS_MOE_ERR_WORKSPACE, "workspace is null");
    if (reinterpret_cast<uintptr_t>(ws) % 256 != 0)
        return fail(XS_MOE_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    if (have < need)
        return fail(XS_MOE_ERR_WORKSPACE, "workspace too small: %zu bytes given, %zu needed", have, need);
    return 0;
}

// ---- launches --------------------------------------------------------------------------------------------
constexpr int kRouterSmallTokens = 32;

constexpr size_t kOffWnorm = 192;        // status block: f32 max router-row norm
constexpr size_t kOffRefineCounters = 200; // status block: two u64 (tokens recomputed in full, exact logits computed)

// Filter + refine (xs_route_tc.cuh): approximate logits on the tensor core, exact recomputation of everything the
// selection can depend on.  `status_block` is the head of the caller's workspace.
int launch_logits_filtered(const XsMoeConfig *c, const void *x, const void *rw, const float *bias, float *logits, uint8_t *status_block,
                           int32_t *cand, int32_t *cand_meta, cudaStream_t st)
{
    const int T = c->num_tokens, H = c->hidden, E = c->num_experts, K = c->top_k;
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    const int n = E >= xs::kRtMaxN ? xs::kRtMaxN : (E + 15) / 16 * 16;
    const int stage_bytes = xs::rt_stage_bytes(n);
    int stages = (di.max_smem - 1024 - 256) / stage_bytes;
    if (stages > 6)
        stages = 6;
    if (stages < 2)
        return fail(XS_MOE_ERR_DEVICE, "not enough shared memory for the router pipeline");
    const int smem = stages * stage_bytes + 1024 + 256;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(xs::router_logits_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
        XS_CUDA(cudaFuncSetAttribute(xs::router_exact_slices_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, xs::kRxSmemBytes));
        if (dev < 64)
            configured[dev] = true;
    }
    CUtensorMap t_x, t_w;
    if (int rc = make_tmap_2d(&t_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, T, H, xs::kRtTokens, xs::kBlockK))
        return rc;
    if (int rc = make_tmap_2d(&t_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rw, E, H, n, xs::kBlockK))
        return rc;
    int32_t *status = reinterpret_cast<int32_t *>(status_block);
    float *wnorm = reinterpret_cast<float *>(status_block + kOffWnorm);
    unsigned long long *counters = reinterpret_cast<unsigned long long *>(status_block + kOffRefineCounters);
    const __nv_bfloat16 *xb = static_cast<const __nv_bfloat16 *>(x), *rwb = static_cast<const __nv_bfloat16 *>(rw);
    XS_CUDA(cudaMemsetAsync(wnorm, 0, sizeof(float), st));
    xs::router_wnorm_kernel<<<(E + 7) / 8, 256, 0, st>>>(rwb, E, H, wnorm);
    note_launch();
    dim3 grid((T + xs::kRtTokens - 1) / xs::kRtTokens, (E + xs::kRtMaxN - 1) / xs::kRtMaxN);
    // few tiles: split the hidden dimension over up to kRtMaxSplits CTAs per tile (partial sums added into zeroed logits)
    int splits = 1;
    while (splits < xs::kRtMaxSplits && static_cast<int>(grid.x * grid.y) * splits * 2 <= di.sms && (H / xs::kBlockK) % (splits * 2) == 0)
        splits *= 2;
    grid.z = splits;
    if (splits > 1)
        XS_CUDA(cudaMemsetAsync(logits, 0, static_cast<size_t>(T) * E * sizeof(float), st));
    xs::router_logits_tc_kernel<<<grid, xs::kRtThreads, smem, st>>>(t_x, t_w, logits, T, H, E, n, status, stages);
    note_launch();
    const int blocks = (T + xs::kRcWarps - 1) / xs::kRcWarps;
    const float coeff = xs::router_delta_coeff(H);
    if (E <= 32)
        xs::router_candidates_kernel<1><<<blocks, xs::kRcWarps * 32, 0, st>>>(xb, bias, logits, wnorm, cand, cand_meta, T, H, E, K, coeff);
    else if (E <= 256)
        xs::router_candidates_kernel<8><<<blocks, xs::kRcWarps * 32, 0, st>>>(xb, bias, logits, wnorm, cand, cand_meta, T, H, E, K, coeff);
    else
        xs::router_candidates_kernel<32><<<blocks, xs::kRcWarps * 32, 0, st>>>(xb, bias, logits, wnorm, cand, cand_meta, T, H, E, K, coeff);
    note_launch();
    if (E <= xs::kRxMaxExperts) {
        // a block's time is set by walking H once and by its chains' shared-memory reads: spread the tokens over the SMs
        int tpb = ((T + di.sms - 1) / di.sms + 7) / 8 * 8;
        tpb = tpb < 8 ? 8 : (tpb > xs::kRxTokens ? xs::kRxTokens : tpb);
        xs::router_exact_slices_kernel<<<(T + tpb - 1) / tpb, xs::kRxThreads, xs::kRxSmemBytes, st>>>(xb, rwb, logits, cand, cand_meta, T, H, E,
                                                                                                  counters, tpb);
    }
    else
        xs::router_exact_rows_kernel<<<T, 32, xs::kReSmemBytes, st>>>(xb, rwb, logits, cand, cand_meta, T, H, E, counters, status);
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

// filter_ws: head of a workspace (status block) if the caller only needs what the SELECTION reads to be exact -- large
// batches then take the tensor-core filter + exact refine path; null: every logit exact (the CUDA-core kernels).
int launch_logits(const XsMoeConfig *c, const void *x, const void *rw, float *logits, cudaStream_t st, const float *bias = nullptr,
                  uint8_t *filter_ws = nullptr)
{
    const int T = c->num_tokens, H = c->hidden, E = c->num_experts;
    if (T == 0)
        return 0;
    if (filter_ws && T > kRouterFilterTokens && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(rw)) % 16 == 0) {
        const ForwardPlan p = plan_forward(c);
        return launch_logits_filtered(c, x, rw, bias, logits, filter_ws, reinterpret_cast<int32_t *>(filter_ws + p.off_cand),
                                      reinterpret_cast<int32_t *>(filter_ws + p.off_cand_meta), st);
    }
    const __nv_bfloat16 *xb = static_cast<const __nv_bfloat16 *>(x), *rwb = static_cast<const __nv_bfloat16 *>(rw);
    if (T <= kRouterSmallTokens) {
        // a few tokens per SM at most: a feeder warp and a chain warp per block, lane = expert, one token per block
        static bool configured_rs[64] = {};
        int dev_rs = 0;
        XS_CUDA(cudaGetDevice(&dev_rs));
        if (dev_rs >= 64 || !configured_rs[dev_rs]) {
            XS_CUDA(cudaFuncSetAttribute(xs::router_logits_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, xs::rs_smem_bytes()));
            if (dev_rs < 64)
                configured_rs[dev_rs] = true;
        }
        XS_CUDA(launch_pdl(xs::router_logits_small_kernel, dim3((E + 31) / 32, T), xs::kRsThreads, xs::rs_smem_bytes(), st, xb, rwb, logits, T, H, E));
        note_launch();
    } else if (T <= 1024) {
        // decode-sized batch: one output per thread, 8 experts x 32 tokens per block, cp.async pipeline
        dim3 grid((E + xs::kRdExperts - 1) / xs::kRdExperts, (T + xs::kRdTokens - 1) / xs::kRdTokens);
        static bool configured_rd[64] = {};
        int dev_rd = 0;
        XS_CUDA(cudaGetDevice(&dev_rd));
        if (dev_rd >= 64 || !configured_rd[dev_rd]) {
            XS_CUDA(cudaFuncSetAttribute(xs::router_logits_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, xs::kRdSmemBytes));
            if (dev_rd < 64)
                configured_rd[dev_rd] = true;
        }
        XS_CUDA(launch_pdl(xs::router_logits_decode_kernel, grid, xs::kRdThreads, xs::kRdSmemBytes, st, xb, rwb, logits, T, H, E));
        note_launch();
    } else {
        static bool configured[64] = {};
        int dev = 0;
        XS_CUDA(cudaGetDevice(&dev));
        if (dev >= 64 || !configured[dev]) {
            XS_CUDA(cudaFuncSetAttribute(xs::router_logits_big_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, xs::rb_smem_bytes<4>()));
            XS_CUDA(cudaFuncSetAttribute(xs::router_logits_mid_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, xs::rm_smem_bytes<2>()));
            if (dev < 64)
                configured[dev] = true;
        }
        const int eg = (E + xs::kRbExperts - 1) / xs::kRbExperts;
        if (static_cast<long>(eg) * ((T + 63) / 64) >= 256) {
            xs::router_logits_big_kernel<4><<<dim3(eg, (T + 63) / 64), xs::kRbThreads, xs::rb_smem_bytes<4>(), st>>>(xb, rwb, logits, T, H, E);
            note_launch();
        } else { // 32-token tiles keep more SMs busy on medium batches
            xs::router_logits_mid_kernel<2><<<dim3(eg, (T + 31) / 32), xs::kRbThreads, xs::rm_smem_bytes<2>(), st>>>(xb, rwb, logits, T, H, E);
            note_launch();
        }
    }
    XS_CUDA(cudaGetLastError());
    return 0;
}

int launch_topk(const XsMoeConfig *c, const float *logits, const float *bias, int32_t *ids, float *w, cudaStream_t st)
{
    const int T = c->num_tokens, E = c->num_experts, K = c->top_k;
    if (T == 0)
        return 0;
    const int blocks = (T + 3) / 4;
    if (E <= 32) {
        XS_CUDA(launch_pdl(xs::topk_kernel<1>, blocks, 128, 0, st, logits, bias, ids, w, T, E, K));
        note_launch();
    } else if (E <= 256) {
        XS_CUDA(launch_pdl(xs::topk_kernel<8>, blocks, 128, 0, st, logits, bias, ids, w, T, E, K));
        note_launch();
    } else {
        XS_CUDA(launch_pdl(xs::topk_kernel<32>, blocks, 128, 0, st, logits, bias, ids, w, T, E, K));
        note_launch();
    }
    XS_CUDA(cudaGetLastError());
    return 0;
}

int launch_route(const XsMoeConfig *c, const void *x, const void *rw, const float *bias, float *logits, int32_t *ids, float *w,
                 cudaStream_t st, uint8_t *filter_ws = nullptr)
{
    if (int rc = launch_logits(c, x, rw, logits, st, bias, filter_ws))
        return rc;
    return launch_topk(c, logits, bias, ids, w, st);
}

// extra_rows >= 0: the always-on expert's rows follow the routed rows and offsets gets one more entry, offsets[E+1]
int launch_permute(const XsMoeConfig *c, const int32_t *ids, int32_t *counts, int32_t *offsets, int32_t *perm, int32_t *inv,
                   int32_t *chunk_counts, int32_t *chunk_base, int chunks, int32_t *status, cudaStream_t st, int extra_rows = -1)
{
    const int T = c->num_tokens, E = c->num_experts, K = c->top_k;
    const size_t smem = static_cast<size_t>(E) * xs::kChunkWords * 4;
    xs::permute_count_kernel<<<chunks, xs::kChunkTokens, smem, st>>>(ids, chunk_counts, T, E, K, status);
    note_launch();
    XS_CUDA(cudaGetLastError());
    const int threads = (E + 31) / 32 * 32;
    xs::permute_scan_kernel<<<1, threads, 0, st>>>(chunk_counts, counts, offsets, chunk_base, chunks, E, extra_rows);
    note_launch();
    XS_CUDA(cudaGetLastError());
    xs::permute_fill_kernel<<<chunks, xs::kChunkTokens, smem, st>>>(ids, chunk_base, perm, inv, T, E, K, status);
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

struct TileBuffers {
    int32_t *tile_expert, *tile_row0, *num_tiles;
};

TileBuffers tile_buffers(uint8_t *scratch, const GroupedPlan &gp)
{
    return {reinterpret_cast<int32_t *>(scratch + gp.off_tile_expert), reinterpret_cast<int32_t *>(scratch + gp.off_tile_row0),
            reinterpret_cast<int32_t *>(scratch + gp.off_num_tiles)};
}

// Permutation + tile table for a decode-sized batch in one launch (T <= 256).
int launch_permute_small(const XsMoeConfig *c, const int32_t *ids, int32_t *counts, int32_t *offsets, int32_t *perm, int32_t *inv,
                         int extra_rows, const GroupedPlan &gp, TileBuffers tb, int32_t *status, cudaStream_t st)
{
    const int T = c->num_tokens, E = c->num_experts, K = c->top_k;
    const size_t smem = static_cast<size_t>(E) * xs::kChunkWords * 4 + static_cast<size_t>(E) * 4;
    XS_CUDA(launch_pdl(xs::permute_small_kernel, 1, xs::kChunkTokens, smem, st, ids, counts, offsets, perm, inv, T, E, K, extra_rows,
                       gp.n_tile, gp.max_tiles, tb.tile_expert, tb.tile_row0, tb.num_tiles, status));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

template <int N_TILE, bool GATE_UP>
int launch_gemm_t(const CUtensorMap &tw, const CUtensorMap &tw2, const CUtensorMap &tx, const int32_t *offsets, xs::TileTable tt,
                  int groups, int w_rows, int n_out, int K, void *out, int32_t *status, int max_work, cudaStream_t st)
{
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    const int stage_bytes = xs::gemm_stage_bytes(N_TILE, GATE_UP);
    int stages = (di.max_smem - 1024 - 256) / stage_bytes;
    if (stages > 8)
        stages = 8;
    if (stages < 2)
        return fail(XS_MOE_ERR_DEVICE, "not enough shared memory for the GEMM pipeline");
    const int smem = stages * stage_bytes + 1024 + 256;
    auto kern = xs::grouped_gemm_bf16_kernel<N_TILE, GATE_UP>;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev < 64)
            configured[dev] = true;
    }
    int grid = di.sms < max_work ? di.sms : max_work;
    if (grid < 1)
        grid = 1;
    XS_CUDA(launch_pdl(kern, grid, xs::kGemmThreads, smem, st, tw, tw2, tx, offsets, tt, groups, w_rows, n_out, K, out, status, stages));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

template <bool GATE_UP>
int launch_gemm(int n_tile, const CUtensorMap &tw, const CUtensorMap &tw2, const CUtensorMap &tx, const int32_t *offsets,
                xs::TileTable tt, int groups, int w_rows, int n_out, int K, void *out, int32_t *status, int max_work, cudaStream_t st)
{
    switch (n_tile) {
    case 16: return launch_gemm_t<16, GATE_UP>(tw, tw2, tx, offsets, tt, groups, w_rows, n_out, K, out, status, max_work, st);
    case 32: return launch_gemm_t<32, GATE_UP>(tw, tw2, tx, offsets, tt, groups, w_rows, n_out, K, out, status, max_work, st);
    case 64: return launch_gemm_t<64, GATE_UP>(tw, tw2, tx, offsets, tt, groups, w_rows, n_out, K, out, status, max_work, st);
    case 128: return launch_gemm_t<128, GATE_UP>(tw, tw2, tx, offsets, tt, groups, w_rows, n_out, K, out, status, max_work, st);
    }
    return fail(XS_MOE_ERR_INVALID_ARG, "internal: bad token tile %d", n_tile);
}

constexpr int kFp8TailBytes = 3072; // barriers (256) + amax exchange (2 x 4 x 64 floats)

template <int N_TILE, bool GATE_UP>
int launch_gemm_fp8_t(const CUtensorMap &tw, const CUtensorMap &tw2, const CUtensorMap &tx, const int32_t *offsets, xs::TileTable tt,
                      xs::Fp8Scales sc, int groups, int w_rows, int n_out, int K, void *out, int32_t *status, int max_work,
                      cudaStream_t st)
{
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    const int stage_bytes = (GATE_UP ? 2 : 1) * xs::kTileM * xs::kBlockK8 + N_TILE * xs::kBlockK8;
    int stages = (di.max_smem - 1024 - kFp8TailBytes) / stage_bytes;
    if (stages > 8)
        stages = 8;
    if (stages < 2)
        return fail(XS_MOE_ERR_DEVICE, "not enough shared memory for the GEMM pipeline");
    const int smem = stages * stage_bytes + 1024 + kFp8TailBytes;
    auto kern = xs::grouped_gemm_fp8_kernel<N_TILE, GATE_UP>;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev < 64)
            configured[dev] = true;
    }
    int grid = di.sms < max_work ? di.sms : max_work;
    if (grid < 1)
        grid = 1;
    XS_CUDA(launch_pdl(kern, grid, xs::kGemmThreads, smem, st, tw, tw2, tx, offsets, tt, sc, groups, w_rows, n_out, K, out, status, stages));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

template <bool GATE_UP>
int launch_gemm_fp8(int n_tile, const CUtensorMap &tw, const CUtensorMap &tw2, const CUtensorMap &tx, const int32_t *offsets,
                    xs::TileTable tt, xs::Fp8Scales sc, int groups, int w_rows, int n_out, int K, void *out, int32_t *status,
                    int max_work, cudaStream_t st)
{
    switch (n_tile) {
    case 16: return launch_gemm_fp8_t<16, GATE_UP>(tw, tw2, tx, offsets, tt, sc, groups, w_rows, n_out, K, out, status, max_work, st);
    case 32: return launch_gemm_fp8_t<32, GATE_UP>(tw, tw2, tx, offsets, tt, sc, groups, w_rows, n_out, K, out, status, max_work, st);
    case 64: return launch_gemm_fp8_t<64, GATE_UP>(tw, tw2, tx, offsets, tt, sc, groups, w_rows, n_out, K, out, status, max_work, st);
    }
    return fail(XS_MOE_ERR_INVALID_ARG, "internal: bad token tile %d for FP8", n_tile);
}

template <bool GATE_UP>
int launch_prefill_fp8(const CUtensorMap &tw, const CUtensorMap &tw2, const CUtensorMap &tx, const int32_t *offsets, xs::TileTable tt,
                       xs::Fp8Scales sc, int groups, int w_rows, int n_out, int K, void *out, int32_t *status, int max_work,
                       cudaStream_t st, int y_bf16 = 0)
{
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    int stages = (di.max_smem - 1024 - xs::kPfTailBytes) / xs::kPfStageBytes;
    if (stages > 6)
        stages = 6;
    if (stages < 2)
        return fail(XS_MOE_ERR_DEVICE, "not enough shared memory for the GEMM pipeline");
    const int smem = stages * xs::kPfStageBytes + 1024 + xs::kPfTailBytes;
    auto kern = xs::prefill_gemm_fp8_kernel<GATE_UP>;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev < 64)
            configured[dev] = true;
    }
    int grid = di.sms < max_work ? di.sms : max_work;
    if (grid < 1)
        grid = 1;
    XS_CUDA(launch_pdl(kern, grid, xs::kPfThreads, smem, st, tw, tw2, tx, offsets, tt, sc, groups, w_rows, n_out, K, out, status, stages, y_bf16));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

constexpr int kFp4TailBytes = 512 + 8 * xs::kFp4SfBytesPerStage; // barriers + per-stage scale blocks

template <int N_TILE, bool GATE_UP>
int launch_gemm_fp4_t(const CUtensorMap &tw, const CUtensorMap &tx, const int32_t *offsets, xs::TileTable tt, xs::MxScales sc, int w_rows,
                      int n_out, int K, void *out, int32_t *status, int max_work, cudaStream_t st)
{
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    const int stage_bytes = (GATE_UP ? 2 : 1) * xs::kTileM * xs::kBlockK8 + N_TILE * xs::kBlockK8;
    int stages = (di.max_smem - 1024 - kFp4TailBytes) / stage_bytes;
    if (stages > 8)
        stages = 8;
    if (stages < 2)
        return fail(XS_MOE_ERR_DEVICE, "not enough shared memory for the GEMM pipeline");
    const int smem = stages * stage_bytes + 1024 + kFp4TailBytes;
    auto kern = xs::grouped_gemm_fp4_kernel<N_TILE, GATE_UP>;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev < 64)
            configured[dev] = true;
    }
    int grid = di.sms < max_work ? di.sms : max_work;
    if (grid < 1)
        grid = 1;
    XS_CUDA(launch_pdl(kern, grid, xs::kFp4Threads, smem, st, tw, tx, offsets, tt, sc, w_rows, n_out, K, out, status, stages));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

template <bool GATE_UP>
int launch_gemm_fp4(int n_tile, const CUtensorMap &tw, const CUtensorMap &tx, const int32_t *offsets, xs::TileTable tt, xs::MxScales sc,
                    int w_rows, int n_out, int K, void *out, int32_t *status, int max_work, cudaStream_t st)
{
    switch (n_tile) {
    case 16: return launch_gemm_fp4_t<16, GATE_UP>(tw, tx, offsets, tt, sc, w_rows, n_out, K, out, status, max_work, st);
    case 32: return launch_gemm_fp4_t<32, GATE_UP>(tw, tx, offsets, tt, sc, w_rows, n_out, K, out, status, max_work, st);
    case 64: return launch_gemm_fp4_t<64, GATE_UP>(tw, tx, offsets, tt, sc, w_rows, n_out, K, out, status, max_work, st);
    }
    return fail(XS_MOE_ERR_INVALID_ARG, "internal: bad token tile %d for FP4", n_tile);
}

// w_scale_rows: rows of the weight-scale matrix (all local experts).  tile_rows: 32 or 128, the token rows of a tile (and of
// the token box of tx).
template <bool GATE_UP>
int launch_prefill_fp4(const CUtensorMap &tw, const CUtensorMap &tx, const int32_t *offsets, xs::TileTable tt, xs::MxScales sc, int w_rows,
                       uint64_t w_scale_rows, int n_out, int K, void *out, int32_t *status, int max_work, int tile_rows, cudaStream_t st,
                       const xs::EpReturnArgs &ret = xs::EpReturnArgs{})
{
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    // scales through the TMA unit where the shapes allow: 16 bytes (four k-blocks) per row and request
    const int kbs = K / 32;
    CUtensorMap t_ws{}, t_xs{};
    int sf_tma = 0;
    if (kbs % 16 == 0 && (K / xs::kBlockK8) % 4 == 0 && reinterpret_cast<uintptr_t>(sc.w_scale) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(sc.x_scale) % 16 == 0) {
        if (int rc = make_tmap_bytes(&t_ws, sc.w_scale, w_scale_rows, kbs, 128, 16))
            return rc;
        if (int rc = make_tmap_bytes(&t_xs, sc.x_scale, sc.max_rows, kbs, 128, 16))
            return rc;
        sf_tma = 1;
    }
    int stages = (di.max_smem - 1024 - xs::kPf4TailBytes) / xs::kPfStageBytes;
    if (stages > 6)
        stages = 6;
    if (stages < 2)
        return fail(XS_MOE_ERR_DEVICE, "not enough shared memory for the GEMM pipeline");
    const int smem = stages * xs::kPfStageBytes + 1024 + xs::kPf4TailBytes;
    auto kern = xs::prefill_gemm_fp4_kernel<GATE_UP>;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev < 64)
            configured[dev] = true;
    }
    int grid = di.sms < max_work ? di.sms : max_work;
    if (grid < 1)
        grid = 1;
    XS_CUDA(launch_pdl(kern, grid, xs::kPf4Threads, smem, st, tw, tx, t_ws, t_xs, offsets, tt, sc, w_rows, n_out, K, out, status, stages, tile_rows,
                       sf_tma, ret));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

// Packed e2m1 matrix (rows, K elements = K/2 bytes per row): the TMA unit expands each 16 codes (8 bytes) to a 16-byte
// shared-memory piece, the form the f8f6f4 MMA kinds read.  Box = 128 elements x box_rows, 128-byte swizzle.
int make_tmap_fp4(CUtensorMap *m, const void *base, uint64_t rows, uint64_t k_elems, uint32_t box_rows)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn)
        return fail(XS_MOE_ERR_CUDA, "CUDA error: cuTensorMapEncodeTiled entry point not available");
    if (reinterpret_cast<uintptr_t>(base) % 32 != 0 || (k_elems / 2) % 32 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "packed FP4 operand must be 32-byte aligned with a 32-byte multiple row pitch");
    cuuint64_t dims[2] = {k_elems, rows};
    cuuint64_t strides[1] = {k_elems / 2};
    cuuint32_t box[2] = {128, box_rows};
    CUresult r = encode_2d_cached(fn, m, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (r != CUDA_SUCCESS)
        return fail(XS_MOE_ERR_CUDA, "CUDA error: cuTensorMapEncodeTiled (packed FP4) failed with code %d (rows=%llu k=%llu)", (int)r,
                    (unsigned long long)rows, (unsigned long long)k_elems);
    return 0;
}

// One grouped SwiGLU MLP over rows grouped by expert segment.  Segments 0..groups-1 use the stacked weights
// (gu, dw); if gu2 is given, segment `groups` (the always-on expert's rows) uses (gu2, dw2) in the SAME launches, so
// its tiles are load-balanced with the routed ones instead of running on a handful of SMs by themselves.
struct GroupedArgs {
    int fmt = XS_MOE_BF16, H = 0, I = 0, groups = 0, gemm_impl = 0;
    const void *gu = nullptr, *gu_scale = nullptr, *dw = nullptr, *dw_scale = nullptr;
    const void *gu2 = nullptr, *gu2_scale = nullptr, *dw2 = nullptr, *dw2_scale = nullptr;
    const void *rows = nullptr;
    const float *row_scale = nullptr;
    const int32_t *offsets = nullptr; // groups + 1 (+ 1 with gu2) entries
    int max_rows = 0;
    float *y = nullptr;
    uint8_t *scratch = nullptr;
    GroupedPlan gp;
    int32_t *status = nullptr;
    bool tiles_ready = false; // the tile table was already built (fused routing kernel)
    xs::EpReturnArgs ret;     // expert-parallel return folded into the down epilogue (kernels that support it)
    bool y_bf16 = false;      // y receives bf16 rows (only honoured by the tokens-as-M FP8 / FP4 kernels: see grouped_writes_bf16)
};

// The quantised tokens-as-M kernels can hand their result rows to the layer's combine as bf16 (half the bytes written and
// read back; the extra rounding is what the expert-parallel wire already applies to these formats).  Which problems they serve:
bool grouped_writes_bf16(int fmt, int H, const GroupedPlan &gp, int gemm_impl)
{
    if (gemm_impl != 0 || H % 256 != 0)
        return false;
    if (fmt == XS_MOE_FP8_BLOCK128)
        return gp.n_tile == 128;
    if (fmt == XS_MOE_FP4_MX32)
        return gp.n_tile == 128 || gp.n_tile == 32;
    return false;
}

// does run_grouped take the tokens-as-M FP4 kernels for this problem (the ones whose down epilogue can store to peers)?
bool grouped_supports_fused_return(int fmt, int H, int I, const GroupedPlan &gp)
{
    return fmt == XS_MOE_FP4_MX32 && H % 256 == 0 && I % 128 == 0 && (gp.n_tile == 128 || gp.n_tile == 32);
}

int run_grouped(const GroupedArgs &a, cudaStream_t st, cudaEvent_t mid = nullptr)
{
    if (a.max_rows == 0) {
        if (mid)
            XS_CUDA(cudaEventRecord(mid, st));
        return 0;
    }
    const int H = a.H, I = a.I, groups = a.groups;
    const int segments = groups + (a.gu2 ? 1 : 0);
    const bool fp8 = a.fmt == XS_MOE_FP8_BLOCK128, fp4 = a.fmt == XS_MOE_FP4_MX32;
    if (fp4 && (a.gu2 || !a.gu_scale || !a.dw_scale || !a.row_scale))
        return fail(XS_MOE_ERR_INVALID_ARG, "missing scale");
    if (fp8 && (!a.gu_scale || !a.dw_scale || !a.row_scale || (a.gu2 && (!a.gu2_scale || !a.dw2_scale))))
        return fail(XS_MOE_ERR_INVALID_ARG, "missing scale");
    void *act = a.scratch + a.gp.off_act;
    if (a.gemm_impl == 1) {
        dim3 grid(a.max_rows, 8);
        const __nv_bfloat16 *rows = static_cast<const __nv_bfloat16 *>(a.rows);
        xs::grouped_gemm_bf16_simt_kernel<true><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(a.gu), rows, a.offsets, groups,
                                                                      2 * I, I, H, act);
        note_launch();
        if (a.gu2) {
            xs::grouped_gemm_bf16_simt_kernel<true><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(a.gu2), rows,
                                                                          a.offsets + groups, 1, 2 * I, I, H, act);
            note_launch();
        }
        XS_CUDA(cudaGetLastError());
        if (mid)
            XS_CUDA(cudaEventRecord(mid, st));
        const __nv_bfloat16 *actb = static_cast<const __nv_bfloat16 *>(act);
        xs::grouped_gemm_bf16_simt_kernel<false><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(a.dw), actb, a.offsets, groups,
                                                                       H, H, I, a.y);
        note_launch();
        if (a.gu2) {
            xs::grouped_gemm_bf16_simt_kernel<false><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(a.dw2), actb,
                                                                           a.offsets + groups, 1, H, H, I, a.y);
            note_launch();
        }
        XS_CUDA(cudaGetLastError());
        return 0;
    }
    TileBuffers tb = tile_buffers(a.scratch, a.gp);
    xs::TileTable tt{tb.tile_expert, tb.tile_row0, tb.num_tiles};
    // The GEMM kernels read segment bounds from `offs`: the caller's offsets clamped to the capacity of the row buffers
    // (a fused routing kernel that already built the tile table produced consistent offsets itself).
    const int32_t *offs = a.offsets;
    if (!a.tiles_ready) {
        const int threads = (segments + 31) / 32 * 32;
        if (threads > 1024)
            return fail(XS_MOE_ERR_UNSUPPORTED, "expert count mismatch: at most 1023 local experts next to an always-on expert");
        int32_t *clamped = reinterpret_cast<int32_t *>(a.scratch + a.gp.off_offsets);
        xs::tile_table_kernel<<<1, threads, 0, st>>>(a.offsets, segments, a.gp.n_tile, a.gp.max_tiles, a.max_rows, clamped, tb.tile_expert,
                                                     tb.tile_row0, tb.num_tiles, a.status);
        note_launch();
        XS_CUDA(cudaGetLastError());
        offs = clamped;
    }
    if (fp4) {
        CUtensorMap t_wgu, t_wd, t_x, t_act;
        if (int rc = make_tmap_fp4(&t_wgu, a.gu, static_cast<uint64_t>(groups) * 2 * I, H, xs::kTileM))
            return rc;
        if (int rc = make_tmap_fp4(&t_wd, a.dw, static_cast<uint64_t>(groups) * H, I, xs::kTileM))
            return rc;
        if (int rc = make_tmap_2d(&t_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.rows, a.max_rows, H, a.gp.n_tile, xs::kBlockK8))
            return rc;
        if (int rc = make_tmap_2d(&t_act, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, act, a.max_rows, I, a.gp.n_tile, xs::kBlockK8))
            return rc;
        uint8_t *act_scale = a.scratch + a.gp.off_act_scale;
        if (H % 256 == 0 && (a.gp.n_tile == 128 || a.gp.n_tile == 32)) {
            // tokens as the M of N = 256 block-scaled MMAs (token box of 32 or 128 rows)
            xs::MxScales p1{static_cast<const uint8_t *>(a.gu_scale), reinterpret_cast<const uint8_t *>(a.row_scale), act_scale, a.max_rows};
            if (int rc = launch_prefill_fp4<true>(t_wgu, t_x, offs, tt, p1, 2 * I, static_cast<uint64_t>(groups) * 2 * I, I, H, act, a.status,
                                                  a.gp.max_tiles * (I / 128), a.gp.n_tile, st))
                return rc;
            if (mid)
                XS_CUDA(cudaEventRecord(mid, st));
            xs::MxScales p2{static_cast<const uint8_t *>(a.dw_scale), act_scale, nullptr, a.max_rows};
            xs::EpReturnArgs ret = a.ret;
            ret.y_bf16 = a.y_bf16 ? 1 : 0;
            return launch_prefill_fp4<false>(t_wd, t_act, offs, tt, p2, H, static_cast<uint64_t>(groups) * H, H, I, a.y, a.status,
                                             a.gp.max_tiles * (H / 256), a.gp.n_tile, st, ret);
        }
        if (a.ret.peer_back)
            return fail(XS_MOE_ERR_UNSUPPORTED, "the fused expert-parallel return needs the tokens-as-M FP4 kernels (hidden % 256 == 0)");
        xs::MxScales s1{static_cast<const uint8_t *>(a.gu_scale), reinterpret_cast<const uint8_t *>(a.row_scale), act_scale, a.max_rows};
        if (int rc = launch_gemm_fp4<true>(a.gp.n_tile, t_wgu, t_x, offs, tt, s1, 2 * I, I, H, act, a.status,
                                           a.gp.max_tiles * (I / xs::kTileM), st))
            return rc;
        if (mid)
            XS_CUDA(cudaEventRecord(mid, st));
        xs::MxScales s2{static_cast<const uint8_t *>(a.dw_scale), act_scale, nullptr, a.max_rows};
        return launch_gemm_fp4<false>(a.gp.n_tile, t_wd, t_act, offs, tt, s2, H, H, I, a.y, a.status,
                                      a.gp.max_tiles * (H / xs::kTileM), st);
    }
    if (a.ret.peer_back)
        return fail(XS_MOE_ERR_UNSUPPORTED, "the fused expert-parallel return is implemented for FP4 experts");
    const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int eb = fp8 ? 1 : 2;
    const uint32_t box_k = fp8 ? xs::kBlockK8 : xs::kBlockK;
    CUtensorMap t_wgu, t_wd, t_wgu2, t_wd2, t_x, t_act;
    if (int rc = make_tmap_2d(&t_wgu, dt, eb, a.gu, static_cast<uint64_t>(groups) * 2 * I, H, xs::kTileM, box_k))
        return rc;
    if (int rc = make_tmap_2d(&t_wd, dt, eb, a.dw, static_cast<uint64_t>(groups) * H, I, xs::kTileM, box_k))
        return rc;
    if (a.gu2) {
        if (int rc = make_tmap_2d(&t_wgu2, dt, eb, a.gu2, 2 * I, H, xs::kTileM, box_k))
            return rc;
        if (int rc = make_tmap_2d(&t_wd2, dt, eb, a.dw2, H, I, xs::kTileM, box_k))
            return rc;
    } else {
        t_wgu2 = t_wgu;
        t_wd2 = t_wd;
    }
    if (int rc = make_tmap_2d(&t_x, dt, eb, a.rows, a.max_rows, H, a.gp.n_tile, box_k))
        return rc;
    if (int rc = make_tmap_2d(&t_act, dt, eb, act, a.max_rows, I, a.gp.n_tile, box_k))
        return rc;
    const int work_gu = a.gp.max_tiles * (I / xs::kTileM), work_d = a.gp.max_tiles * (H / xs::kTileM);
    if (!fp8) {
        if (int rc = launch_gemm<true>(a.gp.n_tile, t_wgu, t_wgu2, t_x, offs, tt, groups, 2 * I, I, H, act, a.status, work_gu, st))
            return rc;
        if (mid)
            XS_CUDA(cudaEventRecord(mid, st));
        return launch_gemm<false>(a.gp.n_tile, t_wd, t_wd2, t_act, offs, tt, groups, H, H, I, a.y, a.status, work_d, st);
    }
    float *act_scale = reinterpret_cast<float *>(a.scratch + a.gp.off_act_scale);
    if (a.gp.n_tile == 128) {
        // many tokens per expert: tokens as the M of N = 256 MMAs (prefill kernel); the maps above already use 128-row boxes
        xs::Fp8Scales p1{static_cast<const float *>(a.gu_scale), static_cast<const float *>(a.gu2_scale), a.row_scale, act_scale, a.max_rows};
        if (int rc = launch_prefill_fp8<true>(t_wgu, t_wgu2, t_x, offs, tt, p1, groups, 2 * I, I, H, act, a.status,
                                              a.gp.max_tiles * (I / 128), st))
            return rc;
        if (mid)
            XS_CUDA(cudaEventRecord(mid, st));
        xs::Fp8Scales p2{static_cast<const float *>(a.dw_scale), static_cast<const float *>(a.dw2_scale), act_scale, nullptr, a.max_rows};
        return launch_prefill_fp8<false>(t_wd, t_wd2, t_act, offs, tt, p2, groups, H, H, I, a.y, a.status,
                                         a.gp.max_tiles * (H / 256), st, a.y_bf16 ? 1 : 0);
    }
    xs::Fp8Scales s1{static_cast<const float *>(a.gu_scale), static_cast<const float *>(a.gu2_scale), a.row_scale, act_scale, a.max_rows};
    if (int rc = launch_gemm_fp8<true>(a.gp.n_tile, t_wgu, t_wgu2, t_x, offs, tt, s1, groups, 2 * I, I, H, act, a.status, work_gu, st))
        return rc;
    if (mid)
        XS_CUDA(cudaEventRecord(mid, st));
    xs::Fp8Scales s2{static_cast<const float *>(a.dw_scale), static_cast<const float *>(a.dw2_scale), act_scale, nullptr, a.max_rows};
    return launch_gemm_fp8<false>(a.gp.n_tile, t_wd, t_wd2, t_act, offs, tt, s2, groups, H, H, I, a.y, a.status, work_d, st);
}

__global__ void set_two_ints_kernel(int32_t *p, int a, int b)
{
    p[0] = a;
    p[1] = b;
}

int launch_quantize_rows_mx(const void *x, const int32_t *dst, int nd, uint8_t *q, uint8_t *scale, int rows, int cols, cudaStream_t st)
{
    if (rows == 0)
        return 0;
    XS_CUDA(launch_pdl(xs::quantize_rows_mxfp8_kernel, rows, 256, 0, st, static_cast<const __nv_bfloat16 *>(x), dst, nd, q, scale, rows, cols));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

int launch_quantize_rows(const void *x, uint8_t *q, float *scale, int rows, int cols, cudaStream_t st)
{
    if (rows == 0)
        return 0;
    const long warps = static_cast<long>(rows) * (cols / 128);
    const int blocks = static_cast<int>((warps + 7) / 8);
    XS_CUDA(launch_pdl(xs::quantize_rows_fp8_kernel, blocks, 256, 0, st, static_cast<const __nv_bfloat16 *>(x), q, scale, rows, cols));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

} // namespace

// =========================================================================================================
extern "C" {

const char *xs_moe_status_string(int status)
{
    switch (status) {
    case XS_MOE_OK: return "ok";
    case XS_MOE_ERR_INVALID_ARG: return "invalid argument";
    case XS_MOE_ERR_UNSUPPORTED: return "unsupported";
    case XS_MOE_ERR_WORKSPACE: return "workspace too small or misaligned";
    case XS_MOE_ERR_CUDA: return "CUDA error";
    case XS_MOE_ERR_DEVICE: return "unsupported device";
    case XS_MOE_ERR_KERNEL_TIMEOUT: return "device-side wait timed out";
    }
    return "unknown status";
}

const char *xs_moe_last_error(void)
{
    return g_last_error.c_str();
}

int xs_moe_device_check(void)
{
    DeviceInfo di;
    return device_info(&di);
}

int xs_moe_device_count(int32_t *count)
{
    if (!count)
        return fail(XS_MOE_ERR_INVALID_ARG, "null out-pointer");
    int n = 0;
    XS_CUDA(cudaGetDeviceCount(&n));
    *count = n;
    return 0;
}
int xs_moe_set_device(int32_t device)
{
    XS_CUDA(cudaSetDevice(device));
    return 0;
}
int xs_moe_current_device(int32_t *device)
{
    if (!device)
        return fail(XS_MOE_ERR_INVALID_ARG, "null out-pointer");
    int d = 0;
    XS_CUDA(cudaGetDevice(&d));
    *device = d;
    return 0;
}

int xs_moe_device_alloc(void **ptr, size_t bytes)
{
    if (!ptr)
        return fail(XS_MOE_ERR_INVALID_ARG, "null out-pointer");
    *ptr = nullptr;
    XS_CUDA(cudaMalloc(ptr, bytes ? bytes : 1));
    return 0;
}
int xs_moe_device_free(void *ptr)
{
    XS_CUDA(cudaFree(ptr));
    return 0;
}
int xs_moe_memcpy_h2d(void *dst, const void *src, size_t bytes)
{
    XS_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
    return 0;
}
int xs_moe_memcpy_d2h(void *dst, const void *src, size_t bytes)
{
    XS_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    return 0;
}
int xs_moe_memcpy_d2d(void *dst, const void *src, size_t bytes)
{
    XS_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice));
    return 0;
}
int xs_moe_device_free_bytes(size_t *bytes)
{
    size_t f = 0, t = 0;
    XS_CUDA(cudaMemGetInfo(&f, &t));
    if (bytes)
        *bytes = f;
    return 0;
}
int xs_moe_stream_synchronize(void *stream)
{
    XS_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return 0;
}

int xs_moe_workspace_bytes(const XsMoeConfig *cfg, size_t *bytes)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!bytes)
        return fail(XS_MOE_ERR_INVALID_ARG, "null out-pointer");
    *bytes = plan_forward(cfg).bytes;
    return 0;
}

int xs_moe_route(const XsMoeConfig *cfg, const void *x, const void *rw, const float *bias, float *logits, int32_t *ids, float *w,
                 void *ws, size_t ws_bytes, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!x || !rw || !ids || !w)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    uint8_t *filter_ws = nullptr;
    if (!logits) {
        ForwardPlan p = plan_forward(cfg);
        if (int rc = check_workspace(ws, ws_bytes, p.off_ids))
            return rc;
        logits = reinterpret_cast<float *>(static_cast<uint8_t *>(ws) + p.off_logits);
        filter_ws = static_cast<uint8_t *>(ws); // nobody reads the logits: only what the selection depends on has to be exact
    }
    return launch_route(cfg, x, rw, bias, logits, ids, w, static_cast<cudaStream_t>(stream), filter_ws);
}

int xs_moe_topk(const XsMoeConfig *cfg, const float *logits, const float *bias, int32_t *ids, float *w, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!logits || !ids || !w)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    return launch_topk(cfg, logits, bias, ids, w, static_cast<cudaStream_t>(stream));
}

int xs_moe_permute(const XsMoeConfig *cfg, const int32_t *ids, int32_t *counts, int32_t *offsets, int32_t *perm, int32_t *inv,
                   void *ws, size_t ws_bytes, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!ids || !counts || !offsets || !perm || !inv)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    ForwardPlan p = plan_forward(cfg);
    if (int rc = check_workspace(ws, ws_bytes, p.off_chunk_base + static_cast<size_t>(p.chunks) * cfg->num_experts * 4))
        return rc;
    uint8_t *b = static_cast<uint8_t *>(ws);
    if (cfg->num_tokens > 0 && cfg->num_tokens <= xs::kChunkTokens) // one block does it all (no tile table asked for here)
        return launch_permute_small(cfg, ids, counts, offsets, perm, inv, -1, GroupedPlan{}, TileBuffers{},
                                    reinterpret_cast<int32_t *>(b), static_cast<cudaStream_t>(stream));
    return launch_permute(cfg, ids, counts, offsets, perm, inv, reinterpret_cast<int32_t *>(b + p.off_chunk_counts),
                          reinterpret_cast<int32_t *>(b + p.off_chunk_base), p.chunks, reinterpret_cast<int32_t *>(b),
                          static_cast<cudaStream_t>(stream));
}

static GroupedPlan plan_grouped_stage(const XsMoeConfig *cfg, int max_rows)
{
    // max_rows is a capacity (the expert-parallel buffers are sized for the worst routing); the tile shape follows the rows
    // this rank expects, tokens x top_k, when that is smaller
    const long expect = static_cast<long>(cfg->num_tokens) * cfg->top_k;
    const int rows = expect > 0 && expect < max_rows ? static_cast<int>(expect) : max_rows;
    return plan_grouped(max_rows, rows, cfg->local_expert_count, cfg->local_expert_count, cfg->intermediate, cfg->routed_format,
                        cfg->hidden);
}

int xs_moe_grouped_mlp_workspace_bytes(const XsMoeConfig *cfg, int32_t max_rows, size_t *bytes)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!bytes || max_rows < 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "bad arguments");
    *bytes = kStatusBytes + plan_grouped_stage(cfg, max_rows).bytes;
    return 0;
}

int xs_moe_grouped_mlp(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *rows, const float *row_scales,
                       const int32_t *offsets, int32_t max_rows, float *y, void *ws, size_t ws_bytes, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!w || !rows || !offsets || !y || !w->gate_up_w_dev || !w->down_w_dev)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (max_rows < 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: negative row capacity");
    if (cfg->gemm_impl == 0)
        if (int rc = xs_moe_device_check())
            return rc;
    GroupedArgs a;
    a.gp = plan_grouped_stage(cfg, max_rows);
    if (int rc = check_workspace(ws, ws_bytes, kStatusBytes + a.gp.bytes))
        return rc;
    uint8_t *b = static_cast<uint8_t *>(ws);
    a.fmt = cfg->routed_format;
    a.H = cfg->hidden;
    a.I = cfg->intermediate;
    a.groups = cfg->local_expert_count;
    a.gemm_impl = cfg->gemm_impl;
    a.gu = w->gate_up_w_dev;
    a.gu_scale = w->gate_up_scale_dev;
    a.dw = w->down_w_dev;
    a.dw_scale = w->down_scale_dev;
    a.rows = rows;
    a.row_scale = row_scales;
    a.offsets = offsets;
    a.max_rows = max_rows;
    a.y = y;
    a.scratch = b + kStatusBytes;
    a.status = reinterpret_cast<int32_t *>(b);
    return run_grouped(a, static_cast<cudaStream_t>(stream));
}

static int check_ep(int32_t ranks, int32_t rank, int32_t experts);

int xs_moe_grouped_mlp_return_supported(const XsMoeConfig *cfg, int32_t max_rows, int32_t *supported)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!supported || max_rows < 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "null out-pointer");
    const GroupedPlan gp = plan_grouped_stage(cfg, max_rows);
    *supported = (cfg->gemm_impl == 0 && grouped_supports_fused_return(cfg->routed_format, cfg->hidden, cfg->intermediate, gp)) ? 1 : 0;
    return 0;
}

int xs_moe_grouped_mlp_return(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *rows, const float *row_scales,
                              const int32_t *offsets, int32_t max_rows, int32_t ranks, int32_t rank, const int32_t *all_counts,
                              const int32_t *src_offsets, void *const *peer_back, int32_t back_capacity_rows, void *ws, size_t ws_bytes,
                              void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (int rc = check_ep(ranks, rank, cfg->num_experts))
        return rc;
    if (!w || !rows || !offsets || !all_counts || !src_offsets || !peer_back || !w->gate_up_w_dev || !w->down_w_dev)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (max_rows < 0 || back_capacity_rows < 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: negative row capacity");
    if (cfg->local_expert_count * ranks != cfg->num_experts || cfg->local_expert_begin != rank * cfg->local_expert_count)
        return fail(XS_MOE_ERR_INVALID_ARG, "expert count mismatch: the config's expert slice is not this rank's");
    if (int rc = xs_moe_device_check())
        return rc;
    GroupedArgs a;
    a.gp = plan_grouped_stage(cfg, max_rows);
    if (cfg->gemm_impl != 0 || !grouped_supports_fused_return(cfg->routed_format, cfg->hidden, cfg->intermediate, a.gp))
        return fail(XS_MOE_ERR_UNSUPPORTED, "the fused expert-parallel return is implemented for FP4 experts with hidden % 256 == 0");
    if (int rc = check_workspace(ws, ws_bytes, kStatusBytes + a.gp.bytes))
        return rc;
    uint8_t *b = static_cast<uint8_t *>(ws);
    a.fmt = cfg->routed_format;
    a.H = cfg->hidden;
    a.I = cfg->intermediate;
    a.groups = cfg->local_expert_count;
    a.gu = w->gate_up_w_dev;
    a.gu_scale = w->gate_up_scale_dev;
    a.dw = w->down_w_dev;
    a.dw_scale = w->down_scale_dev;
    a.rows = rows;
    a.row_scale = row_scales;
    a.offsets = offsets;
    a.max_rows = max_rows;
    a.y = nullptr;
    a.scratch = b + kStatusBytes;
    a.status = reinterpret_cast<int32_t *>(b);
    a.ret.peer_back = reinterpret_cast<uint8_t *const *>(peer_back);
    a.ret.all_counts = all_counts;
    a.ret.src_offsets = src_offsets;
    a.ret.experts = cfg->num_experts;
    a.ret.ranks = ranks;
    a.ret.me = rank;
    a.ret.back_capacity = back_capacity_rows;
    return run_grouped(a, static_cast<cudaStream_t>(stream));
}

int xs_moe_quantize_rows_fp8(const void *x, int32_t rows, int32_t cols, void *codes, float *scales, void *stream)
{
    if (!x || !codes || !scales)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (rows < 0 || cols <= 0 || cols % 128 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: columns must be a positive multiple of 128");
    return launch_quantize_rows(x, static_cast<uint8_t *>(codes), scales, rows, cols, static_cast<cudaStream_t>(stream));
}

int xs_moe_quantize_rows_mxfp8(const void *x, int32_t rows, int32_t cols, void *codes, uint8_t *scales, void *stream)
{
    if (!x || !codes || !scales)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (rows < 0 || cols <= 0 || cols % 128 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: columns must be a positive multiple of 128");
    return launch_quantize_rows_mx(x, nullptr, 1, static_cast<uint8_t *>(codes), scales, rows, cols, static_cast<cudaStream_t>(stream));
}

int xs_moe_gather_rows(const void *src, const int32_t *index, void *dst, int32_t n_rows, int32_t row_bytes, void *stream)
{
    if (!src || !index || !dst)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (n_rows < 0 || row_bytes <= 0 || row_bytes % 4 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: row_bytes must be a positive multiple of 4");
    if (n_rows == 0)
        return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
        xs::gather_rows_kernel<<<n_rows, 256, 0, st>>>(static_cast<const uint8_t *>(src), index, static_cast<uint8_t *>(dst), n_rows,
                                                       n_rows, 1, row_bytes);
        note_launch();
    } else {
        xs::gather_rows4_kernel<<<n_rows, 64, 0, st>>>(static_cast<const uint32_t *>(src), index, static_cast<uint32_t *>(dst), n_rows,
                                                       n_rows, 1, row_bytes / 4);
        note_launch();
    }
    XS_CUDA(cudaGetLastError());
    return 0;
}

static int combine_impl(const XsMoeConfig *cfg, const float *y, const int32_t *inv, const float *topk_w, const float *shared, void *out,
                        const void *residual, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!y || !inv || !topk_w || !out)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    const int T = cfg->num_tokens, H = cfg->hidden, K = cfg->top_k;
    if (T == 0)
        return 0;
    int gy = (H + 1023) / 1024;
    XS_CUDA(launch_pdl(xs::combine_kernel<float, float>, dim3(T, gy), 128, 0, static_cast<cudaStream_t>(stream), y, inv, topk_w, shared,
                       static_cast<__nv_bfloat16 *>(out), T, H, K, static_cast<const __nv_bfloat16 *>(residual)));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

// y rows bf16; the always-on expert's rows f32 or bf16
static int combine_bf16_impl(const XsMoeConfig *cfg, const __nv_bfloat16 *y, const int32_t *inv, const float *topk_w, const void *shared,
                             bool shared_is_bf16, void *out, const void *residual, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!y || !inv || !topk_w || !out)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    const int T = cfg->num_tokens, H = cfg->hidden, K = cfg->top_k;
    if (T == 0)
        return 0;
    const dim3 grid(T, (H + 1023) / 1024);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(out);
    const __nv_bfloat16 *res = static_cast<const __nv_bfloat16 *>(residual);
    if (shared_is_bf16)
        XS_CUDA(launch_pdl(xs::combine_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 128, 0, st, y, inv, topk_w, static_cast<const __nv_bfloat16 *>(shared), o, T,
                           H, K, res));
    else
        XS_CUDA(launch_pdl(xs::combine_kernel<__nv_bfloat16, float>, grid, 128, 0, st, y, inv, topk_w, static_cast<const float *>(shared), o, T, H, K, res));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

int xs_moe_combine(const XsMoeConfig *cfg, const float *y, const int32_t *inv, const float *topk_w, const float *shared, void *out,
                   void *stream)
{
    return combine_impl(cfg, y, inv, topk_w, shared, out, nullptr, stream);
}

int xs_moe_rmsnorm(const void *x, const void *weight, void *out, int32_t rows, int32_t hidden, float eps, void *stream)
{
    if (!x || !weight || !out)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (rows < 0 || hidden <= 0 || hidden % 8 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: hidden must be a positive multiple of 8");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) % 16 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "tensors must be 16-byte aligned");
    if (rows == 0)
        return 0;
    xs::rmsnorm_rows_kernel<<<(rows + xs::kRnRows - 1) / xs::kRnRows, xs::kRnThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(weight), static_cast<__nv_bfloat16 *>(out), rows, hidden, eps);
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

int xs_moe_combine_bf16_rows(const XsMoeConfig *cfg, const void *y_bf16, const int32_t *inv, const float *topk_w, const float *shared,
                             void *out, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!y_bf16 || !inv || !topk_w || !out)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    const int T = cfg->num_tokens, H = cfg->hidden, K = cfg->top_k;
    if (T == 0)
        return 0;
    int gy = (H + 1023) / 1024;
    xs::combine_kernel<__nv_bfloat16, float><<<dim3(T, gy), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16 *>(y_bf16), inv, topk_w, shared, static_cast<__nv_bfloat16 *>(out), T, H, K);
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

int xs_moe_gather_rows_f32_to_bf16(const float *src, const int32_t *index, void *dst_bf16, int32_t n_rows, int32_t cols, void *stream)
{
    if (!src || !index || !dst_bf16)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (n_rows < 0 || cols <= 0 || cols % 8 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: columns must be a positive multiple of 8");
    if (n_rows == 0)
        return 0;
    xs::gather_rows_f32_to_bf16_kernel<<<n_rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, index, static_cast<__nv_bfloat16 *>(dst_bf16),
                                                                                             n_rows, cols);
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

// A second stream per (device, caller stream) for work of a layer call that does not depend on the routing (the always-on
// expert of an FP4 layer, which runs in its own launches): forked from the caller's stream by an event at the start of the
// call and joined before the combine, so the pair behaves like one stream to the caller -- also under stream capture, where
// the fork and join become graph edges.  Created on first use (outside of a capture: creating streams is not a stream
// operation and may be refused while a global-mode capture is active).
struct SideStream {
    cudaStream_t side = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
static int side_stream_for(cudaStream_t user, SideStream *out)
{
    struct Entry {
        int dev;
        cudaStream_t user;
        SideStream s;
    };
    static std::mutex mu;
    static std::vector<Entry> table;
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry &e : table)
        if (e.dev == dev && e.user == user) {
            *out = e.s;
            return 0;
        }
    if (table.size() >= 256) { // more caller streams than anyone keeps alive: run on the caller's stream
        *out = SideStream{};
        return 0;
    }
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(user, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
        (void)cudaGetLastError();
        *out = SideStream{}; // first use inside a capture: no fork this time
        return 0;
    }
    SideStream s;
    XS_CUDA(cudaStreamCreateWithFlags(&s.side, cudaStreamNonBlocking));
    XS_CUDA(cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming));
    XS_CUDA(cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming));
    table.push_back(Entry{dev, user, s});
    *out = s;
    return 0;
}

// Stage marks of xs_moe_forward_profile: logits | select + permute + tile table | scatter (+ quantise) |
// gate/up GEMM | down GEMM | combine
static int forward_impl(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x, void *out, void *ws, size_t ws_bytes,
                        void *stream, cudaEvent_t *ev, const void *residual = nullptr)
{
#define XS_MARK(i)                                                       \
    do {                                                                 \
        if (ev)                                                          \
            XS_CUDA(cudaEventRecord(ev[i], static_cast<cudaStream_t>(stream))); \
    } while (0)
    if (int rc = check_cfg(cfg))
        return rc;
    if (!w || !x || !out || !w->router_w_dev || !w->gate_up_w_dev || !w->down_w_dev)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (cfg->num_shared && (!w->shared_gate_up_w_dev || !w->shared_down_w_dev))
        return fail(XS_MOE_ERR_INVALID_ARG, "shared expert weights missing");
    if (cfg->local_expert_begin != 0 || cfg->local_expert_count != cfg->num_experts)
        return fail(XS_MOE_ERR_INVALID_ARG, "expert count mismatch: xs_moe_forward needs all experts on this device; "
                                            "sharded layers are composed from the stage calls");
    if (cfg->gemm_impl == 0)
        if (int rc = xs_moe_device_check())
            return rc;
    const ForwardPlan p = plan_forward(cfg);
    if (int rc = check_workspace(ws, ws_bytes, p.bytes))
        return rc;
    const int T = cfg->num_tokens, H = cfg->hidden, E = cfg->num_experts, K = cfg->top_k, I = cfg->intermediate, S = cfg->num_shared;
    if (T == 0)
        return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t *b = static_cast<uint8_t *>(ws);
    int32_t *status = reinterpret_cast<int32_t *>(b);
    float *logits = reinterpret_cast<float *>(b + p.off_logits);
    int32_t *ids = reinterpret_cast<int32_t *>(b + p.off_ids);
    float *tw = reinterpret_cast<float *>(b + p.off_w);
    int32_t *counts = reinterpret_cast<int32_t *>(b + p.off_counts);
    int32_t *offsets = reinterpret_cast<int32_t *>(b + p.off_offsets);
    int32_t *perm = reinterpret_cast<int32_t *>(b + p.off_perm);
    int32_t *inv = reinterpret_cast<int32_t *>(b + p.off_inv);
    uint8_t *rows = b + p.off_rows;
    float *y = reinterpret_cast<float *>(b + p.off_y);
    const int n_routed = T * K, n_total = T * K + S * T;
    const bool fp8 = cfg->routed_format == XS_MOE_FP8_BLOCK128, fp4 = cfg->routed_format == XS_MOE_FP4_MX32;
    float *rows_scale = (fp8 || fp4) ? reinterpret_cast<float *>(b + p.off_rows_scale) : nullptr;
    const int extra_rows = (S && !fp4) ? T : -1; // FP4 experts: the FP8 always-on expert runs in its own launches
    const bool tensor_path = cfg->gemm_impl == 0;
    uint8_t *gscratch = b + p.off_grouped;

    // FP4 experts: the always-on expert is FP8 (128x128 scales) and runs in launches of its own -- quantise x per 1x128, then
    // a one-segment grouped MLP.  None of it depends on the routing, so it goes to the side stream and overlaps the router,
    // the permutation and the scatter.
    SideStream side;
    bool joined = false;
    if (fp4 && S) {
        if (int rc = side_stream_for(st, &side))
            return rc;
        cudaStream_t ss = st;
        if (side.side) {
            XS_CUDA(cudaEventRecord(side.fork, st));
            XS_CUDA(cudaStreamWaitEvent(side.side, side.fork, 0));
            ss = side.side;
            joined = true;
        }
        uint8_t *xq = b + p.off_sh_rows;
        float *xs_ = reinterpret_cast<float *>(b + p.off_sh_scale);
        int32_t *sh_off = reinterpret_cast<int32_t *>(b + p.off_sh_offsets);
        if (int rc = launch_quantize_rows(x, xq, xs_, T, H, ss))
            return rc;
        set_two_ints_kernel<<<1, 1, 0, ss>>>(sh_off, 0, T);
        note_launch();
        XS_CUDA(cudaGetLastError());
        GroupedArgs sa;
        sa.fmt = XS_MOE_FP8_BLOCK128;
        sa.H = H;
        sa.I = I;
        sa.groups = 1;
        sa.gu = w->shared_gate_up_w_dev;
        sa.gu_scale = w->shared_gate_up_scale_dev;
        sa.dw = w->shared_down_w_dev;
        sa.dw_scale = w->shared_down_scale_dev;
        sa.rows = xq;
        sa.row_scale = xs_;
        sa.offsets = sh_off;
        sa.max_rows = T;
        sa.y = y + static_cast<size_t>(n_routed) * H;
        sa.scratch = b + p.off_sh_grouped;
        sa.gp = p.sh_grouped;
        sa.status = status;
        const int rc_sh = run_grouped(sa, ss);
        if (joined) // join even when a launch failed: a capture in progress must not be left forked
            XS_CUDA(cudaEventRecord(side.join, side.side));
        if (rc_sh)
            return rc_sh;
    }

    XS_MARK(0);
    if (int rc = launch_logits(cfg, x, w->router_w_dev, logits, st, w->router_bias_dev, b))
        return rc;
    XS_MARK(1);
    bool tiles_ready = false;
    if (T <= xs::kChunkTokens) {
        TileBuffers tb = tile_buffers(gscratch, p.grouped);
        if (!tensor_path)
            tb = TileBuffers{nullptr, nullptr, nullptr};
        if (int rc = launch_topk(cfg, logits, w->router_bias_dev, ids, tw, st))
            return rc;
        if (int rc = launch_permute_small(cfg, ids, counts, offsets, perm, inv, extra_rows, p.grouped, tb, status, st))
            return rc;
        tiles_ready = tensor_path;
    } else {
        if (int rc = launch_topk(cfg, logits, w->router_bias_dev, ids, tw, st))
            return rc;
        if (int rc = launch_permute(cfg, ids, counts, offsets, perm, inv, reinterpret_cast<int32_t *>(b + p.off_chunk_counts),
                                    reinterpret_cast<int32_t *>(b + p.off_chunk_base), p.chunks, status, st, extra_rows))
            return rc;
    }
    XS_MARK(2);
    if (fp4) {
        if (int rc = launch_quantize_rows_mx(x, inv, K, rows, reinterpret_cast<uint8_t *>(rows_scale), T, H, st))
            return rc;
    } else if (fp8) {
        XS_CUDA(launch_pdl(xs::scatter_rows_kernel<true>, T, 256, 0, st, static_cast<const __nv_bfloat16 *>(x), inv, rows, rows_scale, T, H, K,
                           n_routed, S));
        note_launch();
    } else {
        XS_CUDA(launch_pdl(xs::scatter_rows_kernel<false>, T, 256, 0, st, static_cast<const __nv_bfloat16 *>(x), inv, rows, nullptr, T, H, K,
                           n_routed, S));
        note_launch();
    }
    XS_CUDA(cudaGetLastError());
    XS_MARK(3);
    GroupedArgs a;
    a.fmt = cfg->routed_format;
    a.H = H;
    a.I = I;
    a.groups = E;
    a.gemm_impl = cfg->gemm_impl;
    a.gu = w->gate_up_w_dev;
    a.gu_scale = w->gate_up_scale_dev;
    a.dw = w->down_w_dev;
    a.dw_scale = w->down_scale_dev;
    if (S && !fp4) {
        a.gu2 = w->shared_gate_up_w_dev;
        a.gu2_scale = w->shared_gate_up_scale_dev;
        a.dw2 = w->shared_down_w_dev;
        a.dw2_scale = w->shared_down_scale_dev;
    }
    a.rows = rows;
    a.row_scale = rows_scale;
    a.offsets = offsets;
    a.max_rows = fp4 ? n_routed : n_total;
    a.y = y;
    a.scratch = gscratch;
    a.gp = p.grouped;
    a.status = status;
    a.tiles_ready = tiles_ready;
    // quantised experts on the tokens-as-M kernels: result rows as bf16 (the routed rows; for FP8 also the always-on expert's,
    // which ride in the same launches)
    const bool y_bf16 = grouped_writes_bf16(cfg->routed_format, H, p.grouped, cfg->gemm_impl);
    a.y_bf16 = y_bf16;
    if (int rc = run_grouped(a, st, ev ? ev[4] : nullptr))
        return rc;
    if (joined)
        XS_CUDA(cudaStreamWaitEvent(st, side.join, 0));
    XS_MARK(5);
    if (y_bf16) {
        // FP4: the always-on expert ran in launches of its own and wrote f32 rows at the f32 layout's offset; FP8: its rows are
        // bf16 rows n_routed.. of the same buffer
        const __nv_bfloat16 *yb = reinterpret_cast<const __nv_bfloat16 *>(y);
        const void *sh = !S ? nullptr : (fp4 ? static_cast<const void *>(y + static_cast<size_t>(n_routed) * H)
                                             : static_cast<const void *>(yb + static_cast<size_t>(n_routed) * H));
        if (int rc = combine_bf16_impl(cfg, yb, inv, tw, sh, /*shared_is_bf16=*/!fp4, out, residual, stream))
            return rc;
    } else if (int rc = combine_impl(cfg, y, inv, tw, S ? y + static_cast<size_t>(n_routed) * H : nullptr, out, residual, stream))
        return rc;
    XS_MARK(6);
    return 0;
#undef XS_MARK
}

int xs_moe_forward(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x, void *out, void *ws, size_t ws_bytes, void *stream)
{
    return forward_impl(cfg, w, x, out, ws, ws_bytes, stream, nullptr);
}

int xs_moe_block_workspace_bytes(const XsMoeConfig *cfg, size_t *bytes)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!bytes)
        return fail(XS_MOE_ERR_INVALID_ARG, "null out-pointer");
    *bytes = plan_forward(cfg).bytes + align_up(static_cast<size_t>(cfg->num_tokens) * cfg->hidden * 2, 256);
    return 0;
}

int xs_moe_block_forward(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x, const void *norm_weight, float eps, void *out,
                         void *ws, size_t ws_bytes, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!x || !norm_weight || !out)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    const size_t fwd = plan_forward(cfg).bytes;
    const size_t xn_bytes = align_up(static_cast<size_t>(cfg->num_tokens) * cfg->hidden * 2, 256);
    if (int rc = check_workspace(ws, ws_bytes, fwd + xn_bytes))
        return rc;
    void *xn = static_cast<uint8_t *>(ws) + fwd;
    if (int rc = xs_moe_rmsnorm(x, norm_weight, xn, cfg->num_tokens, cfg->hidden, eps, stream))
        return rc;
    return forward_impl(cfg, w, xn, out, ws, fwd, stream, nullptr, x);
}

int xs_moe_forward_profile(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x, void *out, void *ws, size_t ws_bytes,
                           void *stream, float *stage_ms)
{
    if (!stage_ms)
        return fail(XS_MOE_ERR_INVALID_ARG, "null out-pointer");
    cudaEvent_t ev[7];
    for (int i = 0; i < 7; i++)
        XS_CUDA(cudaEventCreate(&ev[i]));
    int rc = forward_impl(cfg, w, x, out, ws, ws_bytes, stream, ev);
    if (rc == 0 && cfg->num_tokens > 0) {
        cudaError_t e = cudaEventSynchronize(ev[6]);
        if (e != cudaSuccess)
            rc = fail(XS_MOE_ERR_CUDA, "CUDA error: %s", cudaGetErrorString(e));
        for (int i = 0; i < 6 && rc == 0; i++)
            if (cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]) != cudaSuccess)
                rc = fail(XS_MOE_ERR_CUDA, "CUDA error: event timing failed");
    } else {
        for (int i = 0; i < 6; i++)
            stage_ms[i] = 0.0f;
    }
    for (int i = 0; i < 7; i++)
        cudaEventDestroy(ev[i]);
    return rc;
}

int xs_moe_check_flags(void *ws, void *stream)
{
    if (!ws)
        return fail(XS_MOE_ERR_WORKSPACE, "workspace is null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t flags = 0;
    XS_CUDA(cudaMemcpyAsync(&flags, ws, sizeof(flags), cudaMemcpyDeviceToHost, st));
    XS_CUDA(cudaStreamSynchronize(st));
    if (flags != 0) {
        XS_CUDA(cudaMemsetAsync(ws, 0, sizeof(flags), st));
        XS_CUDA(cudaStreamSynchronize(st));
        if (flags & xs::kStatusWaitTimeout)
            return fail(XS_MOE_ERR_KERNEL_TIMEOUT, "a kernel gave up a bounded wait (status word 0x%x)", flags);
        return fail(XS_MOE_ERR_INVALID_ARG, "a kernel met an out-of-range index (status word 0x%x)", flags);
    }
    return 0;
}

int xs_moe_probe_mma_rate(int32_t kind, int32_t n, int32_t iters, int32_t chains, void *ws, size_t ws_bytes, double *cycles_per_mma,
                          double *issue_cycles_per_mma, double *tflops, void *stream)
{
    if (int rc = xs_moe_device_check())
        return rc;
    if (kind < 0 || kind > 6 || n < 16 || n > 256 || n % 16 != 0 || iters < 4 || iters % 4 != 0 ||
        (chains != 1 && chains != 2 && chains != 4) || chains * n > ((kind == 2 || kind == 3) ? 496 : 512) || (kind >= 4 && 2 * n > 512))
        return fail(XS_MOE_ERR_INVALID_ARG, "bad probe arguments");
    if (int rc = check_workspace(ws, ws_bytes, kStatusBytes))
        return rc;
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t *b = static_cast<uint8_t *>(ws);
    unsigned long long *ctr = reinterpret_cast<unsigned long long *>(b + 64);
    XS_CUDA(cudaMemsetAsync(ctr, 0, 64, st));
    const int smem = (128 + 256) * 128 + 1536 + 1024;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(xs::mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev < 64)
            configured[dev] = true;
    }
    cudaEvent_t e0, e1;
    XS_CUDA(cudaEventCreate(&e0));
    XS_CUDA(cudaEventCreate(&e1));
    XS_CUDA(cudaEventRecord(e0, st));
    xs::mma_rate_kernel<<<di.sms, 64, smem, st>>>(kind, n, iters, chains, ctr, reinterpret_cast<int32_t *>(b));
    note_launch();
    XS_CUDA(cudaGetLastError());
    XS_CUDA(cudaEventRecord(e1, st));
    XS_CUDA(cudaEventSynchronize(e1));
    float ms = 0;
    XS_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    unsigned long long h[3];
    XS_CUDA(cudaMemcpy(h, ctr, sizeof(h), cudaMemcpyDeviceToHost));
    XS_CUDA(cudaMemsetAsync(ctr, 0, 64, st));
    const double ctas = h[2] ? static_cast<double>(h[2]) : 1.0;
    if (cycles_per_mma)
        *cycles_per_mma = static_cast<double>(h[0]) / ctas / iters;
    if (issue_cycles_per_mma)
        *issue_cycles_per_mma = static_cast<double>(h[1]) / ctas / iters;
    if (tflops) {
        const double k = kind == 0 ? 16.0 : 32.0;
        *tflops = 2.0 * 128.0 * n * k * iters * di.sms / (ms * 1e-3) / 1e12;
    }
    return xs_moe_check_flags(ws, stream);
}

int xs_moe_probe_tmem_ld_rate(int32_t shape, int32_t warps, int32_t iters, int32_t with_mma, void *ws, size_t ws_bytes,
                              double *bytes_per_cycle_per_sm, double *mma_cycles_per_mma, void *stream)
{
    if (int rc = xs_moe_device_check())
        return rc;
    if (shape < 0 || shape > 3 || warps < 4 || warps > 16 || warps % 4 != 0 || iters < 1 || iters > (1 << 20))
        return fail(XS_MOE_ERR_INVALID_ARG, "bad probe arguments");
    if (int rc = check_workspace(ws, ws_bytes, kStatusBytes))
        return rc;
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t *b = static_cast<uint8_t *>(ws);
    unsigned long long *ctr = reinterpret_cast<unsigned long long *>(b + 64);
    XS_CUDA(cudaMemsetAsync(ctr, 0, 64, st));
    const int smem = (128 + 256) * 128 + 1024;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(xs::tmem_ld_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev < 64)
            configured[dev] = true;
    }
    // the MMA stream is sized to outlast the readers at the slowest rate seen so far (64 bytes per cycle) and is bounded
    long mma_iters = with_mma ? (static_cast<long>(warps) * iters * 8192 / 64 / 128 + 64) / 4 * 4 : 0;
    if (mma_iters > (1 << 22))
        mma_iters = 1 << 22;
    xs::tmem_ld_rate_kernel<<<di.sms, (warps + 1) * 32, smem, st>>>(shape, warps, iters, with_mma, static_cast<int>(mma_iters), ctr,
                                                                    reinterpret_cast<int32_t *>(b));
    note_launch();
    XS_CUDA(cudaGetLastError());
    unsigned long long h[3];
    XS_CUDA(cudaMemcpyAsync(h, ctr, sizeof(h), cudaMemcpyDeviceToHost, st));
    XS_CUDA(cudaStreamSynchronize(st));
    XS_CUDA(cudaMemsetAsync(ctr, 0, 64, st));
    const double ctas = h[2] ? static_cast<double>(h[2]) : 1.0;
    if (bytes_per_cycle_per_sm)
        *bytes_per_cycle_per_sm = h[0] ? static_cast<double>(warps) * iters * 8192.0 / (static_cast<double>(h[0]) / ctas) : 0.0;
    if (mma_cycles_per_mma)
        *mma_cycles_per_mma = mma_iters ? static_cast<double>(h[1]) / ctas / static_cast<double>(mma_iters) : 0.0;
    return xs_moe_check_flags(ws, stream);
}

int xs_moe_probe_handoff(int32_t responders, int32_t iters, int32_t mode, int32_t ld_cols, void *ws, size_t ws_bytes,
                         double *cycles_per_kblock, void *stream)
{
    if (int rc = xs_moe_device_check())
        return rc;
    if (responders < 1 || responders > 16 || iters < 2 || iters > (1 << 22) || mode < 0 || mode > 15 || ld_cols < 0 || ld_cols > 64 ||
        ld_cols % 32 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "bad probe arguments");
    if (int rc = check_workspace(ws, ws_bytes, kStatusBytes))
        return rc;
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t *b = static_cast<uint8_t *>(ws);
    unsigned long long *ctr = reinterpret_cast<unsigned long long *>(b + 64);
    XS_CUDA(cudaMemsetAsync(ctr, 0, 64, st));
    const int smem = (128 + 256) * 128 + 1024;
    static bool configured[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        XS_CUDA(cudaFuncSetAttribute(xs::handoff_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev < 64)
            configured[dev] = true;
    }
    xs::handoff_rate_kernel<<<di.sms, 640, smem, st>>>(responders, iters, mode, ld_cols, ctr, reinterpret_cast<int32_t *>(b));
    note_launch();
    XS_CUDA(cudaGetLastError());
    unsigned long long h[3];
    XS_CUDA(cudaMemcpyAsync(h, ctr, sizeof(h), cudaMemcpyDeviceToHost, st));
    XS_CUDA(cudaStreamSynchronize(st));
    XS_CUDA(cudaMemsetAsync(ctr, 0, 64, st));
    const double ctas = h[2] ? static_cast<double>(h[2]) : 1.0;
    if (cycles_per_kblock)
        *cycles_per_kblock = static_cast<double>(h[0]) / ctas / ((mode & 8) ? (iters + 1) / 2 : iters) / ((mode & 8) ? 0.5 : 1.0);
    return xs_moe_check_flags(ws, stream);
}

int xs_moe_plan_info(const XsMoeConfig *cfg, int32_t *token_tile, int32_t *prefill_kernels)
{
    if (int rc = check_cfg(cfg))
        return rc;
    const ForwardPlan p = plan_forward(cfg);
    if (token_tile)
        *token_tile = p.grouped.n_tile;
    if (prefill_kernels)
        *prefill_kernels = (p.grouped.n_tile == 128 && cfg->routed_format != XS_MOE_BF16) ? 1 : 0;
    return 0;
}

int xs_moe_launch_count(unsigned long long *count)
{
    if (!count)
        return fail(XS_MOE_ERR_INVALID_ARG, "null out-pointer");
    *count = g_launches.load(std::memory_order_relaxed);
    return 0;
}

int xs_moe_debug_counters(void *ws, unsigned long long *out16, void *stream)
{
    if (!ws || !out16)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t *p = static_cast<uint8_t *>(ws) + 64;
    XS_CUDA(cudaMemcpyAsync(out16, p, 128, cudaMemcpyDeviceToHost, st));
    XS_CUDA(cudaMemsetAsync(p, 0, 128, st));
    XS_CUDA(cudaStreamSynchronize(st));
    return 0;
}

int xs_moe_workspace_init(void *ws, size_t ws_bytes, void *stream)
{
    if (int rc = check_workspace(ws, ws_bytes, kStatusBytes))
        return rc;
    XS_CUDA(cudaMemsetAsync(ws, 0, kStatusBytes, static_cast<cudaStream_t>(stream)));
    return 0;
}

// ---------------------------------------------------------------------------------------------------------
// Permutation without any allocation.
//
// Some callers cannot obtain device memory at the moment they need a permutation: an engine that gave all
// free HBM to its KV page pool at start-up has nothing left for cudaMalloc to hand out, and a serving thread
// that must keep its latency flat cannot afford cudaMalloc / cudaFree either, because both synchronise the
// whole device.  For them the chunk tables the permutation kernels need live in the array below, which is part
// of the library image: every GPU that loads the library holds these ~513 KB until the process exits.
//
// Limits: at most kNoAllocMaxTokens tokens and kNoAllocMaxExperts experts per call.
// The array is shared by every call on the device and keeps what the previous call left in it; the words that
// must start at zero are cleared (on the caller's stream) at the start of each call.  Two calls that overlap
// on the GPU -- different streams, or different host threads -- race on the array: serialise them.
constexpr int kNoAllocMaxTokens = 16384;
constexpr int kNoAllocMaxExperts = 1024;
constexpr int kNoAllocStatusInts = 64; // 256 bytes: status word + padding
constexpr size_t kNoAllocTableInts = static_cast<size_t>(kNoAllocMaxTokens / xs::kChunkTokens) * kNoAllocMaxExperts;
static __device__ __align__(256) int32_t g_noalloc_scratch[kNoAllocStatusInts + 2 * kNoAllocTableInts];

// In host code the name of a __device__ array is only a handle for the runtime, never an address a kernel may
// be given.  The device address is looked up once per device (with that device current) and cached.
static int noalloc_scratch_address(int32_t **out)
{
    static std::mutex mu;
    static int32_t *addr[64] = {};
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64)
        return fail(XS_MOE_ERR_DEVICE, "device ordinal %d outside the supported range", dev);
    std::lock_guard<std::mutex> g(mu);
    if (!addr[dev]) {
        int32_t *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return fail(XS_MOE_ERR_CUDA, "CUDA error: %s (cudaGetSymbolAddress of the built-in scratch)", cudaGetErrorString(e));
        addr[dev] = p;
    }
    *out = addr[dev];
    return 0;
}

int xs_moe_permute_noalloc(const XsMoeConfig *cfg, const int32_t *ids, int32_t *counts, int32_t *offsets, int32_t *perm,
                           int32_t *inv, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!ids || !counts || !offsets || !perm || !inv)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (cfg->num_tokens > kNoAllocMaxTokens || cfg->num_experts > kNoAllocMaxExperts)
        return fail(XS_MOE_ERR_WORKSPACE,
                    "built-in scratch too small: %d tokens x %d experts asked, at most %d tokens x %d experts per call "
                    "(use xs_moe_permute with a caller workspace)",
                    cfg->num_tokens, cfg->num_experts, kNoAllocMaxTokens, kNoAllocMaxExperts);
    int32_t *base = nullptr;
    if (int rc = noalloc_scratch_address(&base))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int chunks = (cfg->num_tokens + xs::kChunkTokens - 1) / xs::kChunkTokens;
    if (chunks == 0)
        chunks = 1;
    // the status word is OR-ed into by the kernels, so it has to start at zero; the chunk tables are fully
    // rewritten for the (chunks x experts) range this call reads
    XS_CUDA(cudaMemsetAsync(base, 0, kNoAllocStatusInts * sizeof(int32_t), st));
    int32_t *chunk_counts = base + kNoAllocStatusInts;
    int32_t *chunk_base = chunk_counts + kNoAllocTableInts;
    return launch_permute(cfg, ids, counts, offsets, perm, inv, chunk_counts, chunk_base, chunks, base, st);
}

int xs_moe_forward_host(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x_host, void *out_host, void *x_stage, void *out_stage,
                        void *ws, size_t ws_bytes, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (!x_host || !out_host || !x_stage || !out_stage)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(cfg->num_tokens) * cfg->hidden * 2;
    XS_CUDA(cudaMemcpyAsync(x_stage, x_host, bytes, cudaMemcpyHostToDevice, st));
    if (int rc = xs_moe_forward(cfg, w, x_stage, out_stage, ws, ws_bytes, stream))
        return rc;
    XS_CUDA(cudaMemcpyAsync(out_host, out_stage, bytes, cudaMemcpyDeviceToHost, st));
    XS_CUDA(cudaStreamSynchronize(st));
    return xs_moe_check_flags(ws, stream);
}

// ---- expert parallelism over peer memory ---------------------------------------------------------------------------

int xs_moe_ipc_export(void *ptr, uint8_t *handle)
{
    static_assert(sizeof(cudaIpcMemHandle_t) == XS_MOE_IPC_HANDLE_BYTES, "handle size");
    if (!ptr || !handle)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    cudaIpcMemHandle_t h;
    XS_CUDA(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle, &h, sizeof(h));
    return 0;
}

int xs_moe_ipc_import(const uint8_t *handle, void **ptr)
{
    if (!ptr || !handle)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    XS_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return 0;
}

int xs_moe_ipc_close(void *ptr)
{
    if (ptr)
        XS_CUDA(cudaIpcCloseMemHandle(ptr));
    return 0;
}

static int check_ep(int32_t ranks, int32_t rank, int32_t experts)
{
    if (ranks < 1 || ranks > 32 || rank < 0 || rank >= ranks)
        return fail(XS_MOE_ERR_INVALID_ARG, "bad rank %d of %d (at most 32 ranks)", rank, ranks);
    if (experts < 1 || experts > 1024 || experts % ranks != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "expert count mismatch: %d experts must divide evenly over %d ranks (at most 1024)", experts,
                    ranks);
    return 0;
}

int xs_moe_ep_plan(const int32_t *all_counts, int32_t ranks, int32_t experts, int32_t rank, int32_t *dest_base, int32_t *offsets_local,
                   int32_t *src_offsets, void *stream)
{
    if (int rc = check_ep(ranks, rank, experts))
        return rc;
    if (!all_counts || !dest_base || !offsets_local || !src_offsets)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    int threads = ((experts > ranks ? experts : ranks) + 31) / 32 * 32;
    xs::ep_plan_kernel<<<1, threads, 0, static_cast<cudaStream_t>(stream)>>>(all_counts, ranks, experts, rank, dest_base, offsets_local,
                                                                            src_offsets);
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

int xs_moe_ep_signal(int32_t ranks, int32_t rank, const int32_t *counts, int32_t experts, void *const *peer_all_counts,
                     void *const *peer_flags, int32_t *my_flags, int32_t *epoch, void *ws, void *stream)
{
    if (int rc = check_ep(ranks, rank, experts > 0 ? experts : ranks))
        return rc;
    if (!peer_flags || !my_flags || !epoch || !ws || (counts && !peer_all_counts))
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    xs::ep_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(counts, experts, reinterpret_cast<int32_t *const *>(peer_all_counts),
                                                                          reinterpret_cast<int32_t *const *>(peer_flags), my_flags, epoch, ranks, rank,
                                                                          static_cast<int32_t *>(ws));
    note_launch();
    XS_CUDA(cudaGetLastError());
    return 0;
}

int xs_moe_ep_dispatch(const XsMoeConfig *cfg, int32_t ranks, const void *x, const int32_t *ids, const int32_t *inv,
                       const int32_t *my_offsets, const int32_t *dest_base, void *const *peer_rows, void *const *peer_scales,
                       int32_t capacity_rows, void *ws, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (int rc = check_ep(ranks, 0, cfg->num_experts))
        return rc;
    if (!x || !ids || !inv || !my_offsets || !dest_base || !peer_rows || !ws || (cfg->routed_format != XS_MOE_BF16 && !peer_scales))
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (cfg->top_k > 32 || capacity_rows < 0 || cfg->hidden % 128 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch: top_k <= 32 and hidden a multiple of 128 are required");
    if (cfg->num_tokens == 0)
        return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto rows = reinterpret_cast<uint8_t *const *>(peer_rows);
    auto scales = reinterpret_cast<uint8_t *const *>(peer_scales);
    auto xb = static_cast<const __nv_bfloat16 *>(x);
    int32_t *status = static_cast<int32_t *>(ws);
    const int T = cfg->num_tokens, H = cfg->hidden, K = cfg->top_k, E = cfg->num_experts;
    if (cfg->routed_format == XS_MOE_BF16) {
        xs::ep_dispatch_kernel<0><<<T, 256, 0, st>>>(xb, ids, inv, my_offsets, dest_base, rows, scales, T, H, K, E, ranks, capacity_rows,
                                                     status);
        note_launch();
    } else if (cfg->routed_format == XS_MOE_FP8_BLOCK128) {
        xs::ep_dispatch_kernel<1><<<T, 256, 0, st>>>(xb, ids, inv, my_offsets, dest_base, rows, scales, T, H, K, E, ranks, capacity_rows,
                                                     status);
        note_launch();
    } else {
        xs::ep_dispatch_kernel<2><<<T, 256, 0, st>>>(xb, ids, inv, my_offsets, dest_base, rows, scales, T, H, K, E, ranks, capacity_rows,
                                                     status);
        note_launch();
    }
    XS_CUDA(cudaGetLastError());
    return 0;
}

int xs_moe_ep_return(const XsMoeConfig *cfg, int32_t ranks, int32_t rank, const float *y_grouped, const int32_t *all_counts,
                     const int32_t *offsets_local, const int32_t *src_offsets, int32_t y_capacity_rows, void *const *peer_back,
                     int32_t back_capacity_rows, int32_t wire_bf16, void *ws, void *stream)
{
    if (int rc = check_cfg(cfg))
        return rc;
    if (int rc = check_ep(ranks, rank, cfg->num_experts))
        return rc;
    if (!y_grouped || !all_counts || !offsets_local || !src_offsets || !peer_back || !ws)
        return fail(XS_MOE_ERR_INVALID_ARG, "null tensor pointer");
    if (back_capacity_rows < 0 || y_capacity_rows < 0 || cfg->hidden % 8 != 0)
        return fail(XS_MOE_ERR_INVALID_ARG, "shape mismatch");
    DeviceInfo di;
    if (int rc = device_info(&di))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto back = reinterpret_cast<uint8_t *const *>(peer_back);
    int32_t *status = static_cast<int32_t *>(ws);
    const int grid = di.sms * 8;
    if (wire_bf16) {
        xs::ep_return_kernel<true><<<grid, 256, 0, st>>>(y_grouped, all_counts, offsets_local, src_offsets, back, cfg->hidden,
                                                         cfg->num_experts, ranks, rank, y_capacity_rows, back_capacity_rows, status);
        note_launch();
    } else {
        xs::ep_return_kernel<false><<<grid, 256, 0, st>>>(y_grouped, all_counts, offsets_local, src_offsets, back, cfg->hidden,
                                                          cfg->num_experts, ranks, rank, y_capacity_rows, back_capacity_rows, status);
        note_launch();
    }
    XS_CUDA(cudaGetLastError());
    return 0;
}

} // extern "C"

#include "xs_comm.inl"
