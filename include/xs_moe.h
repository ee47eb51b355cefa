/*
 * xs_moe.h -- C ABI of the B200 (sm_100a) MoE forward path.
 *
 * Plain pointers and sizes only; no C++ or framework types cross this boundary, no exception leaves it.
 * Every entry point returns 0 on success or a negative XsMoeStatus; xs_moe_status_string() names it and
 * xs_moe_last_error() gives the detail message of the calling thread's last failure.
 *
 * The reference engine reaches its kernels through per-op `<op>_launch(void*..., DType)` functions that
 * are declared in CUDA-free headers and defined in .cu files (reference: xstar_cpp/include/ops/mlp.h:95-102,
 * xstar_cpp/include/ops/gemm.h:165-176, xstar_cpp/include/ops/softmax.h:75-80,
 * xstar_cpp/include/ops/embedding.h:58-63, xstar_cpp/include/ops/add.h:38) and through the allocator
 * wrappers of xstar_cpp/include/cuda/cuda_allocator.h:32-69.  The functions below are what a `moe` op in
 * that engine binds in the same way; each one cites the reference interface whose role it takes.
 *
 * Device pointers are marked _dev.  All index arrays are int32, row-major, contiguous.
 * Streams are passed as void* (a cudaStream_t; NULL = the default stream).  Calls enqueue work and return;
 * they do not synchronise unless stated.
 */
#ifndef XS_MOE_H
#define XS_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum XsMoeStatus {
    XS_MOE_OK = 0,
    XS_MOE_ERR_INVALID_ARG = -1,   /* null pointer, bad dimension, unsupported combination */
    XS_MOE_ERR_UNSUPPORTED = -2,   /* format / shape not implemented by this build */
    XS_MOE_ERR_WORKSPACE = -3,     /* workspace too small or misaligned */
    XS_MOE_ERR_CUDA = -4,          /* a CUDA runtime/driver call failed; see xs_moe_last_error() */
    XS_MOE_ERR_DEVICE = -5,        /* not an sm_100 device, or the kernel image is missing */
    XS_MOE_ERR_KERNEL_TIMEOUT = -6 /* a bounded device-side wait gave up (reported by xs_moe_check_flags) */
} XsMoeStatus;

/* storage format of expert weights */
typedef enum XsMoeFormat {
    XS_MOE_BF16 = 0,          /* bf16, (rows, K) row-major */
    XS_MOE_FP8_BLOCK128 = 1,  /* e4m3 codes + f32 scale per 128x128 block, scales (rows/128, K/128) */
    XS_MOE_FP4_MX32 = 2       /* e2m1 packed 2/byte (low nibble = even k) + e8m0 scale per 32 along K */
} XsMoeFormat;

typedef struct XsMoeConfig {
    int32_t num_tokens;     /* T: rows of x handled by this call */
    int32_t hidden;         /* H */
    int32_t num_experts;    /* E: routed experts the ROUTER scores (global count) */
    int32_t top_k;          /* k */
    int32_t intermediate;   /* I */
    int32_t num_shared;     /* 0 or 1 shared expert */
    int32_t routed_format;  /* XsMoeFormat of gate_up_w / down_w */
    int32_t shared_format;  /* XsMoeFormat of the shared expert */
    int32_t local_expert_begin; /* expert parallelism: this device owns experts [begin, begin+count) */
    int32_t local_expert_count; /* == num_experts when not sharded */
    int32_t gemm_impl;      /* 0 = tcgen05 tensor-core kernels (the product path);
                               1 = plain CUDA-core cross-check kernels (bf16 only; used by tests to
                                   validate the tensor-core path on the device, never a fallback) */
    int32_t reserved[5];    /* must be zero */
} XsMoeConfig;

typedef struct XsMoeWeights {
    const void *router_w_dev;             /* (E, H) bf16 */
    const float *router_bias_dev;         /* (E) f32, selection only; may be NULL */
    const void *gate_up_w_dev;            /* (E_local, 2I, H) rows [gate; up] as xstar_cpp/include/ops/mlp.h:34 */
    const void *gate_up_scale_dev;        /* FP8: f32 (E_local, 2I/128, H/128); FP4: u8 (E_local, 2I, H/32) */
    const void *down_w_dev;               /* (E_local, H, I) */
    const void *down_scale_dev;           /* FP8: f32 (E_local, H/128, I/128); FP4: u8 (E_local, H, I/32) */
    const void *shared_gate_up_w_dev;     /* (2I, H) or NULL */
    const void *shared_gate_up_scale_dev;
    const void *shared_down_w_dev;        /* (H, I) or NULL */
    const void *shared_down_scale_dev;
} XsMoeWeights;

/* ---- library / device ----------------------------------------------------------------------------- */

/* Takes the role of CHECK_CUDA's message (reference: xstar_cpp/include/cuda/cuda_check.h:23-31). */
const char *xs_moe_status_string(int status);
const char *xs_moe_last_error(void);

/* 0 if the current device can run this library (compute capability 10.x), else XS_MOE_ERR_DEVICE. */
int xs_moe_device_check(void);

/* Device selection for the calling host thread (the reference's ops run on device 0 implicitly,
 * xstar_cpp/src/ops/add.cu:26; an expert-parallel host drives one device per thread). */
int xs_moe_device_count(int32_t *count);
int xs_moe_set_device(int32_t device);
int xs_moe_current_device(int32_t *device);

/* Allocator wrappers with the reference's meaning (xstar_cpp/include/cuda/cuda_allocator.h:32-69):
 * raw device allocation, synchronous copies, free-memory probe. */
int xs_moe_device_alloc(void **ptr_dev, size_t bytes);
int xs_moe_device_free(void *ptr_dev);
int xs_moe_memcpy_h2d(void *dst_dev, const void *src_host, size_t bytes);
int xs_moe_memcpy_d2h(void *dst_host, const void *src_dev, size_t bytes);
int xs_moe_memcpy_d2d(void *dst_dev, const void *src_dev, size_t bytes);
int xs_moe_device_free_bytes(size_t *bytes);
int xs_moe_stream_synchronize(void *stream);

/* ---- workspace ------------------------------------------------------------------------------------ */

/* Bytes of scratch xs_moe_forward needs for `cfg` (an upper bound over all routings).  The caller owns
 * the buffer (256-byte aligned) and may reuse it across calls that do not overlap on the device.
 * Replaces the per-temporary Tensor allocations of the reference's ops (xstar_cpp/src/ops/mlp.cpp:66). */
int xs_moe_workspace_bytes(const XsMoeConfig *cfg, size_t *bytes);

/* Clears the status word at the head of a workspace.  Call once after allocating it (and after a
 * failed xs_moe_check_flags, which also clears it). */
int xs_moe_workspace_init(void *workspace_dev, size_t workspace_bytes, void *stream);

/* ---- the whole layer -------------------------------------------------------------------------------- */

/* out(T,H) bf16 = MoE(x(T,H) bf16).  The slot `mlp(x, gate_up_w, down_w)` fills in the reference's block
 * (xstar_cpp/src/ops/transformer_block.cpp:353; op contract xstar_cpp/include/ops/mlp.h:51). */
int xs_moe_forward(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x_dev, void *out_dev,
                   void *workspace_dev, size_t workspace_bytes, void *stream);

/* The block's feed-forward half, out = x + MoE(rmsnorm(x, norm_weight, eps)): the expression the reference's block ends with
 * (xstar_cpp/src/ops/transformer_block.cpp:353, `add(attention_x, mlp(rmsnorm(attention_x, ln2_w, eps), ...))`) with the MoE
 * layer in mlp's place.  x (T,H) bf16 is the block's residual stream; norm_weight (H) bf16.  The normalised rows are written
 * once (the router's tensor-core pass and the row scatter both read them) with the arithmetic of the reference's rmsnorm
 * (xstar_cpp/src/ops/rmsnorm.cpp:52-72, sum of squares in ascending order: bit-identical); the residual add is fused into the
 * combine kernel with add's two roundings (xstar_cpp/src/ops/add.cpp:27-49).  Workspace: xs_moe_block_workspace_bytes. */
int xs_moe_block_workspace_bytes(const XsMoeConfig *cfg, size_t *bytes);
int xs_moe_block_forward(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x_dev, const void *norm_weight_dev, float eps,
                         void *out_dev, void *workspace_dev, size_t workspace_bytes, void *stream);

/* xs_moe_forward with CUDA events recorded between its stages on `stream`; synchronises and returns SIX stage
 * times in milliseconds: router logits, selection + permutation + tile table, row scatter (+ activation
 * quantisation for FP8), gate/up GEMM, down GEMM, combine.  The always-on expert runs inside the two GEMM
 * launches.  For benchmarks; no counterpart in the reference, whose ops are timed from Python
 * (bench/bench_splitkv.py:86-105 in the reference). */
int xs_moe_forward_profile(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x_dev, void *out_dev,
                           void *workspace_dev, size_t workspace_bytes, void *stream, float *stage_ms);

/* Same with x and out in HOST memory: copies x in, runs, copies out back and synchronises -- the
 * "returns => finished" behaviour of every reference op (xstar_cpp/src/ops/mlp.cu:188-189). */
int xs_moe_forward_host(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *x_host, void *out_host,
                        void *x_staging_dev, void *out_staging_dev, void *workspace_dev, size_t workspace_bytes,
                        void *stream);

/* ---- stages (used by the layer, by expert parallelism and by the parity tests) -------------------- */

/* Router logits + selection.  logits(T,E) f32 are accumulated per output in ascending k (the order of
 * gemm_cpu, xstar_cpp/include/ops/gemm.h:57-83; linear's x*W^T, xstar_cpp/src/ops/linear.cpp:20-31);
 * key = logit + bias (a NaN key orders as -inf); the k largest keys, ties to the lower id; slots in ascending expert id;
 * weights = max-shifted softmax over the selected unbiased logits (xstar_cpp/src/ops/softmax.cpp:56-93).
 * logits_dev may be NULL when the caller does not want them (scratch is then taken from the workspace); batches of more
 * than 256 tokens then take a two-step router -- approximate logits on the tensor core, exact ascending-k recomputation of
 * every logit the selection can depend on (the chosen experts and all within a proven error bound of the k / k+1 boundary)
 * -- whose ids and weights are the same as those of the all-exact path. */
int xs_moe_route(const XsMoeConfig *cfg, const void *x_dev, const void *router_w_dev, const float *router_bias_dev,
                 float *logits_dev, int32_t *topk_ids_dev, float *topk_w_dev, void *workspace_dev,
                 size_t workspace_bytes, void *stream);

/* The selection step of xs_moe_route by itself, on logits(T,E) f32 the caller already holds (same rule: key = logit +
 * bias, a NaN key orders as -inf, ties to the lower id, ascending slots, softmax over the selected unbiased logits).
 * Takes the role of softmax_launch over a row (xstar_cpp/include/ops/softmax.h:75-80) restricted to the k chosen. */
int xs_moe_topk(const XsMoeConfig *cfg, const float *logits_dev, const float *router_bias_dev, int32_t *topk_ids_dev,
                float *topk_w_dev, void *stream);

/* Deterministic permutation: rows sorted by (expert asc, token asc).  counts(E), offsets(E+1),
 * perm(T*k): row -> t*k+slot, inv(T*k): t*k+slot -> row.  The index-array convention (raw integers next
 * to the tensors) is that of the reference's gather op (xstar_cpp/include/ops/embedding.h:12-13,34). */
int xs_moe_permute(const XsMoeConfig *cfg, const int32_t *topk_ids_dev, int32_t *counts_dev, int32_t *offsets_dev,
                   int32_t *perm_dev, int32_t *inv_dev, void *workspace_dev, size_t workspace_bytes, void *stream);

/* xs_moe_permute for callers that cannot allocate device memory.  No counterpart in the reference (every
 * reference op allocates its temporaries with cudaMalloc, xstar_cpp/src/tensor.cpp:34-37).
 *
 * Who needs it: an engine whose start-up gave all free HBM to its KV page pool, so that a later cudaMalloc has
 * nothing to return; a serving thread that must not stall, since cudaMalloc and cudaFree synchronise the whole
 * device.  This call performs no cudaMalloc, cudaFree or any other allocating routine: its chunk tables live in
 * a fixed array inside the library image (about 513 KB, held by every GPU that loads the library until the
 * process exits).  Inputs and outputs are the caller's, exactly as for xs_moe_permute, and the results are
 * identical.
 *
 * Limits: num_tokens <= 16384 and num_experts <= 1024; larger calls fail with XS_MOE_ERR_WORKSPACE and a
 * message that names the limit.
 * The first call on each device looks up the array's device address (one runtime query, with that device
 * current); make that first call before any stream capture begins.
 * All calls on a device share the array and it keeps the previous call's contents; what must start at zero
 * is cleared on `stream` at the start of each call.  Calls that overlap on the GPU (two streams, two threads)
 * race on it -- serialise them.  Out-of-range expert ids are skipped as in xs_moe_permute, but the flag is
 * kept inside the library and not reported; use xs_moe_permute + xs_moe_check_flags for untrusted ids. */
int xs_moe_permute_noalloc(const XsMoeConfig *cfg, const int32_t *topk_ids_dev, int32_t *counts_dev,
                           int32_t *offsets_dev, int32_t *perm_dev, int32_t *inv_dev, void *stream);

/* Per-expert SwiGLU MLPs over already-routed rows: rows_dev(M,H) (bf16; or e4m3 codes with row_scales_dev
 * (M, H/128) f32 for FP8 experts; or e4m3 codes with row_scales_dev pointing at (M, H/32) e8m0 BYTES for FP4
 * experts; NULL for bf16) are grouped by LOCAL expert
 * (expert e owns rows [offsets[e], offsets[e+1]), e in [0, local_expert_count)); y_dev(M,H) f32 receives
 * down(silu(gate x) * up x) per row.  Takes the role of gemm_silu_and_mul_launch + the down linear
 * (xstar_cpp/include/ops/mlp.h:95-102, xstar_cpp/src/ops/mlp.cpp:64-70), once per expert segment.
 * max_rows is the capacity of rows_dev / y_dev (the true M is offsets[E_local], read on the device); offsets that
 * reach beyond it are clamped to it on the device and flagged (xs_moe_check_flags), never written through. */
int xs_moe_grouped_mlp_workspace_bytes(const XsMoeConfig *cfg, int32_t max_rows, size_t *bytes);
int xs_moe_grouped_mlp(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *rows_dev,
                       const float *row_scales_dev, const int32_t *offsets_dev, int32_t max_rows, float *y_dev,
                       void *workspace_dev, size_t workspace_bytes, void *stream);

/* out(rows, hidden) bf16 = rmsnorm(x, weight, eps) with the reference's arithmetic (rmsnorm_launch,
 * xstar_cpp/include/ops/rmsnorm.h:46-52; CPU loop xstar_cpp/src/ops/rmsnorm.cpp:52-72): f32 sum of squares in ascending column
 * order, inv = 1 / sqrt(sum / hidden + eps), out[j] = bf16(bf16(x[j] * inv) * weight[j]).  Bit-identical to the CPU op. */
int xs_moe_rmsnorm(const void *x_dev, const void *weight_dev, void *out_dev, int32_t rows, int32_t hidden, float eps, void *stream);

/* Activation quantisation for FP8 experts: x (rows, cols) bf16 -> e4m3 codes (rows, cols) and one f32 scale
 * per (row, 128 columns): s = max(amax, 1e-10) / 448, code = e4m3_rne_saturating(x / s).  No counterpart in
 * the reference, whose DType has no 8-bit member (xstar_cpp/include/dtype.h:8-12). */
int xs_moe_quantize_rows_fp8(const void *x_dev, int32_t rows, int32_t cols, void *codes_dev, float *scales_dev,
                             void *stream);

/* Activation quantisation for FP4 experts (MX-FP8): e4m3 codes and one e8m0 scale byte per (row, 32 columns):
 * s = the smallest power of two >= max(amax, 1e-30) / 448, code = e4m3_rne_saturating(x / s).  No counterpart
 * in the reference (xstar_cpp/include/dtype.h:8-12 has no 8-bit member). */
int xs_moe_quantize_rows_mxfp8(const void *x_dev, int32_t rows, int32_t cols, void *codes_dev, uint8_t *scales_dev,
                               void *stream);

/* dst[r] = src[index[r]] for r < n_rows, rows of row_bytes bytes (a multiple of 4): the reference's gather
 * (embedding_launch, xstar_cpp/include/ops/embedding.h:58-63) with int32 indices and any row type.  Used to put
 * x into expert order (index = perm / k) and to regroup rows received from other ranks. */
int xs_moe_gather_rows(const void *src_dev, const int32_t *index_dev, void *dst_dev, int32_t n_rows, int32_t row_bytes,
                       void *stream);

/* out[t] = sum_j w[t,j] * y[inv[t,j]] (+ shared[t]), slot order, shared last, f32, one RNE downcast
 * (add's contract, xstar_cpp/src/ops/add.cpp:27-49).  shared_dev (T,H) f32 may be NULL. */
int xs_moe_combine(const XsMoeConfig *cfg, const float *y_dev, const int32_t *inv_dev, const float *topk_w_dev,
                   const float *shared_dev, void *out_dev, void *stream);

/* Expert-parallel return trip with bf16 rows on the wire (used for the quantised formats, whose tolerance allows
 * it): gather + round f32 expert outputs into arrival order, and the combine that reads bf16 rows.  Same contracts as
 * xs_moe_gather_rows / xs_moe_combine otherwise (add_launch, xstar_cpp/include/ops/add.h:38). */
int xs_moe_gather_rows_f32_to_bf16(const float *src_dev, const int32_t *index_dev, void *dst_bf16_dev, int32_t n_rows,
                                   int32_t cols, void *stream);
int xs_moe_combine_bf16_rows(const XsMoeConfig *cfg, const void *y_bf16_dev, const int32_t *inv_dev,
                             const float *topk_w_dev, const float *shared_dev, void *out_dev, void *stream);

/* ---- expert parallelism over peer memory (no counterpart in the reference: the expert all-to-all is a roadmap
 * row there, README.md:30, with no code behind it) ---------------------------------------------------------------
 * The dispatch and return trips of an expert-parallel layer as kernels that store each row straight into the buffer
 * of the rank that needs it, over NVLink peer mappings.  Every address is computed on the device from the (ranks,
 * experts) matrix of row counts, so the layer needs no host synchronisation; no kernel waits for another GPU, the
 * caller puts a barrier collective between the stores and their first reader. */

#define XS_MOE_IPC_HANDLE_BYTES 64
/* Peer mappings of buffers from xs_moe_device_alloc: export a handle here, import it in the other process of the
 * same box (enables peer access on first use), close it before the owner frees the buffer. */
int xs_moe_ipc_export(void *ptr_dev, uint8_t *handle64);
int xs_moe_ipc_import(const uint8_t *handle64, void **ptr_dev);
int xs_moe_ipc_close(void *ptr_dev);

/* From all_counts (ranks, experts) int32: dest_base[e] = first row of THIS rank's rows of expert e inside the
 * grouped buffer of e's owner (rows grouped by local expert, then source rank, then source order);
 * offsets_local[experts/ranks + 1] = segment offsets of this rank's own grouped buffer; src_offsets (ranks, experts) =
 * every rank's exclusive prefix of its counts (its permuted-row offsets). */
int xs_moe_ep_plan(const int32_t *all_counts_dev, int32_t ranks, int32_t num_experts, int32_t rank, int32_t *dest_base_dev,
                   int32_t *offsets_local_dev, int32_t *src_offsets_dev, void *stream);

/* Barrier between the ranks of one box over peer memory, in one warp per GPU: every rank stores its launch epoch into row
 * `rank` of every peer's flag array (peer_flags_dev: `ranks` pointers to arrays of `ranks` int32, zero at start) and polls its
 * own array (my_flags_dev) until every rank's entry has reached the epoch; *epoch_dev (int32, zero at start) advances by one
 * per call, on the device, so the call can be replayed inside a CUDA graph.  Everything the ranks enqueued before the call on
 * their streams (peer stores among them) is visible to what they enqueue after it.  With counts_dev != NULL the call is also
 * the layer's all-gather: this rank's `experts` counts are stored into row `rank` of every rank's all_counts first
 * (peer_all_counts_dev: `ranks` pointers to (ranks, experts) int32).  A replacement for the all-gather and the one-element
 * all-reduces of include/xs_moe_comm.h at a third of their latency; unlike them it WAITS for the peers inside a kernel, with a
 * bound (about two seconds), after which the wait-timeout bit is set in the status word of workspace_dev: call it only once
 * the ranks have agreed on the host that all of them will (EpGroup's check-in), and never for two ranks that share one GPU. */
int xs_moe_ep_signal(int32_t ranks, int32_t rank, const int32_t *counts_dev, int32_t experts, void *const *peer_all_counts_dev,
                     void *const *peer_flags_dev, int32_t *my_flags_dev, int32_t *epoch_dev, void *workspace_dev, void *stream);

/* Quantise (per cfg->routed_format: bf16 rows | e4m3 + 1x128 f32 scales | e4m3 + 1x32 e8m0 scales) each local token
 * once and store it for each of its k experts into row dest_base[e] + (inv[t,j] - my_offsets[e]) of the owner's
 * buffers.  peer_rows_dev / peer_scales_dev: device arrays of `ranks` pointers (this rank's own buffer included).
 * Rows outside [0, capacity_rows) are skipped and flagged in the workspace status word. */
int xs_moe_ep_dispatch(const XsMoeConfig *cfg, int32_t ranks, const void *x_dev, const int32_t *topk_ids_dev,
                       const int32_t *inv_dev, const int32_t *my_offsets_dev, const int32_t *dest_base_dev,
                       void *const *peer_rows_dev, void *const *peer_scales_dev, int32_t capacity_rows, void *workspace_dev,
                       void *stream);

/* Expert outputs (grouped rows, f32) back to row src_offsets[s][e] + j of their source rank's return buffer, as f32
 * or rounded to bf16 (wire_bf16 != 0).  The row count is read on the device from offsets_local and limited to
 * y_capacity_rows, the rows y_grouped_dev holds; rows beyond it, and destination rows outside
 * [0, back_capacity_rows), are skipped and flagged in the workspace status word. */
int xs_moe_ep_return(const XsMoeConfig *cfg, int32_t ranks, int32_t rank, const float *y_grouped_dev,
                     const int32_t *all_counts_dev, const int32_t *offsets_local_dev, const int32_t *src_offsets_dev,
                     int32_t y_capacity_rows, void *const *peer_back_dev, int32_t back_capacity_rows, int32_t wire_bf16,
                     void *workspace_dev, void *stream);

/* xs_moe_grouped_mlp with the return trip folded into the down GEMM: instead of writing f32 rows to y for xs_moe_ep_return
 * to carry, the epilogue rounds each output row to bf16 and stores it straight into its source rank's return buffer
 * (row src_offsets[s][e] + j, as xs_moe_ep_return computes it), tile by tile, so the NVLink transfer overlaps the math and
 * the f32 y buffer is neither written nor read.  `cfg` carries this rank's expert slice (local_expert_begin / _count).
 * Implemented for FP4 experts with hidden % 256 == 0 (the tokens-as-M kernels); xs_moe_grouped_mlp_return_supported says
 * whether a configuration takes it, other configurations get XS_MOE_ERR_UNSUPPORTED and use the two-step form.  Destination
 * rows outside [0, back_capacity_rows) are skipped and flagged.  The caller's barrier after this call takes the place of
 * the one after xs_moe_ep_return. */
int xs_moe_grouped_mlp_return_supported(const XsMoeConfig *cfg, int32_t max_rows, int32_t *supported);
int xs_moe_grouped_mlp_return(const XsMoeConfig *cfg, const XsMoeWeights *w, const void *rows_dev, const float *row_scales_dev,
                              const int32_t *offsets_local_dev, int32_t max_rows, int32_t ranks, int32_t rank,
                              const int32_t *all_counts_dev, const int32_t *src_offsets_dev, void *const *peer_back_dev,
                              int32_t back_capacity_rows, void *workspace_dev, size_t workspace_bytes, void *stream);

/* Reads and clears the device-side status word the kernels of the last calls on this workspace wrote
 * (bounded waits that gave up, index checks that failed).  Synchronises the stream. */
int xs_moe_check_flags(void *workspace_dev, void *stream);

#ifdef __cplusplus
}
#endif
#endif
