/*
 * xs_moe_tuning.h -- tuning aids of the B200 MoE library: hardware rate probes and the role profile of the
 * warp-specialised GEMM kernels.  None of them is part of the layer and none has a counterpart in the reference, whose
 * ops are timed from Python (bench/bench_splitkv.py:86-105 in the reference).  Same conventions as xs_moe.h: plain
 * pointers, 0 or a negative XsMoeStatus.
 */
#ifndef XS_MOE_TUNING_H
#define XS_MOE_TUNING_H

#include "xs_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Tensor-pipe rate probe: every SM issues `iters` (a multiple of 4) tcgen05.mma of M = 128, N = n (16..256) on zeroed
 * shared memory from one thread, round-robin over `chains` (1, 2 or 4) independent TMEM accumulators (chains * n <= 512;
 * <= 496 for the block-scaled kind, whose scales take the last columns).  kind 0 = bf16 (K = 16), 1 = e4m3 (K = 32),
 * 2 = block-scaled e4m3 x e2m1 (K = 32), 3 = the same with three tcgen05.cp scale copies (3 x 512 bytes, shared memory
 * to TMEM) issued by the same thread before every four MMAs, as a block-scaled GEMM's k-block needs; 4 and 5 = e4m3 issued
 * as a loop with per-k-block accumulators issues it (every four MMAs start afresh in the other of two accumulators and are
 * followed by two, resp. one, tcgen05.commit; `chains` is ignored), 6 = 5 with the issuing thread waiting for every
 * group's commit before the next group (four times its cycles per MMA = latency from issue to observed completion).  Returns cycles per MMA until completion, cycles per MMA spent issuing, and
 * whole-chip TFLOP/s by CUDA events.  Needs a workspace of at least 256 bytes (status block).  Synchronises. */
int xs_moe_probe_mma_rate(int32_t kind, int32_t n, int32_t iters, int32_t chains, void *workspace_dev,
                          size_t workspace_bytes, double *cycles_per_mma, double *issue_cycles_per_mma, double *tflops,
                          void *stream);

/* TMEM read-rate probe: on every SM `warps` warps (4, 8, 12 or 16) read 32 lanes x 64 columns per iteration
 * with tcgen05.ld.32x32b and wait; shape 0 = two pairs of .x16 with a wait after each pair, 1 = four .x16 and one wait,
 * 2 = two .x32, 3 = one .x64.  With with_mma != 0 one more warp issues N = 256 e4m3 MMAs into the other half of TMEM for
 * the duration.  Returns the bytes per cycle per SM the readers achieved and (with_mma) the cycles per MMA of the
 * concurrent stream.  Needs a workspace of at least 256 bytes.  Synchronises. */
int xs_moe_probe_tmem_ld_rate(int32_t shape, int32_t warps, int32_t iters, int32_t with_mma, void *workspace_dev,
                              size_t workspace_bytes, double *bytes_per_cycle_per_sm, double *mma_cycles_per_mma,
                              void *stream);

/* Accumulator hand-over probe: on every SM one thread issues `iters` k-blocks of four N = 256 e4m3 MMAs alternately into
 * two TMEM buffers and commits each to a barrier; `responders` warps (1..16) wait for it, read ld_cols (0, 32 or 64) columns
 * of the buffer and arrive on the barrier the issuer waits for before it reuses the buffer.  mode bit 0: responders poll
 * with mbarrier.test_wait, bit 1: the issuer too, bit 2: no tcgen05 fences around the waits, bit 3: two issuer warps take
 * k-blocks alternately.  Returns cycles per k-block.  Needs a workspace of at least 256 bytes.  Synchronises. */
int xs_moe_probe_handoff(int32_t responders, int32_t iters, int32_t mode, int32_t ld_cols, void *workspace_dev,
                         size_t workspace_bytes, double *cycles_per_kblock, void *stream);

/* Role profile of the warp-specialised GEMM kernels that ran on this workspace since the last call: sixteen 64-bit
 * cycle counters summed over CTAs (0 producer blocked on a free stage, 1 MMA issuer blocked on operands, 2 on scales,
 * 3 on a free accumulator, 4 scale writers blocked on a free slot, 5 epilogue blocked on an accumulator, 6 CTA lifetime,
 * 7 CTAs; the FP8 prefill kernel uses 2 and 4 for the cycles of its promotion bodies and of its per-tile tails, 8 for the
 * amax exchange waits and 9 for the MMA thread's issue time; 10..15 are spare).  The counters are compiled into the kernels only when the library is built with -DXS_ROLE_PROFILE=1; the
 * default build returns zeros.  Reads and clears; synchronises. */
int xs_moe_debug_counters(void *workspace_dev, unsigned long long *out16, void *stream);

/* Which GEMM kernels xs_moe_forward will launch for `cfg`: the token tile (16, 32 or 64: tokens as the N of 128-weight-row
 * MMAs, the decode shape; 128: tokens as the M of N = 256 MMAs, the prefill kernels of the FP8 / FP4 formats, or the
 * 128-token decode-shape tile of bf16) and whether the prefill kernels run. */
int xs_moe_plan_info(const XsMoeConfig *cfg, int32_t *token_tile, int32_t *prefill_kernels);

/* Kernels this library has enqueued in this process so far (a launch captured into a CUDA graph counts once, at capture;
 * its replays are the caller's to multiply).  For benchmarks that report how many of the library's kernels a timed region
 * ran. */
int xs_moe_launch_count(unsigned long long *count);

#ifdef __cplusplus
}
#endif
#endif
