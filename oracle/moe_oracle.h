/*
 * CPU oracle for the MoE forward path -- TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the numerics contracts of the reference's CPU ops, composed into the
 * MoE layer the reference plans but does not ship (README.md:28 of the reference is the only mention).
 * It is the checker for the CUDA path: only tests, the smoke check and the benchmark's CPU-baseline leg
 * may load it.  The product library never links or calls anything in this directory.
 *
 * Parity status: the GEMM order, SiLU, rounding points and row gather are pinned bit-for-bit against the
 * reference's own compiled CPU ops (see ref_compose.cpp).  Routing (top-k, tie-break, renormalisation),
 * permutation order, combine order and every FP8/FP4 rule have no reference implementation and no
 * reference test: for those this file is normative and parity is UNPINNED.
 *
 * Contracts followed (paths are inside the reference project):
 *   xstar_cpp/include/ops/gemm.h:57-83      per-output ascending-k f32 accumulation from 0, one RNE downcast
 *   xstar_cpp/src/ops/linear.cpp:20-31      weight stored (out,in), y = x * W^T, leading dims collapsed
 *   xstar_cpp/src/ops/mlp.cpp:10-45         branch-stable sigmoid, silu(g)*u in f32, gate rows first then up rows
 *   xstar_cpp/src/ops/softmax.cpp:56-93     max-shifted f32 softmax
 *   xstar_cpp/src/ops/embedding.cpp:37-46   bit-exact row gather
 *   xstar_cpp/src/ops/add.cpp:27-49         f32 add, one downcast
 *   xstar_cpp/src/bfloat16.cpp:5-25         bf16 <-> f32, round-to-nearest-even on the upper 16 bits
 */
#ifndef XS_MOE_ORACLE_H
#define XS_MOE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* storage / arithmetic modes */
enum {
    XSO_F32 = 0,            /* everything f32, no intermediate rounding (config "fp32 on CPU") */
    XSO_BF16 = 1,           /* act rounded once to bf16, out rounded once to bf16 (the CUDA contract, mlp.h:78-84) */
    XSO_BF16_REFCPU = 2,    /* as the reference CPU mlp: gate_up rounded to bf16 before SiLU, y rounded to bf16 (mlp.cpp:73) */
    XSO_FP8 = 3,            /* e4m3 weights with 128x128 f32 block scales, activations e4m3 per 1x128 */
    XSO_FP4 = 4             /* e2m1 weights with e8m0 scale per 32, activations e4m3 with e8m0 scale per 32 */
};

typedef struct XsOracleDims {
    int32_t T;      /* tokens */
    int32_t H;      /* hidden */
    int32_t E;      /* routed experts */
    int32_t K;      /* top-k */
    int32_t I;      /* intermediate */
    int32_t S;      /* shared experts: 0 or 1 */
} XsOracleDims;

/* ---- scalar format helpers ------------------------------------------------------------------------ */
uint16_t xso_f32_to_bf16(float f);
float xso_bf16_to_f32(uint16_t b);
uint8_t xso_f32_to_e4m3(float f);       /* RNE, saturating to +-448, NaN -> 0x7f */
float xso_e4m3_to_f32(uint8_t c);
uint8_t xso_f32_to_e2m1(float f);       /* RNE (ties to even code), saturating to +-6; returns 4-bit code */
float xso_e2m1_to_f32(uint8_t c);
uint8_t xso_f32_to_e8m0_ceil(float f);  /* smallest power of two >= f, as a biased exponent; f<=0 -> 0 */
float xso_e8m0_to_f32(uint8_t c);

/* ---- stage 1: router logits.  x (T,H) and router_w (E,H) as f32 (bf16 values widened); logits (T,E) f32 */
void xso_router_logits(const float *x, const float *router_w, float *logits, int T, int H, int E);

/* ---- stage 2: selection.  key = logit + bias (bias may be NULL); the K largest keys, ties to the lower
 * expert id; slots written in ascending expert id; w = softmax over the selected UNBIASED logits. */
void xso_topk(const float *logits, const float *bias, int32_t *topk_ids, float *topk_w, int T, int E, int K);

/* ---- stage 3: permutation.  rows sorted by (expert asc, token asc).
 * counts[E], offsets[E+1], perm[T*K] (row -> t*K+slot), inv[T*K] (t*K+slot -> row). */
void xso_permute(const int32_t *topk_ids, int32_t *counts, int32_t *offsets, int32_t *perm, int32_t *inv,
                 int T, int E, int K);

/* ---- activation quantisation, 1x128 groups: s = max(amax,1e-10)/448, q = e4m3(x / s) */
void xso_quant_act_fp8(const float *x, uint8_t *q, float *scale, int rows, int cols);
/* ---- activation quantisation, 1x32 groups with power-of-two scale: s = 2^ceil(log2(amax/448)) */
void xso_quant_act_mxfp8(const float *x, uint8_t *q, uint8_t *scale_e8m0, int rows, int cols);

/*
 * Whole layer.  All weight pointers are in their STORAGE form:
 *   mode F32:            x, router_w, gate_up_w, down_w, shared_* are float
 *   mode BF16/REFCPU:    x, router_w, weights are uint16 bf16 bits; out is uint16 bf16 bits
 *   mode FP8:            x, router_w bf16; gate_up_w/down_w/shared_* uint8 e4m3 codes with f32 block scales
 *                        gate_up_scale (E, 2I/128, H/128), down_scale (E, H/128, I/128); out bf16
 *   mode FP4:            routed weights packed e2m1 (two per byte, low nibble = even k) with e8m0 scales
 *                        gate_up_scale (E, 2I, H/32), down_scale (E, H, I/32) as uint8;
 *                        shared expert is FP8 128x128 as in mode FP8; out bf16
 * router_bias: (E) f32 or NULL.  Optional debug outputs may be NULL.
 * y_rows (T*K, H) f32, if given, receives the per-assignment expert outputs in permuted row order.
 * threads: worker threads over experts / tokens; the result does not depend on it.
 * token_subset / n_subset: if non-NULL, experts are evaluated only for those token ids (routing and
 * permutation are still computed for all tokens); rows of `out` for other tokens are left untouched.
 */
typedef struct XsOracleArgs {
    XsOracleDims d;
    int32_t mode;
    int32_t threads;
    const void *x;
    const void *router_w;
    const float *router_bias;
    const void *gate_up_w;
    const void *gate_up_scale;
    const void *down_w;
    const void *down_scale;
    const void *shared_gate_up_w;
    const void *shared_gate_up_scale;
    const void *shared_down_w;
    const void *shared_down_scale;
    void *out;
    float *logits;      /* (T,E)   optional */
    int32_t *topk_ids;  /* (T,K)   optional */
    float *topk_w;      /* (T,K)   optional */
    int32_t *counts;    /* (E)     optional */
    int32_t *offsets;   /* (E+1)   optional */
    int32_t *perm;      /* (T*K)   optional */
    int32_t *inv;       /* (T*K)   optional */
    float *y_rows;      /* (T*K,H) optional */
    const int32_t *token_subset;
    int32_t n_subset;
} XsOracleArgs;

/* returns 0 on success, negative on bad arguments */
int xso_moe_forward(const XsOracleArgs *a);

/* One dense SwiGLU MLP on `rows` rows (the per-expert body), for known-answer tests.
 * Same storage conventions as xso_moe_forward for the given mode (F32 / BF16 / BF16_REFCPU only);
 * y is f32 (rows,H) for F32/BF16 and bf16-rounded values widened to f32 for BF16_REFCPU. */
int xso_expert_mlp(int mode, const void *x, const void *gate_up_w, const void *down_w, float *y,
                   int rows, int H, int I);

/* The two ops around the layer in the engine's block, `add(x, mlp(rmsnorm(x, w, eps), ...))`
 * (xstar_cpp/src/ops/transformer_block.cpp:353), on bf16 storage (uint16 bits):
 * rmsnorm as xstar_cpp/src/ops/rmsnorm.cpp:52-72 (f32 sum of squares in ascending order, 1 / sqrt(sum / H + eps),
 * out = bf16(bf16(x * inv) * w)); add as xstar_cpp/src/ops/add.cpp:40-49 (f32 add, one rounding). */
void xso_rmsnorm_bf16(const uint16_t *x, const uint16_t *w, uint16_t *out, int rows, int H, float eps);
void xso_add_bf16(const uint16_t *a, const uint16_t *b, uint16_t *out, size_t n);

#ifdef __cplusplus
}
#endif
#endif
