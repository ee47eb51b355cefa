/*
 * CPU oracle for the MoE forward path -- TEST INFRASTRUCTURE ONLY (see moe_oracle.h).
 *
 * Every GEMM here accumulates each output element sequentially in ascending k, in f32, starting from 0,
 * which is the order of gemm_cpu in the reference (xstar_cpp/include/ops/gemm.h:57-83).  The loops are
 * register-blocked over several OUTPUTS at once; that changes which outputs are computed together, never
 * the order of additions inside one output, so results are bit-identical to the reference loop.
 * Build without -ffast-math and with -ffp-contract=off.
 */
#include "moe_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------------ */
/* scalar formats                                                                                    */
/* ------------------------------------------------------------------------------------------------ */

/* xstar_cpp/src/bfloat16.cpp:5-25 -- add 0x7FFF + lsb, keep the upper half; NaN/Inf not special-cased */
uint16_t xso_f32_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

/* xstar_cpp/src/bfloat16.cpp:27-36 */
float xso_bf16_to_f32(uint16_t b)
{
    uint32_t u = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static float g_e4m3_table[256];
static int g_tables_ready = 0;

static void build_tables(void)
{
    if (g_tables_ready)
        return;
    for (int c = 0; c < 256; c++) {
        int sign = c >> 7, ex = (c >> 3) & 15, man = c & 7;
        float v;
        if (ex == 15 && man == 7)
            v = NAN;
        else if (ex == 0)
            v = ldexpf((float)man, -9); /* subnormal: man/8 * 2^-6 */
        else
            v = ldexpf(1.0f + (float)man / 8.0f, ex - 7);
        g_e4m3_table[c] = sign ? -v : v;
    }
    __atomic_store_n(&g_tables_ready, 1, __ATOMIC_RELEASE);
}

float xso_e4m3_to_f32(uint8_t c)
{
    build_tables();
    return g_e4m3_table[c];
}

/* e4m3 (bias 7, max 448, no Inf): round to nearest, ties to even, saturate */
uint8_t xso_f32_to_e4m3(float f)
{
    if (f != f)
        return 0x7f;
    uint8_t sign = (uint8_t)(signbit(f) ? 0x80 : 0);
    float a = fabsf(f);
    if (a >= 448.0f)
        return (uint8_t)(sign | 0x7e);
    if (a < ldexpf(1.0f, -6)) {
        /* subnormal grid: multiples of 2^-9; rintf in the default mode is round-half-even */
        float q = rintf(a * 512.0f);
        return (uint8_t)(sign | (uint8_t)q); /* q==8 encodes 2^-6 (ex=1, man=0) naturally */
    }
    int e;
    float m = frexpf(a, &e); /* a = m * 2^e, m in [0.5,1) */
    /* significand 1.mmm -> scale to [8,16) */
    float q = rintf(m * 16.0f);
    int ex = e - 1 + 7;
    if (q == 16.0f) {
        q = 8.0f;
        ex += 1;
    }
    int man = (int)q - 8;
    if (ex > 15 || (ex == 15 && man == 7))
        return (uint8_t)(sign | 0x7e);
    return (uint8_t)(sign | (ex << 3) | man);
}

static const float g_e2m1_vals[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

float xso_e2m1_to_f32(uint8_t c)
{
    float v = g_e2m1_vals[c & 7];
    return (c & 8) ? -v : v;
}

uint8_t xso_f32_to_e2m1(float f)
{
    uint8_t sign = (uint8_t)(signbit(f) ? 8 : 0);
    float a = fabsf(f);
    if (!(a == a))
        return (uint8_t)(sign | 7);
    /* midpoints; ties go to the code with an even mantissa bit (codes 0,2,4,6) */
    uint8_t c;
    if (a <= 0.25f) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return (uint8_t)(sign | c);
}

float xso_e8m0_to_f32(uint8_t c)
{
    return ldexpf(1.0f, (int)c - 127);
}

uint8_t xso_f32_to_e8m0_ceil(float f)
{
    if (!(f > 0.0f))
        return 0;
    int e;
    float m = frexpf(f, &e); /* f = m*2^e, m in [0.5,1) */
    int p = (m == 0.5f) ? e - 1 : e; /* smallest p with 2^p >= f */
    p += 127;
    if (p < 0) p = 0;
    if (p > 254) p = 254;
    return (uint8_t)p;
}

/* ------------------------------------------------------------------------------------------------ */
/* order-exact GEMM: C[m][n] = sum_k A[m][k] * W[n][k], ascending k, f32                             */
/* ------------------------------------------------------------------------------------------------ */
static void gemm_nt(const float *A, int lda, const float *W, int ldw, float *C, int ldc, int M, int N, int K)
{
    int m = 0;
    for (; m + 2 <= M; m += 2) {
        const float *a0 = A + (size_t)m * lda, *a1 = a0 + lda;
        int n = 0;
        for (; n + 4 <= N; n += 4) {
            const float *w0 = W + (size_t)n * ldw, *w1 = w0 + ldw, *w2 = w1 + ldw, *w3 = w2 + ldw;
            float c00 = 0, c01 = 0, c02 = 0, c03 = 0, c10 = 0, c11 = 0, c12 = 0, c13 = 0;
            for (int k = 0; k < K; k++) {
                float x0 = a0[k], x1 = a1[k];
                c00 += x0 * w0[k]; c01 += x0 * w1[k]; c02 += x0 * w2[k]; c03 += x0 * w3[k];
                c10 += x1 * w0[k]; c11 += x1 * w1[k]; c12 += x1 * w2[k]; c13 += x1 * w3[k];
            }
            float *o0 = C + (size_t)m * ldc + n, *o1 = o0 + ldc;
            o0[0] = c00; o0[1] = c01; o0[2] = c02; o0[3] = c03;
            o1[0] = c10; o1[1] = c11; o1[2] = c12; o1[3] = c13;
        }
        for (; n < N; n++) {
            const float *w0 = W + (size_t)n * ldw;
            float c0 = 0, c1 = 0;
            for (int k = 0; k < K; k++) {
                c0 += a0[k] * w0[k];
                c1 += a1[k] * w0[k];
            }
            C[(size_t)m * ldc + n] = c0;
            C[(size_t)(m + 1) * ldc + n] = c1;
        }
    }
    for (; m < M; m++) {
        const float *a0 = A + (size_t)m * lda;
        int n = 0;
        for (; n + 8 <= N; n += 8) {
            const float *w = W + (size_t)n * ldw;
            float c[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int k = 0; k < K; k++) {
                float x0 = a0[k];
                for (int j = 0; j < 8; j++)
                    c[j] += x0 * w[(size_t)j * ldw + k];
            }
            for (int j = 0; j < 8; j++)
                C[(size_t)m * ldc + n + j] = c[j];
        }
        for (; n < N; n++) {
            const float *w0 = W + (size_t)n * ldw;
            float c0 = 0;
            for (int k = 0; k < K; k++)
                c0 += a0[k] * w0[k];
            C[(size_t)m * ldc + n] = c0;
        }
    }
}

/* block-scaled GEMM: per scale group of G consecutive k, partial = sequential f32 sum of code products,
 * then acc += partial * (sa * sw).  sa: (M, K/G) per-row scales; sw(n, kb) supplied through a callback
 * layout: sw_row_div = rows of W sharing one scale (128 for 128x128 blocks, 1 for per-row MX scales). */
static void gemm_nt_scaled(const float *A, int lda, const float *sa, const float *W, int ldw, const float *sw,
                           int sw_row_div, float *C, int ldc, int M, int N, int K, int G)
{
    int KB = K / G;
    for (int m = 0; m < M; m++) {
        const float *a0 = A + (size_t)m * lda;
        const float *sa0 = sa + (size_t)m * KB;
        int n = 0;
        for (; n + 4 <= N; n += 4) {
            const float *w[4];
            const float *s[4];
            for (int j = 0; j < 4; j++) {
                w[j] = W + (size_t)(n + j) * ldw;
                s[j] = sw + (size_t)((n + j) / sw_row_div) * KB;
            }
            float acc[4] = {0, 0, 0, 0};
            for (int kb = 0; kb < KB; kb++) {
                float p0 = 0, p1 = 0, p2 = 0, p3 = 0;
                int k0 = kb * G;
                for (int k = k0; k < k0 + G; k++) {
                    float x0 = a0[k];
                    p0 += x0 * w[0][k]; p1 += x0 * w[1][k]; p2 += x0 * w[2][k]; p3 += x0 * w[3][k];
                }
                float sx = sa0[kb];
                acc[0] += p0 * (sx * s[0][kb]);
                acc[1] += p1 * (sx * s[1][kb]);
                acc[2] += p2 * (sx * s[2][kb]);
                acc[3] += p3 * (sx * s[3][kb]);
            }
            for (int j = 0; j < 4; j++)
                C[(size_t)m * ldc + n + j] = acc[j];
        }
        for (; n < N; n++) {
            const float *w0 = W + (size_t)n * ldw;
            const float *s0 = sw + (size_t)(n / sw_row_div) * KB;
            float acc = 0;
            for (int kb = 0; kb < KB; kb++) {
                float p = 0;
                for (int k = kb * G; k < (kb + 1) * G; k++)
                    p += a0[k] * w0[k];
                acc += p * (sa0[kb] * s0[kb]);
            }
            C[(size_t)m * ldc + n] = acc;
        }
    }
}

/* xstar_cpp/src/ops/mlp.cpp:10-26 */
static float sigmoid_ref(float x)
{
    if (x >= 0)
        return 1.0f / (1.0f + expf(-x));
    return expf(x) / (1.0f + expf(x));
}
static float silu_ref(float x)
{
    return x * sigmoid_ref(x);
}

/* ------------------------------------------------------------------------------------------------ */
/* stages                                                                                            */
/* ------------------------------------------------------------------------------------------------ */
void xso_router_logits(const float *x, const float *router_w, float *logits, int T, int H, int E)
{
    gemm_nt(x, H, router_w, H, logits, E, T, E, H);
}

void xso_topk(const float *logits, const float *bias, int32_t *topk_ids, float *topk_w, int T, int E, int K)
{
    unsigned char *sel = (unsigned char *)malloc((size_t)E);
    for (int t = 0; t < T; t++) {
        const float *l = logits + (size_t)t * E;
        memset(sel, 0, (size_t)E);
        for (int j = 0; j < K; j++) {
            int best = -1;
            float bk = 0;
            for (int e = 0; e < E; e++) {
                if (sel[e])
                    continue;
                float key = bias ? l[e] + bias[e] : l[e];
                if (key != key)
                    key = -INFINITY; /* a NaN key orders as -inf: the selection stays a total order */
                if (best < 0 || key > bk) { /* strict >: ties keep the lower id */
                    best = e;
                    bk = key;
                }
            }
            sel[best] = 1;
        }
        int j = 0;
        float m = -INFINITY;
        for (int e = 0; e < E; e++)
            if (sel[e]) {
                topk_ids[(size_t)t * K + j++] = e;
                if (l[e] > m)
                    m = l[e];
            }
        float sum = 0;
        for (j = 0; j < K; j++)
            sum += expf(l[topk_ids[(size_t)t * K + j]] - m);
        for (j = 0; j < K; j++)
            topk_w[(size_t)t * K + j] = expf(l[topk_ids[(size_t)t * K + j]] - m) / sum;
    }
    free(sel);
}

void xso_permute(const int32_t *topk_ids, int32_t *counts, int32_t *offsets, int32_t *perm, int32_t *inv,
                 int T, int E, int K)
{
    memset(counts, 0, sizeof(int32_t) * (size_t)E);
    for (int i = 0; i < T * K; i++)
        counts[topk_ids[i]]++;
    offsets[0] = 0;
    for (int e = 0; e < E; e++)
        offsets[e + 1] = offsets[e] + counts[e];
    int32_t *cur = (int32_t *)malloc(sizeof(int32_t) * (size_t)E);
    memcpy(cur, offsets, sizeof(int32_t) * (size_t)E);
    for (int t = 0; t < T; t++)
        for (int j = 0; j < K; j++) {
            int e = topk_ids[(size_t)t * K + j];
            int row = cur[e]++;
            perm[row] = t * K + j;
            inv[(size_t)t * K + j] = row;
        }
    free(cur);
}

void xso_quant_act_fp8(const float *x, uint8_t *q, float *scale, int rows, int cols)
{
    int G = cols / 128;
    for (int r = 0; r < rows; r++)
        for (int g = 0; g < G; g++) {
            const float *p = x + (size_t)r * cols + g * 128;
            float amax = 0;
            for (int i = 0; i < 128; i++) {
                float a = fabsf(p[i]);
                if (a > amax)
                    amax = a;
            }
            float s = fmaxf(amax, 1e-10f) / 448.0f;
            scale[(size_t)r * G + g] = s;
            for (int i = 0; i < 128; i++)
                q[(size_t)r * cols + g * 128 + i] = xso_f32_to_e4m3(p[i] / s);
        }
}

void xso_quant_act_mxfp8(const float *x, uint8_t *q, uint8_t *scale_e8m0, int rows, int cols)
{
    int G = cols / 32;
    for (int r = 0; r < rows; r++)
        for (int g = 0; g < G; g++) {
            const float *p = x + (size_t)r * cols + g * 32;
            float amax = 0;
            for (int i = 0; i < 32; i++) {
                float a = fabsf(p[i]);
                if (a > amax)
                    amax = a;
            }
            uint8_t sc = xso_f32_to_e8m0_ceil(fmaxf(amax, 1e-30f) / 448.0f);
            scale_e8m0[(size_t)r * G + g] = sc;
            float inv = ldexpf(1.0f, 127 - (int)sc); /* exact: power of two */
            for (int i = 0; i < 32; i++)
                q[(size_t)r * cols + g * 32 + i] = xso_f32_to_e4m3(p[i] * inv);
        }
}

/* ------------------------------------------------------------------------------------------------ */
/* expert bodies                                                                                     */
/* ------------------------------------------------------------------------------------------------ */
static void widen_bf16(const uint16_t *src, float *dst, size_t n)
{
    for (size_t i = 0; i < n; i++)
        dst[i] = xso_bf16_to_f32(src[i]);
}
static void decode_e4m3(const uint8_t *src, float *dst, size_t n)
{
    build_tables();
    for (size_t i = 0; i < n; i++)
        dst[i] = g_e4m3_table[src[i]];
}
static void decode_e2m1_packed(const uint8_t *src, float *dst, size_t n_elems)
{
    for (size_t i = 0; i < n_elems / 2; i++) {
        dst[2 * i] = xso_e2m1_to_f32(src[i] & 15);
        dst[2 * i + 1] = xso_e2m1_to_f32(src[i] >> 4);
    }
}

/* float-weight SwiGLU MLP (modes F32, BF16, BF16_REFCPU) on `rows` rows; xs (rows,H) f32; y (rows,H) f32 */
static void mlp_float(int mode, const float *xs, const float *wgu, const float *wd, float *y, int rows, int H, int I)
{
    float *gu = (float *)malloc(sizeof(float) * (size_t)rows * 2 * I);
    float *act = (float *)malloc(sizeof(float) * (size_t)rows * I);
    gemm_nt(xs, H, wgu, H, gu, 2 * I, rows, 2 * I, H);
    if (mode == XSO_BF16_REFCPU) /* linear's output downcast, mlp.cpp:73 */
        for (size_t i = 0; i < (size_t)rows * 2 * I; i++)
            gu[i] = xso_bf16_to_f32(xso_f32_to_bf16(gu[i]));
    for (int r = 0; r < rows; r++)
        for (int j = 0; j < I; j++) {
            float g = gu[(size_t)r * 2 * I + j], u = gu[(size_t)r * 2 * I + I + j];
            float a = silu_ref(g) * u;
            if (mode != XSO_F32)
                a = xso_bf16_to_f32(xso_f32_to_bf16(a));
            act[(size_t)r * I + j] = a;
        }
    gemm_nt(act, I, wd, I, y, H, rows, H, I);
    if (mode == XSO_BF16_REFCPU)
        for (size_t i = 0; i < (size_t)rows * H; i++)
            y[i] = xso_bf16_to_f32(xso_f32_to_bf16(y[i]));
    free(gu);
    free(act);
}

/* FP8 128x128 block-scaled SwiGLU MLP.  xq (rows,H) decoded e4m3 codes as f32, sx (rows,H/128) */
static void mlp_fp8(const float *xq, const float *sx, const uint8_t *wgu_c, const float *sgu, const uint8_t *wd_c,
                    const float *sd, float *y, int rows, int H, int I)
{
    float *wgu = (float *)malloc(sizeof(float) * (size_t)2 * I * H);
    float *wd = (float *)malloc(sizeof(float) * (size_t)H * I);
    decode_e4m3(wgu_c, wgu, (size_t)2 * I * H);
    decode_e4m3(wd_c, wd, (size_t)H * I);
    float *gu = (float *)malloc(sizeof(float) * (size_t)rows * 2 * I);
    float *act = (float *)malloc(sizeof(float) * (size_t)rows * I);
    uint8_t *aq = (uint8_t *)malloc((size_t)rows * I);
    float *aqf = (float *)malloc(sizeof(float) * (size_t)rows * I);
    float *sact = (float *)malloc(sizeof(float) * (size_t)rows * (I / 128));
    gemm_nt_scaled(xq, H, sx, wgu, H, sgu, 128, gu, 2 * I, rows, 2 * I, H, 128);
    for (int r = 0; r < rows; r++)
        for (int j = 0; j < I; j++)
            act[(size_t)r * I + j] = silu_ref(gu[(size_t)r * 2 * I + j]) * gu[(size_t)r * 2 * I + I + j];
    xso_quant_act_fp8(act, aq, sact, rows, I);
    decode_e4m3(aq, aqf, (size_t)rows * I);
    gemm_nt_scaled(aqf, I, sact, wd, I, sd, 128, y, H, rows, H, I, 128);
    free(wgu); free(wd); free(gu); free(act); free(aq); free(aqf); free(sact);
}

/* FP4 (e2m1 + e8m0/32) weights with MX-FP8 activations (e4m3 + e8m0/32). */
static void mlp_fp4(const float *xq, const float *sx, const uint8_t *wgu_p, const uint8_t *sgu8, const uint8_t *wd_p,
                    const uint8_t *sd8, float *y, int rows, int H, int I)
{
    float *wgu = (float *)malloc(sizeof(float) * (size_t)2 * I * H);
    float *wd = (float *)malloc(sizeof(float) * (size_t)H * I);
    float *sgu = (float *)malloc(sizeof(float) * (size_t)2 * I * (H / 32));
    float *sd = (float *)malloc(sizeof(float) * (size_t)H * (I / 32));
    decode_e2m1_packed(wgu_p, wgu, (size_t)2 * I * H);
    decode_e2m1_packed(wd_p, wd, (size_t)H * I);
    for (size_t i = 0; i < (size_t)2 * I * (H / 32); i++) sgu[i] = xso_e8m0_to_f32(sgu8[i]);
    for (size_t i = 0; i < (size_t)H * (I / 32); i++) sd[i] = xso_e8m0_to_f32(sd8[i]);
    float *gu = (float *)malloc(sizeof(float) * (size_t)rows * 2 * I);
    float *act = (float *)malloc(sizeof(float) * (size_t)rows * I);
    uint8_t *aq = (uint8_t *)malloc((size_t)rows * I);
    uint8_t *sa8 = (uint8_t *)malloc((size_t)rows * (I / 32));
    float *aqf = (float *)malloc(sizeof(float) * (size_t)rows * I);
    float *sact = (float *)malloc(sizeof(float) * (size_t)rows * (I / 32));
    gemm_nt_scaled(xq, H, sx, wgu, H, sgu, 1, gu, 2 * I, rows, 2 * I, H, 32);
    for (int r = 0; r < rows; r++)
        for (int j = 0; j < I; j++)
            act[(size_t)r * I + j] = silu_ref(gu[(size_t)r * 2 * I + j]) * gu[(size_t)r * 2 * I + I + j];
    xso_quant_act_mxfp8(act, aq, sa8, rows, I);
    decode_e4m3(aq, aqf, (size_t)rows * I);
    for (size_t i = 0; i < (size_t)rows * (I / 32); i++) sact[i] = xso_e8m0_to_f32(sa8[i]);
    gemm_nt_scaled(aqf, I, sact, wd, I, sd, 1, y, H, rows, H, I, 32);
    free(wgu); free(wd); free(sgu); free(sd); free(gu); free(act); free(aq); free(sa8); free(aqf); free(sact);
}

int xso_expert_mlp(int mode, const void *x, const void *gate_up_w, const void *down_w, float *y, int rows, int H, int I)
{
    if (mode != XSO_F32 && mode != XSO_BF16 && mode != XSO_BF16_REFCPU)
        return -1;
    if (mode == XSO_F32) {
        mlp_float(mode, (const float *)x, (const float *)gate_up_w, (const float *)down_w, y, rows, H, I);
        return 0;
    }
    float *xf = (float *)malloc(sizeof(float) * (size_t)rows * H);
    float *wgu = (float *)malloc(sizeof(float) * (size_t)2 * I * H);
    float *wd = (float *)malloc(sizeof(float) * (size_t)H * I);
    widen_bf16((const uint16_t *)x, xf, (size_t)rows * H);
    widen_bf16((const uint16_t *)gate_up_w, wgu, (size_t)2 * I * H);
    widen_bf16((const uint16_t *)down_w, wd, (size_t)H * I);
    mlp_float(mode, xf, wgu, wd, y, rows, H, I);
    free(xf); free(wgu); free(wd);
    return 0;
}

/* xstar_cpp/src/ops/rmsnorm.cpp:52-72 */
void xso_rmsnorm_bf16(const uint16_t *x, const uint16_t *w, uint16_t *out, int rows, int H, float eps)
{
    for (int r = 0; r < rows; r++) {
        const uint16_t *xr = x + (size_t)r * H;
        float rms = 0;
        for (int j = 0; j < H; j++) {
            float v = xso_bf16_to_f32(xr[j]);
            rms += v * v;
        }
        float inv_rms = 1.0f / sqrtf(rms / (float)H + eps);
        for (int j = 0; j < H; j++) {
            float n = xso_bf16_to_f32(xso_f32_to_bf16(xso_bf16_to_f32(xr[j]) * inv_rms));
            out[(size_t)r * H + j] = xso_f32_to_bf16(n * xso_bf16_to_f32(w[j]));
        }
    }
}

/* xstar_cpp/src/ops/add.cpp:40-49 */
void xso_add_bf16(const uint16_t *a, const uint16_t *b, uint16_t *out, size_t n)
{
    for (size_t i = 0; i < n; i++)
        out[i] = xso_f32_to_bf16(xso_bf16_to_f32(a[i]) + xso_bf16_to_f32(b[i]));
}

/* ------------------------------------------------------------------------------------------------ */
/* whole layer                                                                                       */
/* ------------------------------------------------------------------------------------------------ */
typedef struct Job {
    const XsOracleArgs *a;
    const float *xf;        /* (T,H) widened activations */
    const float *xq8;       /* (T,H) decoded e4m3 codes, 1x128 scales  (FP8; FP4 shared expert) */
    const float *sx8;       /* (T,H/128) */
    const float *xqmx;      /* (T,H) decoded e4m3 codes, 1x32 pow2 scales (FP4 routed) */
    const float *sxmx;      /* (T,H/32) */
    const int32_t *offsets, *perm;
    const unsigned char *in_subset; /* (T) or NULL */
    float *y_rows;          /* (T*K,H) */
    float *y_shared;        /* (T,H) */
    int next;               /* atomic work counter over E + S units */
} Job;

static void run_unit(Job *jb, int unit)
{
    const XsOracleArgs *a = jb->a;
    const int H = a->d.H, I = a->d.I, K = a->d.K, E = a->d.E, T = a->d.T;
    const int mode = a->mode;
    int is_shared = unit >= E;
    int e = unit;
    /* rows of this unit */
    int nrows_all = is_shared ? T : jb->offsets[e + 1] - jb->offsets[e];
    if (nrows_all == 0)
        return;
    int32_t *tok = (int32_t *)malloc(sizeof(int32_t) * (size_t)nrows_all);
    int32_t *dst = (int32_t *)malloc(sizeof(int32_t) * (size_t)nrows_all);
    int rows = 0;
    for (int r = 0; r < nrows_all; r++) {
        int t = is_shared ? r : jb->perm[jb->offsets[e] + r] / K;
        if (jb->in_subset && !jb->in_subset[t])
            continue;
        tok[rows] = t;
        dst[rows] = is_shared ? r : jb->offsets[e] + r;
        rows++;
    }
    if (rows == 0) {
        free(tok); free(dst);
        return;
    }
    float *y = (float *)malloc(sizeof(float) * (size_t)rows * H);
    float *yout = is_shared ? jb->y_shared : jb->y_rows;

    int fmt = mode;
    if (mode == XSO_FP4 && is_shared)
        fmt = XSO_FP8;

    if (fmt == XSO_F32 || fmt == XSO_BF16 || fmt == XSO_BF16_REFCPU) {
        /* row gather: embedding.cpp:37-46 */
        float *xs = (float *)malloc(sizeof(float) * (size_t)rows * H);
        for (int r = 0; r < rows; r++)
            memcpy(xs + (size_t)r * H, jb->xf + (size_t)tok[r] * H, sizeof(float) * (size_t)H);
        const void *gu_src = is_shared ? a->shared_gate_up_w : a->gate_up_w;
        const void *d_src = is_shared ? a->shared_down_w : a->down_w;
        size_t eoff = is_shared ? 0 : (size_t)e;
        if (fmt == XSO_F32) {
            mlp_float(fmt, xs, (const float *)gu_src + eoff * 2 * I * H, (const float *)d_src + eoff * H * I, y, rows, H, I);
        } else {
            float *wgu = (float *)malloc(sizeof(float) * (size_t)2 * I * H);
            float *wd = (float *)malloc(sizeof(float) * (size_t)H * I);
            widen_bf16((const uint16_t *)gu_src + eoff * 2 * I * H, wgu, (size_t)2 * I * H);
            widen_bf16((const uint16_t *)d_src + eoff * H * I, wd, (size_t)H * I);
            mlp_float(fmt, xs, wgu, wd, y, rows, H, I);
            free(wgu); free(wd);
        }
        free(xs);
    } else if (fmt == XSO_FP8) {
        int HB = H / 128, IB = I / 128;
        float *xs = (float *)malloc(sizeof(float) * (size_t)rows * H);
        float *ss = (float *)malloc(sizeof(float) * (size_t)rows * HB);
        for (int r = 0; r < rows; r++) {
            memcpy(xs + (size_t)r * H, jb->xq8 + (size_t)tok[r] * H, sizeof(float) * (size_t)H);
            memcpy(ss + (size_t)r * HB, jb->sx8 + (size_t)tok[r] * HB, sizeof(float) * (size_t)HB);
        }
        const uint8_t *gu_c = (const uint8_t *)(is_shared ? a->shared_gate_up_w : a->gate_up_w);
        const uint8_t *d_c = (const uint8_t *)(is_shared ? a->shared_down_w : a->down_w);
        const float *gu_s = (const float *)(is_shared ? a->shared_gate_up_scale : a->gate_up_scale);
        const float *d_s = (const float *)(is_shared ? a->shared_down_scale : a->down_scale);
        size_t eoff = is_shared ? 0 : (size_t)e;
        mlp_fp8(xs, ss, gu_c + eoff * 2 * I * H, gu_s + eoff * (2 * I / 128) * HB, d_c + eoff * H * I,
                d_s + eoff * HB * IB, y, rows, H, I);
        free(xs); free(ss);
    } else { /* XSO_FP4 routed */
        int HB = H / 32;
        float *xs = (float *)malloc(sizeof(float) * (size_t)rows * H);
        float *ss = (float *)malloc(sizeof(float) * (size_t)rows * HB);
        for (int r = 0; r < rows; r++) {
            memcpy(xs + (size_t)r * H, jb->xqmx + (size_t)tok[r] * H, sizeof(float) * (size_t)H);
            memcpy(ss + (size_t)r * HB, jb->sxmx + (size_t)tok[r] * HB, sizeof(float) * (size_t)HB);
        }
        const uint8_t *gu_p = (const uint8_t *)a->gate_up_w + (size_t)e * 2 * I * (H / 2);
        const uint8_t *d_p = (const uint8_t *)a->down_w + (size_t)e * H * (I / 2);
        const uint8_t *gu_s = (const uint8_t *)a->gate_up_scale + (size_t)e * 2 * I * (H / 32);
        const uint8_t *d_s = (const uint8_t *)a->down_scale + (size_t)e * H * (I / 32);
        mlp_fp4(xs, ss, gu_p, gu_s, d_p, d_s, y, rows, H, I);
        free(xs); free(ss);
    }
    for (int r = 0; r < rows; r++)
        memcpy(yout + (size_t)dst[r] * H, y + (size_t)r * H, sizeof(float) * (size_t)H);
    free(y); free(tok); free(dst);
}

static void *worker(void *p)
{
    Job *jb = (Job *)p;
    int units = jb->a->d.E + (jb->a->d.S ? 1 : 0);
    for (;;) {
        int u = __atomic_fetch_add(&jb->next, 1, __ATOMIC_RELAXED);
        if (u >= units)
            break;
        /* heavy shared expert first: unit order is E (shared), 0, 1, ... */
        int unit = jb->a->d.S ? (u == 0 ? jb->a->d.E : u - 1) : u;
        run_unit(jb, unit);
    }
    return NULL;
}

int xso_moe_forward(const XsOracleArgs *a)
{
    const int T = a->d.T, H = a->d.H, E = a->d.E, K = a->d.K, I = a->d.I, S = a->d.S;
    const int mode = a->mode;
    if (T < 0 || H <= 0 || E <= 0 || K <= 0 || K > E || I <= 0 || S < 0 || S > 1)
        return -1;
    if (mode < XSO_F32 || mode > XSO_FP4)
        return -2;
    if ((mode == XSO_FP8 || mode == XSO_FP4) && (H % 128 || I % 128))
        return -3;
    if (T == 0)
        return 0;
    build_tables();

    /* widen x and router_w */
    float *xf = (float *)malloc(sizeof(float) * (size_t)T * H);
    float *rw = (float *)malloc(sizeof(float) * (size_t)E * H);
    if (mode == XSO_F32) {
        memcpy(xf, a->x, sizeof(float) * (size_t)T * H);
        memcpy(rw, a->router_w, sizeof(float) * (size_t)E * H);
    } else {
        widen_bf16((const uint16_t *)a->x, xf, (size_t)T * H);
        widen_bf16((const uint16_t *)a->router_w, rw, (size_t)E * H);
    }
    float *logits = a->logits ? a->logits : (float *)malloc(sizeof(float) * (size_t)T * E);
    int32_t *ids = a->topk_ids ? a->topk_ids : (int32_t *)malloc(sizeof(int32_t) * (size_t)T * K);
    float *tw = a->topk_w ? a->topk_w : (float *)malloc(sizeof(float) * (size_t)T * K);
    int32_t *counts = a->counts ? a->counts : (int32_t *)malloc(sizeof(int32_t) * (size_t)E);
    int32_t *offsets = a->offsets ? a->offsets : (int32_t *)malloc(sizeof(int32_t) * (size_t)(E + 1));
    int32_t *perm = a->perm ? a->perm : (int32_t *)malloc(sizeof(int32_t) * (size_t)T * K);
    int32_t *inv = a->inv ? a->inv : (int32_t *)malloc(sizeof(int32_t) * (size_t)T * K);
    float *y_rows = a->y_rows ? a->y_rows : (float *)malloc(sizeof(float) * (size_t)T * K * H);

    xso_router_logits(xf, rw, logits, T, H, E);
    xso_topk(logits, a->router_bias, ids, tw, T, E, K);
    xso_permute(ids, counts, offsets, perm, inv, T, E, K);

    unsigned char *in_subset = NULL;
    if (a->token_subset) {
        in_subset = (unsigned char *)calloc((size_t)T, 1);
        for (int i = 0; i < a->n_subset; i++)
            in_subset[a->token_subset[i]] = 1;
    }

    Job jb;
    memset(&jb, 0, sizeof(jb));
    jb.a = a;
    jb.xf = xf;
    jb.offsets = offsets;
    jb.perm = perm;
    jb.in_subset = in_subset;
    jb.y_rows = y_rows;
    jb.y_shared = S ? (float *)malloc(sizeof(float) * (size_t)T * H) : NULL;

    float *xq8 = NULL, *sx8 = NULL, *xqmx = NULL, *sxmx = NULL;
    if (mode == XSO_FP8 || mode == XSO_FP4) {
        uint8_t *q = (uint8_t *)malloc((size_t)T * H);
        xq8 = (float *)malloc(sizeof(float) * (size_t)T * H);
        sx8 = (float *)malloc(sizeof(float) * (size_t)T * (H / 128));
        xso_quant_act_fp8(xf, q, sx8, T, H);
        decode_e4m3(q, xq8, (size_t)T * H);
        if (mode == XSO_FP4) {
            uint8_t *s8 = (uint8_t *)malloc((size_t)T * (H / 32));
            xqmx = (float *)malloc(sizeof(float) * (size_t)T * H);
            sxmx = (float *)malloc(sizeof(float) * (size_t)T * (H / 32));
            xso_quant_act_mxfp8(xf, q, s8, T, H);
            decode_e4m3(q, xqmx, (size_t)T * H);
            for (size_t i = 0; i < (size_t)T * (H / 32); i++)
                sxmx[i] = xso_e8m0_to_f32(s8[i]);
            free(s8);
        }
        free(q);
    }
    jb.xq8 = xq8; jb.sx8 = sx8; jb.xqmx = xqmx; jb.sxmx = sxmx;

    int nthreads = a->threads > 1 ? a->threads : 1;
    if (nthreads == 1) {
        worker(&jb);
    } else {
        pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nthreads);
        for (int i = 0; i < nthreads; i++)
            pthread_create(&th[i], NULL, worker, &jb);
        for (int i = 0; i < nthreads; i++)
            pthread_join(th[i], NULL);
        free(th);
    }

    /* combine: slot order j = 0..K-1, then the shared expert, f32, one downcast (add.cpp:27-49) */
    for (int t = 0; t < T; t++) {
        if (in_subset && !in_subset[t])
            continue;
        for (int h = 0; h < H; h++) {
            float acc = 0.0f;
            for (int j = 0; j < K; j++)
                acc += tw[(size_t)t * K + j] * y_rows[(size_t)inv[(size_t)t * K + j] * H + h];
            if (S)
                acc += jb.y_shared[(size_t)t * H + h];
            if (mode == XSO_F32)
                ((float *)a->out)[(size_t)t * H + h] = acc;
            else
                ((uint16_t *)a->out)[(size_t)t * H + h] = xso_f32_to_bf16(acc);
        }
    }

    free(xf); free(rw);
    if (!a->logits) free(logits);
    if (!a->topk_ids) free(ids);
    if (!a->topk_w) free(tw);
    if (!a->counts) free(counts);
    if (!a->offsets) free(offsets);
    if (!a->perm) free(perm);
    if (!a->inv) free(inv);
    if (!a->y_rows) free(y_rows);
    free(in_subset);
    free(jb.y_shared);
    free(xq8); free(sx8); free(xqmx); free(sxmx);
    return 0;
}
