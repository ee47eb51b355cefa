/*
 * TEST INFRASTRUCTURE ONLY.  Composes the MoE layer out of the reference's OWN compiled CPU ops:
 *   logits   = linear(x_f32, router_w_f32, nullptr)          (xstar_cpp/src/ops/linear.cpp:9-66)
 *   x_e      = embedding(x as a (T,H) table, token ids of e)  (xstar_cpp/src/ops/embedding.cpp:7-56)
 *   y_e      = mlp(x_e, gate_up_w[e], down_w[e])              (xstar_cpp/src/ops/mlp.cpp:47-86)
 *   shared   = mlp(x, shared_gate_up_w, shared_down_w)
 * The reference has no router selection, permutation or weighted combine, so the selection (topk_ids,
 * topk_w) and the permutation (offsets, perm) are INPUTS here, and the final weighted sum is the only
 * arithmetic in this file (slot order, shared expert last, f32, one downcast).
 *
 * The reference sources are compiled where they lie (see the Makefile); nothing is copied.
 * Used (a) to pin moe_oracle.c bit-for-bit and (b) as the timed "reference" CPU baseline.
 * Also exposes the two ops around the layer in the block, rmsnorm and add (xstar_cpp/src/ops/transformer_block.cpp:353).
 */
#include <atomic>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "bfloat16.h"
#include "ops/embedding.h"
#include "ops/linear.h"
#include "ops/add.h"
#include "ops/mlp.h"
#include "ops/rmsnorm.h"
#include "tensor.h"

namespace {

Tensor view(const void *p, std::vector<std::int64_t> shape, DType dt)
{
    return Tensor(p, std::move(shape), dt, Device::CPU);
}

float elem(const Tensor &t, std::size_t i)
{
    if (t.dtype() == DType::Float32)
        return t.data<float>()[i];
    return static_cast<float>(t.data<bfloat16>()[i]);
}

} // namespace

extern "C" {

/* logits (T,E) f32 from f32 copies of x and router_w (bf16 -> f32 widening is lossless, and gemm_cpu
 * widens every operand before multiplying, so this equals an unrounded bf16-input accumulation). */
int xsref_router_logits(const float *x, const float *router_w, float *logits, int T, int H, int E)
{
    try {
        Tensor xt = view(x, {T, H}, DType::Float32);
        Tensor wt = view(router_w, {E, H}, DType::Float32);
        Tensor out = linear(xt, wt, nullptr);
        std::memcpy(logits, out.data(), sizeof(float) * (std::size_t)T * E);
        return 0;
    } catch (...) {
        return -1;
    }
}

/*
 * bf16 != 0 selects BFloat16 tensors (storage = bf16 bits), else Float32.
 * y_rows (T*K,H) f32 receives mlp outputs (widened if bf16) in permuted row order; out has the storage dtype.
 * token_subset may be NULL; otherwise only assignments of those tokens are evaluated.
 */
int xsref_moe_experts_combine(int bf16, int T, int H, int E, int K, int I, int S, const void *x,
                              const void *gate_up_w, const void *down_w, const void *shared_gate_up_w,
                              const void *shared_down_w, const int32_t *topk_ids, const float *topk_w,
                              const int32_t *offsets, const int32_t *perm, const int32_t *inv, float *y_rows,
                              void *out, int threads, const int32_t *token_subset, int n_subset)
{
    (void)topk_ids;
    try {
        const DType dt = bf16 ? DType::BFloat16 : DType::Float32;
        const std::size_t es = bf16 ? 2 : 4;
        Tensor xt = view(x, {T, H}, dt);
        std::vector<unsigned char> in_subset;
        if (token_subset) {
            in_subset.assign((std::size_t)T, 0);
            for (int i = 0; i < n_subset; i++)
                in_subset[(std::size_t)token_subset[i]] = 1;
        }
        std::vector<float> y_shared;
        if (S)
            y_shared.assign((std::size_t)T * H, 0.0f);

        std::atomic<int> next{0};
        std::atomic<int> failed{0};
        const int units = E + (S ? 1 : 0);
        auto work = [&]() {
            try {
                for (;;) {
                    int u = next.fetch_add(1);
                    if (u >= units)
                        break;
                    int unit = S ? (u == 0 ? E : u - 1) : u;
                    bool is_shared = unit >= E;
                    int n_all = is_shared ? T : offsets[unit + 1] - offsets[unit];
                    std::vector<std::int64_t> tok;
                    std::vector<int> dst;
                    for (int r = 0; r < n_all; r++) {
                        int t = is_shared ? r : perm[offsets[unit] + r] / K;
                        if (!in_subset.empty() && !in_subset[(std::size_t)t])
                            continue;
                        tok.push_back(t);
                        dst.push_back(is_shared ? r : offsets[unit] + r);
                    }
                    if (tok.empty())
                        continue;
                    const char *gu = static_cast<const char *>(is_shared ? shared_gate_up_w : gate_up_w);
                    const char *dw = static_cast<const char *>(is_shared ? shared_down_w : down_w);
                    std::size_t eoff = is_shared ? 0 : (std::size_t)unit;
                    Tensor gut = view(gu + eoff * 2 * I * H * es, {2 * I, H}, dt);
                    Tensor dwt = view(dw + eoff * (std::size_t)H * I * es, {H, I}, dt);
                    Tensor xe = embedding(xt, tok.data(), {(std::int64_t)tok.size()});
                    Tensor ye = mlp(xe, gut, dwt);
                    float *yo = is_shared ? y_shared.data() : y_rows;
                    for (std::size_t r = 0; r < tok.size(); r++)
                        for (int h = 0; h < H; h++)
                            yo[(std::size_t)dst[r] * H + h] = elem(ye, r * H + h);
                }
            } catch (...) {
                failed = 1;
            }
        };
        int nt = threads > 1 ? threads : 1;
        if (nt == 1) {
            work();
        } else {
            std::vector<std::thread> th;
            for (int i = 0; i < nt; i++)
                th.emplace_back(work);
            for (auto &t : th)
                t.join();
        }
        if (failed)
            return -2;

        for (int t = 0; t < T; t++) {
            if (!in_subset.empty() && !in_subset[(std::size_t)t])
                continue;
            for (int h = 0; h < H; h++) {
                float acc = 0.0f;
                for (int j = 0; j < K; j++)
                    acc += topk_w[(std::size_t)t * K + j] * y_rows[(std::size_t)inv[(std::size_t)t * K + j] * H + h];
                if (S)
                    acc += y_shared[(std::size_t)t * H + h];
                if (bf16)
                    static_cast<bfloat16 *>(out)[(std::size_t)t * H + h] = bfloat16(acc);
                else
                    static_cast<float *>(out)[(std::size_t)t * H + h] = acc;
            }
        }
        return 0;
    } catch (...) {
        return -1;
    }
}

/* rmsnorm(x (rows,H) bf16, w (H) bf16, eps) -> out bf16, by the reference's own op (xstar_cpp/src/ops/rmsnorm.cpp) */
int xsref_rmsnorm_bf16(const void *x, const void *w, void *out, int rows, int H, float eps)
{
    try {
        Tensor xt = view(x, {rows, H}, DType::BFloat16);
        Tensor wt = view(w, {H}, DType::BFloat16);
        Tensor r = rmsnorm(xt, wt, eps);
        std::memcpy(out, r.data(), sizeof(std::uint16_t) * (std::size_t)rows * H);
        return 0;
    } catch (...) {
        return -1;
    }
}

/* add(a, b) on bf16 tensors of n elements, by the reference's own op (xstar_cpp/src/ops/add.cpp) */
int xsref_add_bf16(const void *a, const void *b, void *out, long long n)
{
    try {
        Tensor at = view(a, {n}, DType::BFloat16);
        Tensor bt = view(b, {n}, DType::BFloat16);
        Tensor r = add(at, bt);
        std::memcpy(out, r.data(), sizeof(std::uint16_t) * (std::size_t)n);
        return 0;
    } catch (...) {
        return -1;
    }
}

} // extern "C"
