// Op-level C ABI: one entry point per Backend method on the Dense path
// (src/backend.zig).  Each accepts host or device pointers; host operands are
// staged through device buffers owned by the context, which reproduces the call
// shape of the reference (operands in, result out, synchronous), while device
// pointers only enqueue on the context's stream.
#include <cmath>

#include "zn_internal.h"

namespace {

zn_status stage_reserve(zn_ctx *ctx, int slot, size_t floats) {
    if (ctx->stage_floats[slot] >= floats) return ZN_OK;
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(ctx->stage[slot]);
    ctx->stage[slot] = nullptr;
    ctx->stage_floats[slot] = 0;
    ZN_CUDA(ctx, cudaMalloc((void **)&ctx->stage[slot], floats * sizeof(float)));
    ctx->stage_floats[slot] = floats;
    return ZN_OK;
}

// Resolves one operand: device pointers pass through, host pointers are staged in `slot`.
struct Operand {
    float *dev = nullptr;
    float *host = nullptr;   // non-null when staged
    size_t count = 0;
};

zn_status resolve(zn_ctx *ctx, int slot, const float *p, size_t count, bool copy_in, Operand *out) {
    out->count = count;
    const int owner = zn_ptr_device(p);
    if (owner >= 0) {
        // a kernel of this context cannot be handed another GPU's memory (a TMA descriptor over it must not exist)
        if (owner != ctx->device)
            return zn_fail(ctx, ZN_ERR_INVALID_DEVICE, "operand lives on device %d, the context on device %d", owner, ctx->device);
        out->dev = const_cast<float *>(p);
        return ZN_OK;
    }
    ZN_TRY(stage_reserve(ctx, slot, count));
    out->dev = ctx->stage[slot];
    out->host = const_cast<float *>(p);
    if (copy_in) ZN_CUDA(ctx, cudaMemcpyAsync(out->dev, p, count * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    return ZN_OK;
}

// Copies a staged result back and synchronizes when any operand lived on the host.
zn_status finish(zn_ctx *ctx, const Operand *result, bool any_host) {
    if (result && result->host)
        ZN_CUDA(ctx, cudaMemcpyAsync(result->host, result->dev, result->count * sizeof(float), cudaMemcpyDeviceToHost,
                                     ctx->stream));
    if (any_host) {
        ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        return zn_check_device_status(ctx);
    }
    return ZN_OK;
}

int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

enum Orient { NN, TN, NT };

// One of the three products at the context's precision, on device operands.
zn_status gemm_dispatch(zn_ctx *ctx, Orient o, const float *a, const float *b, int64_t m, int64_t n, int64_t k,
                        zn_epilogue ep) {
    const zn_precision prec = ctx->precision;
    if (prec == ZN_FP32_SIMT || prec == ZN_FP32_EXACT) {
        const bool exact = prec == ZN_FP32_EXACT;
        switch (o) {
        case NN: return zn_gemm_simt(ctx, a, k, 1, b, n, 1, m, n, k, ep, exact);
        case TN: return zn_gemm_simt(ctx, a, 1, m, b, n, 1, m, n, k, ep, exact);   // A stored [k][m]
        default: return zn_gemm_simt(ctx, a, k, 1, b, 1, k, m, n, k, ep, exact);   // B stored [n][k]
        }
    }
    // Tensor-core modes.  A rows/cols as stored, B rows/cols as stored.
    const int64_t a_rows = (o == TN) ? k : m, a_cols = (o == TN) ? m : k;
    const int64_t b_rows = (o == NT) ? n : k, b_cols = (o == NT) ? k : n;
    const bool a_mn = (o == TN), b_mn = (o != NT);
    if (prec == ZN_BF16_TC) {
        const int64_t lda = round_up(a_cols, 8), ldb = round_up(b_cols, 8);
        const size_t fa = (size_t)(a_rows * lda + 1) / 2, fb = (size_t)(b_rows * ldb + 1) / 2;
        ZN_TRY(stage_reserve(ctx, 4, fa));
        ZN_TRY(stage_reserve(ctx, 5, fb));
        ZN_TRY(zn_k_convert(ctx, a, a_cols, ctx->stage[4], lda, true, a_rows, a_cols));
        ZN_TRY(zn_k_convert(ctx, b, b_cols, ctx->stage[5], ldb, true, b_rows, b_cols));
        return zn_gemm_tc(ctx, 0, ctx->stage[4], lda, a_mn, ctx->stage[5], ldb, b_mn, m, n, k, ep);
    }
    // TF32: fp32 operands feed the tensor cores directly when their pitch allows a TMA descriptor.
    const void *ap = a, *bp = b;
    int64_t lda = a_cols, ldb = b_cols;
    if (a_cols % 4 != 0 || (reinterpret_cast<uintptr_t>(a) & 15)) {
        lda = round_up(a_cols, 8);
        ZN_TRY(stage_reserve(ctx, 4, (size_t)(a_rows * lda)));
        ZN_TRY(zn_k_convert(ctx, a, a_cols, ctx->stage[4], lda, false, a_rows, a_cols));
        ap = ctx->stage[4];
    }
    if (b_cols % 4 != 0 || (reinterpret_cast<uintptr_t>(b) & 15)) {
        ldb = round_up(b_cols, 8);
        ZN_TRY(stage_reserve(ctx, 5, (size_t)(b_rows * ldb)));
        ZN_TRY(zn_k_convert(ctx, b, b_cols, ctx->stage[5], ldb, false, b_rows, b_cols));
        bp = ctx->stage[5];
    }
    return zn_gemm_tc(ctx, 1, ap, lda, a_mn, bp, ldb, b_mn, m, n, k, ep);
}

zn_status matmul_common(zn_ctx *ctx, Orient o, const float *a, const float *b, const float *bias, float *c, size_t m,
                        size_t n, size_t k, int accumulate, int act) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!a || !b || !c) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "matmul: null operand");
    if (m == 0 || n == 0 || k == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "matmul: zero dimension");
    if (act < ZN_ACT_RELU || act > ZN_ACT_ELU) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "unknown activation %d", act);
    cudaSetDevice(ctx->device);
    Operand A, B, C, Bi;
    ZN_TRY(resolve(ctx, 0, a, m * k, true, &A));
    ZN_TRY(resolve(ctx, 1, b, k * n, true, &B));
    ZN_TRY(resolve(ctx, 2, c, m * n, accumulate != 0, &C));
    if (bias) ZN_TRY(resolve(ctx, 3, bias, n, true, &Bi));
    zn_epilogue ep;
    ep.bias = bias ? Bi.dev : nullptr;
    ep.act = act == ZN_ACT_SOFTMAX ? (int)ZN_ACT_LINEAR : act;
    ep.out_f32 = C.dev;
    ep.ld_out_f32 = (int64_t)n;
    ep.accumulate = accumulate ? 1 : 0;
    ZN_TRY(gemm_dispatch(ctx, o, A.dev, B.dev, (int64_t)m, (int64_t)n, (int64_t)k, ep));
    if (act == ZN_ACT_SOFTMAX)     // row by row, as Dense.forward applies it (src/layer.zig:398-406)
        ZN_TRY(zn_k_softmax_rows(ctx, C.dev, false, (int64_t)n, nullptr, false, 0, C.dev, (int64_t)n, (int64_t)m, (int64_t)n,
                                 ctx->precision == ZN_FP32_EXACT));
    return finish(ctx, &C, A.host || B.host || C.host || Bi.host);
}

}   // namespace

extern "C" zn_status zn_matmul(zn_ctx *ctx, const float *a, const float *b, float *c, size_t m, size_t n, size_t k,
                               int32_t accumulate) {
    return matmul_common(ctx, NN, a, b, nullptr, c, m, n, k, accumulate, ZN_ACT_LINEAR);
}

extern "C" zn_status zn_matmul_transpose_a(zn_ctx *ctx, const float *a, const float *b, float *c, size_t m, size_t n,
                                           size_t k, int32_t accumulate) {
    return matmul_common(ctx, TN, a, b, nullptr, c, m, n, k, accumulate, ZN_ACT_LINEAR);
}

extern "C" zn_status zn_matmul_transpose_b(zn_ctx *ctx, const float *a, const float *b, float *c, size_t m, size_t n,
                                           size_t k, int32_t accumulate) {
    return matmul_common(ctx, NT, a, b, nullptr, c, m, n, k, accumulate, ZN_ACT_LINEAR);
}

extern "C" zn_status zn_matmul_bias_act(zn_ctx *ctx, const float *a, const float *b, const float *bias, float *c,
                                        size_t batch, size_t n, size_t k, zn_activation act) {
    if (ctx && !bias) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "matmul_bias_act: null bias");
    return matmul_common(ctx, NN, a, b, bias, c, batch, n, k, 0, (int)act);
}

extern "C" zn_status zn_add_bias(zn_ctx *ctx, float *out, size_t out_len, const float *bias, size_t bias_len) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!out || !bias) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "add_bias: null operand");
    if (bias_len == 0 || out_len % bias_len != 0) return zn_fail(ctx, ZN_ERR_SHAPE, "add_bias: output is not rows x bias_len");
    if (out_len == 0) return ZN_OK;
    Operand O, B;
    ZN_TRY(resolve(ctx, 0, out, out_len, true, &O));
    ZN_TRY(resolve(ctx, 1, bias, bias_len, true, &B));
    ZN_TRY(zn_k_add_bias(ctx, O.dev, (int64_t)(out_len / bias_len), (int64_t)bias_len, B.dev));
    return finish(ctx, &O, O.host || B.host);
}

extern "C" zn_status zn_accumulate_bias(zn_ctx *ctx, float *grad_bias, size_t bias_len, const float *g, size_t g_len) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!grad_bias || !g) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "accumulate_bias: null operand");
    if (bias_len == 0 || g_len % bias_len != 0) return zn_fail(ctx, ZN_ERR_SHAPE, "accumulate_bias: gradient is not rows x bias_len");
    if (g_len == 0) return ZN_OK;
    Operand GB, G;
    ZN_TRY(resolve(ctx, 0, grad_bias, bias_len, true, &GB));
    ZN_TRY(resolve(ctx, 1, g, g_len, true, &G));
    ZN_TRY(zn_k_bias_reduce(ctx, G.dev, false, (int64_t)bias_len, (int64_t)(g_len / bias_len), (int64_t)bias_len, GB.dev,
                            true, ctx->precision == ZN_FP32_EXACT));
    return finish(ctx, &GB, GB.host || G.host);
}

static bool act_supported(int act) { return act >= ZN_ACT_RELU && act <= ZN_ACT_ELU; }

extern "C" zn_status zn_activation_forward(zn_ctx *ctx, zn_activation act, const float *in, float *out, size_t count) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!in || !out) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "activation_forward: null operand");
    if (!act_supported(act)) return zn_fail(ctx, ZN_ERR_UNSUPPORTED, "activation %d is not on the Dense path", (int)act);
    if (count == 0) return ZN_OK;
    Operand I, O;
    ZN_TRY(resolve(ctx, 0, in, count, true, &I));
    if (in == out) O = I;
    else ZN_TRY(resolve(ctx, 1, out, count, false, &O));
    if (act == ZN_ACT_SOFTMAX)     // the whole slice is one vector (src/backend.zig:377-379)
        ZN_TRY(zn_k_softmax_rows(ctx, I.dev, false, (int64_t)count, nullptr, false, 0, O.dev, (int64_t)count, 1, (int64_t)count,
                                 ctx->precision == ZN_FP32_EXACT));
    else
        ZN_TRY(zn_k_act_forward(ctx, act, I.dev, O.dev, (int64_t)count));
    return finish(ctx, &O, I.host || O.host);
}

extern "C" zn_status zn_activation_backward(zn_ctx *ctx, zn_activation act, const float *y, const float *grad_out,
                                            float *grad_in, size_t count) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!y || !grad_out || !grad_in) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "activation_backward: null operand");
    if (!act_supported(act)) return zn_fail(ctx, ZN_ERR_UNSUPPORTED, "activation %d is not on the Dense path", (int)act);
    if (count == 0) return ZN_OK;
    Operand Y, GO, GI;
    ZN_TRY(resolve(ctx, 0, y, count, true, &Y));
    ZN_TRY(resolve(ctx, 1, grad_out, count, true, &GO));
    ZN_TRY(resolve(ctx, 2, grad_in, count, false, &GI));
    if (act == ZN_ACT_SOFTMAX)     // src/backend.zig:2650-2652
        ZN_TRY(zn_k_softmax_backward_rows(ctx, Y.dev, (int64_t)count, GO.dev, (int64_t)count, GI.dev, (int64_t)count, false, 1,
                                          (int64_t)count, ctx->precision == ZN_FP32_EXACT));
    else
        ZN_TRY(zn_k_act_backward(ctx, act, Y.dev, GO.dev, GI.dev, (int64_t)count));
    return finish(ctx, &GI, Y.host || GO.host || GI.host);
}

extern "C" zn_status zn_loss_forward(zn_ctx *ctx, zn_loss loss, const float *output, const float *target, size_t rows,
                                     size_t cols, float *loss_out) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!output || !target || !loss_out) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "loss_forward: null operand");
    if (rows == 0 || cols == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "loss_forward: empty output");
    Operand O, T;
    ZN_TRY(resolve(ctx, 0, output, rows * cols, true, &O));
    ZN_TRY(resolve(ctx, 1, target, rows * cols, true, &T));
    ZN_TRY(stage_reserve(ctx, 3, 16));
    ZN_TRY(zn_k_loss(ctx, loss, O.dev, (int64_t)cols, T.dev, nullptr, false, 0, (int64_t)rows, (int64_t)cols,
                     (float)(rows * cols), ctx->stage[3], ctx->precision == ZN_FP32_EXACT));
    ZN_CUDA(ctx, cudaMemcpyAsync(ctx->pinned_scalar, ctx->stage[3], sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const float sum = ctx->pinned_scalar[0];
    const bool flat = loss == ZN_LOSS_MSE || loss == ZN_LOSS_BINARY_CROSS_ENTROPY;
    *loss_out = flat ? sum / (float)(rows * cols) : (rows > 1 ? sum / (float)rows : sum);
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_loss_backward(zn_ctx *ctx, zn_loss loss, const float *output, const float *target,
                                      float *grad_out, size_t rows, size_t cols) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!output || !target || !grad_out) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "loss_backward: null operand");
    if (rows == 0 || cols == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "loss_backward: empty output");
    Operand O, T, G;
    ZN_TRY(resolve(ctx, 0, output, rows * cols, true, &O));
    ZN_TRY(resolve(ctx, 1, target, rows * cols, true, &T));
    ZN_TRY(resolve(ctx, 2, grad_out, rows * cols, false, &G));
    ZN_TRY(stage_reserve(ctx, 3, 16));
    ZN_TRY(zn_k_loss(ctx, loss, O.dev, (int64_t)cols, T.dev, G.dev, false, (int64_t)cols, (int64_t)rows, (int64_t)cols,
                     (float)(rows * cols), ctx->stage[3], ctx->precision == ZN_FP32_EXACT));
    return finish(ctx, &G, O.host || T.host || G.host);
}

extern "C" zn_status zn_evaluate_classification(zn_ctx *ctx, const float *outputs, const float *targets, size_t rows,
                                                size_t cols, size_t num_classes, uint64_t *confusion, float *metrics4) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (rows == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "EmptyInput: no samples to evaluate");
    if (!outputs || !targets) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "evaluate_classification: null operand");
    if (cols == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "evaluate_classification: zero columns");
    cudaSetDevice(ctx->device);
    Operand O, T;
    ZN_TRY(resolve(ctx, 0, outputs, rows * cols, true, &O));
    ZN_TRY(resolve(ctx, 1, targets, rows * cols, true, &T));
    return zn_k_classification_metrics(ctx, O.dev, (int64_t)cols, T.dev, (int64_t)cols, rows, cols, num_classes, confusion, metrics4);
}

extern "C" zn_status zn_sgd_update(zn_ctx *ctx, float *weights, const float *grads, size_t count, float learning_rate,
                                   float weight_decay) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!weights || !grads) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "sgd_update: null operand");
    if (count == 0) return ZN_OK;
    Operand W, G;
    ZN_TRY(resolve(ctx, 0, weights, count, true, &W));
    ZN_TRY(resolve(ctx, 1, grads, count, true, &G));
    zn_opt_args a{};
    a.w = W.dev; a.g = G.dev; a.count = count; a.lr = learning_rate; a.wd = weight_decay; a.w_clamp = 100.0f;
    ZN_TRY(zn_k_sgd(ctx, a, false));
    return finish(ctx, &W, W.host || G.host);
}

extern "C" zn_status zn_sgd_update_bias(zn_ctx *ctx, float *bias, const float *grads, size_t count, float learning_rate) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!bias || !grads) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "sgd_update_bias: null operand");
    if (count == 0) return ZN_OK;
    Operand W, G;
    ZN_TRY(resolve(ctx, 0, bias, count, true, &W));
    ZN_TRY(resolve(ctx, 1, grads, count, true, &G));
    zn_opt_args a{};
    a.w = W.dev; a.g = G.dev; a.count = count; a.lr = learning_rate; a.w_clamp = 50.0f;
    ZN_TRY(zn_k_sgd(ctx, a, true));
    return finish(ctx, &W, W.host || G.host);
}

extern "C" zn_status zn_adam_update(zn_ctx *ctx, float *weights, const float *grads, float *m, float *v, size_t count,
                                    float lr, float beta1, float beta2, float eps, float bias_corr1, float bias_corr2) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!weights || !grads || !m || !v) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "adam_update: null operand");
    if (count == 0) return ZN_OK;
    Operand W, G, M, V;
    ZN_TRY(resolve(ctx, 0, weights, count, true, &W));
    ZN_TRY(resolve(ctx, 1, grads, count, true, &G));
    ZN_TRY(resolve(ctx, 2, m, count, true, &M));
    ZN_TRY(resolve(ctx, 3, v, count, true, &V));
    zn_opt_args a{};
    a.w = W.dev; a.g = G.dev; a.m = M.dev; a.v = V.dev; a.count = count;
    a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.bc1 = bias_corr1; a.bc2 = bias_corr2; a.w_clamp = 100.0f;
    ZN_TRY(zn_k_adam(ctx, a));
    const bool any_host = W.host || G.host || M.host || V.host;
    if (M.host) ZN_CUDA(ctx, cudaMemcpyAsync(M.host, M.dev, count * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    if (V.host) ZN_CUDA(ctx, cudaMemcpyAsync(V.host, V.dev, count * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    return finish(ctx, &W, any_host);
}

extern "C" zn_status zn_rmsprop_update(zn_ctx *ctx, float *weights, const float *grads, float *g_avg, size_t count,
                                       float lr, float rho, float eps) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!weights || !grads || !g_avg) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "rmsprop_update: null operand");
    if (count == 0) return ZN_OK;
    Operand W, G, S;
    ZN_TRY(resolve(ctx, 0, weights, count, true, &W));
    ZN_TRY(resolve(ctx, 1, grads, count, true, &G));
    ZN_TRY(resolve(ctx, 2, g_avg, count, true, &S));
    zn_opt_args a{};
    a.w = W.dev; a.g = G.dev; a.m = S.dev; a.count = count;
    a.lr = lr; a.rho = rho; a.eps = eps; a.w_clamp = 100.0f;
    ZN_TRY(zn_k_rmsprop(ctx, a));
    if (S.host) ZN_CUDA(ctx, cudaMemcpyAsync(S.host, S.dev, count * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    return finish(ctx, &W, W.host || G.host || S.host);
}

extern "C" zn_status zn_clip_grad_norm(zn_ctx *ctx, float *const *grads, const size_t *counts, size_t tensor_count,
                                       float *norm_out, float *factor_out) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!grads || !counts || tensor_count == 0 || tensor_count > 32)
        return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "clip_grad_norm: 1..32 tensors");
    const bool dev = zn_is_device_ptr(grads[0]);
    size_t total = 0;
    for (size_t i = 0; i < tensor_count; ++i) {
        if (!grads[i]) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "clip_grad_norm: null tensor");
        if (zn_is_device_ptr(grads[i]) != dev) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "clip_grad_norm: mixed host and device tensors");
        total += (counts[i] + 3) / 4 * 4;
    }
    ZN_TRY(stage_reserve(ctx, 3, 16));
    std::vector<zn_seg> segs(tensor_count);
    std::vector<float *> dptr(tensor_count);
    if (dev) {
        for (size_t i = 0; i < tensor_count; ++i) { dptr[i] = grads[i]; segs[i] = {grads[i], counts[i]}; }
    } else {
        ZN_TRY(stage_reserve(ctx, 0, total));
        size_t off = 0;
        for (size_t i = 0; i < tensor_count; ++i) {
            dptr[i] = ctx->stage[0] + off;
            ZN_CUDA(ctx, cudaMemcpyAsync(dptr[i], grads[i], counts[i] * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
            segs[i] = {dptr[i], counts[i]};
            off += (counts[i] + 3) / 4 * 4;
        }
    }
    ZN_TRY(zn_k_grad_norm(ctx, segs.data(), (int)tensor_count, ctx->stage[3], ctx->precision == ZN_FP32_EXACT));
    for (size_t i = 0; i < tensor_count; ++i) ZN_TRY(zn_k_scale(ctx, dptr[i], counts[i], ctx->stage[3] + 1));
    if (!dev)
        for (size_t i = 0; i < tensor_count; ++i)
            ZN_CUDA(ctx, cudaMemcpyAsync(grads[i], dptr[i], counts[i] * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    if (!dev || norm_out || factor_out) {
        ZN_CUDA(ctx, cudaMemcpyAsync(ctx->pinned_scalar, ctx->stage[3], 2 * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
        ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (norm_out) *norm_out = ctx->pinned_scalar[0];
        if (factor_out) *factor_out = ctx->pinned_scalar[1];
        return zn_check_device_status(ctx);
    }
    return ZN_OK;
}
