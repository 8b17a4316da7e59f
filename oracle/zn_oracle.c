/*
 * zn_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Single-threaded CPU restatement of ZigNeuron's CPU Dense-layer training
 * path.  It exists only so that tests, the smoke check and the CPU-baseline
 * leg of the benchmark have something to compare the CUDA path against.  The
 * shipped library never links, loads or calls anything in this file.
 *
 * Every function cites the reference source (path within the ZigNeuron
 * tree : line) whose arithmetic it follows, operation by operation: the same
 * loop order, the same association of the floating point expressions, a
 * multiply followed by a separate add where the reference writes `a * b + c`
 * (Zig does not contract that into an FMA; build this file with
 * -ffp-contract=off so GCC does not either).
 *
 * Arithmetic that lives in Zig's standard library (std.math.exp, @log,
 * std.math.pow, @sqrt, std.math.tanh) is restated with libm expf/logf/powf/
 * sqrtf/tanhf; the difference is at most an ulp or two, inside every
 * tolerance the reference's own tests use.  The exp and log of the softmax and
 * cross-entropy paths are evaluated in double precision and rounded once
 * (zo_exp1 / zo_log1): that is the correctly rounded float in all but isolated
 * cases, a definition that does not move with the libm at hand, and one a GPU
 * can reproduce bit for bit.  An ulp there matters: under Adam a one-ulp
 * difference in a softmax sends a 100-step run down another path.
 *
 * Pinning: the known-answer values of the reference's unit tests
 * (tests/golden/reference_kat.json, transcribed from the files under src/test/unit)
 * are checked against this file by tests/test_oracle_golden.py.  Initial
 * weight VALUES are "parity unpinned": no reference test fixes a single
 * initial weight and Zig's PRNG is not restated here; callers inject weights.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

static inline float zo_exp1(float x) { return (float)exp((double)x); }
static inline float zo_log1(float x) { return (float)log((double)x); }
#include <string.h>

#define ZO_API __attribute__((visibility("default")))

/* Activation tags: order of `Activation` in src/activation.zig:14-22. */
enum { ZO_RELU = 0, ZO_SIGMOID = 1, ZO_TANH = 2, ZO_SOFTMAX = 3, ZO_LINEAR = 4,
       ZO_GELU = 5, ZO_LEAKY_RELU = 6, ZO_ELU = 7 };
/* Loss tags: order of `Loss` in src/loss.zig:12-22. */
enum { ZO_MSE = 0, ZO_CE = 1, ZO_CE_LOGITS = 2, ZO_BCE = 3, ZO_KL = 4 };
enum { ZO_OPT_SGD = 0, ZO_OPT_ADAM = 1, ZO_OPT_MOMENTUM = 2, ZO_OPT_ADAMW = 3, ZO_OPT_RMSPROP = 4 };

/* ------------------------------------------------------------------ GEMMs */

/* NN product, one output row at a time.
 * src/backend.zig:169-173 (matMul with m>1 -> matMulBatch), :2609-2613
 * (cpuMatMulBatch calls cpuMatMul with m=1 per row), :2520-2607 (cpuMatMul:
 * row zeroed unless accumulating, then for p ascending c[j] += a[p]*b[p][j];
 * the 8-wide vector branch does the same multiply and add per element). */
ZO_API void zo_matmul(const float *a, const float *b, float *c,
                      size_t m, size_t n, size_t k, int accumulate) {
    for (size_t i = 0; i < m; ++i) {
        const float *a_row = a + i * k;
        float *c_row = c + i * n;
        if (!accumulate) memset(c_row, 0, n * sizeof(float));
        for (size_t p = 0; p < k; ++p) {
            const float a_val = a_row[p];
            const float *b_row = b + p * n;
            for (size_t j = 0; j < n; ++j) c_row[j] += a_val * b_row[j];
        }
    }
}

/* TN product, A stored [k][m].  src/backend.zig:2615-2630. */
ZO_API void zo_matmul_transpose_a(const float *a, const float *b, float *c,
                                  size_t m, size_t n, size_t k, int accumulate) {
    for (size_t i = 0; i < m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (size_t p = 0; p < k; ++p) sum += a[p * m + i] * b[p * n + j];
            if (accumulate) c[i * n + j] += sum; else c[i * n + j] = sum;
        }
    }
}

/* Rows [row0,row1) of the TN product only; used to time a slab of a product
 * too large to finish on one core (rows are independent, :2617). */
ZO_API void zo_matmul_transpose_a_rows(const float *a, const float *b, float *c,
                                       size_t m, size_t n, size_t k,
                                       size_t row0, size_t row1) {
    for (size_t i = row0; i < row1 && i < m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (size_t p = 0; p < k; ++p) sum += a[p * m + i] * b[p * n + j];
            c[i * n + j] = sum;
        }
    }
}

/* NT product, B stored [n][k].  src/backend.zig:2632-2647. */
ZO_API void zo_matmul_transpose_b(const float *a, const float *b, float *c,
                                  size_t m, size_t n, size_t k, int accumulate) {
    for (size_t i = 0; i < m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (size_t p = 0; p < k; ++p) sum += a[i * k + p] * b[j * k + p];
            if (accumulate) c[i * n + j] += sum; else c[i * n + j] = sum;
        }
    }
}

/* ------------------------------------------------------ bias, activations */

/* src/backend.zig:658-671 (cpu arm of addBias). */
ZO_API void zo_add_bias(float *out, size_t out_len, const float *bias, size_t bias_len) {
    const size_t batch = out_len / bias_len;
    for (size_t b = 0; b < batch; ++b)
        for (size_t i = 0; i < bias_len; ++i) out[b * bias_len + i] += bias[i];
}

/* src/backend.zig:706-713 (cpuAccumulateBias): rows ascending, += into gb. */
ZO_API void zo_accumulate_bias(float *grad_bias, size_t bias_len,
                               const float *grad_after_act, size_t g_len) {
    const size_t batch = g_len / bias_len;
    for (size_t b = 0; b < batch; ++b)
        for (size_t i = 0; i < bias_len; ++i) grad_bias[i] += grad_after_act[b * bias_len + i];
}

/* src/activation.zig:24-35 with :97-99 (relu), :105-112 (sigmoid),
 * :118-120 (tanh), :30 (linear). */
static float act_forward(int act, float x) {
    switch (act) {
    case ZO_RELU: return x > 0 ? x : 0;
    case ZO_SIGMOID:
        if (x >= 0) return 1 / (1 + expf(-x));
        else { const float e = expf(x); return e / (1 + e); }
    case ZO_TANH: return tanhf(x);
    case ZO_GELU: {                                  /* src/activation.zig:128-134 */
        const float c = 0.7978845608f, k = 0.044715f;
        const float x3 = x * x * x;
        const float inner = c * (x + k * x3);
        return 0.5f * x * (1.0f + tanhf(inner));
    }
    case ZO_LEAKY_RELU: return x > 0 ? x : 0.01f * x;
    case ZO_ELU: return x > 0 ? x : 1.0f * (expf(x) - 1.0f);
    default: return x;
    }
}

/* src/activation.zig:37-48 with :101-103, :114-116, :122-124; takes the
 * ACTIVATED output y.  relu follows src/optimization.zig:229-251
 * (y > 0 ? grad : 0, a select, not a multiply). */
static float act_backward(int act, float y, float g) {
    switch (act) {
    case ZO_RELU: return y > 0 ? g : 0;
    case ZO_SIGMOID: return g * y * (1 - y);          /* optimization.zig sigmoidBackwardVectorized scalar tail */
    case ZO_TANH: return g * (1 - y * y);
    case ZO_GELU: {                                  /* src/activation.zig:139-150: derivative taken at x = y */
        const float c = 0.7978845608f, k = 0.044715f;
        const float x = y;
        const float x3 = x * x * x;
        const float inner = c * (x + k * x3);
        const float t = tanhf(inner);
        const float sech2 = 1.0f - t * t;
        return (0.5f * (1.0f + t) + 0.5f * x * sech2 * c * (1.0f + 3.0f * k * x * x)) * g;
    }
    case ZO_LEAKY_RELU: return (y > 0 ? 1.0f : 0.01f) * g;
    case ZO_ELU: return (y > 0 ? 1.0f : y + 1.0f) * g;
    default: return g;
    }
}

/* Activation.softmaxForward, src/activation.zig:51-78: one vector, in == out allowed. */
ZO_API void zo_softmax_forward(const float *in, float *out, size_t n) {
    float max_val = -INFINITY;
    for (size_t i = 0; i < n; ++i) if (in[i] > max_val) max_val = in[i];
    float sum = 0;
    for (size_t i = 0; i < n; ++i) { out[i] = zo_exp1(in[i] - max_val); sum += out[i]; }
    if (sum > 0) { for (size_t i = 0; i < n; ++i) out[i] /= sum; }
    else { const float u = 1.0f / (float)n; for (size_t i = 0; i < n; ++i) out[i] = u; }
}

/* Activation.softmaxBackward, src/activation.zig:82-95. */
ZO_API void zo_softmax_backward(const float *s, const float *grad_out, float *grad_in, size_t n) {
    float dot = 0;
    for (size_t i = 0; i < n; ++i) dot += grad_out[i] * s[i];
    for (size_t i = 0; i < n; ++i) grad_in[i] = s[i] * (grad_out[i] - dot);
}

/* src/backend.zig:367-386 (cpu arm): element-wise, in == out allowed; softmax takes the whole
 * slice as one vector. */
ZO_API void zo_activation_forward(int act, const float *in, float *out, size_t n) {
    if (act == ZO_SOFTMAX) { zo_softmax_forward(in, out, n); return; }
    for (size_t i = 0; i < n; ++i) out[i] = act_forward(act, in[i]);
}

/* src/backend.zig:2649-2669 (cpuActivationBackward). */
ZO_API void zo_activation_backward(int act, const float *y, const float *grad_out,
                                   float *grad_in, size_t n) {
    if (act == ZO_LINEAR) { memcpy(grad_in, grad_out, n * sizeof(float)); return; }
    if (act == ZO_SOFTMAX) { zo_softmax_backward(y, grad_out, grad_in, n); return; }
    for (size_t i = 0; i < n; ++i) grad_in[i] = act_backward(act, y[i], grad_out[i]);
}

/* ------------------------------------------------------------------- loss */

/* src/loss.zig:93-101. */
ZO_API float zo_mse_forward(const float *o, const float *t, size_t n) {
    float sum = 0;
    for (size_t i = 0; i < n; ++i) { const float d = o[i] - t[i]; sum += d * d; }
    return sum / (float)n;
}

/* src/loss.zig:103-109: 2*(o-t)/n, n = number of elements handed in. */
ZO_API void zo_mse_backward(const float *o, const float *t, float *g, size_t n) {
    const float nf = (float)n;
    for (size_t i = 0; i < n; ++i) g[i] = 2 * (o[i] - t[i]) / nf;
}

/* src/loss.zig:202-229: one vector = one sample. */
ZO_API float zo_ce_logits_forward(const float *logits, const float *target, size_t n) {
    float mx = logits[0];
    for (size_t i = 1; i < n; ++i) if (logits[i] > mx) mx = logits[i];
    float sum_exp = 0;
    for (size_t i = 0; i < n; ++i) sum_exp += zo_exp1(logits[i] - mx);
    const float lse = zo_log1(sum_exp) + mx;
    float loss = 0;
    for (size_t i = 0; i < n; ++i) if (target[i] > 0.5f) { loss = -(logits[i] - lse); break; }
    return loss;
}

/* src/loss.zig:233-254: softmax(logits) - target. */
ZO_API void zo_ce_logits_backward(const float *logits, const float *target, float *g, size_t n) {
    if (n == 0) return;
    float mx = logits[0];
    for (size_t i = 1; i < n; ++i) if (logits[i] > mx) mx = logits[i];
    float sum_exp = 0;
    for (size_t i = 0; i < n; ++i) { g[i] = zo_exp1(logits[i] - mx); sum_exp += g[i]; }
    for (size_t i = 0; i < n; ++i) g[i] = (g[i] / sum_exp) - target[i];
}

/* Loss.crossEntropyForward, src/loss.zig:110-169: despite the enum's comment it takes LOGITS; the
 * exponent is clamped to [-50, 50], every target entry above 0.5 contributes and the result is
 * their mean; degenerate inputs give 0. */
ZO_API float zo_ce_forward(const float *o, const float *t, size_t n) {
    if (n == 0) return 0;
    float mx = -INFINITY;
    for (size_t i = 0; i < n; ++i) if (o[i] > mx) mx = o[i];
    if (mx == -INFINITY) return 0;
    float lse = 0;
    for (size_t i = 0; i < n; ++i) {
        const float diff = o[i] - mx;
        const float cd = diff > 50 ? 50 : (diff < -50 ? -50 : diff);
        lse += zo_exp1(cd);
    }
    if (!isfinite(lse) || lse <= 0) return 0;
    lse = zo_log1(lse) + mx;
    float loss_sum = 0, count = 0;
    for (size_t i = 0; i < n; ++i)
        if (t[i] > 0.5f) { loss_sum += lse - o[i]; count += 1; }
    if (count == 0) return 0;
    return loss_sum / count;
}

/* Loss.crossEntropyBackward, src/loss.zig:171-196: softmax(output) - target. */
ZO_API void zo_ce_backward(const float *o, const float *t, float *g, size_t n) {
    zo_ce_logits_backward(o, t, g, n);      /* the same arithmetic, statement for statement */
}

/* Loss.binaryCrossEntropyForward, src/loss.zig:255-274 (outputs are probabilities). */
ZO_API float zo_bce_forward(const float *o, const float *t, size_t n) {
    float sum = 0;
    const float eps = 1e-7f;
    for (size_t i = 0; i < n; ++i) {
        float p = o[i];
        if (p < eps) p = eps;
        if (p > 1 - eps) p = 1 - eps;
        float q = 1 - p;
        if (q < eps) q = eps;
        if (q > 1 - eps) q = 1 - eps;
        sum -= t[i] * logf(p) + (1 - t[i]) * logf(q);
    }
    return sum / (float)n;
}

/* Loss.binaryCrossEntropyBackward, src/loss.zig:286-302: (p - t) / n, n = elements handed in. */
ZO_API void zo_bce_backward(const float *o, const float *t, float *g, size_t n, size_t divisor) {
    const float nf = (float)divisor, eps = 1e-7f;
    for (size_t i = 0; i < n; ++i) {
        float p = o[i];
        if (p < eps) p = eps;
        if (p > 1.0f - eps) p = 1.0f - eps;
        g[i] = (p - t[i]) / nf;
    }
}

/* Row-wise batching of the per-vector cross-entropies: gradient per row with no 1/B
 * (kernels/loss.cu:123-155), loss = mean over rows (kernels/loss.cu:175-213,
 * `total_loss / num_samples`); each row uses the src/loss.zig formulas. */
ZO_API float zo_ce_logits_rows(const float *logits, const float *target, float *g,
                               size_t rows, size_t cols) {
    float total = 0;
    for (size_t r = 0; r < rows; ++r) {
        total += zo_ce_logits_forward(logits + r * cols, target + r * cols, cols);
        if (g) zo_ce_logits_backward(logits + r * cols, target + r * cols, g + r * cols, cols);
    }
    return total / (float)rows;
}

static int loss_is_flat(int loss) { return loss == ZO_MSE || loss == ZO_BCE; }

/* src/loss.zig:34-60 dispatch.  MSE and BCE are flat over all rows*cols elements; the
 * cross-entropies are taken row by row and averaged over the rows (one row: the plain call). */
ZO_API float zo_loss_forward(int loss, const float *o, const float *t, size_t rows, size_t cols) {
    if (loss == ZO_MSE) return zo_mse_forward(o, t, rows * cols);
    if (loss == ZO_BCE) return zo_bce_forward(o, t, rows * cols);
    if (loss == ZO_CE) {
        if (rows == 1) return zo_ce_forward(o, t, cols);
        float total = 0;
        for (size_t r = 0; r < rows; ++r) total += zo_ce_forward(o + r * cols, t + r * cols, cols);
        return total / (float)rows;
    }
    if (rows == 1) return zo_ce_logits_forward(o, t, cols);
    return zo_ce_logits_rows(o, t, NULL, rows, cols);
}

ZO_API void zo_loss_backward(int loss, const float *o, const float *t, float *g, size_t rows, size_t cols) {
    if (loss == ZO_MSE) { zo_mse_backward(o, t, g, rows * cols); return; }
    if (loss == ZO_BCE) { zo_bce_backward(o, t, g, rows * cols, rows * cols); return; }
    for (size_t r = 0; r < rows; ++r)
        zo_ce_logits_backward(o + r * cols, t + r * cols, g + r * cols, cols);
}

/* ------------------------------------------------------------- optimizers */

static float clamp_grad(float g) {              /* NaN -> 0, else clamp to [-5,5] */
    if (isnan(g)) return 0.0f;
    return fminf(5.0f, fmaxf(-5.0f, g));
}

/* src/backend.zig:2722-2739 (cpuSgdUpdate). */
ZO_API void zo_sgd_update(float *w, const float *g_raw, size_t n, float lr, float wd) {
    for (size_t i = 0; i < n; ++i) {
        const float g = clamp_grad(g_raw[i]);
        w[i] -= lr * (g + wd * w[i]);
        w[i] = fminf(100.0f, fmaxf(-100.0f, w[i]));
    }
}

/* src/backend.zig:2741-2758 (cpuSgdUpdateBias): clamp +-50, no decay. */
ZO_API void zo_sgd_update_bias(float *b, const float *g_raw, size_t n, float lr) {
    for (size_t i = 0; i < n; ++i) {
        const float g = clamp_grad(g_raw[i]);
        b[i] -= lr * g;
        b[i] = fminf(50.0f, fmaxf(-50.0f, b[i]));
    }
}

/* src/backend.zig:2760-2772 (cpuAdamUpdate); the association of each product
 * is the reference's: (1-b2)*g*g is ((1-b2)*g)*g, lr*m_hat/(...) is
 * (lr*m_hat)/(...). */
ZO_API void zo_adam_update(float *w, const float *g_raw, float *m, float *v, size_t n,
                           float lr, float beta1, float beta2, float eps,
                           float bias_corr1, float bias_corr2) {
    for (size_t i = 0; i < n; ++i) {
        const float g = clamp_grad(g_raw[i]);
        m[i] = beta1 * m[i] + (1.0f - beta1) * g;
        v[i] = beta2 * v[i] + (1.0f - beta2) * g * g;
        const float m_hat = m[i] / bias_corr1;
        const float v_hat = v[i] / bias_corr2;
        w[i] -= lr * m_hat / (sqrtf(v_hat) + eps);
        w[i] = fminf(100.0f, fmaxf(-100.0f, w[i]));
    }
}

/* The two host-side bias corrections of Adam.step, src/optimizer.zig:210-213. */
ZO_API void zo_adam_bias_corrections(float beta1, float beta2, size_t t, float *bc1, float *bc2) {
    const float tf = (float)t;
    *bc1 = 1.0f - powf(beta1, tf);
    *bc2 = 1.0f - powf(beta2, tf);
}

/* src/backend.zig:2774-2783 (cpuRmspropUpdate). */
ZO_API void zo_rmsprop_update(float *w, const float *g_raw, float *g_avg, size_t n, float lr, float rho, float eps) {
    for (size_t i = 0; i < n; ++i) {
        const float g = clamp_grad(g_raw[i]);
        g_avg[i] = rho * g_avg[i] + (1.0f - rho) * g * g;
        w[i] -= lr * g / (sqrtf(g_avg[i]) + eps);
        w[i] = fminf(100.0f, fmaxf(-100.0f, w[i]));
    }
}

/* Sgd.step with momentum > 0, src/optimizer.zig:114-159: v = momentum*v - lr*g; w = w + v, built from
 * Backend.scale and Backend.elementWise, so without the gradient or weight clamps of the plain path. */
ZO_API void zo_sgd_momentum_update(float *w, const float *g, float *vel, size_t n, float lr, float momentum) {
    for (size_t i = 0; i < n; ++i) {
        const float scaled_v = vel[i] * momentum;
        const float scaled_g = g[i] * lr;
        vel[i] = scaled_v - scaled_g;
        w[i] = w[i] + vel[i];
    }
}

/* The decoupled decay AdamW.step applies after adamUpdate, src/optimizer.zig:288-296. */
ZO_API void zo_decoupled_decay(float *w, size_t n, float lr, float weight_decay) {
    const float wdlr = lr * weight_decay;
    for (size_t i = 0; i < n; ++i) w[i] = w[i] * (1.0f - wdlr);
}

/* Global gradient-norm clip of Network.trainStep, src/network.zig:513-535:
 * one running f32 sum over every tensor in the order given, sqrt, and when
 * the norm exceeds 1.0 every gradient is multiplied by 1/(norm + 1e-6).
 * Returns the norm; *clip_factor is 1.0 when no clipping happened. */
ZO_API float zo_clip_grad_norm(float **grads, const size_t *lens, size_t count, float *clip_factor) {
    const float max_norm = 1.0f;
    float total = 0.0f;
    for (size_t t = 0; t < count; ++t)
        for (size_t i = 0; i < lens[t]; ++i) total += grads[t][i] * grads[t][i];
    total = sqrtf(total);
    float f = 1.0f;
    if (total > max_norm) {
        f = max_norm / (total + 1e-6f);
        for (size_t t = 0; t < count; ++t)
            for (size_t i = 0; i < lens[t]; ++i) grads[t][i] *= f;
    }
    if (clip_factor) *clip_factor = f;
    return total;
}

/* src/cuda_multi_gpu.zig:247-265 (distributeWorkload, .round_robin):
 * contiguous shard i gets total/n rows, plus one for i < total % n. */
ZO_API void zo_distribute_round_robin(size_t total, size_t n, size_t i, size_t *start, size_t *end) {
    const size_t base = total / n, rem = total % n;
    size_t off = 0;
    for (size_t d = 0; d < i; ++d) off += base + (d < rem ? 1 : 0);
    *start = off;
    *end = off + base + (i < rem ? 1 : 0);
}

/* ---------------------------------------------------------------- network */

typedef struct {
    size_t in, out;
    int act;
    float *W, *b, *gW, *gb;            /* src/layer.zig:291-301 */
    float *x_cache, *y_cache;          /* LayerCache, src/network.zig:33-36 */
    size_t cache_rows;
    int opt;                           /* Network.optimizers[i], src/network.zig:44 */
    float beta1, beta2, eps, wd, momentum, rho;
    size_t t;
    float *mW, *vW, *mb, *vb;          /* Adam state, src/optimizer.zig:169-184 */
} zo_layer;

typedef struct zo_net {
    zo_layer *layers;
    size_t count, cap;
    float *work1, *work2;              /* grad_work_1/2, src/network.zig:425-426 */
    size_t work_len;
    float last_norm, last_clip;
} zo_net;

ZO_API zo_net *zo_net_create(void) { return (zo_net *)calloc(1, sizeof(zo_net)); }

ZO_API void zo_net_destroy(zo_net *net) {
    if (!net) return;
    for (size_t i = 0; i < net->count; ++i) {
        zo_layer *l = &net->layers[i];
        free(l->W); free(l->b); free(l->gW); free(l->gb); free(l->x_cache); free(l->y_cache);
        free(l->mW); free(l->vW); free(l->mb); free(l->vb);
    }
    free(net->layers); free(net->work1); free(net->work2); free(net);
}

/* Network.addDense -> Dense.init, src/layer.zig:306-348.  Weights start at 0
 * here; callers inject values (initial weights are parity-unpinned). */
ZO_API int zo_net_add_dense(zo_net *net, size_t in, size_t out, int act) {
    if (in == 0 || out == 0) return -1;
    if (net->count == net->cap) {
        net->cap = net->cap ? net->cap * 2 : 4;
        net->layers = (zo_layer *)realloc(net->layers, net->cap * sizeof(zo_layer));
    }
    zo_layer *l = &net->layers[net->count];
    memset(l, 0, sizeof(*l));
    l->in = in; l->out = out; l->act = act;
    l->W = (float *)calloc(in * out, sizeof(float));
    l->b = (float *)calloc(out, sizeof(float));
    l->gW = (float *)calloc(in * out, sizeof(float));
    l->gb = (float *)calloc(out, sizeof(float));
    l->opt = ZO_OPT_SGD;
    return (int)net->count++;
}

ZO_API size_t zo_net_layer_count(const zo_net *net) { return net->count; }

ZO_API void zo_net_set_params(zo_net *net, size_t layer, const float *W, const float *b) {
    zo_layer *l = &net->layers[layer];
    if (W) memcpy(l->W, W, l->in * l->out * sizeof(float));
    if (b) memcpy(l->b, b, l->out * sizeof(float));
}

ZO_API void zo_net_get_params(const zo_net *net, size_t layer, float *W, float *b) {
    const zo_layer *l = &net->layers[layer];
    if (W) memcpy(W, l->W, l->in * l->out * sizeof(float));
    if (b) memcpy(b, l->b, l->out * sizeof(float));
}

ZO_API void zo_net_get_grads(const zo_net *net, size_t layer, float *gW, float *gb) {
    const zo_layer *l = &net->layers[layer];
    if (gW) memcpy(gW, l->gW, l->in * l->out * sizeof(float));
    if (gb) memcpy(gb, l->gb, l->out * sizeof(float));
}

/* Per-layer SGD (momentum 0), src/optimizer.zig:160-164. */
ZO_API void zo_net_set_sgd(zo_net *net, size_t layer, float weight_decay) {
    zo_layer *l = &net->layers[layer];
    l->opt = ZO_OPT_SGD; l->wd = weight_decay;
}

/* Per-layer Adam with its own step counter, src/optimizer.zig:169-207. */
ZO_API void zo_net_set_adam(zo_net *net, size_t layer, float beta1, float beta2, float eps, float weight_decay) {
    zo_layer *l = &net->layers[layer];
    l->opt = ZO_OPT_ADAM; l->beta1 = beta1; l->beta2 = beta2; l->eps = eps; l->wd = weight_decay; l->t = 0;
    free(l->mW); free(l->vW); free(l->mb); free(l->vb);
    l->mW = (float *)calloc(l->in * l->out, sizeof(float));
    l->vW = (float *)calloc(l->in * l->out, sizeof(float));
    l->mb = (float *)calloc(l->out, sizeof(float));
    l->vb = (float *)calloc(l->out, sizeof(float));
}

static void alloc_state(zo_layer *l, int two) {
    free(l->mW); free(l->vW); free(l->mb); free(l->vb);
    l->mW = (float *)calloc(l->in * l->out, sizeof(float));
    l->mb = (float *)calloc(l->out, sizeof(float));
    l->vW = two ? (float *)calloc(l->in * l->out, sizeof(float)) : NULL;
    l->vb = two ? (float *)calloc(l->out, sizeof(float)) : NULL;
}

/* Sgd{ .momentum = m } with its velocity tensors, src/optimizer.zig:96-104. */
ZO_API void zo_net_set_sgd_momentum(zo_net *net, size_t layer, float momentum) {
    zo_layer *l = &net->layers[layer];
    l->opt = ZO_OPT_MOMENTUM; l->momentum = momentum;
    alloc_state(l, 0);
}

/* AdamW, src/optimizer.zig:236-297. */
ZO_API void zo_net_set_adamw(zo_net *net, size_t layer, float beta1, float beta2, float eps, float weight_decay) {
    zo_layer *l = &net->layers[layer];
    l->opt = ZO_OPT_ADAMW; l->beta1 = beta1; l->beta2 = beta2; l->eps = eps; l->wd = weight_decay; l->t = 0;
    alloc_state(l, 1);
}

/* Rmsprop, src/optimizer.zig:300-345. */
ZO_API void zo_net_set_rmsprop(zo_net *net, size_t layer, float rho, float eps, float weight_decay) {
    zo_layer *l = &net->layers[layer];
    l->opt = ZO_OPT_RMSPROP; l->rho = rho; l->eps = eps; l->wd = weight_decay;
    alloc_state(l, 0);
}

static void ensure_cache(zo_layer *l, size_t rows) {
    if (l->cache_rows >= rows) return;
    free(l->x_cache); free(l->y_cache);
    l->x_cache = (float *)malloc(rows * l->in * sizeof(float));
    l->y_cache = (float *)malloc(rows * l->out * sizeof(float));
    l->cache_rows = rows;
}

/* Dense.forward, src/layer.zig:380-409: matMul, addBias, activation in place. */
static void dense_forward(zo_layer *l, const float *x, float *y, size_t rows) {
    zo_matmul(x, l->W, y, rows, l->out, l->in, 0);
    zo_add_bias(y, rows * l->out, l->b, l->out);
    if (l->act == ZO_SOFTMAX) {                      /* one sample at a time, src/layer.zig:398-406 */
        for (size_t r = 0; r < rows; ++r) zo_softmax_forward(y + r * l->out, y + r * l->out, l->out);
    } else {
        zo_activation_forward(l->act, y, y, rows * l->out);
    }
}

/* Network.forward, src/network.zig:309-386: every layer keeps a copy of its
 * input and its activated output; `out` (may be NULL) gets the last output. */
ZO_API void zo_net_forward(zo_net *net, const float *x, size_t rows, float *out) {
    const float *cur = x;
    for (size_t i = 0; i < net->count; ++i) {
        zo_layer *l = &net->layers[i];
        ensure_cache(l, rows);
        memcpy(l->x_cache, cur, rows * l->in * sizeof(float));
        dense_forward(l, l->x_cache, l->y_cache, rows);
        cur = l->y_cache;
    }
    if (out && net->count) {
        const zo_layer *last = &net->layers[net->count - 1];
        memcpy(out, last->y_cache, rows * last->out * sizeof(float));
    }
}

/* Dense.backward, src/layer.zig:411-475: activation derivative on the
 * activated output, dX = G*W^T, gb += column sums of G, gW = X^T*G. */
static void dense_backward(zo_layer *l, const float *x, const float *grad_out,
                           float *grad_in, const float *y, float *gaa, size_t rows) {
    if (l->act == ZO_SOFTMAX) {                      /* src/layer.zig:429-438 */
        for (size_t r = 0; r < rows; ++r)
            zo_softmax_backward(y + r * l->out, grad_out + r * l->out, gaa + r * l->out, l->out);
    } else {
        zo_activation_backward(l->act, y, grad_out, gaa, rows * l->out);
    }
    zo_matmul_transpose_b(gaa, l->W, grad_in, rows, l->in, l->out, 0);
    zo_accumulate_bias(l->gb, l->out, gaa, rows * l->out);
    zo_matmul_transpose_a(x, gaa, l->gW, l->in, l->out, rows, 0);
}

/* Gradient-only pass: clearGradients (src/network.zig:388-393), forward,
 * computeGradients (:395-479), the clip (:513-535).  `mse_count` is the n of
 * the MSE gradient: rows*cols of this call unless a data-parallel caller
 * passes the global element count.  Returns the loss of the forward output
 * (:574) -- for MSE the mean uses mse_count as well. */
static float net_gradients(zo_net *net, const float *x, const float *t, size_t rows,
                           int loss, size_t mse_count, int do_clip) {
    size_t widest = 0;
    for (size_t i = 0; i < net->count; ++i) {
        zo_layer *l = &net->layers[i];
        memset(l->gW, 0, l->in * l->out * sizeof(float));
        memset(l->gb, 0, l->out * sizeof(float));
        if (l->in > widest) widest = l->in;
        if (l->out > widest) widest = l->out;
    }
    zo_net_forward(net, x, rows, NULL);

    if (net->work_len < rows * widest) {
        free(net->work1); free(net->work2);
        net->work_len = rows * widest;
        net->work1 = (float *)malloc(net->work_len * sizeof(float));
        net->work2 = (float *)malloc(net->work_len * sizeof(float));
    }
    float *gaa = (float *)malloc(rows * widest * sizeof(float));
    float *grad = net->work1, *next = net->work2;

    zo_layer *last = &net->layers[net->count - 1];
    const size_t cols = last->out;
    float loss_val;
    if (loss == ZO_MSE) {
        const float nf = (float)mse_count;
        float sum = 0;
        for (size_t i = 0; i < rows * cols; ++i) {
            const float d = last->y_cache[i] - t[i];
            sum += d * d;
            grad[i] = 2 * (last->y_cache[i] - t[i]) / nf;
        }
        loss_val = sum / nf;
    } else if (loss == ZO_BCE) {                     /* flat like MSE: the divisor is the (global) element count */
        zo_bce_backward(last->y_cache, t, grad, rows * cols, mse_count);
        loss_val = zo_bce_forward(last->y_cache, t, rows * cols) * ((float)(rows * cols) / (float)mse_count);
    } else {
        zo_loss_backward(loss, last->y_cache, t, grad, rows, cols);
        loss_val = zo_loss_forward(loss, last->y_cache, t, rows, cols);
    }

    for (size_t i = net->count; i-- > 0;) {
        zo_layer *l = &net->layers[i];
        dense_backward(l, l->x_cache, grad, next, l->y_cache, gaa, rows);
        float *tmp = grad; grad = next; next = tmp;
    }
    free(gaa);

    net->last_norm = 0; net->last_clip = 1.0f;
    if (do_clip) {
        float **gs = (float **)malloc(2 * net->count * sizeof(float *));
        size_t *ls = (size_t *)malloc(2 * net->count * sizeof(size_t));
        for (size_t i = 0; i < net->count; ++i) {
            gs[2 * i] = net->layers[i].gW; ls[2 * i] = net->layers[i].in * net->layers[i].out;
            gs[2 * i + 1] = net->layers[i].gb; ls[2 * i + 1] = net->layers[i].out;
        }
        net->last_norm = zo_clip_grad_norm(gs, ls, 2 * net->count, &net->last_clip);
        free(gs); free(ls);
    }
    return loss_val;
}

/* Optimizer dispatch of trainStep, src/network.zig:541-549 ->
 * Sgd.step (src/optimizer.zig:160-164) / Adam.step (:209-233). */
static void net_apply_optimizers(zo_net *net, float lr) {
    for (size_t i = 0; i < net->count; ++i) {
        zo_layer *l = &net->layers[i];
        const size_t nw = l->in * l->out;
        if (l->opt == ZO_OPT_ADAM) {
            l->t += 1;
            float bc1, bc2;
            zo_adam_bias_corrections(l->beta1, l->beta2, l->t, &bc1, &bc2);
            if (l->wd > 0.0f) {
                for (size_t j = 0; j < nw; ++j) l->gW[j] += l->wd * l->W[j];
                for (size_t j = 0; j < l->out; ++j) l->gb[j] += l->wd * l->b[j];
            }
            zo_adam_update(l->W, l->gW, l->mW, l->vW, nw, lr, l->beta1, l->beta2, l->eps, bc1, bc2);
            zo_adam_update(l->b, l->gb, l->mb, l->vb, l->out, lr, l->beta1, l->beta2, l->eps, bc1, bc2);
        } else if (l->opt == ZO_OPT_ADAMW) {
            l->t += 1;
            float bc1, bc2;
            zo_adam_bias_corrections(l->beta1, l->beta2, l->t, &bc1, &bc2);
            zo_adam_update(l->W, l->gW, l->mW, l->vW, nw, lr, l->beta1, l->beta2, l->eps, bc1, bc2);
            zo_adam_update(l->b, l->gb, l->mb, l->vb, l->out, lr, l->beta1, l->beta2, l->eps, bc1, bc2);
            zo_decoupled_decay(l->W, nw, lr, l->wd);
            zo_decoupled_decay(l->b, l->out, lr, l->wd);
        } else if (l->opt == ZO_OPT_RMSPROP) {
            if (l->wd > 0.0f) {
                for (size_t j = 0; j < nw; ++j) l->gW[j] += l->wd * l->W[j];
                for (size_t j = 0; j < l->out; ++j) l->gb[j] += l->wd * l->b[j];
            }
            zo_rmsprop_update(l->W, l->gW, l->mW, nw, lr, l->rho, l->eps);
            zo_rmsprop_update(l->b, l->gb, l->mb, l->out, lr, l->rho, l->eps);
        } else if (l->opt == ZO_OPT_MOMENTUM) {
            zo_sgd_momentum_update(l->W, l->gW, l->mW, nw, lr, l->momentum);
            zo_sgd_momentum_update(l->b, l->gb, l->mb, l->out, lr, l->momentum);
        } else {
            zo_sgd_update(l->W, l->gW, nw, lr, l->wd);
            zo_sgd_update_bias(l->b, l->gb, l->out, lr);
        }
    }
}

/* One training step on a block of `rows` samples: Network.trainStep,
 * src/network.zig:481-579, with the two batching changes the benchmark
 * configurations need (the target-length guard at :490-491 lifted; CE taken
 * per row).  rows == 1 is the literal reference step. */
ZO_API float zo_net_train_step(zo_net *net, const float *x, const float *t, size_t rows,
                               float lr, int loss) {
    const size_t cols = net->layers[net->count - 1].out;
    const float l = net_gradients(net, x, t, rows, loss, rows * cols, 1);
    net_apply_optimizers(net, lr);
    return l;
}

/* Gradients of a shard of a larger batch without clip or update: what one
 * data-parallel rank computes before the gradient sum.  `global_rows` sets
 * the MSE divisor; CE gradients are unscaled sums.  Returns the shard's loss
 * SUM (MSE: sum of squared errors / global n; CE: sum of row losses). */
ZO_API float zo_net_shard_gradients(zo_net *net, const float *x, const float *t, size_t rows,
                                    size_t global_rows, int loss) {
    const size_t cols = net->layers[net->count - 1].out;
    const float l = net_gradients(net, x, t, rows, loss, global_rows * cols, 0);
    return loss_is_flat(loss) ? l : l * (float)rows;
}

/* Second half of a data-parallel step: gradients already summed into the
 * net (zo_net_set_grads), then clip and update exactly as trainStep does. */
ZO_API void zo_net_set_grads(zo_net *net, size_t layer, const float *gW, const float *gb) {
    zo_layer *l = &net->layers[layer];
    memcpy(l->gW, gW, l->in * l->out * sizeof(float));
    memcpy(l->gb, gb, l->out * sizeof(float));
}

ZO_API void zo_net_clip_and_update(zo_net *net, float lr) {
    float **gs = (float **)malloc(2 * net->count * sizeof(float *));
    size_t *ls = (size_t *)malloc(2 * net->count * sizeof(size_t));
    for (size_t i = 0; i < net->count; ++i) {
        gs[2 * i] = net->layers[i].gW; ls[2 * i] = net->layers[i].in * net->layers[i].out;
        gs[2 * i + 1] = net->layers[i].gb; ls[2 * i + 1] = net->layers[i].out;
    }
    net->last_norm = zo_clip_grad_norm(gs, ls, 2 * net->count, &net->last_clip);
    free(gs); free(ls);
    net_apply_optimizers(net, lr);
}

ZO_API void zo_net_last_clip(const zo_net *net, float *norm, float *factor) {
    if (norm) *norm = net->last_norm;
    if (factor) *factor = net->last_clip;
}

/* Network.train, src/network.zig:596-616 with the constant scheduler: for
 * each epoch, one trainStep per sample in order; epoch_loss[e] is the mean of
 * the per-sample losses (:615). */
ZO_API void zo_net_train(zo_net *net, const float *inputs, const float *targets, size_t samples,
                         size_t epochs, float lr, int loss, float *epoch_loss) {
    const size_t in = net->layers[0].in, out = net->layers[net->count - 1].out;
    for (size_t e = 0; e < epochs; ++e) {
        float total = 0;
        for (size_t s = 0; s < samples; ++s)
            total += zo_net_train_step(net, inputs + s * in, targets + s * out, 1, lr, loss);
        if (epoch_loss) epoch_loss[e] = total / (float)samples;
    }
}

/* ---------------------------------------------------------------- evaluation */

/* getPredictedClass, src/metrics.zig:213-227: first index of the maximum (strict >). */
ZO_API size_t zo_predicted_class(const float *output, size_t n) {
    size_t idx = 0;
    float best = output[0];
    for (size_t i = 1; i < n; ++i)
        if (output[i] > best) { best = output[i]; idx = i; }
    return idx;
}

/* getTrueClass, src/metrics.zig:230-235: first entry above 0.5, else class 0. */
ZO_API size_t zo_true_class(const float *target, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (target[i] > 0.5f) return i;
    return 0;
}

/* computeClassificationMetrics, src/metrics.zig:85-163.  cm[target][pred], row-major classes x classes;
 * out4 = accuracy, macro precision, macro recall, F1 of those two.  Returns 0, 1 = EmptyInput, 2 = InvalidClass. */
ZO_API int zo_classification_metrics(const size_t *pred, const size_t *targ, size_t n, size_t classes,
                                     unsigned long long *cm, float *out4) {
    if (n == 0) return 1;
    memset(cm, 0, classes * classes * sizeof(unsigned long long));
    for (size_t i = 0; i < n; ++i) {
        if (pred[i] >= classes || targ[i] >= classes) return 2;
        cm[targ[i] * classes + pred[i]] += 1;
    }
    size_t correct = 0;
    float total_precision = 0, total_recall = 0;
    for (size_t c = 0; c < classes; ++c) {
        const size_t tp = (size_t)cm[c * classes + c];
        size_t fp = 0, fn = 0;
        for (size_t i = 0; i < classes; ++i)
            if (i != c) { fp += (size_t)cm[i * classes + c]; fn += (size_t)cm[c * classes + i]; }
        correct += tp;
        total_precision += (tp + fp > 0) ? (float)tp / (float)(tp + fp) : 0.0f;
        total_recall += (tp + fn > 0) ? (float)tp / (float)(tp + fn) : 0.0f;
    }
    const float accuracy = (float)correct / (float)n;
    const float precision = total_precision / (float)classes;
    const float recall = total_recall / (float)classes;
    out4[0] = accuracy; out4[1] = precision; out4[2] = recall;
    out4[3] = (precision + recall > 0) ? 2.0f * precision * recall / (precision + recall) : 0.0f;
    return 0;
}

/* evaluateClassification, src/metrics.zig:239-264, on row-major blocks of `rows` outputs and targets. */
ZO_API int zo_evaluate_classification(const float *outputs, const float *targets, size_t rows, size_t cols,
                                      size_t classes, unsigned long long *cm, float *out4) {
    size_t *pred = (size_t *)malloc((rows ? rows : 1) * sizeof(size_t));
    size_t *targ = (size_t *)malloc((rows ? rows : 1) * sizeof(size_t));
    for (size_t r = 0; r < rows; ++r) {
        pred[r] = zo_predicted_class(outputs + r * cols, cols);
        targ[r] = zo_true_class(targets + r * cols, cols);
    }
    const int rc = zo_classification_metrics(pred, targ, rows, classes, cm, out4);
    free(pred); free(targ);
    return rc;
}
