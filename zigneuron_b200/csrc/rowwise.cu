// Bandwidth-bound kernels of the Dense step: operand conversion, bias add,
// activations, the column reduction behind accumulateBias, and the fused
// loss value + gradient kernels.  All are sized for coalesced 16-byte accesses
// and grids that are multiples of the SM count; reductions are two-stage
// (block partials in the context's scratch, then one block adds them in a fixed
// order), so results do not depend on scheduling.
#include <atomic>

#include "zn_internal.h"
#include "zn_act.cuh"

namespace {

constexpr int TPB = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the block; the result is valid in thread 0.
__device__ __forceinline__ float block_sum(float v) {
    __shared__ float part[32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) part[w] = v;
    __syncthreads();
    if (w == 0) {
        v = lane < (int)((blockDim.x + 31) >> 5) ? part[lane] : 0.f;
        v = warp_sum(v);
    }
    return v;
}

__device__ __forceinline__ float act_fwd(int act, float x) {
    switch (act) {
    case ZN_ACT_RELU: return x > 0.f ? x : 0.f;
    case ZN_ACT_SIGMOID:
        if (x >= 0.f) return 1.f / (1.f + expf(-x));
        else { const float e = expf(x); return e / (1.f + e); }
    case ZN_ACT_TANH: return tanhf(x);
    case ZN_ACT_GELU: return zn_gelu_fwd(x);
    case ZN_ACT_LEAKY_RELU: return zn_leaky_fwd(x);
    case ZN_ACT_ELU: return zn_elu_fwd(x);
    default: return x;
    }
}
__device__ __forceinline__ float act_bwd(int act, float y, float g) {
    switch (act) {
    case ZN_ACT_RELU: return y > 0.f ? g : 0.f;
    case ZN_ACT_SIGMOID: return __fmul_rn(__fmul_rn(g, y), (1.f - y));
    case ZN_ACT_TANH: return __fmul_rn(g, (1.f - __fmul_rn(y, y)));
    case ZN_ACT_GELU: return zn_gelu_bwd(y, g);
    case ZN_ACT_LEAKY_RELU: return zn_leaky_bwd(y, g);
    case ZN_ACT_ELU: return zn_elu_bwd(y, g);
    default: return g;
    }
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- f32 -> operand type, with zeroed padding columns --------------------------------
template <typename T>
__global__ void convert_kernel(const float *__restrict__ src, int64_t ld_src, T *__restrict__ dst, int64_t ld_dst,
                               int64_t rows, int64_t cols) {
    zn_pdl_release();
    zn_pdl_wait();
    // one thread per group of 8 destination columns
    const int64_t groups_per_row = ld_dst / 8;
    const int64_t total = rows * groups_per_row;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = g / groups_per_row, c0 = (g % groups_per_row) * 8;
        const float *s = src + r * ld_src + c0;
        float v[8];
        if (c0 + 8 <= cols && ((reinterpret_cast<uintptr_t>(s) & 15) == 0)) {
            const float4 a = *reinterpret_cast<const float4 *>(s), b = *reinterpret_cast<const float4 *>(s + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (c0 + j < cols) ? s[j] : 0.f;
        }
        T *d = dst + r * ld_dst + c0;
        if (sizeof(T) == 2) {
            uint32_t w[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * h], v[2 * h + 1]);
                w[h] = *reinterpret_cast<const uint32_t *>(&b2);
            }
            *reinterpret_cast<uint4 *>(d) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            float *df = reinterpret_cast<float *>(d);
            *reinterpret_cast<float4 *>(df) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(df + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
}

__global__ void add_bias_kernel(float *__restrict__ out, int64_t total, int64_t cols, const float *__restrict__ bias) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __fadd_rn(out[i], bias[i % cols]);
}

__global__ void act_forward_kernel(int act, const float *in, float *out, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = act_fwd(act, in[i]);
}

__global__ void act_backward_kernel(int act, const float *__restrict__ y, const float *__restrict__ go,
                                    float *__restrict__ gi, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        gi[i] = act_bwd(act, y[i], go[i]);
}

// In-place activation derivative on an operand-typed gradient block: g = act'(y) (*) g.
template <typename T>
__global__ void act_backward_t_kernel(int act, const T *__restrict__ y, int64_t ld_y, T *__restrict__ g, int64_t ld_g,
                                      int64_t rows, int64_t cols) {
    const int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols, c = i % cols;
        const float yv = to_f32(y[r * ld_y + c]);
        const float gv = to_f32(g[r * ld_g + c]);
        g[r * ld_g + c] = from_f32<T>(act_bwd(act, yv, gv));
    }
}

// exp and log of the exact mode.  The reference's CPU path calls its math library, whose float routines return the
// correctly rounded result in all but isolated cases; the device's expf / logf are allowed 1-2 ulp.  One ulp in a
// softmax is enough to send an Adam run down another path after a few dozen steps, so the exact mode evaluates in
// double precision and rounds once, which gives the correctly rounded float in all but about one case in 10^8.
__device__ __forceinline__ float exp_rounded_once(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float log_rounded_once(float x) { return (float)log((double)x); }

// ---- row-wise softmax -------------------------------------------------------------------
// Activation.softmaxForward (src/activation.zig:51-78) on every row of a block, the way Dense.forward
// applies it sample by sample (src/layer.zig:398-406).  One warp per row.  `exact`: lane 0 takes the
// maximum and the sum of exponentials in column order, as the reference does; otherwise lanes take
// strided partial sums.  Either output may be null; in == out is allowed.
template <typename TIN, typename TOUT>
__global__ void softmax_rows_kernel(const TIN *in, int64_t ld_in, TOUT *out_t, int64_t ld_t, float *out_f32,
                                    int64_t ld_f, int64_t rows, int64_t cols, int exact) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const TIN *x = in + r * ld_in;
        float mx = -INFINITY, sum = 0.f;
        if (exact) {
            if (lane == 0) {
                for (int64_t c = 0; c < cols; ++c) { const float v = to_f32(x[c]); if (v > mx) mx = v; }
                for (int64_t c = 0; c < cols; ++c) sum = __fadd_rn(sum, exp_rounded_once(__fsub_rn(to_f32(x[c]), mx)));
            }
            mx = __shfl_sync(0xffffffffu, mx, 0);
            sum = __shfl_sync(0xffffffffu, sum, 0);
        } else {
            for (int64_t c = lane; c < cols; c += 32) mx = fmaxf(mx, to_f32(x[c]));
            mx = warp_max(mx);
            for (int64_t c = lane; c < cols; c += 32) sum += expf(to_f32(x[c]) - mx);
            sum = warp_sum(sum);
        }
        const bool ok = sum > 0.f;                       // false also for NaN: uniform, as the reference
        const float uniform = __fdiv_rn(1.0f, (float)cols);
        for (int64_t c = lane; c < cols; c += 32) {
            const float ex = exact ? exp_rounded_once(__fsub_rn(to_f32(x[c]), mx)) : expf(__fsub_rn(to_f32(x[c]), mx));
            const float v = ok ? __fdiv_rn(ex, sum) : uniform;
            if (out_t) out_t[r * ld_t + c] = from_f32<TOUT>(v);
            if (out_f32) out_f32[r * ld_f + c] = v;
        }
    }
}

// Activation.softmaxBackward (src/activation.zig:82-95) per row: gi = s * (go - sum(go * s)); gi == go allowed.
template <typename T>
__global__ void softmax_backward_rows_kernel(const T *s, int64_t ld_s, const T *go, int64_t ld_go, T *gi, int64_t ld_gi,
                                             int64_t rows, int64_t cols, int exact) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const T *sr = s + r * ld_s, *gr = go + r * ld_go;
        float dot = 0.f;
        if (exact) {
            if (lane == 0)
                for (int64_t c = 0; c < cols; ++c) dot = __fadd_rn(dot, __fmul_rn(to_f32(gr[c]), to_f32(sr[c])));
            dot = __shfl_sync(0xffffffffu, dot, 0);
        } else {
            for (int64_t c = lane; c < cols; c += 32) dot += to_f32(gr[c]) * to_f32(sr[c]);
            dot = warp_sum(dot);
        }
        for (int64_t c = lane; c < cols; c += 32)
            gi[r * ld_gi + c] = from_f32<T>(__fmul_rn(to_f32(sr[c]), __fsub_rn(to_f32(gr[c]), dot)));
    }
}

// ---- column sums ------------------------------------------------------------------------

// Exact order: one thread per column, rows ascending (cpuAccumulateBias, src/backend.zig:706-713).
template <typename T>
__global__ void bias_reduce_exact_kernel(const T *__restrict__ g, int64_t ld, int64_t rows, int64_t cols,
                                         float *__restrict__ gb, int accumulate) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = accumulate ? gb[c] : 0.f;
    for (int64_t r = 0; r < rows; ++r) s = __fadd_rn(s, to_f32(g[r * ld + c]));
    gb[c] = s;
}

// Stage 1: block (strip, split) sums rows [split*rows_per, ...) of a 32*VEC-column strip.
// Each warp walks rows warp, warp+8, ...; a lane owns VEC adjacent columns (16 bytes).
// With `counters` (one per strip, zero between launches) the block of a strip that finishes last also adds the
// strip's partial sums up, in split order, and writes gb: the whole reduction in one launch.  Without, stage 2 is
// the kernel below.  Either way the additions are the same ones in the same order.
template <typename T, int VEC>
__global__ void bias_reduce_partial_kernel(const T *__restrict__ g, int64_t ld, int64_t rows, int64_t cols,
                                           int64_t rows_per, float *__restrict__ partial, float *__restrict__ gb,
                                           int accumulate, unsigned int *counters) {
    constexpr int STRIP = 32 * VEC;
    __shared__ float sm[TPB / 32][STRIP];
    __shared__ bool last;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t c0 = (int64_t)blockIdx.x * STRIP + lane * VEC;
    const int64_t r_begin = (int64_t)blockIdx.y * rows_per;
    const int64_t r_end = min(rows, r_begin + rows_per);
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    const bool vec_ok = (c0 + VEC <= cols) && ((ld * sizeof(T)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(g) & 15) == 0);
    for (int64_t r = r_begin + w; r < r_end; r += TPB / 32) {
        const T *p = g + r * ld + c0;
        if (vec_ok) {
            const uint4 u = *reinterpret_cast<const uint4 *>(p);
            if (sizeof(T) == 2) {
                const uint32_t wv[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    acc[2 * h] += __uint_as_float(wv[h] << 16);
                    acc[2 * h + 1] += __uint_as_float(wv[h] & 0xFFFF0000u);
                }
            } else {
                acc[0] += __uint_as_float(u.x); acc[1] += __uint_as_float(u.y);
                acc[2] += __uint_as_float(u.z); acc[3] += __uint_as_float(u.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                if (c0 + j < cols) acc[j] += to_f32(p[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) sm[w][lane * VEC + j] = acc[j];
    __syncthreads();
    for (int c = threadIdx.x; c < STRIP; c += TPB) {
        float s = 0.f;
#pragma unroll
        for (int ww = 0; ww < TPB / 32; ++ww) s += sm[ww][c];
        const int64_t gc = (int64_t)blockIdx.x * STRIP + c;
        if (gc < cols) partial[(int64_t)blockIdx.y * cols + gc] = s;
    }
    if (!counters) return;
    __threadfence();                                   // this block's partial sums are visible before its arrival is
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&counters[blockIdx.x], 1u) == gridDim.y - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (int c = threadIdx.x; c < STRIP; c += TPB) {
        const int64_t gc = (int64_t)blockIdx.x * STRIP + c;
        if (gc >= cols) continue;
        float s = 0.f;
        for (unsigned int i = 0; i < gridDim.y; ++i) s += __ldcg(partial + (int64_t)i * cols + gc);
        gb[gc] = accumulate ? gb[gc] + s : s;
    }
    if (threadIdx.x == 0) counters[blockIdx.x] = 0u;   // ready for the next launch on this lane
}

// Stage 2: gb[c] (+)= sum over splits, in split order.
__global__ void bias_reduce_final_kernel(const float *__restrict__ partial, int64_t cols, int splits,
                                         float *__restrict__ gb, int accumulate) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.f;
    for (int i = 0; i < splits; ++i) s += partial[(int64_t)i * cols + c];
    gb[c] = accumulate ? gb[c] + s : s;
}

// ---- losses ---------------------------------------------------------------------------------

// End of a loss kernel: the block's partial sum is stored; with an arrival counter the block that arrives last also
// adds all partial sums up (double, fixed order: thread i takes partial[i], partial[i + TPB], ..., then a tree) and
// writes the loss sum, so the loss needs no second launch.  Called by every thread of the block.
__device__ __forceinline__ void finish_loss_sum(float block_total, float *partial, float *loss_sum, unsigned int *counter) {
    __shared__ double fin[TPB];
    __shared__ bool last;
    if (threadIdx.x == 0) {
        partial[blockIdx.x] = block_total;
        if (counter) {
            __threadfence();
            last = atomicAdd(counter, 1u) == gridDim.x - 1;
        }
    }
    if (!counter) return;
    __syncthreads();
    if (!last) return;
    __threadfence();
    double s = 0.0;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) s += (double)__ldcg(partial + i);
    fin[threadIdx.x] = s;
    __syncthreads();
    for (int o = TPB / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) fin[threadIdx.x] += fin[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        *loss_sum = (float)fin[0];
        *counter = 0u;
    }
}

// MSE (src/loss.zig:93-109): grad = 2*(o-t)/n, partial[block] = sum (o-t)^2 over the block's elements.
template <typename T>
__global__ void mse_kernel(const float *__restrict__ out, int64_t ld_o, const float *__restrict__ target,
                           T *__restrict__ grad, int64_t ld_g, int64_t rows, int64_t cols, float n_div,
                           float *__restrict__ partial, float *loss_sum, unsigned int *counter) {
    const int64_t total = rows * cols;
    float s = 0.f;
    const bool flat = (ld_o == cols) && (!grad || ld_g == cols);
    if (flat && (total % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
        ((reinterpret_cast<uintptr_t>(target) & 15) == 0) && (sizeof(T) == 4 ? ((reinterpret_cast<uintptr_t>(grad) & 15) == 0)
                                                                              : ((reinterpret_cast<uintptr_t>(grad) & 7) == 0))) {
        const int64_t n4 = total / 4;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
            const float4 o = reinterpret_cast<const float4 *>(out)[i];
            const float4 t = reinterpret_cast<const float4 *>(target)[i];
            const float d0 = o.x - t.x, d1 = o.y - t.y, d2 = o.z - t.z, d3 = o.w - t.w;
            s += d0 * d0; s += d1 * d1; s += d2 * d2; s += d3 * d3;
            if (grad) {
                const float g0 = __fdiv_rn(2.f * d0, n_div), g1 = __fdiv_rn(2.f * d1, n_div);
                const float g2 = __fdiv_rn(2.f * d2, n_div), g3 = __fdiv_rn(2.f * d3, n_div);
                if (sizeof(T) == 4) {
                    reinterpret_cast<float4 *>(grad)[i] = make_float4(g0, g1, g2, g3);
                } else {
                    const __nv_bfloat162 a = __floats2bfloat162_rn(g0, g1), b = __floats2bfloat162_rn(g2, g3);
                    reinterpret_cast<uint2 *>(grad)[i] =
                        make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
                }
            }
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = i / cols, c = i % cols;
            const float d = out[r * ld_o + c] - target[i];
            s += d * d;
            if (grad) grad[r * ld_g + c] = from_f32<T>(__fdiv_rn(2.f * d, n_div));
        }
    }
    s = block_sum(s);
    finish_loss_sum(s, partial, loss_sum, counter);
}

// Binary cross-entropy on probabilities (src/loss.zig:255-302): p clamped to [1e-7, 1 - 1e-7], so is 1 - p;
// loss term -(t*log(p) + (1-t)*log(1-p)), grad = (p - t)/n.  partial[block] = sum of the block's terms.
__device__ __forceinline__ float bce_term(float o, float t, float &p) {
    const float eps = 1e-7f;
    p = o;
    if (p < eps) p = eps;
    if (p > 1.f - eps) p = 1.f - eps;
    float q = __fsub_rn(1.f, p);
    if (q < eps) q = eps;
    if (q > 1.f - eps) q = 1.f - eps;
    return __fadd_rn(__fmul_rn(t, logf(p)), __fmul_rn(__fsub_rn(1.f, t), logf(q)));
}

template <typename T>
__global__ void bce_kernel(const float *__restrict__ out, int64_t ld_o, const float *__restrict__ target,
                           T *__restrict__ grad, int64_t ld_g, int64_t rows, int64_t cols, float n_div,
                           float *__restrict__ partial, float *loss_sum, unsigned int *counter) {
    const int64_t total = rows * cols;
    float s = 0.f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols, c = i % cols;
        const float t = target[i];
        float p;
        s -= bce_term(out[r * ld_o + c], t, p);
        if (grad) grad[r * ld_g + c] = from_f32<T>(__fdiv_rn(__fsub_rn(p, t), n_div));
    }
    s = block_sum(s);
    finish_loss_sum(s, partial, loss_sum, counter);
}

// Row loss of Loss.crossEntropyForward (src/loss.zig:110-169), the variant WITHOUT "_logits" in its name,
// which takes logits all the same: exponents clamped to [-50, 50], every target entry above 0.5
// contributes lse - o, the row's loss is their mean, degenerate rows give 0.
__device__ __forceinline__ float ce_plain_row_loss(float mx, float sum_clamped, float loss_sum, float count) {
    if (mx == -INFINITY || !isfinite(sum_clamped) || sum_clamped <= 0.f || count == 0.f) return 0.f;
    return __fdiv_rn(loss_sum, count);
}

// Softmax cross-entropy with logits, one warp per row (src/loss.zig:202-254 per row;
// rows batched as kernels/loss.cu:123-155): grad = exp(l-max)/sum - t, row loss =
// -(l[target] - (log(sum) + max)) with target = first column whose t > 0.5.
template <typename T>
__global__ void ce_kernel(const float *__restrict__ logits, int64_t ld_o, const float *__restrict__ target,
                          T *__restrict__ grad, int64_t ld_g, int64_t rows, int64_t cols, float *__restrict__ partial,
                          int exact, int plain, float *loss_sum, unsigned int *counter) {
    zn_pdl_release();
    zn_pdl_wait();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    float loss_acc = 0.f;
    for (int64_t r = (int64_t)blockIdx.x * wpb + w; r < rows; r += (int64_t)gridDim.x * wpb) {
        const float *l = logits + r * ld_o;
        const float *t = target + r * cols;
        float mx = -INFINITY;
        for (int64_t c = lane; c < cols; c += 32) mx = fmaxf(mx, l[c]);
        mx = warp_max(mx);
        float se = 0.f;
        int64_t first = INT64_MAX;
        for (int64_t c = lane; c < cols; c += 32) {
            se += expf(l[c] - mx);
            if (t[c] > 0.5f && c < first) first = c;
        }
        se = warp_sum(se);
        if (exact) {   // the reference's order: one running sum over the columns (src/loss.zig:243-247)
            se = 0.f;
            for (int64_t c = 0; c < cols; ++c) se = __fadd_rn(se, exp_rounded_once(__fsub_rn(l[c], mx)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
        if (grad) {
            T *g = grad + r * ld_g;
            for (int64_t c = lane; c < cols; c += 32) {
                const float e = exact ? exp_rounded_once(__fsub_rn(l[c], mx)) : expf(l[c] - mx);
                g[c] = from_f32<T>(__fsub_rn(__fdiv_rn(e, se), t[c]));
            }
        }
        if (!plain) {
            if (lane == 0 && first != INT64_MAX) loss_acc += -(l[first] - (logf(se) + mx));
        } else {
            float sec = 0.f;
            for (int64_t c = lane; c < cols; c += 32) sec += expf(fminf(50.f, fmaxf(-50.f, l[c] - mx)));
            sec = warp_sum(sec);
            const float lse = logf(sec) + mx;
            float ls = 0.f, cnt = 0.f;
            for (int64_t c = lane; c < cols; c += 32)
                if (t[c] > 0.5f) { ls += lse - l[c]; cnt += 1.f; }
            ls = warp_sum(ls);
            cnt = warp_sum(cnt);
            if (lane == 0) loss_acc += ce_plain_row_loss(mx, sec, ls, cnt);
        }
    }
    loss_acc = block_sum(loss_acc);
    finish_loss_sum(loss_acc, partial, loss_sum, counter);
}

// FP32_EXACT mode: the loss SUM in the reference's order.  MSE: one running f32 sum of (o-t)^2 over all
// elements (src/loss.zig:93-101).  CE: row losses added row by row (kernels/loss.cu:175-213).
__global__ void loss_sum_exact_kernel(int loss, const float *__restrict__ out, int64_t ld_o, const float *__restrict__ target,
                                      int64_t rows, int64_t cols, float *__restrict__ result) {
    float total = 0.f;
    for (int64_t r = 0; r < rows; ++r) {
        const float *o = out + r * ld_o, *t = target + r * cols;
        if (loss == ZN_LOSS_MSE) {
            for (int64_t c = 0; c < cols; ++c) {
                const float d = __fsub_rn(o[c], t[c]);
                total = __fadd_rn(total, __fmul_rn(d, d));
            }
        } else if (loss == ZN_LOSS_BINARY_CROSS_ENTROPY) {
            for (int64_t c = 0; c < cols; ++c) {
                float p;
                total = __fsub_rn(total, bce_term(o[c], t[c], p));
            }
        } else if (loss == ZN_LOSS_CROSS_ENTROPY) {
            float mx = -INFINITY;
            for (int64_t c = 0; c < cols; ++c) if (o[c] > mx) mx = o[c];
            float sec = 0.f;
            for (int64_t c = 0; c < cols; ++c) sec = __fadd_rn(sec, exp_rounded_once(fminf(50.f, fmaxf(-50.f, __fsub_rn(o[c], mx)))));
            const float lse = __fadd_rn(log_rounded_once(sec), mx);
            float ls = 0.f, cnt = 0.f;
            for (int64_t c = 0; c < cols; ++c)
                if (t[c] > 0.5f) { ls = __fadd_rn(ls, __fsub_rn(lse, o[c])); cnt += 1.f; }
            total = __fadd_rn(total, ce_plain_row_loss(mx, sec, ls, cnt));
        } else {
            float mx = o[0];
            for (int64_t c = 1; c < cols; ++c) if (o[c] > mx) mx = o[c];
            float se = 0.f;
            for (int64_t c = 0; c < cols; ++c) se = __fadd_rn(se, exp_rounded_once(__fsub_rn(o[c], mx)));
            const float lse = __fadd_rn(log_rounded_once(se), mx);
            float l = 0.f;
            for (int64_t c = 0; c < cols; ++c) if (t[c] > 0.5f) { l = -(__fsub_rn(o[c], lse)); break; }
            total = __fadd_rn(total, l);
        }
    }
    *result = total;
}

// The column reduction runs on a side lane underneath the persistent GEMM, whose CTAs need the SM set up
// for maximum shared memory; a kernel left to another shared-memory / L1 split cannot share an SM with
// them.  Ask for the same split (see the same note in optim.cu).
void prefer_gemm_compatible_carveout(zn_ctx *ctx) {
    static std::atomic<uint64_t> done_mask{0};
    const uint64_t bit = 1ull << (ctx->device & 63);
    if (done_mask.load() & bit) return;
    done_mask.fetch_or(bit);
    const int c = cudaSharedmemCarveoutMaxShared;
    const cudaFuncAttribute at = cudaFuncAttributePreferredSharedMemoryCarveout;
    cudaFuncSetAttribute(bias_reduce_partial_kernel<float, 4>, at, c);
    cudaFuncSetAttribute(bias_reduce_partial_kernel<__nv_bfloat16, 8>, at, c);
    cudaFuncSetAttribute(bias_reduce_final_kernel, at, c);
    cudaFuncSetAttribute(bias_reduce_exact_kernel<float>, at, c);
    cudaFuncSetAttribute(bias_reduce_exact_kernel<__nv_bfloat16>, at, c);
    cudaGetLastError();
}

int grid_for(zn_ctx *ctx, int64_t work_items, int per_sm = 8) {
    int64_t blocks = (work_items + TPB - 1) / TPB;
    const int64_t cap = (int64_t)ctx->sm_count * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}   // namespace

zn_status zn_k_convert(zn_ctx *ctx, const float *src, int64_t ld_src, void *dst, int64_t ld_dst, bool dst_bf16,
                       int64_t rows, int64_t cols) {
    if (ld_dst % 8 != 0) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "convert: destination pitch must be a multiple of 8");
    zn_launch_scope scope(ctx, ZN_PROF_CONVERT, 0, (double)rows * cols * (4 + (dst_bf16 ? 2 : 4)));
    const int grid = grid_for(ctx, rows * (ld_dst / 8));
    if (dst_bf16)
        zn_launch_pdl(convert_kernel<__nv_bfloat16>, dim3(grid), dim3(TPB), 0, ctx->stream, src, ld_src, (__nv_bfloat16 *)dst, ld_dst, rows, cols);
    else
        zn_launch_pdl(convert_kernel<float>, dim3(grid), dim3(TPB), 0, ctx->stream, src, ld_src, (float *)dst, ld_dst, rows, cols);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_add_bias(zn_ctx *ctx, float *out, int64_t rows, int64_t cols, const float *bias) {
    zn_launch_scope scope(ctx, ZN_PROF_ELEMENTWISE, 0, 8.0 * rows * cols);
    add_bias_kernel<<<grid_for(ctx, rows * cols), TPB, 0, ctx->stream>>>(out, rows * cols, cols, bias);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_act_forward(zn_ctx *ctx, int act, const float *in, float *out, int64_t n) {
    zn_launch_scope scope(ctx, ZN_PROF_ELEMENTWISE, 0, 8.0 * n);
    act_forward_kernel<<<grid_for(ctx, n), TPB, 0, ctx->stream>>>(act, in, out, n);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_act_backward(zn_ctx *ctx, int act, const float *y, const float *go, float *gi, int64_t n) {
    zn_launch_scope scope(ctx, ZN_PROF_ELEMENTWISE, 0, 12.0 * n);
    act_backward_kernel<<<grid_for(ctx, n), TPB, 0, ctx->stream>>>(act, y, go, gi, n);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

static int row_grid(zn_ctx *ctx, int64_t rows) {
    int64_t blocks = (rows + TPB / 32 - 1) / (TPB / 32);
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    return (int)(blocks < 1 ? 1 : blocks > cap ? cap : blocks);
}

zn_status zn_k_softmax_rows(zn_ctx *ctx, const void *in, bool in_bf16, int64_t ld_in, void *out_t, bool out_bf16,
                            int64_t ld_t, float *out_f32, int64_t ld_f, int64_t rows, int64_t cols, bool exact) {
    zn_launch_scope scope(ctx, ZN_PROF_ELEMENTWISE, 0, (double)rows * cols * 8);
    const int grid = row_grid(ctx, rows);
    if (in_bf16) {
        if (out_t && !out_bf16) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "softmax: bf16 input needs a bf16 typed output");
        softmax_rows_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(
            (const __nv_bfloat16 *)in, ld_in, (__nv_bfloat16 *)out_t, ld_t, out_f32, ld_f, rows, cols, exact ? 1 : 0);
    } else if (out_t && out_bf16) {
        softmax_rows_kernel<float, __nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(
            (const float *)in, ld_in, (__nv_bfloat16 *)out_t, ld_t, out_f32, ld_f, rows, cols, exact ? 1 : 0);
    } else {
        softmax_rows_kernel<float, float><<<grid, TPB, 0, ctx->stream>>>(
            (const float *)in, ld_in, (float *)out_t, ld_t, out_f32, ld_f, rows, cols, exact ? 1 : 0);
    }
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_softmax_backward_rows(zn_ctx *ctx, const void *s, int64_t ld_s, const void *go, int64_t ld_go, void *gi,
                                     int64_t ld_gi, bool bf16, int64_t rows, int64_t cols, bool exact) {
    zn_launch_scope scope(ctx, ZN_PROF_ELEMENTWISE, 0, (double)rows * cols * (bf16 ? 8 : 16));
    const int grid = row_grid(ctx, rows);
    if (bf16)
        softmax_backward_rows_kernel<__nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(
            (const __nv_bfloat16 *)s, ld_s, (const __nv_bfloat16 *)go, ld_go, (__nv_bfloat16 *)gi, ld_gi, rows, cols, exact ? 1 : 0);
    else
        softmax_backward_rows_kernel<float><<<grid, TPB, 0, ctx->stream>>>(
            (const float *)s, ld_s, (const float *)go, ld_go, (float *)gi, ld_gi, rows, cols, exact ? 1 : 0);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_act_backward_t(zn_ctx *ctx, int act, const void *y, int64_t ld_y, void *g, int64_t ld_g, bool bf16,
                              int64_t rows, int64_t cols, bool exact) {
    if (act == ZN_ACT_SOFTMAX) return zn_k_softmax_backward_rows(ctx, y, ld_y, g, ld_g, g, ld_g, bf16, rows, cols, exact);
    zn_launch_scope scope(ctx, ZN_PROF_ELEMENTWISE, 0, (double)rows * cols * (bf16 ? 6 : 12));
    const int grid = grid_for(ctx, rows * cols);
    if (bf16)
        act_backward_t_kernel<__nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(act, (const __nv_bfloat16 *)y, ld_y, (__nv_bfloat16 *)g, ld_g, rows, cols);
    else
        act_backward_t_kernel<float><<<grid, TPB, 0, ctx->stream>>>(act, (const float *)y, ld_y, (float *)g, ld_g, rows, cols);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_bias_reduce(zn_ctx *ctx, const void *g, bool g_bf16, int64_t ld, int64_t rows, int64_t cols, float *gb,
                           bool accumulate, bool exact) {
    const double bytes = (double)rows * cols * (g_bf16 ? 2 : 4) + 4.0 * cols;
    prefer_gemm_compatible_carveout(ctx);
    if (exact) {
        zn_launch_scope scope(ctx, ZN_PROF_BIAS_REDUCE, 0, bytes);
        const int grid = (int)((cols + 127) / 128);
        if (g_bf16)
            bias_reduce_exact_kernel<__nv_bfloat16><<<grid, 128, 0, ctx->stream>>>((const __nv_bfloat16 *)g, ld, rows, cols, gb, accumulate);
        else
            bias_reduce_exact_kernel<float><<<grid, 128, 0, ctx->stream>>>((const float *)g, ld, rows, cols, gb, accumulate);
        ZN_CUDA(ctx, cudaGetLastError());
        return ZN_OK;
    }
    const int vec = g_bf16 ? 8 : 4, strip = 32 * vec;
    const int strips = (int)((cols + strip - 1) / strip);
    // enough row splits to fill the machine about four times over, at least 64 rows each
    int64_t splits = ((int64_t)ctx->sm_count * 4 + strips - 1) / strips;
    const int64_t max_splits = (rows + 63) / 64;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
    const int64_t rows_per = (rows + splits - 1) / splits;
    splits = (rows + rows_per - 1) / rows_per;
    ZN_TRY(zn_scratch_reserve(ctx, (size_t)(splits * cols)));
    // one launch when every strip has an arrival counter of its own, else the two-kernel form
    unsigned int *counters = nullptr;
    if (strips <= ZN_COUNTER_SUMSQ) ZN_TRY(zn_lane_counters(ctx, &counters));
    zn_launch_scope scope(ctx, ZN_PROF_BIAS_REDUCE, 0, bytes, counters ? 1 : 2);
    dim3 grid((unsigned)strips, (unsigned)splits);
    if (g_bf16)
        bias_reduce_partial_kernel<__nv_bfloat16, 8><<<grid, TPB, 0, ctx->stream>>>((const __nv_bfloat16 *)g, ld, rows, cols, rows_per, ctx->scratch, gb, accumulate ? 1 : 0, counters);
    else
        bias_reduce_partial_kernel<float, 4><<<grid, TPB, 0, ctx->stream>>>((const float *)g, ld, rows, cols, rows_per, ctx->scratch, gb, accumulate ? 1 : 0, counters);
    if (!counters)
        bias_reduce_final_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, ctx->stream>>>(ctx->scratch, cols, (int)splits, gb, accumulate);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

// ---- bias-gradient accumulation that never allocates ------------------------------------------
//
// zn_accumulate_bias keeps its per-split partial sums in a scratch block that the context grows with
// cudaMalloc when a larger problem arrives.  Some users of this library cannot afford that call: a host
// program that has already handed every byte of device memory to its own pool (so cudaMalloc fails), or a
// training loop that must not stall on the device-wide synchronisation cudaMalloc/cudaFree imply.  For them
// the same two kernels run here with their partial sums in a fixed block that is part of the library image:
// ZN_NOALLOC_SCRATCH_FLOATS floats (4 MiB) of global memory that every GPU loading the library holds until
// the process exits.
//
// The block is shared by every call on a device and keeps whatever the previous call left in it.  Nothing
// in it has to start at zero: the first kernel writes every slot (split, column) that the second one reads.
// Two calls that run on the same GPU at the same time (different streams or contexts) would overwrite each
// other's partial sums; callers must order them.
constexpr size_t ZN_NOALLOC_SCRATCH_FLOATS = (size_t)1 << 20;
static __device__ __align__(256) float zn_noalloc_scratch[ZN_NOALLOC_SCRATCH_FLOATS];

// In host code `zn_noalloc_scratch` is only a stand-in for the symbol, not an address a kernel can use; the
// device address is looked up once per device, with that device current, and cached here.  The cache is
// atomic: two threads that meet in the first call on a device both look the address up and store the same value.
static float *noalloc_scratch_address(zn_ctx *ctx, zn_status *status) {
    static std::atomic<float *> per_device[64];
    *status = ZN_OK;
    if (ctx->device < 0 || ctx->device >= 64) {
        *status = zn_fail(ctx, ZN_ERR_INVALID_DEVICE, "device index %d outside the supported range", ctx->device);
        return nullptr;
    }
    float *p = per_device[ctx->device].load(std::memory_order_acquire);
    if (!p) {
        cudaError_t e = cudaGetSymbolAddress((void **)&p, zn_noalloc_scratch);   // the caller made ctx->device current
        if (e != cudaSuccess || !p) {
            *status = zn_cuda_status(ctx, e == cudaSuccess ? cudaErrorInvalidSymbol : e, "cudaGetSymbolAddress(zn_noalloc_scratch)");
            return nullptr;
        }
        per_device[ctx->device].store(p, std::memory_order_release);
    }
    return p;
}

extern "C" zn_status zn_accumulate_bias_noalloc(zn_ctx *ctx, float *grad_bias, size_t bias_len, const float *g,
                                                size_t g_len) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!grad_bias || !g) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "accumulate_bias_noalloc: null operand");
    if (bias_len == 0 || g_len % bias_len != 0)
        return zn_fail(ctx, ZN_ERR_SHAPE, "accumulate_bias_noalloc: gradient is not rows x bias_len");
    if (g_len == 0) return ZN_OK;
    if (!zn_is_device_ptr(grad_bias) || !zn_is_device_ptr(g))
        return zn_fail(ctx, ZN_ERR_INVALID_VALUE,
                       "accumulate_bias_noalloc: operands must be device pointers (staging host memory would allocate)");
    // every call, not only the first: the calling thread's current device may be another GPU
    ZN_CUDA(ctx, cudaSetDevice(ctx->device));
    prefer_gemm_compatible_carveout(ctx);
    const int64_t cols = (int64_t)bias_len, rows = (int64_t)(g_len / bias_len);
    if (ctx->precision == ZN_FP32_EXACT) {
        // The reference's order of additions (one running sum per column, rows ascending), as zn_accumulate_bias
        // gives on such a context.  That kernel keeps its sum in a register: no scratch of any kind, no size limit.
        ctx->launches += 1;
        bias_reduce_exact_kernel<float><<<(unsigned)((cols + 127) / 128), 128, 0, ctx->stream>>>(g, cols, rows, cols, grad_bias, 1);
        ZN_CUDA(ctx, cudaGetLastError());
        return ZN_OK;
    }
    // same split of the rows as zn_accumulate_bias, so both entry points add in the same order
    const int strip = 32 * 4;
    const int strips = (int)((cols + strip - 1) / strip);
    int64_t splits = ((int64_t)ctx->sm_count * 4 + strips - 1) / strips;
    const int64_t max_splits = (rows + 63) / 64;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
    const int64_t rows_per = (rows + splits - 1) / splits;
    splits = (rows + rows_per - 1) / rows_per;
    const size_t need = (size_t)(splits * cols);
    if (need > ZN_NOALLOC_SCRATCH_FLOATS)
        return zn_fail(ctx, ZN_ERR_INVALID_VALUE,
                       "accumulate_bias_noalloc: %zu rows x %zu columns needs %zu floats of scratch, the fixed block holds %zu; "
                       "use zn_accumulate_bias or fewer columns",
                       (size_t)rows, (size_t)cols, need, ZN_NOALLOC_SCRATCH_FLOATS);
    zn_status st;
    float *scratch = noalloc_scratch_address(ctx, &st);
    if (!scratch) return st;
    ctx->launches += 2;
    dim3 grid((unsigned)strips, (unsigned)splits);
    // two kernels and no arrival counters: the counters of the one-launch form live in memory the context allocates
    bias_reduce_partial_kernel<float, 4><<<grid, TPB, 0, ctx->stream>>>(g, cols, rows, cols, rows_per, scratch, nullptr, 0, nullptr);
    bias_reduce_final_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, ctx->stream>>>(scratch, cols, (int)splits, grad_bias, 1);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_loss(zn_ctx *ctx, int loss, const float *out, int64_t ld_o, const float *target, void *grad, bool grad_bf16,
                    int64_t ld_g, int64_t rows, int64_t cols, float mse_divisor, float *loss_sum_dev, bool exact) {
    if (loss != ZN_LOSS_MSE && loss != ZN_LOSS_CROSS_ENTROPY_LOGITS && loss != ZN_LOSS_CROSS_ENTROPY && loss != ZN_LOSS_BINARY_CROSS_ENTROPY)
        return zn_fail(ctx, ZN_ERR_UNSUPPORTED, "loss %d is not on the Dense path (kl_divergence has no batched form)", loss);
    const int64_t total = rows * cols;
    const bool flat = loss == ZN_LOSS_MSE || loss == ZN_LOSS_BINARY_CROSS_ENTROPY;
    int grid;
    if (loss == ZN_LOSS_MSE) grid = grid_for(ctx, (total + 3) / 4, 4);
    else if (flat) grid = grid_for(ctx, total, 4);
    else grid = grid_for(ctx, rows * 32, 8);
    ZN_TRY(zn_scratch_reserve(ctx, (size_t)grid));
    // the loss sum is formed by the last block of the loss kernel itself; the exact mode forms it in the
    // reference's order with a kernel of its own
    unsigned int *counter = nullptr;
    if (!exact) {
        ZN_TRY(zn_lane_counters(ctx, &counter));
        counter += ZN_COUNTER_LOSS;
    }
    zn_launch_scope scope(ctx, ZN_PROF_LOSS, 0, (double)total * (8 + (grad ? (grad_bf16 ? 2 : 4) : 0)), exact ? 2 : 1);
    if (loss == ZN_LOSS_MSE) {
        if (grad_bf16)
            mse_kernel<__nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(out, ld_o, target, (__nv_bfloat16 *)grad, ld_g, rows, cols, mse_divisor, ctx->scratch, loss_sum_dev, counter);
        else
            mse_kernel<float><<<grid, TPB, 0, ctx->stream>>>(out, ld_o, target, (float *)grad, ld_g, rows, cols, mse_divisor, ctx->scratch, loss_sum_dev, counter);
    } else if (loss == ZN_LOSS_BINARY_CROSS_ENTROPY) {
        if (grad_bf16)
            bce_kernel<__nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(out, ld_o, target, (__nv_bfloat16 *)grad, ld_g, rows, cols, mse_divisor, ctx->scratch, loss_sum_dev, counter);
        else
            bce_kernel<float><<<grid, TPB, 0, ctx->stream>>>(out, ld_o, target, (float *)grad, ld_g, rows, cols, mse_divisor, ctx->scratch, loss_sum_dev, counter);
    } else {
        const int plain = loss == ZN_LOSS_CROSS_ENTROPY ? 1 : 0;
        if (grad_bf16)
            zn_launch_pdl(ce_kernel<__nv_bfloat16>, dim3(grid), dim3(TPB), 0, ctx->stream, out, ld_o, target, (__nv_bfloat16 *)grad, ld_g, rows, cols, ctx->scratch, exact ? 1 : 0, plain, loss_sum_dev, counter);
        else
            zn_launch_pdl(ce_kernel<float>, dim3(grid), dim3(TPB), 0, ctx->stream, out, ld_o, target, (float *)grad, ld_g, rows, cols, ctx->scratch, exact ? 1 : 0, plain, loss_sum_dev, counter);
    }
    if (exact) loss_sum_exact_kernel<<<1, 1, 0, ctx->stream>>>(loss, out, ld_o, target, rows, cols, loss_sum_dev);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}
