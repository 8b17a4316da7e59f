// Gradient-norm clip and the SGD / Adam parameter updates.
//
// Network.trainStep's clip (src/network.zig:513-535) needs the norm of every
// gradient before any parameter moves, so the step is two passes: (1) sum of
// squares over all gradient tensors -> norm and clip factor, kept on the device;
// (2) one pass per parameter tensor that applies the factor, the reference's
// clamps and the update (cpuSgdUpdate / cpuSgdUpdateBias / cpuAdamUpdate,
// src/backend.zig:2722-2772) and refreshes the tensor-core operand copy of the
// weights.  12 bytes per parameter for SGD, 28 for Adam, plus the operand copy.
#include <cstdlib>
#include <atomic>

#include "zn_internal.h"

namespace {

constexpr int TPB = 256;
constexpr int MAX_SEGS = 32;

struct SegTable {
    const float *ptr[MAX_SEGS];
    unsigned long long count[MAX_SEGS];
    int first_block[MAX_SEGS + 1];   // blocks [first_block[i], first_block[i+1]) belong to segment i
    int nseg;
};

constexpr int ELEMS_PER_BLOCK = TPB * 4 * 8;   // 8 float4 per thread

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum of the block partials in double, by one block: thread i adds partial[i], partial[i + TPB], ...; then a tree.
__device__ __forceinline__ double sum_partials_double(const float *partial, int n, double *sm) {
    double s = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += (double)__ldcg(partial + i);
    sm[threadIdx.x] = s;
    __syncthreads();
    for (int o = TPB / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
        __syncthreads();
    }
    return sm[0];
}

// finish: 0 = partials only (a second kernel adds them up); 1 = the block that arrives last adds all partials and
// writes the sum of squares as a double; 2 = ... and writes norm and clip factor (src/network.zig:513-524).  The
// adding order is that of the two-kernel form, so the results are the same to the bit.
__global__ void sq_partial_kernel(const __grid_constant__ SegTable tab, float *__restrict__ partial,
                                  unsigned int *counter, int finish, void *out) {
    __shared__ float part[TPB / 32];
    __shared__ double fin[TPB];
    __shared__ bool last;
    int seg = 0;
    while (seg + 1 < tab.nseg && (int)blockIdx.x >= tab.first_block[seg + 1]) ++seg;
    const float *p = tab.ptr[seg];
    const unsigned long long n = tab.count[seg];
    const unsigned long long base = (unsigned long long)((int)blockIdx.x - tab.first_block[seg]) * ELEMS_PER_BLOCK;
    const unsigned long long end = min(n, base + ELEMS_PER_BLOCK);
    float s = 0.f;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        for (unsigned long long i = base + threadIdx.x * 4ull; i < end; i += TPB * 4ull) {
            if (i + 4 <= end) {
                const float4 v = __ldcs(reinterpret_cast<const float4 *>(p + i));   // read once: keep it out of L2's way
                s += v.x * v.x; s += v.y * v.y; s += v.z * v.z; s += v.w * v.w;
            } else {
                for (unsigned long long j = i; j < end; ++j) s += p[j] * p[j];
            }
        }
    } else {
        for (unsigned long long i = base + threadIdx.x; i < end; i += TPB) s += p[i] * p[i];
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < TPB / 32; ++i) t += part[i];
        partial[blockIdx.x] = t;
        if (finish) {
            __threadfence();                                       // the partial is visible before the arrival is
            last = atomicAdd(counter, 1u) == gridDim.x - 1;
        }
    }
    if (!finish) return;
    __syncthreads();
    if (!last) return;
    __threadfence();
    const double total_sq = sum_partials_double(partial, (int)gridDim.x, fin);
    if (threadIdx.x == 0) {
        if (finish == 1) {
            *static_cast<double *>(out) = total_sq;
        } else {
            float *o = static_cast<float *>(out);
            const float total = sqrtf((float)total_sq);
            o[0] = total;
            o[1] = total > 1.0f ? __fdiv_rn(1.0f, __fadd_rn(total, 1e-6f)) : 1.0f;
        }
        *counter = 0u;                                             // ready for the next launch on this lane
    }
}

// The reference's own order: one running f32 sum over every tensor in turn (src/network.zig:513-521).
// One thread; used only by the FP32_EXACT mode, where matching the reference's rounding matters more
// than speed.
__global__ void norm_exact_kernel(const __grid_constant__ SegTable tab, float *__restrict__ out) {
    float total = 0.f;
    for (int s = 0; s < tab.nseg; ++s) {
        const float *p = tab.ptr[s];
        const unsigned long long n = tab.count[s];
        unsigned long long i = 0;
        for (; i + 4 <= n; i += 4) {
            const float a = p[i], b = p[i + 1], c = p[i + 2], d = p[i + 3];
            total = __fadd_rn(total, __fmul_rn(a, a));
            total = __fadd_rn(total, __fmul_rn(b, b));
            total = __fadd_rn(total, __fmul_rn(c, c));
            total = __fadd_rn(total, __fmul_rn(d, d));
        }
        for (; i < n; ++i) total = __fadd_rn(total, __fmul_rn(p[i], p[i]));
    }
    total = sqrtf(total);
    out[0] = total;
    out[1] = total > 1.0f ? __fdiv_rn(1.0f, __fadd_rn(total, 1e-6f)) : 1.0f;
}

__global__ void scale_kernel(float *p, size_t n, const float *factor) {
    const float f = *factor;
    if (f == 1.0f) return;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        p[i] = __fmul_rn(p[i], f);
}

__device__ __forceinline__ float clamp_grad(float g) {
    if (isnan(g)) return 0.0f;
    return fminf(5.0f, fmaxf(-5.0f, g));
}

template <typename ST>
__device__ __forceinline__ void store_shadow(ST *shadow, size_t i, long long cols, long long ld, float w) {
    const size_t idx = (ld == cols) ? i : (i / (size_t)cols) * (size_t)ld + (i % (size_t)cols);
    if (sizeof(ST) == 2) reinterpret_cast<__nv_bfloat16 *>(shadow)[idx] = __float2bfloat16_rn(w);
    else reinterpret_cast<float *>(shadow)[idx] = w;
}

// w -= lr * (g + wd * w), clamps as the reference; bias: no decay, clamp +-50.
template <typename ST>
__global__ void sgd_kernel(zn_opt_args a, int is_bias) {
    const float f = a.factor_dev ? *a.factor_dev : 1.0f;
    const bool write_g = f != 1.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.count; i += (size_t)gridDim.x * blockDim.x) {
        float g = a.g[i];
        if (write_g) { g = __fmul_rn(g, f); a.g[i] = g; }
        g = clamp_grad(g);
        float w = a.w[i];
        if (is_bias) w = __fsub_rn(w, __fmul_rn(a.lr, g));
        else w = __fsub_rn(w, __fmul_rn(a.lr, __fadd_rn(g, __fmul_rn(a.wd, w))));
        w = fminf(a.w_clamp, fmaxf(-a.w_clamp, w));
        a.w[i] = w;
        if (a.shadow) store_shadow<ST>(static_cast<ST *>(a.shadow), i, a.cols, a.ld_shadow, w);
    }
}

__device__ __forceinline__ void sgd_one(const zn_opt_args &a, float f, int is_bias, float &g, float &w) {
    if (f != 1.0f) g = __fmul_rn(g, f);
    const float gc = clamp_grad(g);
    if (is_bias) w = __fsub_rn(w, __fmul_rn(a.lr, gc));
    else w = __fsub_rn(w, __fmul_rn(a.lr, __fadd_rn(gc, __fmul_rn(a.wd, w))));
    w = fminf(a.w_clamp, fmaxf(-a.w_clamp, w));
}

// Four parameters per thread, 16-byte streaming accesses (same conditions as adam_vec4_kernel).
template <typename ST>
__global__ void sgd_vec4_kernel(zn_opt_args a, int is_bias) {
    const float f = a.factor_dev ? *a.factor_dev : 1.0f;
    const bool write_g = f != 1.0f;
    const size_t n4 = a.count / 4;
    float4 *W = reinterpret_cast<float4 *>(a.w), *G = reinterpret_cast<float4 *>(a.g);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 g = __ldcs(&G[i]), w = __ldcs(&W[i]);
        sgd_one(a, f, is_bias, g.x, w.x);
        sgd_one(a, f, is_bias, g.y, w.y);
        sgd_one(a, f, is_bias, g.z, w.z);
        sgd_one(a, f, is_bias, g.w, w.w);
        if (write_g) __stcs(&G[i], g);
        __stcs(&W[i], w);
        if (a.shadow) {
            if (sizeof(ST) == 2) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
                reinterpret_cast<uint2 *>(a.shadow)[i] =
                    make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
            } else {
                reinterpret_cast<float4 *>(a.shadow)[i] = w;
            }
        }
    }
}

// cpuAdamUpdate, src/backend.zig:2760-2772, with Adam.step's L2 term (src/optimizer.zig:221-228) folded in.
__device__ __forceinline__ void adam_one(const zn_opt_args &a, float f, float omb1, float omb2, float &g, float &w,
                                         float &m, float &v) {
    if (f != 1.0f) g = __fmul_rn(g, f);
    if (a.wd > 0.0f) g = __fadd_rn(g, __fmul_rn(a.wd, w));
    const float gc = clamp_grad(g);
    m = __fadd_rn(__fmul_rn(a.beta1, m), __fmul_rn(omb1, gc));
    v = __fadd_rn(__fmul_rn(a.beta2, v), __fmul_rn(__fmul_rn(omb2, gc), gc));
    const float m_hat = __fdiv_rn(m, a.bc1);
    const float v_hat = __fdiv_rn(v, a.bc2);
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(a.lr, m_hat), __fadd_rn(__fsqrt_rn(v_hat), a.eps)));
    w = fminf(a.w_clamp, fmaxf(-a.w_clamp, w));
    // AdamW's decoupled decay, applied to the clamped weight (src/optimizer.zig:288-296)
    if (a.decay_mul != 0.0f) w = __fmul_rn(w, a.decay_mul);
}

// Four parameters per thread with 16-byte accesses; the host picks this variant when every pointer is
// 16-byte aligned, the count is a multiple of 4 and the operand copy (if any) has the weights' own pitch.
template <typename ST>
__global__ void adam_vec4_kernel(zn_opt_args a) {
    const float f = a.factor_dev ? *a.factor_dev : 1.0f;
    const bool write_g = (f != 1.0f) || (a.wd > 0.0f);
    const float omb1 = 1.0f - a.beta1, omb2 = 1.0f - a.beta2;
    const size_t n4 = a.count / 4;
    float4 *W = reinterpret_cast<float4 *>(a.w), *G = reinterpret_cast<float4 *>(a.g);
    float4 *M = reinterpret_cast<float4 *>(a.m), *V = reinterpret_cast<float4 *>(a.v);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        // streaming accesses: this pass touches every parameter once while GEMMs of the next step run on the
        // same GPU; it should not push their operand tiles out of L2
        float4 g = __ldcs(&G[i]), w = __ldcs(&W[i]), m = __ldcs(&M[i]), v = __ldcs(&V[i]);
        adam_one(a, f, omb1, omb2, g.x, w.x, m.x, v.x);
        adam_one(a, f, omb1, omb2, g.y, w.y, m.y, v.y);
        adam_one(a, f, omb1, omb2, g.z, w.z, m.z, v.z);
        adam_one(a, f, omb1, omb2, g.w, w.w, m.w, v.w);
        if (write_g) __stcs(&G[i], g);
        __stcs(&M[i], m);
        __stcs(&V[i], v);
        __stcs(&W[i], w);
        if (a.shadow) {
            if (sizeof(ST) == 2) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
                reinterpret_cast<uint2 *>(a.shadow)[i] =
                    make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
            } else {
                reinterpret_cast<float4 *>(a.shadow)[i] = w;
            }
        }
    }
}

template <typename ST>
__global__ void adam_kernel(zn_opt_args a) {
    const float f = a.factor_dev ? *a.factor_dev : 1.0f;
    const bool write_g = (f != 1.0f) || (a.wd > 0.0f);
    const float omb1 = 1.0f - a.beta1, omb2 = 1.0f - a.beta2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.count; i += (size_t)gridDim.x * blockDim.x) {
        float g = a.g[i];
        float w = a.w[i];
        if (f != 1.0f) g = __fmul_rn(g, f);
        if (a.wd > 0.0f) g = __fadd_rn(g, __fmul_rn(a.wd, w));
        if (write_g) a.g[i] = g;
        g = clamp_grad(g);
        const float m = __fadd_rn(__fmul_rn(a.beta1, a.m[i]), __fmul_rn(omb1, g));
        const float v = __fadd_rn(__fmul_rn(a.beta2, a.v[i]), __fmul_rn(__fmul_rn(omb2, g), g));
        a.m[i] = m;
        a.v[i] = v;
        const float m_hat = __fdiv_rn(m, a.bc1);
        const float v_hat = __fdiv_rn(v, a.bc2);
        w = __fsub_rn(w, __fdiv_rn(__fmul_rn(a.lr, m_hat), __fadd_rn(__fsqrt_rn(v_hat), a.eps)));
        w = fminf(a.w_clamp, fmaxf(-a.w_clamp, w));
        if (a.decay_mul != 0.0f) w = __fmul_rn(w, a.decay_mul);
        a.w[i] = w;
        if (a.shadow) store_shadow<ST>(static_cast<ST *>(a.shadow), i, a.cols, a.ld_shadow, w);
    }
}

// Optimizers with one state tensor (held in a.m).
//   MOMENTUM  Sgd.step with momentum > 0 (src/optimizer.zig:114-159): v = momentum*v - lr*g; w = w + v.  The
//             reference builds this from Backend.scale and Backend.elementWise, so neither clamp applies.
//   RMSPROP   Rmsprop.step's L2 term (src/optimizer.zig:346-355) and cpuRmspropUpdate (src/backend.zig:2774-2783).
enum { STATE1_MOMENTUM = 0, STATE1_RMSPROP = 1 };

template <int KIND>
__device__ __forceinline__ void state1_one(const zn_opt_args &a, float f, float omr, float &g, float &w, float &s) {
    if (f != 1.0f) g = __fmul_rn(g, f);
    if (KIND == STATE1_MOMENTUM) {
        s = __fsub_rn(__fmul_rn(s, a.momentum), __fmul_rn(g, a.lr));
        w = __fadd_rn(w, s);
    } else {
        if (a.wd > 0.0f) g = __fadd_rn(g, __fmul_rn(a.wd, w));
        const float gc = clamp_grad(g);
        s = __fadd_rn(__fmul_rn(a.rho, s), __fmul_rn(__fmul_rn(omr, gc), gc));
        w = __fsub_rn(w, __fdiv_rn(__fmul_rn(a.lr, gc), __fadd_rn(__fsqrt_rn(s), a.eps)));
        w = fminf(a.w_clamp, fmaxf(-a.w_clamp, w));
    }
}

template <int KIND, typename ST>
__global__ void state1_kernel(zn_opt_args a) {
    const float f = a.factor_dev ? *a.factor_dev : 1.0f;
    const bool write_g = (f != 1.0f) || (KIND == STATE1_RMSPROP && a.wd > 0.0f);
    const float omr = 1.0f - a.rho;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.count; i += (size_t)gridDim.x * blockDim.x) {
        float g = a.g[i], w = a.w[i], s = a.m[i];
        state1_one<KIND>(a, f, omr, g, w, s);
        if (write_g) a.g[i] = g;
        a.m[i] = s;
        a.w[i] = w;
        if (a.shadow) store_shadow<ST>(static_cast<ST *>(a.shadow), i, a.cols, a.ld_shadow, w);
    }
}

// Four parameters per thread, 16-byte streaming accesses (same conditions as adam_vec4_kernel).
template <int KIND, typename ST>
__global__ void state1_vec4_kernel(zn_opt_args a) {
    const float f = a.factor_dev ? *a.factor_dev : 1.0f;
    const bool write_g = (f != 1.0f) || (KIND == STATE1_RMSPROP && a.wd > 0.0f);
    const float omr = 1.0f - a.rho;
    const size_t n4 = a.count / 4;
    float4 *W = reinterpret_cast<float4 *>(a.w), *G = reinterpret_cast<float4 *>(a.g), *S = reinterpret_cast<float4 *>(a.m);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 g = __ldcs(&G[i]), w = __ldcs(&W[i]), s = __ldcs(&S[i]);
        state1_one<KIND>(a, f, omr, g.x, w.x, s.x);
        state1_one<KIND>(a, f, omr, g.y, w.y, s.y);
        state1_one<KIND>(a, f, omr, g.z, w.z, s.z);
        state1_one<KIND>(a, f, omr, g.w, w.w, s.w);
        if (write_g) __stcs(&G[i], g);
        __stcs(&S[i], s);
        __stcs(&W[i], w);
        if (a.shadow) {
            if (sizeof(ST) == 2) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
                reinterpret_cast<uint2 *>(a.shadow)[i] =
                    make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
            } else {
                reinterpret_cast<float4 *>(a.shadow)[i] = w;
            }
        }
    }
}

// The training step runs these kernels on side lanes underneath the persistent GEMM, whose CTAs need the
// SM configured for maximum shared memory.  A kernel that lets the driver pick another shared-memory /
// L1 split cannot share an SM with them and would only run between GEMM launches; ask for the same split.
void prefer_gemm_compatible_carveout(zn_ctx *ctx) {
    static std::atomic<uint64_t> done_mask{0};
    const uint64_t bit = 1ull << (ctx->device & 63);
    if (done_mask.load() & bit) return;
    done_mask.fetch_or(bit);
    const int c = cudaSharedmemCarveoutMaxShared;
    const cudaFuncAttribute at = cudaFuncAttributePreferredSharedMemoryCarveout;
    cudaFuncSetAttribute(sq_partial_kernel, at, c);
    cudaFuncSetAttribute(norm_exact_kernel, at, c);
    cudaFuncSetAttribute(scale_kernel, at, c);
    cudaFuncSetAttribute(sgd_kernel<float>, at, c);
    cudaFuncSetAttribute(sgd_kernel<__nv_bfloat16>, at, c);
    cudaFuncSetAttribute(sgd_vec4_kernel<float>, at, c);
    cudaFuncSetAttribute(sgd_vec4_kernel<__nv_bfloat16>, at, c);
    cudaFuncSetAttribute(adam_kernel<float>, at, c);
    cudaFuncSetAttribute(adam_kernel<__nv_bfloat16>, at, c);
    cudaFuncSetAttribute(adam_vec4_kernel<float>, at, c);
    cudaFuncSetAttribute(adam_vec4_kernel<__nv_bfloat16>, at, c);
    cudaFuncSetAttribute(state1_kernel<STATE1_MOMENTUM, float>, at, c);
    cudaFuncSetAttribute(state1_kernel<STATE1_MOMENTUM, __nv_bfloat16>, at, c);
    cudaFuncSetAttribute(state1_kernel<STATE1_RMSPROP, float>, at, c);
    cudaFuncSetAttribute(state1_kernel<STATE1_RMSPROP, __nv_bfloat16>, at, c);
    cudaFuncSetAttribute(state1_vec4_kernel<STATE1_MOMENTUM, float>, at, c);
    cudaFuncSetAttribute(state1_vec4_kernel<STATE1_MOMENTUM, __nv_bfloat16>, at, c);
    cudaFuncSetAttribute(state1_vec4_kernel<STATE1_RMSPROP, float>, at, c);
    cudaFuncSetAttribute(state1_vec4_kernel<STATE1_RMSPROP, __nv_bfloat16>, at, c);
    cudaGetLastError();
}

int grid_for(zn_ctx *ctx, size_t n) {
    prefer_gemm_compatible_carveout(ctx);
    size_t blocks = (n + TPB - 1) / TPB;
    // Two blocks per SM: the update kernels run beside a persistent GEMM CTA on every SM, and each of their
    // threads keeps four 16-byte loads in flight, which is enough to stream at the rate the GEMM leaves them;
    // more resident warps only take issue slots from the GEMM's epilogue warps (measured with 8 per SM: the
    // 8192-row Adam step 8.25 -> 8.10 ms, the 65536-row step 61.0 -> 59.7 ms).  ZN_OPT_BLOCKS_PER_SM overrides.
    static const int per_sm = getenv("ZN_OPT_BLOCKS_PER_SM") ? atoi(getenv("ZN_OPT_BLOCKS_PER_SM")) : 2;
    const size_t cap = (size_t)ctx->sm_count * (size_t)(per_sm > 0 ? per_sm : 2);
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}   // namespace

zn_status zn_k_grad_norm(zn_ctx *ctx, const zn_seg *segs, int nseg, float *norm_factor_dev, bool exact) {
    if (nseg <= 0 || nseg > MAX_SEGS) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "grad norm: 1..%d tensors supported", MAX_SEGS);
    SegTable tab;
    int blocks = 0;
    double bytes = 0;
    for (int i = 0; i < nseg; ++i) {
        tab.ptr[i] = segs[i].ptr;
        tab.count[i] = segs[i].count;
        tab.first_block[i] = blocks;
        blocks += (int)((segs[i].count + ELEMS_PER_BLOCK - 1) / ELEMS_PER_BLOCK);
        bytes += 4.0 * segs[i].count;
    }
    tab.first_block[nseg] = blocks;
    tab.nseg = nseg;
    if (blocks == 0) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "grad norm: empty tensors");
    if (exact) {
        zn_launch_scope scope(ctx, ZN_PROF_GRAD_NORM, 0, bytes, 1);
        norm_exact_kernel<<<1, 1, 0, ctx->stream>>>(tab, norm_factor_dev);
        ZN_CUDA(ctx, cudaGetLastError());
        return ZN_OK;
    }
    ZN_TRY(zn_scratch_reserve(ctx, (size_t)blocks));
    unsigned int *counters = nullptr;
    ZN_TRY(zn_lane_counters(ctx, &counters));
    zn_launch_scope scope(ctx, ZN_PROF_GRAD_NORM, 0, bytes, 1);
    sq_partial_kernel<<<blocks, TPB, 0, ctx->stream>>>(tab, ctx->scratch, counters + ZN_COUNTER_SUMSQ, 2, norm_factor_dev);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

namespace {

__global__ void norm_combine_kernel(const double *__restrict__ sums, int count, float *__restrict__ out) {
    double s = 0.0;
    for (int i = 0; i < count; ++i) s += sums[i];
    const float total = sqrtf((float)s);
    out[0] = total;
    out[1] = total > 1.0f ? __fdiv_rn(1.0f, __fadd_rn(total, 1e-6f)) : 1.0f;
}

}   // namespace

zn_status zn_k_sumsq(zn_ctx *ctx, const zn_seg *segs, int nseg, double *sumsq_dev) {
    if (nseg <= 0 || nseg > MAX_SEGS) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "sum of squares: 1..%d tensors supported", MAX_SEGS);
    SegTable tab;
    int blocks = 0;
    double bytes = 0;
    for (int i = 0; i < nseg; ++i) {
        tab.ptr[i] = segs[i].ptr;
        tab.count[i] = segs[i].count;
        tab.first_block[i] = blocks;
        blocks += (int)((segs[i].count + ELEMS_PER_BLOCK - 1) / ELEMS_PER_BLOCK);
        bytes += 4.0 * segs[i].count;
    }
    tab.first_block[nseg] = blocks;
    tab.nseg = nseg;
    if (blocks == 0) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "sum of squares: empty tensors");
    prefer_gemm_compatible_carveout(ctx);
    {
        static std::atomic<uint64_t> done_mask{0};
        const uint64_t bit = 1ull << (ctx->device & 63);
        if (!(done_mask.load() & bit)) {
            done_mask.fetch_or(bit);
            cudaFuncSetAttribute(sq_partial_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            cudaFuncSetAttribute(norm_combine_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            cudaGetLastError();
        }
    }
    ZN_TRY(zn_scratch_reserve(ctx, (size_t)blocks));
    unsigned int *counters = nullptr;
    ZN_TRY(zn_lane_counters(ctx, &counters));
    zn_launch_scope scope(ctx, ZN_PROF_GRAD_NORM, 0, bytes, 1);
    sq_partial_kernel<<<blocks, TPB, 0, ctx->stream>>>(tab, ctx->scratch, counters + ZN_COUNTER_SUMSQ, 1, sumsq_dev);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_norm_combine(zn_ctx *ctx, const double *sumsq_dev, int count, float *norm_factor_dev) {
    zn_launch_scope scope(ctx, ZN_PROF_GRAD_NORM, 0, 8.0 * count, 1);
    norm_combine_kernel<<<1, 1, 0, ctx->stream>>>(sumsq_dev, count, norm_factor_dev);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_scale(zn_ctx *ctx, float *p, size_t n, const float *factor_dev) {
    zn_launch_scope scope(ctx, ZN_PROF_OPTIMIZER, 0, 8.0 * n);
    scale_kernel<<<grid_for(ctx, n), TPB, 0, ctx->stream>>>(p, n, factor_dev);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_sgd(zn_ctx *ctx, const zn_opt_args &a, bool is_bias) {
    zn_launch_scope scope(ctx, ZN_PROF_OPTIMIZER, 0, (12.0 + (a.shadow ? (a.shadow_bf16 ? 2 : 4) : 0)) * a.count);
    auto aligned = [](const void *p, uintptr_t to) { return (reinterpret_cast<uintptr_t>(p) & (to - 1)) == 0; };
    const bool vec4 = a.count % 4 == 0 && a.count >= 4096 && aligned(a.w, 16) && aligned(a.g, 16) &&
                      (!a.shadow || (a.ld_shadow == a.cols && aligned(a.shadow, a.shadow_bf16 ? 8 : 16)));
    if (vec4) {
        const int grid = grid_for(ctx, a.count / 4);
        if (a.shadow && a.shadow_bf16) sgd_vec4_kernel<__nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(a, is_bias ? 1 : 0);
        else sgd_vec4_kernel<float><<<grid, TPB, 0, ctx->stream>>>(a, is_bias ? 1 : 0);
        ZN_CUDA(ctx, cudaGetLastError());
        return ZN_OK;
    }
    if (a.shadow && a.shadow_bf16) sgd_kernel<__nv_bfloat16><<<grid_for(ctx, a.count), TPB, 0, ctx->stream>>>(a, is_bias ? 1 : 0);
    else sgd_kernel<float><<<grid_for(ctx, a.count), TPB, 0, ctx->stream>>>(a, is_bias ? 1 : 0);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_adam(zn_ctx *ctx, const zn_opt_args &a) {
    zn_launch_scope scope(ctx, ZN_PROF_OPTIMIZER, 0, (28.0 + (a.shadow ? (a.shadow_bf16 ? 2 : 4) : 0)) * a.count);
    auto aligned = [](const void *p, uintptr_t to) { return (reinterpret_cast<uintptr_t>(p) & (to - 1)) == 0; };
    const bool vec4 = a.count % 4 == 0 && a.count >= 4096 && aligned(a.w, 16) && aligned(a.g, 16) && aligned(a.m, 16) &&
                      aligned(a.v, 16) && (!a.shadow || (a.ld_shadow == a.cols && aligned(a.shadow, a.shadow_bf16 ? 8 : 16)));
    if (vec4) {
        const int grid = grid_for(ctx, a.count / 4);
        if (a.shadow && a.shadow_bf16) adam_vec4_kernel<__nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(a);
        else adam_vec4_kernel<float><<<grid, TPB, 0, ctx->stream>>>(a);
        ZN_CUDA(ctx, cudaGetLastError());
        return ZN_OK;
    }
    if (a.shadow && a.shadow_bf16) adam_kernel<__nv_bfloat16><<<grid_for(ctx, a.count), TPB, 0, ctx->stream>>>(a);
    else adam_kernel<float><<<grid_for(ctx, a.count), TPB, 0, ctx->stream>>>(a);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

namespace {

template <int KIND>
zn_status launch_state1(zn_ctx *ctx, const zn_opt_args &a) {
    zn_launch_scope scope(ctx, ZN_PROF_OPTIMIZER, 0, (20.0 + (a.shadow ? (a.shadow_bf16 ? 2 : 4) : 0)) * a.count);
    auto aligned = [](const void *p, uintptr_t to) { return (reinterpret_cast<uintptr_t>(p) & (to - 1)) == 0; };
    const bool vec4 = a.count % 4 == 0 && a.count >= 4096 && aligned(a.w, 16) && aligned(a.g, 16) && aligned(a.m, 16) &&
                      (!a.shadow || (a.ld_shadow == a.cols && aligned(a.shadow, a.shadow_bf16 ? 8 : 16)));
    const bool bf16 = a.shadow && a.shadow_bf16;
    if (vec4) {
        const int grid = grid_for(ctx, a.count / 4);
        if (bf16) state1_vec4_kernel<KIND, __nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(a);
        else state1_vec4_kernel<KIND, float><<<grid, TPB, 0, ctx->stream>>>(a);
    } else {
        const int grid = grid_for(ctx, a.count);
        if (bf16) state1_kernel<KIND, __nv_bfloat16><<<grid, TPB, 0, ctx->stream>>>(a);
        else state1_kernel<KIND, float><<<grid, TPB, 0, ctx->stream>>>(a);
    }
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

}   // namespace

namespace {

struct MultiUpdateTable {
    zn_opt_args a[ZN_MULTI_UPDATE_MAX];
    int kind[ZN_MULTI_UPDATE_MAX], is_bias[ZN_MULTI_UPDATE_MAX];
    int first_block[ZN_MULTI_UPDATE_MAX + 1];
    int n;
};
constexpr int MULTI_ELEMS_PER_BLOCK = TPB * 8;

// One launch for every parameter tensor of a small network (where a launch costs more than the update itself).
// Each block belongs to one tensor and walks its own 2048 elements with that tensor's rule.
__global__ void multi_update_kernel(const __grid_constant__ MultiUpdateTable tab) {
    int t = 0;
    while (t + 1 < tab.n && (int)blockIdx.x >= tab.first_block[t + 1]) ++t;
    const zn_opt_args &a = tab.a[t];
    const int kind = tab.kind[t], is_bias = tab.is_bias[t];
    const float f = a.factor_dev ? *a.factor_dev : 1.0f;
    const size_t base = (size_t)((int)blockIdx.x - tab.first_block[t]) * MULTI_ELEMS_PER_BLOCK;
    const size_t end = min(a.count, base + MULTI_ELEMS_PER_BLOCK);
    const float omb1 = 1.0f - a.beta1, omb2 = 1.0f - a.beta2, omr = 1.0f - a.rho;
    for (size_t i = base + threadIdx.x; i < end; i += TPB) {
        float g = a.g[i], w = a.w[i];
        bool write_g = f != 1.0f;
        if (kind == 1) {
            float m = a.m[i], v = a.v[i];
            write_g = write_g || a.wd > 0.0f;
            adam_one(a, f, omb1, omb2, g, w, m, v);
            a.m[i] = m;
            a.v[i] = v;
        } else if (kind == 2) {
            float st = a.m[i];
            state1_one<STATE1_MOMENTUM>(a, f, omr, g, w, st);
            a.m[i] = st;
        } else if (kind == 4) {
            float st = a.m[i];
            write_g = write_g || a.wd > 0.0f;
            state1_one<STATE1_RMSPROP>(a, f, omr, g, w, st);
            a.m[i] = st;
        } else {
            sgd_one(a, f, is_bias, g, w);
        }
        if (write_g) a.g[i] = g;
        a.w[i] = w;
        if (a.shadow) {
            if (a.shadow_bf16) store_shadow<__nv_bfloat16>(static_cast<__nv_bfloat16 *>(a.shadow), i, a.cols, a.ld_shadow, w);
            else store_shadow<float>(static_cast<float *>(a.shadow), i, a.cols, a.ld_shadow, w);
        }
    }
}

}   // namespace

zn_status zn_k_multi_update(zn_ctx *ctx, const zn_opt_args *args, const int *kinds, const int *is_bias, int count) {
    if (count <= 0 || count > ZN_MULTI_UPDATE_MAX)
        return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "multi update: 1..%d tensors supported", (int)ZN_MULTI_UPDATE_MAX);
    MultiUpdateTable tab;
    int blocks = 0;
    double bytes = 0;
    for (int i = 0; i < count; ++i) {
        tab.a[i] = args[i];
        tab.kind[i] = kinds[i];
        tab.is_bias[i] = is_bias[i];
        tab.first_block[i] = blocks;
        blocks += (int)((args[i].count + MULTI_ELEMS_PER_BLOCK - 1) / MULTI_ELEMS_PER_BLOCK);
        bytes += (kinds[i] == 1 ? 28.0 : kinds[i] == 0 ? 12.0 : 20.0) * (double)args[i].count;
    }
    tab.first_block[count] = blocks;
    tab.n = count;
    if (blocks == 0) return ZN_OK;
    prefer_gemm_compatible_carveout(ctx);
    zn_launch_scope scope(ctx, ZN_PROF_OPTIMIZER, 0, bytes);
    multi_update_kernel<<<blocks, TPB, 0, ctx->stream>>>(tab);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_sgd_momentum(zn_ctx *ctx, const zn_opt_args &a) { return launch_state1<STATE1_MOMENTUM>(ctx, a); }
zn_status zn_k_rmsprop(zn_ctx *ctx, const zn_opt_args &a) { return launch_state1<STATE1_RMSPROP>(ctx, a); }

namespace {
__global__ void f32_to_f64_kernel(const float *__restrict__ src, double *__restrict__ dst) { *dst = (double)*src; }
__global__ void f64_to_f32_kernel(const double *__restrict__ src, float *__restrict__ dst) { *dst = (float)*src; }
}   // namespace

// One value between the float loss slot and the double array the ranks exchange with the sums of squares.
zn_status zn_k_f32_to_f64(zn_ctx *ctx, const float *src, double *dst) {
    zn_launch_scope scope(ctx, ZN_PROF_GRAD_NORM, 0, 12.0);
    f32_to_f64_kernel<<<1, 1, 0, ctx->stream>>>(src, dst);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

zn_status zn_k_f64_to_f32(zn_ctx *ctx, const double *src, float *dst) {
    zn_launch_scope scope(ctx, ZN_PROF_GRAD_NORM, 0, 12.0);
    f64_to_f32_kernel<<<1, 1, 0, ctx->stream>>>(src, dst);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}
