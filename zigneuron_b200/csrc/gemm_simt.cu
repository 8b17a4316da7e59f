// fp32 CUDA-core GEMM for the three Dense products, with the bias / activation /
// activation-derivative mask / accumulate epilogue fused in.
//
// Stands where the reference has Backend.matMul, matMulTransposeA and
// matMulTransposeB (src/backend.zig:169-195, :298-325) and their CPU kernels
// (:2520-2647).  Every C[i][j] is summed over k in ascending order by a single
// thread, exactly the order of the reference loops; with EXACT the multiply and
// the add are separate roundings as well (the reference has no FMA), which makes
// the product bit-identical to the reference's.
#include "zn_internal.h"
#include "zn_act.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256;

__device__ __forceinline__ float apply_act(int act, float v) {
    switch (act) {
    case ZN_ACT_RELU: return v > 0.f ? v : 0.f;
    case ZN_ACT_SIGMOID:
        if (v >= 0.f) return 1.f / (1.f + expf(-v));
        else { const float e = expf(v); return e / (1.f + e); }
    case ZN_ACT_TANH: return tanhf(v);
    case ZN_ACT_GELU: return zn_gelu_fwd(v);
    case ZN_ACT_LEAKY_RELU: return zn_leaky_fwd(v);
    case ZN_ACT_ELU: return zn_elu_fwd(v);
    default: return v;
    }
}

struct Epi {
    const float *bias;
    const float *mask;
    float *out;
    int64_t ld_mask, ld_out;
    int act, accumulate;
    int acc_init;   // NN with accumulate: start the running sum from C, as cpuMatMul does (src/backend.zig:2521)
};

template <bool EXACT>
__device__ __forceinline__ float mac(float acc, float a, float b) {
    if (EXACT) return __fadd_rn(acc, __fmul_rn(a, b));
    return fmaf(a, b, acc);
}

// A_KC: A is contiguous along k (row-major [m][k]); otherwise contiguous along m ([k][m]).
// B_NC: B is contiguous along n (row-major [k][n]); otherwise contiguous along k ([n][k]).
template <bool A_KC, bool B_NC, bool EXACT>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const float *__restrict__ a, int64_t lda, const float *__restrict__ b, int64_t ldb,
                 int64_t M, int64_t N, int64_t K, Epi ep) {
    __shared__ __align__(16) float As[BK][BM];
    __shared__ __align__(16) float Bs[BK][BN];

    const int t = threadIdx.x;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
    const int tx = t & 15, ty = t >> 4;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    if (ep.acc_init) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t r = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int64_t c = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
                if (r < M && c < N) acc[i][j] = ep.out[r * ep.ld_out + c];
            }
        }
    }

    const bool a_vec = ((reinterpret_cast<uintptr_t>(a) & 15) == 0) && (lda % 4 == 0);
    const bool b_vec = ((reinterpret_cast<uintptr_t>(b) & 15) == 0) && (ldb % 4 == 0);

    for (int64_t k0 = 0; k0 < K; k0 += BK) {
        float ra[8], rb[8];
        // ---- A tile: 128 (m) x 16 (k)
        if (A_KC) {
            const int row = t & 127, ks = (t >> 7) * 8;
            const int64_t gm = m0 + row, gk = k0 + ks;
            const float *src = a + gm * lda + gk;
            if (gm < M && gk + 8 <= K && a_vec) {
                const float4 v0 = *reinterpret_cast<const float4 *>(src);
                const float4 v1 = *reinterpret_cast<const float4 *>(src + 4);
                ra[0] = v0.x; ra[1] = v0.y; ra[2] = v0.z; ra[3] = v0.w;
                ra[4] = v1.x; ra[5] = v1.y; ra[6] = v1.z; ra[7] = v1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) ra[i] = (gm < M && gk + i < K) ? src[i] : 0.f;
            }
        } else {
            const int kr = t >> 4, ms = (t & 15) * 8;
            const int64_t gk = k0 + kr, gm = m0 + ms;
            const float *src = a + gk * lda + gm;
            if (gk < K && gm + 8 <= M && a_vec) {
                const float4 v0 = *reinterpret_cast<const float4 *>(src);
                const float4 v1 = *reinterpret_cast<const float4 *>(src + 4);
                ra[0] = v0.x; ra[1] = v0.y; ra[2] = v0.z; ra[3] = v0.w;
                ra[4] = v1.x; ra[5] = v1.y; ra[6] = v1.z; ra[7] = v1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) ra[i] = (gk < K && gm + i < M) ? src[i] : 0.f;
            }
        }
        // ---- B tile: 16 (k) x 128 (n)
        if (B_NC) {
            const int kr = t >> 4, ns = (t & 15) * 8;
            const int64_t gk = k0 + kr, gn = n0 + ns;
            const float *src = b + gk * ldb + gn;
            if (gk < K && gn + 8 <= N && b_vec) {
                const float4 v0 = *reinterpret_cast<const float4 *>(src);
                const float4 v1 = *reinterpret_cast<const float4 *>(src + 4);
                rb[0] = v0.x; rb[1] = v0.y; rb[2] = v0.z; rb[3] = v0.w;
                rb[4] = v1.x; rb[5] = v1.y; rb[6] = v1.z; rb[7] = v1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) rb[i] = (gk < K && gn + i < N) ? src[i] : 0.f;
            }
        } else {
            const int col = t & 127, ks = (t >> 7) * 8;
            const int64_t gn = n0 + col, gk = k0 + ks;
            const float *src = b + gn * ldb + gk;
            if (gn < N && gk + 8 <= K && b_vec) {
                const float4 v0 = *reinterpret_cast<const float4 *>(src);
                const float4 v1 = *reinterpret_cast<const float4 *>(src + 4);
                rb[0] = v0.x; rb[1] = v0.y; rb[2] = v0.z; rb[3] = v0.w;
                rb[4] = v1.x; rb[5] = v1.y; rb[6] = v1.z; rb[7] = v1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) rb[i] = (gn < N && gk + i < K) ? src[i] : 0.f;
            }
        }
        __syncthreads();   // previous tile fully consumed
        if (A_KC) {
            const int row = t & 127, ks = (t >> 7) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) As[ks + i][row] = ra[i];
        } else {
            const int kr = t >> 4, ms = (t & 15) * 8;
            *reinterpret_cast<float4 *>(&As[kr][ms]) = make_float4(ra[0], ra[1], ra[2], ra[3]);
            *reinterpret_cast<float4 *>(&As[kr][ms + 4]) = make_float4(ra[4], ra[5], ra[6], ra[7]);
        }
        if (B_NC) {
            const int kr = t >> 4, ns = (t & 15) * 8;
            *reinterpret_cast<float4 *>(&Bs[kr][ns]) = make_float4(rb[0], rb[1], rb[2], rb[3]);
            *reinterpret_cast<float4 *>(&Bs[kr][ns + 4]) = make_float4(rb[4], rb[5], rb[6], rb[7]);
        } else {
            const int col = t & 127, ks = (t >> 7) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) Bs[ks + i][col] = rb[i];
        }
        __syncthreads();

#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[kk][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = mac<EXACT>(acc[i][j], av[i], bv[j]);
        }
    }

    // ---- epilogue
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t r = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (r >= M) continue;
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            const int64_t c0 = n0 + jh * 64 + tx * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int64_t c = c0 + j;
                if (c >= N) continue;
                float v = acc[i][jh * 4 + j];
                if (ep.bias) v = __fadd_rn(v, ep.bias[c]);
                v = apply_act(ep.act, v);
                if (ep.mask) v = ep.mask[r * ep.ld_mask + c] > 0.f ? v : 0.f;
                float *dst = ep.out + r * ep.ld_out + c;
                if (ep.accumulate) v = __fadd_rn(*dst, v);
                *dst = v;
            }
        }
    }
}

template <bool A_KC, bool B_NC>
void launch(zn_ctx *ctx, const float *a, int64_t lda, const float *b, int64_t ldb, int64_t m, int64_t n, int64_t k,
            const Epi &ep, bool exact) {
    dim3 grid((unsigned)((n + BN - 1) / BN), (unsigned)((m + BM - 1) / BM));
    if (exact) gemm_simt_kernel<A_KC, B_NC, true><<<grid, THREADS, 0, ctx->stream>>>(a, lda, b, ldb, m, n, k, ep);
    else gemm_simt_kernel<A_KC, B_NC, false><<<grid, THREADS, 0, ctx->stream>>>(a, lda, b, ldb, m, n, k, ep);
}

// ---- small-tile variant ------------------------------------------------------------------------------
// 64 x 64 tiles, 4 x 4 outputs per thread.  Same arithmetic and the same k order per element as the kernel
// above; used when the 128 x 128 grid would leave most SMs idle (the layers of small networks).
constexpr int SM_T = 64;

template <bool KC /* source contiguous along k */>
__device__ __forceinline__ void load4(const float *__restrict__ src, int64_t ld, int64_t mn0, int64_t k0, int64_t MN,
                                      int64_t K, int t, bool vec_ok, float (&r)[4]) {
    // KC:  the tile is [64 mn][16 k], thread -> (mn = t & 63, k = (t >> 6) * 4 .. +3), element (mn, k) at src[mn * ld + k]
    // !KC: the tile is [16 k][64 mn], thread -> (k = t >> 4, mn = (t & 15) * 4 .. +3), element (mn, k) at src[k * ld + mn]
    if (KC) {
        const int64_t gmn = mn0 + (t & 63), gk = k0 + (t >> 6) * 4;
        const float *p = src + gmn * ld + gk;
        if (gmn < MN && gk + 4 <= K && vec_ok) {
            const float4 v = *reinterpret_cast<const float4 *>(p);
            r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) r[i] = (gmn < MN && gk + i < K) ? p[i] : 0.f;
        }
    } else {
        const int64_t gk = k0 + (t >> 4), gmn = mn0 + (t & 15) * 4;
        const float *p = src + gk * ld + gmn;
        if (gk < K && gmn + 4 <= MN && vec_ok) {
            const float4 v = *reinterpret_cast<const float4 *>(p);
            r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) r[i] = (gk < K && gmn + i < MN) ? p[i] : 0.f;
        }
    }
}

template <bool A_KC, bool B_NC, bool EXACT>
__global__ void __launch_bounds__(THREADS)
gemm_simt_small_kernel(const float *__restrict__ a, int64_t lda, const float *__restrict__ b, int64_t ldb,
                       int64_t M, int64_t N, int64_t K, Epi ep) {
    __shared__ __align__(16) float As[BK][SM_T];
    __shared__ __align__(16) float Bs[BK][SM_T];
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * SM_T, n0 = (int64_t)blockIdx.x * SM_T;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t r = m0 + ty * 4 + i, c = n0 + tx * 4 + j;
            acc[i][j] = (ep.acc_init && r < M && c < N) ? ep.out[r * ep.ld_out + c] : 0.f;
        }
    const bool a_vec = ((reinterpret_cast<uintptr_t>(a) & 15) == 0) && (lda % 4 == 0);
    const bool b_vec = ((reinterpret_cast<uintptr_t>(b) & 15) == 0) && (ldb % 4 == 0);

    for (int64_t k0 = 0; k0 < K; k0 += BK) {
        float ra[4], rb[4];
        load4<A_KC>(a, lda, m0, k0, M, K, t, a_vec, ra);
        load4<!B_NC>(b, ldb, n0, k0, N, K, t, b_vec, rb);     // B is contiguous along k exactly when it is not along n
        __syncthreads();
        if (A_KC) {
#pragma unroll
            for (int i = 0; i < 4; ++i) As[(t >> 6) * 4 + i][t & 63] = ra[i];
        } else {
            *reinterpret_cast<float4 *>(&As[t >> 4][(t & 15) * 4]) = make_float4(ra[0], ra[1], ra[2], ra[3]);
        }
        if (!B_NC) {
#pragma unroll
            for (int i = 0; i < 4; ++i) Bs[(t >> 6) * 4 + i][t & 63] = rb[i];
        } else {
            *reinterpret_cast<float4 *>(&Bs[t >> 4][(t & 15) * 4]) = make_float4(rb[0], rb[1], rb[2], rb[3]);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a4 = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = mac<EXACT>(acc[i][j], av[i], bv[j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = m0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = n0 + tx * 4 + j;
            if (c >= N) continue;
            float v = acc[i][j];
            if (ep.bias) v = __fadd_rn(v, ep.bias[c]);
            v = apply_act(ep.act, v);
            if (ep.mask) v = ep.mask[r * ep.ld_mask + c] > 0.f ? v : 0.f;
            float *dst = ep.out + r * ep.ld_out + c;
            if (ep.accumulate) v = __fadd_rn(*dst, v);
            *dst = v;
        }
    }
}

template <bool A_KC, bool B_NC>
void launch_small(zn_ctx *ctx, const float *a, int64_t lda, const float *b, int64_t ldb, int64_t m, int64_t n, int64_t k,
                  const Epi &ep, bool exact) {
    dim3 grid((unsigned)((n + SM_T - 1) / SM_T), (unsigned)((m + SM_T - 1) / SM_T));
    if (exact) gemm_simt_small_kernel<A_KC, B_NC, true><<<grid, THREADS, 0, ctx->stream>>>(a, lda, b, ldb, m, n, k, ep);
    else gemm_simt_small_kernel<A_KC, B_NC, false><<<grid, THREADS, 0, ctx->stream>>>(a, lda, b, ldb, m, n, k, ep);
}

}   // namespace

zn_status zn_gemm_simt(zn_ctx *ctx, const float *a, int64_t a_rs, int64_t a_cs, const float *b, int64_t b_rs,
                       int64_t b_cs, int64_t m, int64_t n, int64_t k, const zn_epilogue &e, bool exact) {
    if (!a || !b || !e.out_f32) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "gemm: null operand");
    if (m <= 0 || n <= 0 || k <= 0) return zn_fail(ctx, ZN_ERR_SHAPE, "gemm: non-positive dimension");
    if ((m + BM - 1) / BM > 65535) return zn_fail(ctx, ZN_ERR_SHAPE, "gemm: m too large for the fp32 path");
    const bool a_kc = (a_cs == 1), b_nc = (b_cs == 1);
    if (!a_kc && a_rs != 1) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "gemm: A must be contiguous along m or k");
    if (!b_nc && b_rs != 1) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "gemm: B must be contiguous along n or k");
    Epi ep{e.bias, static_cast<const float *>(e.mask), e.out_f32, e.ld_mask, e.ld_out_f32, e.act, e.accumulate, 0};
    if (e.accumulate && a_kc && b_nc && !e.bias && e.act == ZN_ACT_LINEAR && !e.mask) { ep.acc_init = 1; ep.accumulate = 0; }
    const int64_t lda = a_kc ? a_rs : a_cs, ldb = b_nc ? b_rs : b_cs;
    zn_launch_scope scope(ctx, ZN_PROF_GEMM_SIMT, 2.0 * m * n * k, 4.0 * (m * k + k * n + m * n));
    // few large tiles would leave most of the machine idle: use 64 x 64 tiles then
    const int64_t big_tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    if (big_tiles < 2 * (int64_t)ctx->sm_count && (m + SM_T - 1) / SM_T <= 65535) {
        if (a_kc && b_nc) launch_small<true, true>(ctx, a, lda, b, ldb, m, n, k, ep, exact);
        else if (a_kc && !b_nc) launch_small<true, false>(ctx, a, lda, b, ldb, m, n, k, ep, exact);
        else if (!a_kc && b_nc) launch_small<false, true>(ctx, a, lda, b, ldb, m, n, k, ep, exact);
        else launch_small<false, false>(ctx, a, lda, b, ldb, m, n, k, ep, exact);
        ZN_CUDA(ctx, cudaGetLastError());
        return ZN_OK;
    }
    if (a_kc && b_nc) launch<true, true>(ctx, a, lda, b, ldb, m, n, k, ep, exact);
    else if (a_kc && !b_nc) launch<true, false>(ctx, a, lda, b, ldb, m, n, k, ep, exact);
    else if (!a_kc && b_nc) launch<false, true>(ctx, a, lda, b, ldb, m, n, k, ep, exact);
    else launch<false, false>(ctx, a, lda, b, ldb, m, n, k, ep, exact);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}
