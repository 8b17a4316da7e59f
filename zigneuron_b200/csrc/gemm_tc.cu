// tcgen05 / TMEM GEMM for the three Dense products on sm_100a.
//
// One persistent CTA per SM walks 128 x 256 output tiles (128 x 128 where the wide tiles would leave
// most SMs idle).  Warp 0 feeds a 3-stage (narrow tiles: 4-stage) shared-memory ring with TMA
// (cp.async.bulk.tensor, 128-byte swizzle, every CTA loads its own tiles); one thread of warp 1 issues
// tcgen05.mma (cta_group::1, M=128, N=256 or 128) into one of two fp32 accumulators in tensor memory; warps
// 2..9 drain the other accumulator with tcgen05.ld (two warps per quarter of the rows, half the columns
// each) and apply the fused epilogue (bias, activation, activation-derivative mask, accumulate,
// down-convert), so the epilogue of tile i overlaps the main loop of tile i+1.  Results leave through
// shared memory and bulk tensor stores (whole 128-byte lines) or, where that is not possible, as
// per-thread stores.  A two-CTA variant of the same kernel (further down) takes every product with a
// long main loop.
//
// The three orientations of the reference (Backend.matMul, matMulTransposeB,
// matMulTransposeA; src/backend.zig:169-195, :298-325) differ only in which
// operand is K-major and which is MN-major; that is a bit in the instruction
// descriptor plus a different shared-memory tile shape, never a transpose pass:
//   NN  C = A[m][k] . B[k][n]      A K-major,  B N-major
//   NT  C = A[m][k] . B[n][k]^T    A K-major,  B K-major
//   TN  C = A[k][m]^T . B[k][n]    A M-major,  B N-major
//
// Every wait on an mbarrier is bounded: after about a second without progress
// the waiting thread raises a CTA-wide abort flag, records a code in the
// context's status word, and all roles fall through to the common exit, where
// tensor memory is released.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include <atomic>

#include "zn_internal.h"
#include "zn_act.cuh"

namespace {

constexpr int BM = 128, BN = 256;
// one-CTA kernel, beside 64 KiB of output staging: 3 x 48 KiB of operands for 256-column tiles, 4 x 32 KiB for
// 128-column ones; a launch that stores per thread has the room for a fourth stage of 48 KiB
__host__ __device__ constexpr int onecta_stages(int bn, bool staging) { return bn == 256 ? (staging ? 3 : 4) : 4; }
constexpr int TQ = 4;                               // depth of the tile-index ring inside a CTA
constexpr int ROW_BYTES = 128;                    // one swizzle row
constexpr int A_STAGE = BM * ROW_BYTES;           // 16 KiB
constexpr int THREADS = 192;                        // two-CTA kernel: producer warp, MMA warp, 4 epilogue warps
constexpr int EPI1 = 8;                             // one-CTA kernel: 8 epilogue warps, two per quarter of the accumulator's rows
constexpr int THREADS1 = 64 + 32 * EPI1;
constexpr int TMEM_COLS = 512;
constexpr int BIAS_SMEM = 4 * BN * 4;                 // one tile's bias values, a private copy per epilogue warp
constexpr int STG_BUF = 4096;                         // one staged 32 x 32 output block (fp32; 16-bit blocks use half)
constexpr int STAGING1_BYTES = EPI1 * 2 * STG_BUF;    // two blocks per epilogue warp of the one-CTA kernel
// after the operand ring: barriers (256 B), the bias strips, then (1024-aligned) the output staging buffers
constexpr int RING_TAIL = ((256 + BIAS_SMEM + 1023) / 1024) * 1024;
constexpr int onecta_smem(int bn, bool staging) {
    return 1024 /* alignment slack */ + onecta_stages(bn, staging) * (A_STAGE + bn * ROW_BYTES) + RING_TAIL +
           (staging ? STAGING1_BYTES : 0);
}
static_assert(onecta_smem(256, true) <= 232448 && onecta_smem(256, false) <= 232448 && onecta_smem(128, true) <= 232448,
              "the one-CTA kernel must fit the 227 KB of shared memory a CTA may have");
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;

struct TcParams {
    int M, N, K;
    int num_m_tiles, num_n_tiles, num_k_blocks;
    int a_mn, b_mn;           // operand majorness
    uint32_t idesc;
    uint32_t mn_lbo, mn_sbo;  // byte strides of an MN-major operand tile (see the MMA warp)
    // epilogue
    const float *bias;
    int act;
    const void *mask;
    long long ld_mask;
    float *out_f32;
    long long ld_out_f32;
    void *out_t;
    long long ld_out_t;
    int accumulate;
    int *status;
    // Dynamic tile scheduling: a CTA takes tile blockIdx.x first, then gridDim.x + atomicAdd(tile_counter).
    // Each launch also clears the counter the NEXT launch on the stream will use.
    unsigned int *tile_counter, *next_counter;
    int dynamic_tiles;       // 0: plain round-robin over the grid (diagnostic)
    // Output path of the two-CTA kernel: 0 = each thread stores its row straight to global memory; 1 / 2 = the
    // epilogue warps stage 32 x 32 blocks of fp32 (1) or 16-bit (2) results in shared memory and hand them to the
    // TMA unit (tensor map tmC), which writes whole 128-byte lines and clips at the edges of C.
    int out_mode;
    int band;                // m-tiles per band of the tile order (see tile_coords)
#ifdef ZN_DIAG
    unsigned long long *phase_ts;   // diagnostic builds: CTA 0 of the one-CTA kernel writes %globaltimer per phase here
#endif
};

// ---- PTX wrappers -----------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

#ifdef ZN_DIAG
// diagnostic builds: nanosecond time stamp of one phase of CTA 0 (first visit only)
#define ZN_PHASE(p, i)                                                                                 \
    do {                                                                                               \
        if ((p).phase_ts && blockIdx.x == 0 && (p).phase_ts[i] == 0ull) {                              \
            unsigned long long t__;                                                                    \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                                    \
            (p).phase_ts[i] = t__;                                                                     \
        }                                                                                              \
    } while (0)
// diagnostic builds: SM clock of one point of the epilogue of block `c` (warp 2, lane 0 of CTA 0), posted to device memory
__device__ long long zn_diag_clk[128];
#define ZN_CLK(c, point)                                                                               \
    do {                                                                                               \
        if (blockIdx.x == 0 && threadIdx.x == 64 && (c) < 8) zn_diag_clk[(c) * 8 + (point)] = clock64(); \
    } while (0)
// diagnostic builds: SM clock of one point of tile number `it` (as counted by the role) in the leader CTA of cluster 0
__device__ long long zn_diag_tile[8 * 16];
// diagnostic builds, one-CTA kernel, CTA 0: cycles its MMA thread spent waiting for a free accumulator [0] and for
// operands [1], its cycles from first to last tile [2], its tiles [3]; cycles epilogue warp 2 spent waiting for a
// full accumulator [4] and working on one [5]
__device__ long long zn_diag_wait[8];
#define ZN_WAIT_BEGIN() const long long w0__ = clock64()
#define ZN_WAIT_END(slot) do { if (blockIdx.x == 0) zn_diag_wait[slot] += clock64() - w0__; } while (0)
#define ZN_TILE_CLK(it, point)                                                                         \
    do {                                                                                               \
        if (blockIdx.x == 0 && (it) < 8) zn_diag_tile[(it) * 16 + (point)] = clock64();               \
    } while (0)
#else
#define ZN_PHASE(p, i) do { } while (0)
#define ZN_CLK(c, point) do { } while (0)
#define ZN_TILE_CLK(it, point) do { } while (0)
#define ZN_WAIT_BEGIN() do { } while (0)
#define ZN_WAIT_END(slot) do { } while (0)
#endif

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {   // acquire at cluster scope
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the CTA has been aborted or the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          int code, long long limit = WAIT_LIMIT_CYCLES) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                __threadfence_system();
                return false;
            }
        }
    }
}

// Same, for a barrier that a thread of the partner CTA arrives on after writing this CTA's shared memory.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                                  int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                __threadfence_system();
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// Bulk tensor store of one shared-memory box into C (this GPU's own memory, no multicast), as a bulk async-group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int c0, int c1, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(src)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most N of this thread's bulk groups may still be READING their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// orders this thread's ordinary shared-memory writes before later reads of them by the TMA unit
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <bool TF32>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    if (TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
    }
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Shared-memory matrix descriptor, descriptor version 1.  layout_type 2 = 128-byte swizzle on 16-byte
// units; 1 = 128-byte swizzle on 32-byte units, the only swizzled layout the tensor cores accept for an
// MN-major operand of a 32-bit type (tf32).  lbo / sbo in bytes.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout_type = 2) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout_type << 61;
    return d;
}

__device__ __forceinline__ float act_apply(int act, float v) {
    switch (act) {
    case ZN_ACT_RELU: return v > 0.f ? v : 0.f;
    case ZN_ACT_SIGMOID:
        if (v >= 0.f) return 1.f / (1.f + __expf(-v));
        else { const float e = __expf(v); return e / (1.f + e); }
    case ZN_ACT_TANH: return tanhf(v);
    default: return v;
    }
}

// Tile order: bands of G m-tiles, inside a band m fastest.  The CTAs of a wave then share G strips of A and about
// (CTAs / G) strips of B, which they read in step (one DRAM read per strip and wave, the rest L2 hits).
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int G, int &tm, int &tn) {
    const int per_band = G * num_n;
    const int band = t / per_band, first_m = band * G;
    const int rows = min(num_m - first_m, G);
    const int r = t - band * per_band;
    tm = first_m + r % rows;
    tn = r / rows;
}

// 256-bit global accesses (sm_100): one full 32-byte sector per thread and instruction.
__device__ __forceinline__ void st_global_v8(void *p, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}
__device__ __forceinline__ void ld_global_v8(const void *p, uint32_t (&w)[8]) {
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p));
}

// The arithmetic of the epilogue for 32 consecutive columns of one output row: bias, activation and the
// activation-derivative mask, from the raw accumulator words r into v.
template <bool TF32>
__device__ __forceinline__ void epilogue_values(const TcParams &p, long long row, int col0, const uint32_t (&r)[32],
                                                const float *bias_s, float (&v)[32]) {
    constexpr bool t_bf16 = !TF32;
    const int valid = min(32, p.N - col0);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (bias_s) {   // every lane reads the same shared-memory word: a broadcast, no bank conflict
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += bias_s[j];
    }
    // one branch on the (uniform) activation outside the element loop: a switch per element makes the
    // compiler issue every activation's code, predicated off, for each of the 32 values
    if (p.act == ZN_ACT_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
    } else if (p.act == ZN_ACT_SIGMOID) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = act_apply(ZN_ACT_SIGMOID, v[j]);
    } else if (p.act == ZN_ACT_TANH) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = act_apply(ZN_ACT_TANH, v[j]);
    } else if (p.act == ZN_ACT_GELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = zn_gelu_fwd(v[j]);
    } else if (p.act == ZN_ACT_LEAKY_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = zn_leaky_fwd(v[j]);
    } else if (p.act == ZN_ACT_ELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = zn_elu_fwd(v[j]);
    }
    if (p.mask) {
        if (t_bf16) {
            const __nv_bfloat16 *mrow = static_cast<const __nv_bfloat16 *>(p.mask) + row * p.ld_mask + col0;
            if (valid == 32 && ((reinterpret_cast<uintptr_t>(mrow) & 31) == 0)) {
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    uint32_t w[8];
                    ld_global_v8(mrow + g * 16, w);
#pragma unroll
                    for (int h = 0; h < 8; ++h) {
                        const uint32_t lo = w[h] & 0xFFFFu, hi = w[h] >> 16;
                        if (!(lo != 0u && lo < 0x8000u)) v[g * 16 + h * 2] = 0.f;
                        if (!(hi != 0u && hi < 0x8000u)) v[g * 16 + h * 2 + 1] = 0.f;
                    }
                }
            } else if (valid == 32 && ((reinterpret_cast<uintptr_t>(mrow) & 15) == 0)) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint4 u = *reinterpret_cast<const uint4 *>(mrow + g * 8);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        // bf16 > 0  <=>  sign bit clear and magnitude bits non-zero
                        const uint32_t lo = w[h] & 0xFFFFu, hi = w[h] >> 16;
                        if (!(lo != 0u && lo < 0x8000u)) v[g * 8 + h * 2] = 0.f;
                        if (!(hi != 0u && hi < 0x8000u)) v[g * 8 + h * 2 + 1] = 0.f;
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < valid && !(__bfloat162float(mrow[j]) > 0.f)) v[j] = 0.f;
            }
        } else {
            const float *mrow = static_cast<const float *>(p.mask) + row * p.ld_mask + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < valid && !(mrow[j] > 0.f)) v[j] = 0.f;
        }
    }
}

// Fused epilogue for 32 consecutive columns of one output row held by this thread:
// bias, activation, activation-derivative mask, accumulate, stores (fp32 and/or operand type).
template <bool TF32>
__device__ __forceinline__ void epilogue_chunk(const TcParams &p, long long row, int col0, const uint32_t (&r)[32],
                                               const float *bias_s /* 32 staged bias values of these columns, or null */) {
    constexpr bool t_bf16 = !TF32;
    const int valid = min(32, p.N - col0);
    float v[32];
    epilogue_values<TF32>(p, row, col0, r, bias_s, v);
    if (p.out_f32) {
        float *orow = p.out_f32 + row * p.ld_out_f32 + col0;
        const bool vec = valid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
        if (p.accumulate) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < valid) v[j] += orow[j];
        }
        if (vec && ((reinterpret_cast<uintptr_t>(orow) & 31) == 0)) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t w[8];
#pragma unroll
                for (int h = 0; h < 8; ++h) w[h] = __float_as_uint(v[g * 8 + h]);
                st_global_v8(orow + g * 8, w);
            }
        } else if (vec) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
                *reinterpret_cast<float4 *>(orow + g * 4) =
                    make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < valid) orow[j] = v[j];
        }
    }
    if (p.out_t) {
        if (t_bf16) {
            __nv_bfloat16 *orow = static_cast<__nv_bfloat16 *>(p.out_t) + row * p.ld_out_t + col0;
            if (valid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 31) == 0)) {
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    uint32_t w[8];
#pragma unroll
                    for (int h = 0; h < 8; ++h) {
                        const __nv_bfloat162 b2 =
                            __floats2bfloat162_rn(v[g * 16 + h * 2], v[g * 16 + h * 2 + 1]);
                        w[h] = *reinterpret_cast<const uint32_t *>(&b2);
                    }
                    st_global_v8(orow + g * 16, w);
                }
            } else if (valid == 32 && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0)) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint32_t w[4];
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        const __nv_bfloat162 b2 =
                            __floats2bfloat162_rn(v[g * 8 + h * 2], v[g * 8 + h * 2 + 1]);
                        w[h] = *reinterpret_cast<const uint32_t *>(&b2);
                    }
                    *reinterpret_cast<uint4 *>(orow + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < valid) orow[j] = __float2bfloat16_rn(v[j]);
            }
        } else {
            float *orow = static_cast<float *>(p.out_t) + row * p.ld_out_t + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < valid) orow[j] = v[j];
        }
    }
}

// Staged output.  One epilogue warp owns two 4 KiB shared-memory buffers; a buffer holds the warp's 32 rows of one
// 32-column block in the layout the tensor map's swizzle expects (fp32: 128-byte rows, 16-byte unit j of row r at
// position j ^ (r & 7); 16-bit: 64-byte rows, unit j at j ^ ((r >> 1) & 3)), which also spreads the 16-byte stores
// of a quarter warp over all 32 banks.  Lane 0 then issues one bulk tensor store per block and keeps at most one
// store reading shared memory behind it, so the warp returns to the next accumulator words at once.
__device__ __forceinline__ void stage_block_f32(uint32_t buf, int lane, const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
        st_shared_v4(buf + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) << 4), __float_as_uint(v[4 * j]),
                     __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
}
__device__ __forceinline__ void stage_block_bf16(uint32_t buf, int lane, const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[8 * j + 2 * h], v[8 * j + 2 * h + 1]);
            w[h] = *reinterpret_cast<const uint32_t *>(&b2);
        }
        st_shared_v4(buf + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) << 4), w[0], w[1], w[2], w[3]);
    }
}

// One 32 x 32 block of results of one epilogue warp through shared memory and the TMA unit.  `stores` counts the
// blocks this warp has handed over so far (it picks the buffer and tells when a buffer's previous store must have
// finished reading it).  Rows at or below M inside the block are written as zeros and dropped by the store.
template <bool TF32>
__device__ __forceinline__ void staged_block(const TcParams &p, const CUtensorMap *tmC, uint32_t warp_staging, int lane,
                                             int warp_row0, int col0, const uint32_t (&r)[32], const float *bias_s,
                                             uint32_t &stores, int c = 0 /* block number, diagnostic builds only */) {
    float v[32];
    const long long row = (long long)warp_row0 + lane;
    ZN_CLK(c, 1);
    if (row < p.M) epilogue_values<TF32>(p, row, col0, r, bias_s, v);
    else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
    }
    ZN_CLK(c, 2);
    const uint32_t sbuf = warp_staging + (stores & 1u) * STG_BUF;
    if (stores >= 2) {                       // the store that last used this buffer has read it
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
    }
    ZN_CLK(c, 3);
    if (p.out_mode == 1) stage_block_f32(sbuf, lane, v);
    else stage_block_bf16(sbuf, lane, v);
    ZN_CLK(c, 4);
    fence_proxy_async_smem();
    ZN_CLK(c, 5);
    __syncwarp();
    if (lane == 0) {
        tma_store_2d(tmC, col0, warp_row0, sbuf);
        bulk_commit();
    }
    ZN_CLK(c, 6);
    ++stores;
}

// ET: operand element type (__nv_bfloat16 or float-as-tf32).  BN_: columns of one output tile, 256 or 128; the
// narrow tile is for problems whose 128 x 256 tiles would leave most SMs idle (it doubles the tile count and
// halves the padding a narrow N pays for).  STAGED_: room for the output staging buffers; without them (launches
// that store per thread) the operand ring of the wide tile gets a fourth stage.
template <typename ET, int BN_, bool STAGED_>
__global__ void __launch_bounds__(THREADS1, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const TcParams p) {
    constexpr bool TF32 = sizeof(ET) == 4;
    constexpr int ES = sizeof(ET);
    constexpr int BK = ROW_BYTES / ES;            // k elements per stage: 64 bf16 / 32 tf32
    constexpr int CH = ROW_BYTES / ES;            // MN elements per 128-byte chunk of an MN-major tile
    constexpr int UMMA_K_BYTES = 32;              // 16 bf16 / 8 tf32 per instruction
    constexpr int KSTEPS = ROW_BYTES / UMMA_K_BYTES;   // 4 instructions per stage
    constexpr int STAGES = onecta_stages(BN_, STAGED_);
    constexpr int STAGE_BYTES = A_STAGE + BN_ * ROW_BYTES;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - raw);
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    // barrier slots (8 bytes each): full[S], empty[S], tmem_full[2], tmem_empty[2], sched_full[TQ],
    // sched_empty[TQ]; then tmem ptr, abort flag, and the ring of tile indices the producer publishes
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    auto sfull_bar = [&](int q) { return bars + 8u * (2 * STAGES + 4 + q); };
    auto sempty_bar = [&](int q) { return bars + 8u * (2 * STAGES + 4 + TQ + q); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4 + 2 * TQ));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile int *tile_ring = reinterpret_cast<volatile int *>(tmem_slot + 2);
    float *bias_smem = reinterpret_cast<float *>(gen + STAGES * STAGE_BYTES + 256);
    const uint32_t staging = base + STAGES * STAGE_BYTES + RING_TAIL;      // 1024-byte aligned

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Launched with programmatic stream serialization (see zn_gemm_tc), the kernel may start while the kernel before it
    // in the stream still runs: whatever touches global memory waits for that kernel below, after the set-up.  The
    // launch of the kernel AFTER this one is released at once, so that its set-up overlaps this kernel in turn.
    zn_pdl_release();
    if (threadIdx.x == 0) ZN_PHASE(p, 0);
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
        if (p.out_mode) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmC) : "memory");
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), EPI1); }
        for (int q = 0; q < TQ; ++q) { mbar_init(sfull_bar(q), 1); mbar_init(sempty_bar(q), 1 + EPI1); }   // MMA thread + the epilogue warps
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    zn_pdl_wait();      // the stream's previous kernel is complete and its writes are visible
    if (threadIdx.x == 0 && blockIdx.x == 0 && p.dynamic_tiles) *p.next_counter = 0u;
    if (threadIdx.x == 0) ZN_PHASE(p, 1);

    const int num_tiles = p.num_m_tiles * p.num_n_tiles;
    const int nkb = p.num_k_blocks;

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            int q = 0;
            uint32_t qphase = 0;
            // Tiles: the CTA's own first, then whatever the grid has not started yet.  The index of the tile AFTER the
            // one about to be loaded is drawn now, so that the atomic's round trip to L2 hides behind a tile of loads.
            int t_next = (int)blockIdx.x;
            while (ok) {
                int t = t_next;
                if (t >= num_tiles) t = -1;
                if (t >= 0) t_next = p.dynamic_tiles ? (int)(gridDim.x + atomicAdd(p.tile_counter, 1u)) : t + (int)gridDim.x;
                if (!mbar_wait(sempty_bar(q), qphase ^ 1u, abort_flag, p.status, 5)) { ok = false; break; }
                tile_ring[q] = t;
                mbar_arrive(sfull_bar(q));            // release: the MMA and epilogue warps read the slot after this
                if (++q == TQ) { q = 0; qphase ^= 1u; }
                if (t < 0) break;
                int tm, tn;
                tile_coords(t, p.num_m_tiles, p.num_n_tiles, p.band, tm, tn);
                const int m0 = tm * BM, n0 = tn * BN_;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_STAGE;
                    mbar_expect_tx(full_bar(s), STAGE_BYTES);
                    ZN_PHASE(p, 2);
                    const int k0 = kb * BK;
                    if (!p.a_mn) {
                        tma_load_2d(sa, &tmA, k0, m0, full_bar(s));                       // box {BK, 128}
                    } else {
#pragma unroll
                        for (int c = 0; c < BM / CH; ++c)                                   // box {CH, BK} each
                            tma_load_2d(sa + c * (BK * ROW_BYTES), &tmA, m0 + c * CH, k0, full_bar(s));
                    }
                    if (!p.b_mn) {
                        tma_load_2d(sb, &tmB, k0, n0, full_bar(s));                       // box {BK, BN_}
                    } else {
#pragma unroll
                        for (int c = 0; c < BN_ / CH; ++c)
                            tma_load_2d(sb + c * (BK * ROW_BYTES), &tmB, n0 + c * CH, k0, full_bar(s));
                    }
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            // Byte strides of the canonical 128B-swizzle layouts:
            //   K-major : 8-row groups 1024 B apart (SBO); LBO unused.  k advances 32 B inside the row.
            //   MN-major: 8-row (k) groups 1024 B apart (SBO) -- 4-row groups, 512 B, in the 32-byte-unit
            //             swizzle tf32 needs; 128-byte MN chunks BK*128 B apart (LBO).
            //             k advances by whole rows: UMMA_K rows * 128 B.
            const uint32_t a_lbo = p.a_mn ? p.mn_lbo : 16, b_lbo = p.b_mn ? p.mn_lbo : 16;
            const uint32_t a_sbo = p.a_mn ? p.mn_sbo : 1024, b_sbo = p.b_mn ? p.mn_sbo : 1024;
            const uint32_t a_lt = (TF32 && p.a_mn) ? 1u : 2u, b_lt = (TF32 && p.b_mn) ? 1u : 2u;
            const uint32_t a_kstep = p.a_mn ? (UMMA_K_BYTES / ES) * ROW_BYTES : UMMA_K_BYTES;
            const uint32_t b_kstep = p.b_mn ? (UMMA_K_BYTES / ES) * ROW_BYTES : UMMA_K_BYTES;
            int it = 0, q = 0;
            uint32_t qphase = 0;
            for (; ok; ++it) {
                if (!mbar_wait(sfull_bar(q), qphase, abort_flag, p.status, 6)) { ok = false; break; }
                const int t = tile_ring[q];
                mbar_arrive(sempty_bar(q));
                if (++q == TQ) { q = 0; qphase ^= 1u; }
                if (t < 0) break;
                const int buf = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                {
                    ZN_WAIT_BEGIN();
                    if (!mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
                    ZN_WAIT_END(0);
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN_);
                for (int kb = 0; kb < nkb; ++kb) {
                    {
                        ZN_WAIT_BEGIN();
                        if (!mbar_wait(full_bar(s), phase, abort_flag, p.status, 3)) { ok = false; break; }
                        ZN_WAIT_END(1);
                    }
                    ZN_PHASE(p, 3);
                    tc_fence_after();
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_STAGE;
#pragma unroll
                    for (int ks = 0; ks < KSTEPS; ++ks) {
                        const uint64_t ad = make_desc(sa + ks * a_kstep, a_lbo, a_sbo, a_lt);
                        const uint64_t bd = make_desc(sb + ks * b_kstep, b_lbo, b_sbo, b_lt);
                        tc_mma<TF32>(d_tmem, ad, bd, p.idesc, (kb | ks) != 0 ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));          // frees the stage when these MMAs have read it
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (ok) tc_commit(tfull_bar(buf));    // accumulator complete
                ZN_PHASE(p, 4);
#ifdef ZN_DIAG
                if (blockIdx.x == 0) {
                    if (it == 0) zn_diag_wait[6] = clock64();
                    zn_diag_wait[2] = clock64() - zn_diag_wait[6];
                    zn_diag_wait[3] = it + 1;
                }
#endif
            }
        }
    } else {
        // ================= epilogue: warps 2..9 =================
        // A warp reads the TMEM lanes 32 * (warp % 4) .., i.e. that quarter of the tile's rows; the two warps of a
        // quarter take one half of the tile's columns each.
        const int ew = warp - 2;                       // 0..7: staging buffers and bias strip of this warp
        const int q = warp & 3;
        const int h = ew >> 2;                         // which half of the columns
        constexpr int HALF_CHUNKS = BN_ / 64;          // 32-column blocks per half
        float *bias_strip = bias_smem + ew * (BN_ / 2);
        int it = 0, sq = 0;
        uint32_t sqphase = 0, stores = 0;
        bool ok = true;
        for (; ok; ++it) {
            if (!mbar_wait(sfull_bar(sq), sqphase, abort_flag, p.status, 7)) { ok = false; break; }
            const int t = tile_ring[sq];
            __syncwarp();
            if (lane == 0) mbar_arrive(sempty_bar(sq));
            if (++sq == TQ) { sq = 0; sqphase ^= 1u; }
            if (t < 0) break;
            int tm, tn;
            tile_coords(t, p.num_m_tiles, p.num_n_tiles, p.band, tm, tn);
            const int buf = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int warp_row0 = tm * BM + q * 32;
            const long long row = (long long)warp_row0 + lane;
            const int n0 = tn * BN_;
            const int nchunks = min(BN_ / 32, (p.N - n0 + 31) / 32);
            const int c_begin = h * HALF_CHUNKS, c_end = min(nchunks, c_begin + HALF_CHUNKS);
            if (p.bias) {
                // The warp copies its half of the tile's bias values into its own strip of shared memory once, instead
                // of every thread fetching all of them from global memory through an L1 that the shared-memory split
                // leaves tiny.  A private strip per warp needs no barrier between warps.
                __syncwarp();                          // the previous tile's reads of the strip are done
                for (int j = lane; j < BN_ / 2; j += 32) {
                    const int col = n0 + c_begin * 32 + j;
                    bias_strip[j] = col < p.N ? __ldg(p.bias + col) : 0.f;
                }
                __syncwarp();
            }
            {
                ZN_WAIT_BEGIN();
                if (!mbar_wait(tfull_bar(buf), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
                if (threadIdx.x == 64) ZN_WAIT_END(4);
            }
            if (warp == 2 && lane == 0) ZN_PHASE(p, 5);
#ifdef ZN_DIAG
            const long long e0__ = clock64();
#endif
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN_);
            if (c_begin >= c_end) {                    // a ragged last tile may leave this warp's half empty
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(buf));
            }
            for (int c = c_begin; c < c_end; ++c) {
                uint32_t r[32];
                ZN_CLK(c, 0);
                tc_ld32(taddr + (uint32_t)(c * 32), r);
                tc_wait_ld();
                if (c == c_end - 1) {
                    // all of this warp's reads of the accumulator are done: hand it back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(buf));
                }
                const float *bias_s = p.bias ? bias_strip + (c - c_begin) * 32 : nullptr;
                if (!STAGED_ || p.out_mode == 0) {
                    ZN_CLK(c, 1);
                    if (row < p.M) epilogue_chunk<TF32>(p, row, n0 + c * 32, r, bias_s);
                    ZN_CLK(c, 6);
                } else if (warp_row0 < p.M) {            // uniform over the warp
                    staged_block<TF32>(p, &tmC, staging + (uint32_t)(ew * 2) * STG_BUF, lane, warp_row0, n0 + c * 32, r, bias_s,
                                       stores, c);
                }
            }
            if (warp == 2 && lane == 0) ZN_PHASE(p, 6);
#ifdef ZN_DIAG
            if (blockIdx.x == 0 && threadIdx.x == 64) zn_diag_wait[5] += clock64() - e0__;
#endif
        }
        if (STAGED_ && lane == 0 && p.out_mode) bulk_wait_read<0>();   // the TMA unit has read every staged block; the writes complete with the kernel
    }
    if (threadIdx.x == 0) ZN_PHASE(p, 7);

    // ---- common exit
    if (*abort_flag) {
        // Something gave up: let copies and MMAs already in flight land before the CTA's memory goes away.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        if (lane == 0) ZN_PHASE(p, 8);
    }
}

// =====================================================================================================
// Two-CTA variant.  A cluster of two CTAs on a pair of SMs computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and its own half (128 of the 256
// columns) of B, the leader CTA's single thread issues the MMAs, and each CTA ends up with its 128 rows of
// the accumulator in its own tensor memory.  Per SM that is 32 KB of operands per k-block instead of the
// 48 KB of the one-CTA kernel, which is what the L2 -> shared-memory path can sustain at full tensor rate.
// Barriers: the leader's `full` barrier counts the bytes of BOTH CTAs' TMA loads (each CTA's loads name
// the leader's barrier); `empty` and `tmem_full` are signalled in both CTAs by one multicast
// tcgen05.commit; the epilogue warps of both CTAs arrive on the leader's `tmem_empty`.

constexpr int STAGES2 = 5;                        // default ring depth; 4 is built as well (see zn_gemm_tc)
constexpr int HALF = 128;                         // rows of A, and columns of B, staged per CTA
constexpr int A2_STAGE = HALF * ROW_BYTES;        // 16 KiB
constexpr int B2_STAGE = HALF * ROW_BYTES;        // 16 KiB
constexpr int STAGE2_BYTES = A2_STAGE + B2_STAGE;
constexpr int PAIR_TAIL = RING_TAIL;
constexpr int smem2_bytes(int stages, bool staging, int epi_warps = 4) {
    return 1024 /* alignment slack */ + stages * STAGE2_BYTES + PAIR_TAIL + (staging ? epi_warps * 2 * STG_BUF : 0);
}
static_assert(smem2_bytes(4, true, 8) <= 232448, "the two-CTA kernel with 8 epilogue warps keeps 4 stages");
static_assert(smem2_bytes(STAGES2, true) <= 232448 && smem2_bytes(6, false) <= smem2_bytes(STAGES2, true),
              "the two-CTA kernel must fit the 227 KB of shared memory a CTA may have");

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion bytes go to a barrier that may live in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar)
        : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both)
                 : "memory");
}
template <bool TF32>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    if (TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
    }
}

// EPI_: epilogue warps per CTA.  4 (one per quarter of the CTA's rows), the form every default route uses: a long
// main loop hides the epilogue.  8 (two per quarter, half the columns each, always with staged stores) is an
// option for short main loops (see zn_gemm_tc).
template <typename ET, int NST, int EPI_>
__global__ void __launch_bounds__(64 + 32 * EPI_, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const TcParams p) {
    constexpr bool TF32 = sizeof(ET) == 4;
    constexpr int ES = sizeof(ET);
    constexpr int BK = ROW_BYTES / ES;
    constexpr int CH = ROW_BYTES / ES;
    constexpr int UMMA_K_BYTES = 32;
    constexpr int KSTEPS = ROW_BYTES / UMMA_K_BYTES;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - raw);
    const uint32_t bars = base + NST * STAGE2_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (NST + s); };
    auto tfull_bar = [&](int b) { return bars + 8u * (2 * NST + b); };
    auto tempty_bar = [&](int b) { return bars + 8u * (2 * NST + 2 + b); };
    auto sfull_bar = [&](int q) { return bars + 8u * (2 * NST + 4 + q); };
    auto sempty_bar = [&](int q) { return bars + 8u * (2 * NST + 4 + TQ + q); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + NST * STAGE2_BYTES + 8 * (2 * NST + 4 + 2 * TQ));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile int *tile_ring = reinterpret_cast<volatile int *>(tmem_slot + 2);
    float *bias_smem = reinterpret_cast<float *>(gen + NST * STAGE2_BYTES + 256);
    const uint32_t staging = base + NST * STAGE2_BYTES + PAIR_TAIL;      // 1024-byte aligned

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0: leader (issues the MMAs), 1: peer

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
        if (p.out_mode) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmC) : "memory");
        for (int s = 0; s < NST; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 2 * EPI_); }   // the epilogue warps of both CTAs
        // tile-index ring: the leader's producer publishes into both CTAs; its `empty` side counts every reader
        // of the pair: leader MMA thread + leader epilogue warps + peer producer + peer epilogue warps
        for (int q = 0; q < TQ; ++q) { mbar_init(sfull_bar(q), 1); mbar_init(sempty_bar(q), 2 + 2 * EPI_); }
        if (blockIdx.x == 0 && p.dynamic_tiles) *p.next_counter = 0u;
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // both CTAs' barriers exist before anything remote touches them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_m_pairs = (p.M + 2 * HALF - 1) / (2 * HALF);
    const int num_tiles = num_m_pairs * p.num_n_tiles;
    const int nkb = p.num_k_blocks;
    const int cluster_id = (int)(blockIdx.x >> 1), num_clusters = (int)(gridDim.x >> 1);

    if (warp == 0) {
        // ================= TMA producer (both CTAs) =================
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            int q = 0;
            uint32_t qphase = 0;
            // The leader draws the index of the tile AFTER the one it is about to load while that one's loads are
            // still being issued: the atomic's round trip to L2 is then hidden behind a whole tile of loads.
            // Publishing an index (remote store + release at cluster scope) still costs this thread about 3,300
            // cycles between two tiles, which the clock stamps of diagnostic builds show as 3,660 cycles without
            // operands at the MMA thread per 8192-deep tile.  Handing the next index over in the MIDDLE of a tile
            // removes that gap (600 cycles) and was measured: the k-blocks then take 647 instead of 611 cycles
            // each and the training step 57.69 against 57.42 ms (three alternating runs on one box).  The main
            // loop runs at the rate L2 delivers operands to the SMs, not at the rate the producer asks for them.
            int t_next = cluster_id;
            int ptile = 0;                                    // tiles this producer has started (diagnostic builds)
            for (bool first = true; ok; first = false, ++ptile) {
                int t;
                if (rank == 0) {
                    // the leader picks the pair's next tile and publishes it into both CTAs' rings
                    t = t_next;
                    if (t >= num_tiles) t = -1;
                    if (t >= 0)
                        t_next = p.dynamic_tiles ? (int)(num_clusters + atomicAdd(p.tile_counter, 1u)) : t + num_clusters;
                    if (!mbar_wait_cluster(sempty_bar(q), qphase ^ 1u, abort_flag, p.status, 15)) { ok = false; break; }
                    ZN_TILE_CLK(ptile, 7);
                    tile_ring[q] = t;
                    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(smem_u32((const void *)&tile_ring[q]), 1)), "r"(t)
                                 : "memory");
                    mbar_arrive(sfull_bar(q));
                    mbar_arrive_cluster(map_to_cta(sfull_bar(q), 1));
                } else {
                    if (!mbar_wait_cluster(sfull_bar(q), qphase, abort_flag, p.status, 16)) { ok = false; break; }
                    t = tile_ring[q];
                    mbar_arrive_cluster(map_to_cta(sempty_bar(q), 0));
                }
                if (++q == TQ) { q = 0; qphase ^= 1u; }
                if (t < 0) break;
                int tm, tn;
                tile_coords(t, num_m_pairs, p.num_n_tiles, p.band, tm, tn);
                const int m0 = tm * 2 * HALF + (int)rank * HALF;       // this CTA's rows of A
                const int n0 = tn * BN + (int)rank * HALF;             // this CTA's columns of B
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
                    if (rank == 0) { if (kb == 0) ZN_TILE_CLK(ptile, 8); if (kb == nkb - 1) ZN_TILE_CLK(ptile, 9); }
                    const uint32_t sa = base + s * STAGE2_BYTES, sb = sa + A2_STAGE;
                    const uint32_t lead_full = map_to_cta(full_bar(s), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE2_BYTES);
                    const int k0 = kb * BK;
                    if (!p.a_mn) {
                        tma_load_2d_pair(sa, &tmA, k0, m0, lead_full);                       // box {BK, 128}
                    } else {
#pragma unroll
                        for (int c = 0; c < HALF / CH; ++c)
                            tma_load_2d_pair(sa + c * (BK * ROW_BYTES), &tmA, m0 + c * CH, k0, lead_full);
                    }
                    if (!p.b_mn) {
                        tma_load_2d_pair(sb, &tmB, k0, n0, lead_full);                       // box {BK, 128}
                    } else {
#pragma unroll
                        for (int c = 0; c < HALF / CH; ++c)
                            tma_load_2d_pair(sb + c * (BK * ROW_BYTES), &tmB, n0 + c * CH, k0, lead_full);
                    }
                    if (++s == NST) { s = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer (leader CTA only) =================
        if (lane == 0 && rank == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint32_t a_lbo = p.a_mn ? p.mn_lbo : 16, b_lbo = p.b_mn ? p.mn_lbo : 16;
            const uint32_t a_sbo = p.a_mn ? p.mn_sbo : 1024, b_sbo = p.b_mn ? p.mn_sbo : 1024;
            const uint32_t a_lt = (TF32 && p.a_mn) ? 1u : 2u, b_lt = (TF32 && p.b_mn) ? 1u : 2u;
            const uint32_t a_kstep = p.a_mn ? (UMMA_K_BYTES / ES) * ROW_BYTES : UMMA_K_BYTES;
            const uint32_t b_kstep = p.b_mn ? (UMMA_K_BYTES / ES) * ROW_BYTES : UMMA_K_BYTES;
            int it = 0, q = 0;
            uint32_t qphase = 0;
            for (; ok; ++it) {
                if (!mbar_wait(sfull_bar(q), qphase, abort_flag, p.status, 17)) { ok = false; break; }
                const int t = tile_ring[q];
                mbar_arrive(sempty_bar(q));
                if (++q == TQ) { q = 0; qphase ^= 1u; }
                if (t < 0) break;
                ZN_TILE_CLK(it, 0);
                const int buf = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, p.status, 12)) { ok = false; break; }
                ZN_TILE_CLK(it, 1);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(full_bar(s), phase, abort_flag, p.status, 13)) { ok = false; break; }
                    if (kb == 0) ZN_TILE_CLK(it, 2);
                    tc_fence_after();
                    const uint32_t sa = base + s * STAGE2_BYTES, sb = sa + A2_STAGE;
#pragma unroll
                    for (int ks = 0; ks < KSTEPS; ++ks) {
                        const uint64_t ad = make_desc(sa + ks * a_kstep, a_lbo, a_sbo, a_lt);
                        const uint64_t bd = make_desc(sb + ks * b_kstep, b_lbo, b_sbo, b_lt);
                        tc_mma_pair<TF32>(d_tmem, ad, bd, p.idesc, (kb | ks) != 0 ? 1u : 0u);
                    }
                    tc_commit_pair(empty_bar(s));         // frees the stage in both CTAs
                    if (++s == NST) { s = 0; phase ^= 1u; }
                }
                if (ok) tc_commit_pair(tfull_bar(buf));   // accumulator complete, in both CTAs
                ZN_TILE_CLK(it, 3);
            }
        }
    } else {
        // ================= epilogue (both CTAs): warps 2.., this CTA's 128 rows =================
        // A warp reads the TMEM lanes 32 * (warp % 4) ..; with 8 warps the two warps of a quarter take half the
        // columns each.
        const int ew = warp - 2;
        const int q = warp & 3;
        constexpr int PARTS = EPI_ / 4;                    // column parts of a tile: 1 or 2
        constexpr int PART_CHUNKS = (BN / 32) / PARTS;     // 32-column blocks per part
        const int c_first = (ew >> 2) * PART_CHUNKS;
        float *bias_strip = bias_smem + ew * (BN / PARTS);
        int it = 0, sq = 0;
        uint32_t stores = 0;                              // staged blocks this warp has handed to the TMA unit
        uint32_t sqphase = 0;
        bool ok = true;
        for (; ok; ++it) {
            if (!mbar_wait_cluster(sfull_bar(sq), sqphase, abort_flag, p.status, 18)) { ok = false; break; }
            const int t = tile_ring[sq];
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(sempty_bar(sq), 0));
            if (++sq == TQ) { sq = 0; sqphase ^= 1u; }
            if (t < 0) break;
            if (threadIdx.x == 64) ZN_TILE_CLK(it, 4);
            int tm, tn;
            tile_coords(t, num_m_pairs, p.num_n_tiles, p.band, tm, tn);
            const int buf = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int warp_row0 = tm * 2 * HALF + (int)rank * HALF + q * 32;
            const long long row = (long long)warp_row0 + lane;
            const int n0 = tn * BN;
            const int nchunks = min(BN / 32, (p.N - n0 + 31) / 32);
            const int c_end = min(nchunks, c_first + PART_CHUNKS);
            if (p.bias) {
                // the warp's own copy of its part of the tile's bias values (no barrier between warps needed)
                __syncwarp();                              // the previous tile's reads of the strip are done
                for (int j = lane; j < BN / PARTS; j += 32) {
                    const int col = n0 + c_first * 32 + j;
                    bias_strip[j] = col < p.N ? __ldg(p.bias + col) : 0.f;
                }
                __syncwarp();
            }
            if (!mbar_wait(tfull_bar(buf), acc_phase, abort_flag, p.status, 14)) { ok = false; break; }
            if (threadIdx.x == 64) ZN_TILE_CLK(it, 5);
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
            if (c_first >= c_end) {                        // a ragged last tile may leave this warp's part empty
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0));
            }
            for (int c = c_first; c < c_end; ++c) {
                uint32_t r[32];
                tc_ld32(taddr + (uint32_t)(c * 32), r);
                tc_wait_ld();
                if (c == c_end - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0));   // to the leader's MMA thread
                }
                const float *bias_s = p.bias ? bias_strip + (c - c_first) * 32 : nullptr;
                if (p.out_mode == 0) {
                    if (row >= p.M) continue;
                    epilogue_chunk<TF32>(p, row, n0 + c * 32, r, bias_s);
                    continue;
                }
                if (warp_row0 >= p.M) continue;          // the warp's 32 rows all lie below C (uniform over the warp)
                staged_block<TF32>(p, &tmC, staging + (uint32_t)(ew * 2) * STG_BUF, lane, warp_row0, n0 + c * 32, r, bias_s, stores);
            }
            if (threadIdx.x == 64) ZN_TILE_CLK(it, 6);
        }
        if (lane == 0 && p.out_mode) bulk_wait_read<0>();   // the TMA unit has read every staged block; the writes complete with the kernel
    }

    // ---- common exit: neither CTA may leave while its partner can still reach its shared or tensor memory
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// One CTA, one barrier that nothing arrives at: the wait runs out after `limit` cycles, the waiting thread raises
// the abort flag and records code 99, and every thread leaves through the ordinary end of the kernel.
__global__ void bounded_wait_probe_kernel(int *status, long long limit) {
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ int abort_flag_s;
    const uint32_t bar = smem_u32(&bar_storage);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        abort_flag_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile int *abort_flag = &abort_flag_s;
    if (threadIdx.x == 0) mbar_wait(bar, 0u, abort_flag, status, 99, limit);
    __syncthreads();
}

// ---- host side ----------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// 2-D row-major tensor [outer][inner], row pitch ld elements; box {box_inner, box_outer}.  Swizzle kinds:
// 0 = 128 B on 16-byte units, 1 = 128 B on 32-byte units (to match descriptor layout type 1), 2 = 64 B (the
// staged output blocks of 16-bit results); out-of-bounds reads give zero, out-of-bounds parts of a store are dropped.
// Encoded maps are cached per context under the bytes of this key.
struct TmapKey {
    const void *ptr;
    long long inner, outer, ld;
    int es, box_inner, box_outer, swizzle;
};

zn_status make_tmap(zn_ctx *ctx, CUtensorMap *out, int es, const void *ptr, int64_t inner, int64_t outer, int64_t ld,
                    int box_inner, int box_outer, int swizzle_kind) {
    TmapKey k;
    memset(&k, 0, sizeof k);                      // padding bytes are part of the key
    k.ptr = ptr; k.inner = inner; k.outer = outer; k.ld = ld;
    k.es = es; k.box_inner = box_inner; k.box_outer = box_outer; k.swizzle = swizzle_kind;
    const std::string key(reinterpret_cast<const char *>(&k), sizeof k);
    auto it = ctx->tmap_cache.find(key);
    if (it != ctx->tmap_cache.end()) {
        memcpy(out, it->second.data(), sizeof(CUtensorMap));
        return ZN_OK;
    }
    EncodeTiledFn enc = get_encode();
    if (!enc) return zn_fail(ctx, ZN_ERR_NOT_INITIALIZED, "cuTensorMapEncodeTiled is not available from the driver");
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld * es) % 16 != 0)
        return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "tensor-core GEMM operand needs a 16-byte aligned base and row pitch");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)(ld * es)};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = es == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const CUtensorMapSwizzle sw = swizzle_kind == 1 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                  : swizzle_kind == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
    CUresult r = enc(out, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return zn_fail(ctx, ZN_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    if (ctx->tmap_cache.size() > 4096) ctx->tmap_cache.clear();
    std::vector<uint8_t> bytes(sizeof(CUtensorMap));
    memcpy(bytes.data(), out, sizeof(CUtensorMap));
    ctx->tmap_cache.emplace(key, std::move(bytes));
    return ZN_OK;
}

// Which kernel, tile width, output path and band height a product gets.  Pure host arithmetic on the shape, the SM
// count and the environment's diagnostic switches, so that it can be checked without a device (zn_debug_tc_route).
struct TcRoute {
    bool use_pair, pair8, narrow, want_staged;
    int bn, num_k_blocks, band;
};
TcRoute tc_route(int elem_type, int64_t m, int64_t n, int64_t k, int sm_count, int reserve_sms, bool stageable) {
    const int es = elem_type == 0 ? 2 : 4;
    const int bk = ROW_BYTES / es;
    // Which kernel.  The two-CTA kernel halves the operand traffic per SM and wins wherever the main loop is long.
    // With a short main loop (K of at most 16 k-blocks: 1024 bf16 / 512 tf32 values) a tile is over before the
    // pair's cluster-wide hand-shakes pay off and the one-CTA kernel is faster: measured in bf16, 65536 x 512 x 512
    // 665 against 510-530 TFLOP/s, 1024^3 114-128 against 103, 256^3 12.8 against 16.8 us per launch.
    // ZN_TC_PAIR=0 / 2: one-CTA kernel only / two-CTA kernel wherever it can run (diagnostic).
    static const int pair_mode = getenv("ZN_TC_PAIR") ? atoi(getenv("ZN_TC_PAIR")) : 1;
    const int num_k_blocks = (int)((k + bk - 1) / bk);
    // A product whose 256 x 256 tiles do not fill the SM pairs more than once also goes to the one-CTA kernel: in a
    // single wave nothing hides the epilogue of the large tile, and the smaller tiles reach more SMs.  Measured,
    // one-CTA against two-CTA kernel: 2048^3 bf16 692-741 against 635-639 TFLOP/s, 1024^3 tf32 88-103 against 73-86,
    // the 784-512-256-10 training step at batch 1024 in tf32 0.205 against 0.238 ms.
    const long long pair_tiles_all = (long long)((m + 2 * BM - 1) / (2 * BM)) * ((n + BN - 1) / BN);
    const int pair_clusters = sm_count / 2 - (reserve_sms + 1) / 2;
    const bool long_pair = m > BM && (pair_mode == 2 || (pair_mode == 1 && num_k_blocks > 16 && pair_tiles_all > pair_clusters));
    // Option: a form of the two-CTA kernel with 8 epilogue warps and staged stores for short main loops with more
    // than one wave of 256 x 256 tiles (per 128 x 256 of output and k-block it takes in 32 KB where the one-CTA
    // kernel takes in 48 KB).  Measured against the one-CTA kernel in bf16: 65536 x 512 x 512 578-594 against
    // 633-683 TFLOP/s, 4096 x 4096 x 512 488-493 against 552-573, 8192 x 2048 x 256 273-275 against 342-371 (tf32
    // within 5 % either way): the pair's hand-over of tile indices across the cluster costs more per tile than
    // the operand bytes saved, so it is off unless asked for.  It needs C to be stageable (see below).
    // ZN_TC_PAIR8=1 / 2: for those short main loops / for every product the two-CTA kernel takes.
    static const int pair8_mode = getenv("ZN_TC_PAIR8") ? atoi(getenv("ZN_TC_PAIR8")) : 0;
    static const int staged_mode = getenv("ZN_TC_STAGED_STORE") ? atoi(getenv("ZN_TC_STAGED_STORE")) : -1;
    const bool short_pair = pair_mode == 1 && pair8_mode == 1 && m > BM && num_k_blocks <= 16 && pair_tiles_all > pair_clusters;
    const bool pair8 = stageable && staged_mode != 0 && (short_pair || (long_pair && pair8_mode == 2));
    const bool use_pair = long_pair || (short_pair && pair8);
    // Tile width of the one-CTA kernel: 128 columns instead of 256 where N fits one narrow tile, or where the wide
    // tiles would occupy at most half the SMs (twice the tiles, each half the work).
    // ZN_TC_NARROW=0 / 2: never / always in the one-CTA kernel (diagnostic).
    static const int narrow_mode = getenv("ZN_TC_NARROW") ? atoi(getenv("ZN_TC_NARROW")) : 1;
    const long long wide_tiles = (long long)((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const bool narrow = !use_pair && (narrow_mode == 2 || (narrow_mode == 1 && (n <= 128 || 2 * wide_tiles <= sm_count - reserve_sms)));
    const int bn = narrow ? 128 : BN;

    // Output path.  Either every thread stores its own row of the tile straight from the registers the accumulator
    // was read into (32-byte pieces, one row per lane: an instruction touches 32 different lines, and the L1 store
    // path takes about two cycles per line, 5 us for a 128 x 256 fp32 tile), or the epilogue warps stage 32 x 32
    // blocks in shared memory and the TMA unit writes them as whole 128-byte lines.  The one-CTA kernel, whose tiles
    // have a short main loop and so wait for their epilogue, stages; the two-CTA kernel, whose epilogue hides under
    // the next tile's long main loop and whose TMA unit is busy with operand loads, stores per thread (measured
    // there, staged against per-thread: 16384^3 TN 1188 against 1245 TFLOP/s, the 8192-wide training step 58.1
    // against 57.5 ms); its variant for short main loops stages.  ZN_TC_STAGED_STORE=0 / 1 forces one path in both
    // kernels (diagnostic).  Staging needs C to be ONE block the unit can address (16-byte aligned base and row
    // pitch) that is only written; C += ..., two outputs at once and odd pitches always take the per-thread stores.
    const bool want_staged = stageable && (pair8 || (staged_mode < 0 ? !use_pair : staged_mode != 0));
    // Rows of tiles per band.  A wave of 74 tile pairs shares `band` strips of A and about 74 / band strips of B;
    // 8 gives the fewest distinct strips (8 + 9.25), i.e. the fewest DRAM reads per wave, and 16 keeps a band's A
    // strips (band x 256 rows x K) in L2 across the waves of the band as long as they are small enough.  So: 16
    // while the A strips of such a band stay within 34 MB (K up to 4096 bf16), else 8.  Measured on the 8192-wide
    // training step (ncu, 8192 rows): an 8192 x 8192 x 8192 product reads 0.99 GB from DRAM with bands of 8 and
    // 1.25 GB with 16, an 8192 x 8192 x 4096 product 0.34 GB against 0.22 GB; under the 1 kW cap the DRAM power
    // saved raises the SM clock (median 1567 -> 1634 MHz) and the step went from 57.2 to 56.5 ms.
    // ZN_TC_BAND overrides (diagnostic).
    static const int band_env = [] { const char *e = getenv("ZN_TC_BAND"); const int v = e ? atoi(e) : 0; return v >= 1 && v <= 64 ? v : 0; }();
    const int band = band_env ? band_env : ((long long)16 * 256 * k * es <= (34ll << 20) ? 16 : 8);
    return TcRoute{use_pair, pair8, narrow, want_staged, bn, num_k_blocks, band};
}

}   // namespace

extern "C" zn_status zn_debug_bounded_wait_probe(zn_ctx *ctx, int64_t limit_cycles) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (limit_cycles < 0 || limit_cycles > 2000000000LL)
        return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "bounded_wait_probe: limit of %lld cycles outside 0..2e9", (long long)limit_cycles);
    ZN_CUDA(ctx, cudaSetDevice(ctx->device));
    ctx->launches += 1;
    bounded_wait_probe_kernel<<<1, 64, 0, ctx->stream>>>(ctx->status_dev, (long long)limit_cycles);
    ZN_CUDA(ctx, cudaGetLastError());
    return ZN_OK;
}

extern "C" zn_status zn_debug_tc_route(int32_t elem_type, int64_t m, int64_t n, int64_t k, int32_t sm_count, int32_t reserve_sms,
                                        int32_t stageable, int32_t out[6]) {
    if (!out || m <= 0 || n <= 0 || k <= 0 || sm_count <= 0 || (elem_type != 0 && elem_type != 1)) return ZN_ERR_INVALID_VALUE;
    const TcRoute r = tc_route(elem_type, m, n, k, sm_count, reserve_sms, stageable != 0);
    out[0] = r.use_pair ? 1 : 0;
    out[1] = r.use_pair ? 256 : r.bn;
    out[2] = r.want_staged ? 1 : 0;
    out[3] = r.use_pair ? (r.pair8 ? 8 : 4) : EPI1;
    out[4] = r.band;
    out[5] = r.num_k_blocks;
    return ZN_OK;
}

zn_status zn_gemm_tc(zn_ctx *ctx, int elem_type, const void *a, int64_t lda, bool a_mn, const void *b, int64_t ldb,
                     bool b_mn, int64_t m, int64_t n, int64_t k, const zn_epilogue &e) {
    if (!a || !b || (!e.out_f32 && !e.out_t)) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "gemm: null operand");
    if (m <= 0 || n <= 0 || k <= 0) return zn_fail(ctx, ZN_ERR_SHAPE, "gemm: non-positive dimension");
    if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return zn_fail(ctx, ZN_ERR_SHAPE, "gemm: dimension too large");
    const int es = elem_type == 0 ? 2 : 4;
    const int bk = ROW_BYTES / es, ch = ROW_BYTES / es;

    using OneFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const TcParams);
    static std::atomic<uint64_t> attr_set_mask{0};   // cudaFuncSetAttribute is per device
    const uint64_t dev_bit = 1ull << (ctx->device & 63);
    if (!(attr_set_mask.load() & dev_bit)) {
        // Ask for the full 228 KB shared-memory split rather than the smallest one that fits this kernel:
        // the ~30 KB left over let the small reduction and update kernels of the other lanes share the SM.
        const struct { OneFn f; int smem; } fns[] = {
            {(OneFn)gemm_tc_kernel<__nv_bfloat16, 256, true>, onecta_smem(256, true)}, {(OneFn)gemm_tc_kernel<float, 256, true>, onecta_smem(256, true)},
            {(OneFn)gemm_tc_kernel<__nv_bfloat16, 256, false>, onecta_smem(256, false)}, {(OneFn)gemm_tc_kernel<float, 256, false>, onecta_smem(256, false)},
            {(OneFn)gemm_tc_kernel<__nv_bfloat16, 128, true>, onecta_smem(128, true)}, {(OneFn)gemm_tc_kernel<float, 128, true>, onecta_smem(128, true)}};
        for (const auto &k : fns) {
            ZN_CUDA(ctx, cudaFuncSetAttribute(k.f, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem));
            cudaFuncSetAttribute(k.f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        }
        cudaGetLastError();
        attr_set_mask.fetch_or(dev_bit);
    }

    const bool tf32 = elem_type != 0;
    bool stageable = false;        // C is one block the TMA unit can address and is only written
    if (!e.accumulate && (e.out_f32 != nullptr) != (e.out_t != nullptr)) {
        const void *cptr = e.out_f32 ? (const void *)e.out_f32 : (const void *)e.out_t;
        const int64_t ldc = e.out_f32 ? e.ld_out_f32 : e.ld_out_t;
        const int ces = (e.out_f32 != nullptr || tf32) ? 4 : 2;
        stageable = (reinterpret_cast<uintptr_t>(cptr) & 15) == 0 && (ldc * ces) % 16 == 0 && ldc >= n;
    }
    const TcRoute route = tc_route(elem_type, m, n, k, ctx->sm_count, e.reserve_sms, stageable);
    const bool use_pair = route.use_pair, pair8 = route.pair8, narrow = route.narrow;
    const int bn = route.bn, num_k_blocks = route.num_k_blocks;

    CUtensorMap tmA, tmB;
    if (!a_mn) ZN_TRY(make_tmap(ctx, &tmA, es, a, k, m, lda, bk, BM, 0));         // [m][k]: inner k
    else ZN_TRY(make_tmap(ctx, &tmA, es, a, m, k, lda, ch, bk, tf32 ? 1 : 0));    // [k][m]: inner m
    if (!b_mn) ZN_TRY(make_tmap(ctx, &tmB, es, b, k, n, ldb, bk, use_pair ? HALF : bn, 0));   // [n][k]: inner k; the pair stages B in halves of 128 columns per CTA
    else ZN_TRY(make_tmap(ctx, &tmB, es, b, n, k, ldb, ch, bk, tf32 ? 1 : 0));    // [k][n]: inner n

    TcParams p;
    p.M = (int)m; p.N = (int)n; p.K = (int)k;
    p.num_m_tiles = (int)((m + BM - 1) / BM);
    p.num_n_tiles = (int)((n + bn - 1) / bn);
    p.num_k_blocks = num_k_blocks;
    p.a_mn = a_mn ? 1 : 0;
    p.b_mn = b_mn ? 1 : 0;
    const uint32_t fmt = elem_type == 0 ? 1u /* bf16 */ : 2u /* tf32 */;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) |
              ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    p.mn_lbo = (uint32_t)(bk * ROW_BYTES);
    p.mn_sbo = tf32 ? 512 : 1024;
#ifdef ZN_DIAG
    if (const char *dbg = getenv("ZN_TC_MN_STRIDES")) {   // diagnostic builds only (-DZN_DIAG): override "lbo,sbo" in bytes
        unsigned l = 0, sb = 0;
        if (sscanf(dbg, "%u,%u", &l, &sb) == 2) { p.mn_lbo = l; p.mn_sbo = sb; }
    }
#endif
    p.bias = e.bias; p.act = e.act; p.mask = e.mask; p.ld_mask = e.ld_mask;
    p.out_f32 = e.out_f32; p.ld_out_f32 = e.ld_out_f32; p.out_t = e.out_t; p.ld_out_t = e.ld_out_t;
    p.accumulate = e.accumulate;
    p.out_mode = 0;
    p.band = route.band;
#ifdef ZN_DIAG
    // ZN_TC_PHASES=1 (diagnostic builds): CTA 0 of every one-CTA launch stamps its phases; the host waits for the launch
    // and prints them relative to the kernel's first stamp
    static unsigned long long *phase_host = nullptr, *phase_dev = nullptr;
    static const bool phases = getenv("ZN_TC_PHASES") != nullptr;
    p.phase_ts = nullptr;
    if (phases) {
        if (!phase_host) {
            cudaHostAlloc((void **)&phase_host, 16 * sizeof(unsigned long long), cudaHostAllocMapped);
            cudaHostGetDevicePointer((void **)&phase_dev, phase_host, 0);
        }
        cudaStreamSynchronize(ctx->stream);
        for (int i = 0; i < 16; ++i) phase_host[i] = 0ull;
        p.phase_ts = phase_dev;
    }
#endif
    p.status = ctx->status_dev;
    if (!ctx->tile_counters) {
        ZN_CUDA(ctx, cudaMalloc((void **)&ctx->tile_counters, 2 * sizeof(unsigned int)));
        ZN_CUDA(ctx, cudaMemsetAsync(ctx->tile_counters, 0, 2 * sizeof(unsigned int), ctx->stream));
    }
    // The two work counters are used in turn by successive launches ON THE MAIN LANE (each clears the one its
    // successor will use).  A GEMM issued on any other lane would race with them, so it walks its tiles in the
    // fixed round-robin order and touches neither counter.
    static const int dyn = getenv("ZN_TC_STATIC_TILES") ? 0 : 1;
    p.dynamic_tiles = (dyn && ctx->lane == ZN_LANE_MAIN) ? 1 : 0;
    {
        // a launch in which every CTA (or CTA pair) has at most one tile has nothing to hand out
        const bool would_pair = use_pair;
        const long long units = would_pair ? (long long)((m + 2 * BM - 1) / (2 * BM)) * p.num_n_tiles : (long long)p.num_m_tiles * p.num_n_tiles;
        const long long workers = would_pair ? ctx->sm_count / 2 - (e.reserve_sms + 1) / 2 : ctx->sm_count - e.reserve_sms;
        if (units <= workers) p.dynamic_tiles = 0;
    }
    p.tile_counter = ctx->tile_counters + (ctx->tile_counter_turn & 1);
    p.next_counter = ctx->tile_counters + ((ctx->tile_counter_turn + 1) & 1);
    if (p.dynamic_tiles) ctx->tile_counter_turn += 1;
    // a launch that fails never cleared its successor's counter: start both from zero again
    auto launch_failed = [&](cudaError_t e, const char *what) {
        cudaMemsetAsync(ctx->tile_counters, 0, 2 * sizeof(unsigned int), ctx->stream);
        ctx->tile_counter_turn = 0;
        return zn_cuda_status(ctx, e, what);
    };

    zn_launch_scope scope(ctx, ZN_PROF_GEMM_TC, 2.0 * m * n * k,
                          (double)es * (m * k + k * n) + (e.out_f32 ? 4.0 : (double)es) * m * n);
    CUtensorMap tmC;
    memset(&tmC, 0, sizeof tmC);
    if (route.want_staged) {
        const bool wide = e.out_f32 != nullptr || tf32;                  // 4-byte results
        const void *cptr = e.out_f32 ? (const void *)e.out_f32 : (const void *)e.out_t;
        const int64_t ldc = e.out_f32 ? e.ld_out_f32 : e.ld_out_t;
        ZN_TRY(make_tmap(ctx, &tmC, wide ? 4 : 2, cptr, n, m, ldc, 32, 32, wide ? 0 : 2));
        p.out_mode = wide ? 1 : 2;
    }
    if (use_pair) {
        // two-CTA kernel: 256 x 256 tiles
        p.idesc = (p.idesc & ~(0x1Fu << 24)) | ((uint32_t)((2 * HALF) >> 4) << 24);   // M = 256 across the pair
        const long long pair_tiles = (long long)((m + 2 * HALF - 1) / (2 * HALF)) * p.num_n_tiles;
        int max_clusters = ctx->sm_count / 2 - (e.reserve_sms + 1) / 2;
        if (max_clusters < 1) max_clusters = 1;
        const int clusters = (int)(pair_tiles < max_clusters ? pair_tiles : max_clusters);
        // Ring depth: 5 stages beside the 32 KB of output staging; a launch that stores per thread has that room
        // for a sixth stage.  ZN_TC_PAIR_STAGES = 4 / 5 / 6 overrides (diagnostic; 6 only without staging).
        static const int nst_env = [] { const char *e = getenv("ZN_TC_PAIR_STAGES"); return e ? atoi(e) : 0; }();
        int nst = STAGES2;
        if (nst_env == 4 || nst_env == 5) nst = nst_env;
        if (nst_env == 6 && p.out_mode == 0) nst = 6;
        using PairFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const TcParams);
        PairFn fn;
        if (pair8) fn = elem_type == 0 ? (PairFn)gemm_tc_pair_kernel<__nv_bfloat16, 4, 8> : (PairFn)gemm_tc_pair_kernel<float, 4, 8>;
        else if (elem_type == 0) fn = nst == 4 ? gemm_tc_pair_kernel<__nv_bfloat16, 4, 4> : nst == 6 ? gemm_tc_pair_kernel<__nv_bfloat16, 6, 4> : gemm_tc_pair_kernel<__nv_bfloat16, STAGES2, 4>;
        else fn = nst == 4 ? gemm_tc_pair_kernel<float, 4, 4> : nst == 6 ? gemm_tc_pair_kernel<float, 6, 4> : gemm_tc_pair_kernel<float, STAGES2, 4>;
        static std::atomic<uint64_t> pair_attr_mask{0};
        if (!(pair_attr_mask.load() & dev_bit)) {
            for (PairFn f : {(PairFn)gemm_tc_pair_kernel<__nv_bfloat16, 4, 4>, (PairFn)gemm_tc_pair_kernel<__nv_bfloat16, STAGES2, 4>, (PairFn)gemm_tc_pair_kernel<__nv_bfloat16, 6, 4>,
                             (PairFn)gemm_tc_pair_kernel<float, 4, 4>, (PairFn)gemm_tc_pair_kernel<float, STAGES2, 4>, (PairFn)gemm_tc_pair_kernel<float, 6, 4>,
                             (PairFn)gemm_tc_pair_kernel<__nv_bfloat16, 4, 8>, (PairFn)gemm_tc_pair_kernel<float, 4, 8>}) {
                ZN_CUDA(ctx, cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2_bytes(STAGES2, true)));
                cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            }
            cudaGetLastError();
            pair_attr_mask.fetch_or(dev_bit);
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(2 * clusters));
        cfg.blockDim = dim3(pair8 ? 64 + 32 * 8 : THREADS);
        cfg.dynamicSmemBytes = pair8 ? smem2_bytes(4, true, 8) : smem2_bytes(nst, nst != 6);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t le = cudaLaunchKernelEx(&cfg, fn, tmA, tmB, tmC, p);
        if (le != cudaSuccess) return launch_failed(le, "launch of the two-CTA tensor-core GEMM");
#ifdef ZN_DIAG
        if (phases) {
            cudaStreamSynchronize(ctx->stream);
            long long tc[8 * 16];
            cudaMemcpyFromSymbol(tc, zn_diag_tile, sizeof tc);
            fprintf(stderr, "pair tiles m=%lld n=%lld k=%lld clusters=%d; leader CTA of cluster 0, cycles from its first stamp\n"
                            "  per tile: producer publish / first load / last load | MMA index / accumulator free / first operands / last issue | "
                            "epilogue index / accumulator full / done\n", (long long)m, (long long)n, (long long)k, clusters);
            long long t0 = tc[7] ? tc[7] : tc[0];
            for (int i = 0; i < 8; ++i) {
                if (!tc[i * 16 + 0]) break;
                fprintf(stderr, "  tile %d: P %lld %lld %lld | M %lld %lld %lld %lld | E %lld %lld %lld\n", i, tc[i * 16 + 7] - t0, tc[i * 16 + 8] - t0,
                        tc[i * 16 + 9] - t0, tc[i * 16 + 0] - t0, tc[i * 16 + 1] - t0, tc[i * 16 + 2] - t0, tc[i * 16 + 3] - t0,
                        tc[i * 16 + 4] - t0, tc[i * 16 + 5] - t0, tc[i * 16 + 6] - t0);
            }
            static const long long zeros[8 * 16] = {0};
            cudaMemcpyToSymbol(zn_diag_tile, zeros, sizeof zeros);
        }
#endif
        return ZN_OK;
    }
    const long long tiles = (long long)p.num_m_tiles * p.num_n_tiles;
    const int sms = ctx->sm_count - e.reserve_sms > 0 ? ctx->sm_count - e.reserve_sms : 1;
    const int grid = (int)(tiles < sms ? tiles : sms);
    OneFn fn;
    int smem;
    if (narrow) {
        fn = elem_type == 0 ? (OneFn)gemm_tc_kernel<__nv_bfloat16, 128, true> : (OneFn)gemm_tc_kernel<float, 128, true>;
        smem = onecta_smem(128, true);
    } else if (p.out_mode != 0) {
        fn = elem_type == 0 ? (OneFn)gemm_tc_kernel<__nv_bfloat16, 256, true> : (OneFn)gemm_tc_kernel<float, 256, true>;
        smem = onecta_smem(256, true);
    } else {
        fn = elem_type == 0 ? (OneFn)gemm_tc_kernel<__nv_bfloat16, 256, false> : (OneFn)gemm_tc_kernel<float, 256, false>;
        smem = onecta_smem(256, false);
    }
    // Programmatic stream serialization: the kernel's set-up (barriers, tensor memory, descriptor prefetch) may run
    // while the stream's previous kernel drains; the kernel itself waits for that kernel before it touches global
    // memory.  Measured on the 784-512-256-10 training step (9 such launches): 0.136 -> 0.125 ms.
    zn_launch_pdl(fn, dim3((unsigned)grid), dim3(THREADS1), (size_t)smem, ctx->stream, tmA, tmB, tmC, p);
    const cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return launch_failed(le, "launch of the tensor-core GEMM");
#ifdef ZN_DIAG
    if (phases) {
        cudaStreamSynchronize(ctx->stream);
        fprintf(stderr, "phases m=%lld n=%lld k=%lld grid=%d:", (long long)m, (long long)n, (long long)k, grid);
        for (int i = 1; i <= 8; ++i)
            fprintf(stderr, " %d:%+.2fus", i, phase_host[i] ? (double)((long long)phase_host[i] - (long long)phase_host[0]) / 1e3 : -1.0);
        fprintf(stderr, "\n");
        long long wt[8];
        cudaMemcpyFromSymbol(wt, zn_diag_wait, sizeof wt);
        fprintf(stderr, "  CTA 0: %lld tiles, %lld cycles from the first tile's last MMA to the last tile's; MMA thread waited %lld for a free accumulator, "
                        "%lld for operands; epilogue warp 2 waited %lld for accumulators and worked %lld on them\n",
                wt[3], wt[2], wt[0], wt[1], wt[4], wt[5]);
        static const long long wzeros[8] = {0};
        cudaMemcpyToSymbol(zn_diag_wait, wzeros, sizeof wzeros);
        long long clk[128];
        cudaMemcpyFromSymbol(clk, zn_diag_clk, sizeof clk);
        fprintf(stderr, "  epilogue clocks of warp 2 (cycles from the block's start: wait_ld, values, buffer free, staged, fence, issued):");
        for (int c = 0; c < 8; ++c) {
            fprintf(stderr, " [b%d @%lld:", c, c ? clk[c * 8] - clk[0] : 0ll);
            for (int k2 = 1; k2 <= 6; ++k2) fprintf(stderr, " %lld", clk[c * 8 + k2] ? clk[c * 8 + k2] - clk[c * 8] : -1ll);
            fprintf(stderr, "]");
        }
        fprintf(stderr, "\n");
    }
#endif
    return ZN_OK;
}
