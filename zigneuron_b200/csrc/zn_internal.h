// Internal declarations shared by the translation units of libzn_b200.so.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>
#include <cuda_bf16.h>

#include <cstdint>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <vector>

#include "zn_b200.h"

#define ZN_MAX_ERR 512

struct zn_prof_slot {
    double ms = 0, flops = 0, bytes = 0;
    uint64_t launches = 0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;   // recorded, not yet read back
};

struct zn_trace_rec { int family, lane; cudaEvent_t e0, e1; };   // one launch of a traced run

struct zn_dp_state;   // dp.cu

struct zn_ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;        // every kernel of this library runs here
    cudaStream_t copy_stream = nullptr;   // host<->device copies of the pipelined step
    cudaStream_t comm_stream = nullptr;   // gradient all-reduces
    zn_precision precision = ZN_FP32_SIMT;
    int batch_depth = 0;
    char err[ZN_MAX_ERR] = {0};

    // One pinned word the kernels' bounded waits write into when they give up.
    int *status_host = nullptr;           // cudaHostAlloc'd, mapped
    int *status_dev = nullptr;            // device alias of status_host

    // Scratch for two-stage reductions (block partials); grown on demand.
    float *scratch = nullptr;
    size_t scratch_floats = 0;
    // Lanes.  `stream` / `scratch` above are those of the ACTIVE lane; every launcher uses them.  The
    // training step runs its column reductions, its all-reduces and its parameter updates on lanes of
    // their own so that they overlap the GEMMs; each lane has its own scratch so concurrent reductions
    // never share partial-sum storage.  0 = main, 1 = communication, 2 = optimizer, 3 = auxiliary.
    struct lane_state { cudaStream_t stream = nullptr; float *scratch = nullptr; size_t scratch_floats = 0; };
    lane_state lanes[4];
    int lane = 0;
    cudaStream_t opt_stream = nullptr, aux_stream = nullptr;
    cudaEvent_t lane_join[4] = {nullptr, nullptr, nullptr, nullptr};
    // Staging for ops called with host pointers; grown on demand.
    float *stage[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t stage_floats[6] = {0, 0, 0, 0, 0, 0};
    float *pinned_scalar = nullptr;       // 16 floats of pinned host memory for scalar read-backs

    std::unordered_map<float *, size_t> tensors;   // zn_tensor_alloc registry (ptr -> count)
    std::unordered_map<std::string, std::vector<uint8_t>> tmap_cache;   // encoded TMA descriptors

    uint64_t launches = 0;
    bool profiling = false;
    zn_prof_slot prof[ZN_PROF_FAMILY_COUNT];
    std::vector<cudaEvent_t> event_pool;
    // ZN_TRACE_FILE=<path> (diagnostic): while profiling is on, every launch is also written as a line
    // "family lane start_ms end_ms" (times from the moment profiling was switched on) when the profile is read
    const char *trace_path = nullptr;
    cudaEvent_t trace_origin = nullptr;
    std::vector<zn_trace_rec> trace;
    cudaEvent_t timer0 = nullptr, timer1 = nullptr;
    // Two work counters for the persistent GEMM's dynamic tile scheduler, used in turn by successive launches
    // on the main stream (each launch clears the one the next launch will use).
    unsigned int *tile_counters = nullptr;
    unsigned int tile_counter_turn = 0;
    // Arrival counters of the reductions that finish in their own last block (column sums, sums of squares, loss
    // sums): 1024 per lane, all zero between launches (the block that finishes a reduction clears what it used).
    unsigned int *block_counters = nullptr;

    zn_dp_state *dp = nullptr;
};

zn_status zn_fail(zn_ctx *ctx, zn_status s, const char *fmt, ...);
zn_status zn_cuda_status(zn_ctx *ctx, cudaError_t e, const char *what);
#define ZN_CUDA(ctx, call)                                                            \
    do {                                                                              \
        cudaError_t e__ = (call);                                                     \
        if (e__ != cudaSuccess) return zn_cuda_status((ctx), e__, #call);             \
    } while (0)
#define ZN_TRY(call)                                                                  \
    do {                                                                              \
        zn_status s__ = (call);                                                       \
        if (s__ != ZN_OK) return s__;                                                 \
    } while (0)

// Launch bookkeeping: counts the launch and, when profiling, brackets it with events.
struct zn_launch_scope {
    zn_ctx *ctx;
    int family;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    zn_launch_scope(zn_ctx *c, int fam, double flops, double bytes, int n_launches = 1);
    ~zn_launch_scope();
};

// Launch with programmatic stream serialization: the kernel may be scheduled while the stream's previous kernel
// still runs, so it MUST execute zn_pdl_wait() before its first access to global memory.  Kernels that call
// zn_pdl_release() at their start let the kernel after them (if launched this way) be scheduled at once.
// ZN_TC_PDL=0 in the environment makes these ordinary launches (diagnostic).
#ifdef __CUDACC__
__device__ __forceinline__ void zn_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void zn_pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... Params, typename... Args>
inline cudaError_t zn_launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    static const bool pdl = !(getenv("ZN_TC_PDL") && atoi(getenv("ZN_TC_PDL")) == 0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}
#endif

enum { ZN_LANE_MAIN = 0, ZN_LANE_COMM = 1, ZN_LANE_OPT = 2, ZN_LANE_AUX = 3 };
void zn_lane_switch(zn_ctx *ctx, int lane);       // makes `lane` the active one (stream + scratch)
struct zn_lane_guard {                            // active lane for the lifetime of the guard
    zn_ctx *ctx;
    int prev;
    zn_lane_guard(zn_ctx *c, int lane) : ctx(c), prev(c->lane) { zn_lane_switch(c, lane); }
    ~zn_lane_guard() { zn_lane_switch(ctx, prev); }
};
// Host waits.  On a data-parallel context they poll (work done? communicator error? deadline?) instead of
// blocking, abort the communicator on an error or a missed deadline, and return ZN_ERR_NCCL (dp.cu).
zn_status zn_wait_event(zn_ctx *ctx, cudaEvent_t ev);
zn_status zn_wait_stream(zn_ctx *ctx, cudaStream_t s);
zn_status zn_sync_all_lanes(zn_ctx *ctx);         // host waits for every lane
zn_status zn_join_lanes_into_main(zn_ctx *ctx);   // the main stream waits (on the device) for the other lanes

zn_status zn_scratch_reserve(zn_ctx *ctx, size_t floats);
// The active lane's 1024 arrival counters (allocated and cleared on first use); see zn_ctx::block_counters.
enum { ZN_COUNTERS_PER_LANE = 1024, ZN_COUNTER_SUMSQ = 1000, ZN_COUNTER_LOSS = 1001 };   // [0, 1000): column strips
zn_status zn_lane_counters(zn_ctx *ctx, unsigned int **out);
zn_status zn_check_device_status(zn_ctx *ctx);   // reads the pinned status word after a sync
bool zn_is_device_ptr(const void *p);
int zn_ptr_device(const void *p);                 // owning device of a device pointer, -1 for host memory

// ---- kernels (each launcher enqueues on ctx->stream and returns) ------------------

// Epilogue applied by both GEMM families to the fp32 accumulator v of C[r][c]:
//   v += bias[c]; v = act(v); if (mask) v = mask[r][c] > 0 ? v : 0; if (accumulate) v += C_old[r][c]
// and stored as fp32 (out_f32) and/or as the activation type (out_t).
struct zn_epilogue {
    const float *bias = nullptr;
    int act = ZN_ACT_LINEAR;
    const void *mask = nullptr;        // activation type of the GEMM (float for SIMT/TF32, bf16 for BF16)
    int64_t ld_mask = 0;
    float *out_f32 = nullptr;
    int64_t ld_out_f32 = 0;
    void *out_t = nullptr;             // only the tensor-core path: output in the operand type
    int64_t ld_out_t = 0;
    int accumulate = 0;                // += into out_f32
    int reserve_sms = 0;               // tensor-core path: leave this many SMs to kernels on other streams
};

// fp32 CUDA-core GEMM.  A(i,p) = a[i*a_rs + p*a_cs], B(p,j) = b[p*b_rs + j*b_cs].
zn_status zn_gemm_simt(zn_ctx *ctx, const float *a, int64_t a_rs, int64_t a_cs, const float *b, int64_t b_rs,
                       int64_t b_cs, int64_t m, int64_t n, int64_t k, const zn_epilogue &ep, bool exact);

// tcgen05 GEMM.  Operand element type: 0 = bf16, 1 = tf32 (fp32 storage).
// A is K-major when a_mn_major == false (memory [m][lda]) and M-major otherwise ([k][lda]);
// B is K-major when b_mn_major == false (memory [n][ldb]) and N-major otherwise ([k][ldb]).
// lda/ldb are in elements and must make the row pitch a multiple of 16 bytes.
zn_status zn_gemm_tc(zn_ctx *ctx, int elem_type, const void *a, int64_t lda, bool a_mn_major, const void *b,
                     int64_t ldb, bool b_mn_major, int64_t m, int64_t n, int64_t k, const zn_epilogue &ep);

// Row-major helpers.  T = float or __nv_bfloat16 selected by is_bf16.
zn_status zn_k_convert(zn_ctx *ctx, const float *src, int64_t ld_src, void *dst, int64_t ld_dst, bool dst_bf16,
                       int64_t rows, int64_t cols);   // pads columns [cols, ld_dst) with zeros
zn_status zn_k_add_bias(zn_ctx *ctx, float *out, int64_t rows, int64_t cols, const float *bias);
zn_status zn_k_act_forward(zn_ctx *ctx, int act, const float *in, float *out, int64_t n);
zn_status zn_k_act_backward(zn_ctx *ctx, int act, const float *y, const float *go, float *gi, int64_t n);
// In place g = act'(y) (*) g on operand-typed blocks (activations whose derivative is not fused in a GEMM epilogue).
// For softmax this is the row-wise backward (`exact`: the dot product in column order).
zn_status zn_k_act_backward_t(zn_ctx *ctx, int act, const void *y, int64_t ld_y, void *g, int64_t ld_g, bool bf16,
                              int64_t rows, int64_t cols, bool exact = false);
// Softmax over each row of a block.  in: f32 or bf16; out_t (f32 or bf16) and out_f32 may each be null; in place allowed.
zn_status zn_k_softmax_rows(zn_ctx *ctx, const void *in, bool in_bf16, int64_t ld_in, void *out_t, bool out_bf16,
                            int64_t ld_t, float *out_f32, int64_t ld_f, int64_t rows, int64_t cols, bool exact);
zn_status zn_k_softmax_backward_rows(zn_ctx *ctx, const void *s, int64_t ld_s, const void *go, int64_t ld_go, void *gi,
                                     int64_t ld_gi, bool bf16, int64_t rows, int64_t cols, bool exact);
// gb[c] (+)= sum_r g[r][c]; exact = one thread per column, rows ascending.
zn_status zn_k_bias_reduce(zn_ctx *ctx, const void *g, bool g_bf16, int64_t ld, int64_t rows, int64_t cols,
                           float *gb, bool accumulate, bool exact);
// Loss value and gradient in one pass over output (fp32, row pitch ld_o) and target (fp32, dense).
// grad (type by grad_bf16, pitch ld_g) may be null (value only).  loss_sum_dev gets the SUM (squared errors
// for MSE, row losses for CE); the caller divides.  mse_divisor is the n of 2(o-t)/n.
zn_status zn_k_loss(zn_ctx *ctx, int loss, const float *out, int64_t ld_o, const float *target, void *grad,
                    bool grad_bf16, int64_t ld_g, int64_t rows, int64_t cols, float mse_divisor,
                    float *loss_sum_dev, bool exact = false);   // exact: sums in the reference's order, one thread

struct zn_seg { const float *ptr; size_t count; };
// norm_factor_dev[0] = sqrt(sum g^2), [1] = clip factor (1 when norm <= 1); extra_sq_dev optional.
zn_status zn_k_grad_norm(zn_ctx *ctx, const zn_seg *segs, int nseg, float *norm_factor_dev, bool exact = false);
zn_status zn_k_scale(zn_ctx *ctx, float *p, size_t n, const float *factor_dev);
// The same norm in two steps, so that each layer's share can be summed as soon as its gradients are final:
// sumsq_dev[0] = sum of squares over the segments (double); combine adds `count` such sums in order and
// writes norm / clip factor as zn_k_grad_norm does.
zn_status zn_k_sumsq(zn_ctx *ctx, const zn_seg *segs, int nseg, double *sumsq_dev);
zn_status zn_k_norm_combine(zn_ctx *ctx, const double *sumsq_dev, int count, float *norm_factor_dev);
zn_status zn_k_f32_to_f64(zn_ctx *ctx, const float *src, double *dst);   // one value
zn_status zn_k_f64_to_f32(zn_ctx *ctx, const double *src, float *dst);

// metrics.evaluateClassification on fp32 device blocks; confusion / metrics4 are host memory (either may be null).
zn_status zn_k_classification_metrics(zn_ctx *ctx, const float *out_dev, int64_t ld_o, const float *tgt_dev, int64_t ld_t,
                                      size_t rows, size_t cols, size_t num_classes, uint64_t *confusion, float *metrics4);

struct zn_opt_args {
    float *w; float *g; float *m; float *v; size_t count;
    float lr, wd, beta1, beta2, eps, bc1, bc2;
    float momentum, rho;            // momentum-SGD and RMSprop (their one state tensor is m)
    float decay_mul;                // AdamW: w *= decay_mul after the Adam update; 0 = no decoupled decay
    float w_clamp;                  // 100 for weights, 50 for SGD bias
    const float *factor_dev;        // clip factor on the device, or null
    void *shadow;                   // operand-type copy of w for the tensor-core GEMMs, or null
    bool shadow_bf16;
    int64_t cols, ld_shadow;        // shadow[(i / cols) * ld_shadow + i % cols]
};
// Every parameter tensor of a small network in ONE launch: `kinds[i]` says which update tensor i gets
// (0 sgd, 1 adam / adamw, 2 momentum sgd, 4 rmsprop; the OPT_* values of net.cu), is_bias[i] selects the plain
// SGD bias rule.  At most ZN_MULTI_UPDATE_MAX tensors.  Same arithmetic per element as the kernels below.
enum { ZN_MULTI_UPDATE_MAX = 16 };
zn_status zn_k_multi_update(zn_ctx *ctx, const zn_opt_args *args, const int *kinds, const int *is_bias, int count);
zn_status zn_k_sgd(zn_ctx *ctx, const zn_opt_args &a, bool is_bias);
zn_status zn_k_adam(zn_ctx *ctx, const zn_opt_args &a);
zn_status zn_k_sgd_momentum(zn_ctx *ctx, const zn_opt_args &a);
zn_status zn_k_rmsprop(zn_ctx *ctx, const zn_opt_args &a);
