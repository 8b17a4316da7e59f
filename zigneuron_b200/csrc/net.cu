// Device-resident Network of Dense layers: the reference's Network.forward /
// computeGradients / trainStep / train (src/network.zig:309-616), Dense.forward /
// backward (src/layer.zig:380-475) and Sgd.step / Adam.step (src/optimizer.zig:
// 160-164, 209-233) restated as one stream of fused kernels.
//
// Per layer and step the stream holds: one GEMM for Y = act(X.W + b); one
// column reduction for gb; one GEMM for gW = X^T.G; one GEMM for
// dX = (G.W^T) (*) act'(Y_prev), whose epilogue produces the next layer's G
// directly; then the global norm (two launches) and one update launch per
// parameter tensor.  Only the inputs of each layer and the activated outputs are
// kept, as in the reference's LayerCache (src/network.zig:33-36).
//
// HBM layout.  Per layer one parameter block [W (in*out) | pad to 4 | b (out)],
// with gradient, Adam-m and Adam-v blocks of the same shape, all fp32.  In the
// tensor-core modes W also has an operand copy (bf16, or fp32 with a pitch TMA
// accepts) that the optimizer kernel refreshes.  Activations are [rows][ld] in
// the operand type, ld = width rounded up to 8 elements in tensor-core modes.
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "zn_internal.h"

zn_status zn_dp_allreduce(zn_ctx *ctx, float *buf, size_t count, cudaStream_t stream);   // dp.cu
bool zn_dp_active(const zn_ctx *ctx);
// Gradient memory NCCL can reduce in place (dp.cu); ZN_ERR_NOT_AVAILABLE = keep the ordinary allocation.
zn_status zn_dp_alloc_registered(zn_ctx *ctx, size_t bytes, void **ptr_out, void **handle_out);
void zn_dp_free_registered(zn_ctx *ctx, void *ptr, void *handle);
int zn_dp_rank(const zn_ctx *ctx);
int zn_dp_world(const zn_ctx *ctx);
bool zn_dp_can_shard(const zn_ctx *ctx);
zn_status zn_dp_allreduce_f64(zn_ctx *ctx, double *buf, size_t count, cudaStream_t stream);
zn_status zn_dp_reduce_scatter(zn_ctx *ctx, float *buf, size_t shard, cudaStream_t stream);
zn_status zn_dp_all_gather(zn_ctx *ctx, float *buf, size_t shard, cudaStream_t stream);
bool zn_dp_can_gather_bf16(const zn_ctx *ctx);
zn_status zn_dp_all_gather_bf16(zn_ctx *ctx, void *buf, size_t shard, cudaStream_t stream);
zn_status zn_dp_broadcast(zn_ctx *ctx, float *buf, size_t count, int root, cudaStream_t stream);

namespace {

int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

enum { OPT_SGD = 0, OPT_ADAM = 1, OPT_MOMENTUM = 2, OPT_ADAMW = 3, OPT_RMSPROP = 4 };

struct Layer {
    size_t in = 0, out = 0;
    int act = ZN_ACT_LINEAR;
    size_t b_off = 0, len = 0, blk = 0;   // bias offset, used length, used length rounded up to a multiple of 4
    size_t cap = 0;                       // floats allocated per block: >= blk + 4; the last four are the tail
    size_t shard = 0;                     // sharded update: floats per rank, world * shard >= blk
    bool gather_bf16 = false;             // sharded update: the ranks exchange the bf16 operand copy, not the fp32 weights
    float *params = nullptr, *grads = nullptr, *m = nullptr, *v = nullptr;
    void *grads_reg = nullptr, *params_reg = nullptr;   // registration handles of blocks that come from NCCL
    bool grads_nccl = false, params_nccl = false;       // the block was allocated by NCCL and is registered
    void *w_op = nullptr;                 // operand copy of W (tensor-core modes), null when W itself is usable
    int64_t ld_w = 0;
    int opt = OPT_SGD;                    // OPT_* below
    float momentum = 0.0f, rho = 0.9f;
    float beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, wd = 0.f;
    size_t t = 0;
    // ordering between the lanes of a step (see step_dev)
    cudaEvent_t g_ready = nullptr, bias_done = nullptr, grads_ready = nullptr, reduced = nullptr, updated = nullptr;
    cudaEvent_t stepped = nullptr;        // sharded update: this rank's piece of the layer has been updated
    bool update_pending = false;          // `updated` has been recorded and not yet waited for by the host
};

struct Slot {                             // one in-flight pipelined step
    float *x = nullptr, *t = nullptr;     // device staging of the host block
    size_t x_cap = 0, t_cap = 0;
    cudaEvent_t copied = nullptr, done = nullptr;
    float *loss_host = nullptr;           // pinned: [loss_sum, norm, factor]
    size_t rows = 0;
    int loss = 0;
    bool busy = false;
};

}   // namespace

struct zn_net {
    zn_ctx *ctx = nullptr;
    zn_precision prec = ZN_FP32_SIMT;
    bool tc = false, bf16 = false;
    std::vector<Layer> layers;
    size_t cap_rows = 0;
    std::vector<void *> acts;             // acts[0] = operand copy of the input (or null when the input is used in place)
    std::vector<int64_t> lds;             // lds[i] = pitch of acts[i]
    float *out_f32 = nullptr;             // fp32 output of the last layer (tensor-core modes)
    void *gwork[2] = {nullptr, nullptr};
    int64_t g_ld_max = 0;
    float *scalars = nullptr;             // device: [0] norm, [1] clip factor
    double *sumsq = nullptr;              // device: per-layer sum of squared gradients (64 slots)
    Slot slots[2];
    int head = 0, inflight = 0;
    size_t global_rows = 0;               // > 0: data parallel
    bool shard_update = false;            // data parallel with the update split over the ranks (see step_dev)
    bool params_stale = false;            // sharded update with bf16 hand-over: fp32 W of the other ranks' pieces is out of date
    cudaEvent_t norm_ready = nullptr;     // sharded update: the global sums of squares and the loss sum are in
    float last_norm = 0.f, last_factor = 1.f;
    const void *last_input_grad = nullptr;
    size_t last_rows = 0;
    uint64_t seed_counter = 0;
};

namespace {

size_t esize(const zn_net *n) { return n->bf16 ? 2 : 4; }

void free_acts(zn_net *n) {
    for (void *p : n->acts) cudaFree(p);
    n->acts.clear();
    n->lds.clear();
    cudaFree(n->out_f32); n->out_f32 = nullptr;
    cudaFree(n->gwork[0]); cudaFree(n->gwork[1]);
    n->gwork[0] = n->gwork[1] = nullptr;
    n->cap_rows = 0;
}

int64_t pitch_of(const zn_net *n, size_t width) { return n->tc ? round_up((int64_t)width, 8) : (int64_t)width; }

// (Re)allocates activation and gradient work buffers for `rows` samples.
zn_status ensure_rows(zn_net *n, size_t rows) {
    zn_ctx *ctx = n->ctx;
    if (rows <= n->cap_rows && n->acts.size() == n->layers.size() + 1) return ZN_OK;
    ZN_TRY(zn_sync_all_lanes(ctx));
    const size_t keep = rows > n->cap_rows ? rows : n->cap_rows;
    free_acts(n);
    const size_t L = n->layers.size();
    n->acts.assign(L + 1, nullptr);
    n->lds.assign(L + 1, 0);
    n->g_ld_max = 0;
    for (size_t i = 0; i <= L; ++i) {
        const size_t width = i == 0 ? n->layers[0].in : n->layers[i - 1].out;
        n->lds[i] = pitch_of(n, width);
        if (n->lds[i] > n->g_ld_max) n->g_ld_max = n->lds[i];
        // acts[0] is only materialised when the input must be converted or re-pitched
        if (i == 0 && !n->tc) continue;
        ZN_CUDA(ctx, cudaMalloc(&n->acts[i], keep * (size_t)n->lds[i] * esize(n)));
        ZN_CUDA(ctx, cudaMemsetAsync(n->acts[i], 0, keep * (size_t)n->lds[i] * esize(n), ctx->stream));
    }
    if (n->tc) ZN_CUDA(ctx, cudaMalloc((void **)&n->out_f32, keep * n->layers[L - 1].out * sizeof(float)));
    for (int i = 0; i < 2; ++i) {
        ZN_CUDA(ctx, cudaMalloc(&n->gwork[i], keep * (size_t)n->g_ld_max * esize(n)));
        ZN_CUDA(ctx, cudaMemsetAsync(n->gwork[i], 0, keep * (size_t)n->g_ld_max * esize(n), ctx->stream));
    }
    n->cap_rows = keep;
    return ZN_OK;
}

zn_status refresh_operand_copy(zn_net *n, Layer &l) {
    if (!l.w_op) return ZN_OK;
    return zn_k_convert(n->ctx, l.params, (int64_t)l.out, l.w_op, l.ld_w, n->bf16, (int64_t)l.in, (int64_t)l.out);
}

// One of the three products in the network's precision.  a/b are operand-typed.
zn_status net_gemm(zn_net *n, int orient /*0 NN,1 TN,2 NT*/, const void *a, int64_t lda, const void *b, int64_t ldb,
                   int64_t m, int64_t nn, int64_t k, const zn_epilogue &ep) {
    zn_ctx *ctx = n->ctx;
    if (!n->tc) {
        const float *fa = (const float *)a, *fb = (const float *)b;
        const bool exact = n->prec == ZN_FP32_EXACT;
        if (orient == 0) return zn_gemm_simt(ctx, fa, lda, 1, fb, ldb, 1, m, nn, k, ep, exact);
        if (orient == 1) return zn_gemm_simt(ctx, fa, 1, lda, fb, ldb, 1, m, nn, k, ep, exact);
        return zn_gemm_simt(ctx, fa, lda, 1, fb, 1, ldb, m, nn, k, ep, exact);
    }
    const int et = n->bf16 ? 0 : 1;
    return zn_gemm_tc(ctx, et, a, lda, orient == 1, b, ldb, orient != 2, m, nn, k, ep);
}

// Forward over `rows` samples whose fp32 input block x_dev is on the device.
zn_status forward_dev(zn_net *n, const float *x_dev, size_t rows) {
    zn_ctx *ctx = n->ctx;
    const size_t L = n->layers.size();
    ZN_TRY(ensure_rows(n, rows));
    const void *cur = x_dev;
    if (n->tc) {
        ZN_TRY(zn_k_convert(ctx, x_dev, (int64_t)n->layers[0].in, n->acts[0], n->lds[0], n->bf16, (int64_t)rows,
                            (int64_t)n->layers[0].in));
        cur = n->acts[0];
    }
    for (size_t i = 0; i < L; ++i) {
        Layer &l = n->layers[i];
        zn_epilogue ep;
        ep.bias = l.params + l.b_off;
        // softmax needs whole rows: the GEMM writes the biased pre-activations, a row kernel follows
        const bool softmax = l.act == ZN_ACT_SOFTMAX;
        ep.act = softmax ? (int)ZN_ACT_LINEAR : l.act;
        const bool last = i + 1 == L;
        if (!n->tc) {
            ep.out_f32 = (float *)n->acts[i + 1];
            ep.ld_out_f32 = n->lds[i + 1];
        } else {
            if (last) { ep.out_f32 = n->out_f32; ep.ld_out_f32 = (int64_t)l.out; }
            if ((!last || l.act != ZN_ACT_LINEAR) && !(last && softmax)) { ep.out_t = n->acts[i + 1]; ep.ld_out_t = n->lds[i + 1]; }
        }
        const void *w = l.w_op ? l.w_op : (const void *)l.params;
        const int64_t ldw = l.w_op ? l.ld_w : (int64_t)l.out;
        // the previous step's update of this layer may still be running on the optimizer lane
        if (l.update_pending) ZN_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, l.updated, 0));
        ZN_TRY(net_gemm(n, 0, cur, n->lds[i], w, ldw, (int64_t)rows, (int64_t)l.out, (int64_t)l.in, ep));
        if (softmax) {     // Dense.forward, src/layer.zig:398-406
            const bool exact = n->prec == ZN_FP32_EXACT;
            const int64_t ld = n->lds[i + 1];
            if (!n->tc)          // fp32 block, in place
                ZN_TRY(zn_k_softmax_rows(ctx, n->acts[i + 1], false, ld, nullptr, false, 0, (float *)n->acts[i + 1], ld,
                                         (int64_t)rows, (int64_t)l.out, exact));
            else if (last)       // fp32 logits -> fp32 probabilities in place, plus the operand-typed copy the backward reads
                ZN_TRY(zn_k_softmax_rows(ctx, n->out_f32, false, (int64_t)l.out, n->acts[i + 1], n->bf16, ld, n->out_f32,
                                         (int64_t)l.out, (int64_t)rows, (int64_t)l.out, exact));
            else                 // hidden layer: operand-typed block, in place
                ZN_TRY(zn_k_softmax_rows(ctx, n->acts[i + 1], n->bf16, ld, n->acts[i + 1], n->bf16, ld, nullptr, 0,
                                         (int64_t)rows, (int64_t)l.out, exact));
        }
        cur = n->acts[i + 1];
    }
    return ZN_OK;
}

float *final_output(zn_net *n) { return n->tc ? n->out_f32 : (float *)n->acts[n->layers.size()]; }

// Everything of one training step after the inputs are on the device.  x_dev / t_dev fp32.
// The loss SUM lands in the tail slot of the last layer's gradient block.
//
// Lanes (streams) of one step, so that only the GEMMs and the loss sit on the critical path:
//   main  forward GEMMs, loss, and per layer (last to first) gW GEMM and dX GEMM
//   aux   per layer the column reduction G -> gb, as soon as G exists
//   comm  per layer, once gW and gb exist: all-reduce over ranks (data parallel), then that layer's sum of
//         squared gradients
//   opt   once every layer is reduced: norm and clip factor, loss/norm read-back into loss_dst, then the
//         update of every layer; `done` is recorded after the read-back, BEFORE the updates
// The updates of step k therefore run under the forward GEMMs of step k+1: the forward GEMM of layer l
// waits (on the device) for the update of layer l only.
zn_status step_dev(zn_net *n, const float *x_dev, const float *t_dev, size_t rows, float lr, int loss, float *loss_dst,
                   cudaEvent_t done) {
    zn_ctx *ctx = n->ctx;
    const size_t L = n->layers.size();
    const bool exact = n->prec == ZN_FP32_EXACT;
    const bool dp = n->global_rows > 0 && zn_dp_active(ctx);
    const bool shard = dp && n->shard_update && !exact;
    // Small networks (a few million parameters at most, one GPU) are bound by launches and stream hand-overs, not
    // by any kernel.  ZN_COMPACT_STEP=1 runs their whole step on the main stream with the norm of all gradients in
    // one launch and the update of every tensor in one launch: 16 launches instead of 24 on 784-512-256-10, but
    // 0.173 against 0.156 ms per step in bf16 -- the lanes' overlap is worth more than the launches saved -- so
    // it is an option, not the default.
    static const bool compact_allowed = getenv("ZN_COMPACT_STEP") && atoi(getenv("ZN_COMPACT_STEP")) != 0;
    size_t total_params = 0;
    for (const Layer &l : n->layers) total_params += l.len;
    const bool compact = compact_allowed && !dp && !exact && total_params <= ((size_t)1 << 22) && 2 * L <= ZN_MULTI_UPDATE_MAX;
    const int lane_comm = compact ? ZN_LANE_MAIN : ZN_LANE_COMM, lane_opt = compact ? ZN_LANE_MAIN : ZN_LANE_OPT;
    const int lane_aux = compact ? ZN_LANE_MAIN : ZN_LANE_AUX;
    cudaStream_t s_main = ctx->stream;   // lane 0 is active here; its slot in lanes[] is only refreshed on a switch
    cudaStream_t s_comm = compact ? s_main : ctx->lanes[ZN_LANE_COMM].stream;
    cudaStream_t s_opt = compact ? s_main : ctx->lanes[ZN_LANE_OPT].stream;
    cudaStream_t s_aux = compact ? s_main : ctx->lanes[ZN_LANE_AUX].stream;
    // ordering between two lanes; inside one stream the order of submission is the order of execution
    auto hand_over = [&](cudaEvent_t ev, cudaStream_t from, cudaStream_t to) -> zn_status {
        if (from == to) return ZN_OK;
        ZN_CUDA(ctx, cudaEventRecord(ev, from));
        ZN_CUDA(ctx, cudaStreamWaitEvent(to, ev, 0));
        return ZN_OK;
    };
    ZN_TRY(forward_dev(n, x_dev, rows));

    Layer &last = n->layers[L - 1];
    const size_t out_cols = last.out;
    const size_t total_rows = dp ? n->global_rows : rows;
    float *loss_slot = last.grads + (last.cap - 4);   // first float of the tail
    int cur = 0;
    ZN_TRY(zn_k_loss(ctx, loss, final_output(n), (int64_t)out_cols, t_dev, n->gwork[cur], n->bf16, n->lds[L],
                     (int64_t)rows, (int64_t)out_cols, (float)(total_rows * out_cols), loss_slot, exact));
    if (last.act != ZN_ACT_LINEAR)   // Dense.backward applies the derivative of every layer, the last included
        ZN_TRY(zn_k_act_backward_t(ctx, last.act, n->acts[L], n->lds[L], n->gwork[cur], n->lds[L], n->bf16,
                                   (int64_t)rows, (int64_t)out_cols, exact));

    for (size_t idx = L; idx-- > 0;) {
        Layer &l = n->layers[idx];
        const void *g = n->gwork[cur];
        const int64_t ld_g = n->lds[idx + 1];
        const void *x_in = (idx == 0 && !n->tc) ? (const void *)x_dev : (const void *)n->acts[idx];
        // gb = column sums of G   (accumulateBias into a cleared gb, src/layer.zig:459), on the aux lane
        ZN_TRY(hand_over(l.g_ready, s_main, s_aux));
        {
            zn_lane_guard lane(ctx, lane_aux);
            ZN_TRY(zn_k_bias_reduce(ctx, g, n->bf16, ld_g, (int64_t)rows, (int64_t)l.out, l.grads + l.b_off, false, exact));
        }
        if (!compact) ZN_CUDA(ctx, cudaEventRecord(l.bias_done, s_aux));
        // gW = X^T . G           (matMulTransposeA, src/layer.zig:466)
        // (Computing layer 0's gW as two halves and putting the first half on the wire while the second is computed
        // was measured on 8 GPUs: 8.464 against 8.390 ms per step.  Two launches of half the tiles lose more to
        // their partial last waves than the earlier start of the exchange gains.  Not kept.)
        {
            zn_epilogue ep;
            ep.out_f32 = l.grads;
            ep.ld_out_f32 = (int64_t)l.out;
            ZN_TRY(net_gemm(n, 1, x_in, n->lds[idx], g, ld_g, (int64_t)l.in, (int64_t)l.out, (int64_t)rows, ep));
        }
        // this layer's gradients are final: sum them over ranks and square-sum them while earlier layers run
        ZN_TRY(hand_over(l.grads_ready, s_main, s_comm));
        if (!compact) ZN_CUDA(ctx, cudaStreamWaitEvent(s_comm, l.bias_done, 0));
        // the last layer's block carries the loss sum in its tail; the other three tail floats stay zero and
        // ride along so that every exchanged count is a multiple of four floats
        if (dp && !shard) ZN_TRY(zn_dp_allreduce(ctx, l.grads, idx + 1 == L ? l.cap : l.blk, s_comm));
        if (shard) {
            // sharded update: this rank ends with the summed gradients of its own piece of the block only, and
            // squares just that piece (the padding inside a block is zero and adds nothing)
            ZN_TRY(zn_dp_reduce_scatter(ctx, l.grads, l.shard, s_comm));
            zn_lane_guard lane(ctx, ZN_LANE_COMM);
            const size_t lo = (size_t)zn_dp_rank(ctx) * l.shard, hi = lo + l.shard < l.blk ? lo + l.shard : l.blk;
            if (lo < hi) {
                const zn_seg seg = {l.grads + lo, hi - lo};
                ZN_TRY(zn_k_sumsq(ctx, &seg, 1, n->sumsq + idx));
            } else {
                ZN_CUDA(ctx, cudaMemsetAsync(n->sumsq + idx, 0, sizeof(double), s_comm));
            }
        } else if (!exact && !compact) {
            zn_lane_guard lane(ctx, ZN_LANE_COMM);
            const zn_seg segs[2] = {{l.grads, l.in * l.out}, {l.grads + l.b_off, l.out}};
            ZN_TRY(zn_k_sumsq(ctx, segs, 2, n->sumsq + idx));
        }
        if (!compact) ZN_CUDA(ctx, cudaEventRecord(l.reduced, s_comm));
        // G of the layer above lives in the block the next dX overwrites: its column sums must be done
        if (idx + 1 < L && !compact) ZN_CUDA(ctx, cudaStreamWaitEvent(s_main, n->layers[idx + 1].bias_done, 0));
        // dX = G . W^T, masked by the previous layer's activation derivative (src/layer.zig:440-448)
        {
            zn_epilogue ep;
            const int prev_act = idx > 0 ? n->layers[idx - 1].act : ZN_ACT_LINEAR;
            if (prev_act == ZN_ACT_RELU) { ep.mask = n->acts[idx]; ep.ld_mask = n->lds[idx]; }
            if (n->tc) { ep.out_t = n->gwork[cur ^ 1]; ep.ld_out_t = n->lds[idx]; }
            else { ep.out_f32 = (float *)n->gwork[cur ^ 1]; ep.ld_out_f32 = n->lds[idx]; }
            // The exchange of layer 0's gradients is the one nothing else hides: its kernel must start the moment
            // gW is done, not after this last GEMM has taken every SM.  So the first rows of this GEMM, about as
            // many as the exchange lasts (8192 rows of the wide MLP = 0.4 ms, the time 134 MB take through NVSwitch),
            // run on 32 SMs fewer; the rest runs on all of them.  Measured on 8 GPUs: 8.65 -> 8.53 ms per step.
            // ZN_DP_RESERVE_SMS / ZN_DP_RESERVE_ROWS override the two figures (0 SMs switches it off).
            static const int reserve = getenv("ZN_DP_RESERVE_SMS") ? atoi(getenv("ZN_DP_RESERVE_SMS")) : 32;
            static const long long reserve_rows = getenv("ZN_DP_RESERVE_ROWS") ? atoll(getenv("ZN_DP_RESERVE_ROWS")) : 8192;
            const void *w = l.w_op ? l.w_op : (const void *)l.params;
            const int64_t ldw = l.w_op ? l.ld_w : (int64_t)l.out;
            if (dp && idx == 0 && n->tc && reserve > 0 && reserve_rows > 0) {
                const size_t first = rows < (size_t)reserve_rows ? rows : (size_t)reserve_rows;
                zn_epilogue e1 = ep;
                e1.reserve_sms = reserve;
                ZN_TRY(net_gemm(n, 2, g, ld_g, w, ldw, (int64_t)first, (int64_t)l.in, (int64_t)l.out, e1));
                if (rows > first) {
                    zn_epilogue e2 = ep;
                    e2.out_t = (char *)ep.out_t + first * (size_t)ep.ld_out_t * esize(n);
                    const void *g2 = (const char *)g + first * (size_t)ld_g * esize(n);
                    ZN_TRY(net_gemm(n, 2, g2, ld_g, w, ldw, (int64_t)(rows - first), (int64_t)l.in, (int64_t)l.out, e2));
                }
            } else {
                ZN_TRY(net_gemm(n, 2, g, ld_g, w, ldw, (int64_t)rows, (int64_t)l.in, (int64_t)l.out, ep));
            }
            if (idx > 0 && prev_act != ZN_ACT_RELU && prev_act != ZN_ACT_LINEAR)
                ZN_TRY(zn_k_act_backward_t(ctx, prev_act, n->acts[idx], n->lds[idx], n->gwork[cur ^ 1], n->lds[idx],
                                           n->bf16, (int64_t)rows, (int64_t)l.in, exact));
        }
        cur ^= 1;
    }
    n->last_input_grad = n->gwork[cur];
    n->last_rows = rows;

    // ---- optimizer lane: everything below waits for all layers' reductions, not for the main stream
    if (!compact)
        for (size_t i = 0; i < L; ++i) ZN_CUDA(ctx, cudaStreamWaitEvent(s_opt, n->layers[i].reduced, 0));
    zn_lane_guard opt_lane(ctx, lane_opt);
    (void)lane_comm;

    // global norm over every gradient tensor, weights then bias, layer by layer (src/network.zig:513-521)
    if (exact || compact) {
        std::vector<zn_seg> segs;
        for (size_t i = 0; i < L; ++i) {
            segs.push_back({n->layers[i].grads, n->layers[i].in * n->layers[i].out});
            segs.push_back({n->layers[i].grads + n->layers[i].b_off, n->layers[i].out});
        }
        ZN_TRY(zn_k_grad_norm(ctx, segs.data(), (int)segs.size(), n->scalars, exact));
    } else {
        if (shard) {
            // one exchange of L + 1 doubles: every layer's sum of squares and the loss sum; the communication lane
            // has every layer's reduce-scatter and square-sum in front of it
            zn_lane_guard lane(ctx, ZN_LANE_COMM);
            ZN_TRY(zn_k_f32_to_f64(ctx, loss_slot, n->sumsq + L));
            ZN_TRY(zn_dp_allreduce_f64(ctx, n->sumsq, L + 1, s_comm));
            ZN_TRY(zn_k_f64_to_f32(ctx, n->sumsq + L, loss_slot));
            ZN_CUDA(ctx, cudaEventRecord(n->norm_ready, s_comm));
            ZN_CUDA(ctx, cudaStreamWaitEvent(s_opt, n->norm_ready, 0));
        }
        ZN_TRY(zn_k_norm_combine(ctx, n->sumsq, (int)L, n->scalars));
    }
    if (loss_dst) {
        ZN_CUDA(ctx, cudaMemcpyAsync(loss_dst, loss_slot, sizeof(float), cudaMemcpyDefault, s_opt));
        if (!zn_is_device_ptr(loss_dst))
            ZN_CUDA(ctx, cudaMemcpyAsync(loss_dst + 1, n->scalars, 2 * sizeof(float), cudaMemcpyDeviceToHost, s_opt));
    }
    if (done) ZN_CUDA(ctx, cudaEventRecord(done, s_opt));

    // optimizer per layer (src/network.zig:541-549)
    zn_opt_args multi_args[ZN_MULTI_UPDATE_MAX];
    int multi_kind[ZN_MULTI_UPDATE_MAX], multi_bias[ZN_MULTI_UPDATE_MAX], multi_n = 0;
    for (size_t i = 0; i < L; ++i) {
        Layer &l = n->layers[i];
        zn_opt_args a{};
        a.lr = lr; a.wd = l.wd; a.factor_dev = n->scalars + 1;
        a.beta1 = l.beta1; a.beta2 = l.beta2; a.eps = l.eps; a.momentum = l.momentum; a.rho = l.rho;
        const bool adam = l.opt == OPT_ADAM || l.opt == OPT_ADAMW;
        if (adam) {
            l.t += 1;
            const float tf = (float)l.t;
            a.bc1 = 1.0f - powf(l.beta1, tf);
            a.bc2 = 1.0f - powf(l.beta2, tf);
        }
        if (l.opt == OPT_ADAMW) {      // decay is decoupled: nothing joins the gradient
            const float wdlr = lr * l.wd;
            a.wd = 0.0f;
            a.decay_mul = 1.0f - wdlr;
        }
        // a small layer's weights and bias share one launch (the launch costs more than either update)
        const bool pair_update = !compact && !shard && l.len <= ((size_t)1 << 20);
        auto update = [&](bool is_bias) -> zn_status {
            if (compact || pair_update) {      // queued: one launch for all tensors after the loop (compact) or per layer
                a.w_clamp = (l.opt == OPT_SGD && is_bias) ? 50.0f : 100.0f;
                multi_args[multi_n] = a;
                multi_kind[multi_n] = l.opt == OPT_ADAMW ? (int)OPT_ADAM : l.opt;
                multi_bias[multi_n] = is_bias ? 1 : 0;
                ++multi_n;
                return ZN_OK;
            }
            switch (l.opt) {
            case OPT_ADAM: case OPT_ADAMW: a.w_clamp = 100.0f; return zn_k_adam(ctx, a);
            case OPT_MOMENTUM: return zn_k_sgd_momentum(ctx, a);
            case OPT_RMSPROP: a.w_clamp = 100.0f; return zn_k_rmsprop(ctx, a);
            default: a.w_clamp = is_bias ? 50.0f : 100.0f; return zn_k_sgd(ctx, a, is_bias);
            }
        };
        if (shard) {
            // Each rank updates its own piece of the block (weights part and bias part of it separately, as the
            // plain SGD path treats them differently), then the pieces are gathered in place and the operand
            // copy of W is rebuilt from the gathered fp32 weights; the forward GEMM of this layer waits for that.
            const size_t lo = (size_t)zn_dp_rank(ctx) * l.shard, hi = lo + l.shard;
            const size_t region[2][2] = {{0, l.in * l.out}, {l.b_off, l.b_off + l.out}};
            for (int part = 0; part < 2; ++part) {
                const size_t a0 = lo > region[part][0] ? lo : region[part][0];
                const size_t a1 = hi < region[part][1] ? hi : region[part][1];
                if (a0 >= a1) continue;
                a.w = l.params + a0; a.g = l.grads + a0; a.count = a1 - a0; a.shadow = nullptr;
                a.m = l.m ? l.m + a0 : nullptr;
                a.v = l.v ? l.v + a0 : nullptr;
                if (part == 0 && l.gather_bf16) {
                    // the update writes this piece of the bf16 operand copy as well: W and its copy have the same
                    // flat layout (pitch = width), so the piece sits at the same offset
                    a.shadow = static_cast<__nv_bfloat16 *>(l.w_op) + a0;
                    a.shadow_bf16 = true;
                    a.cols = a.ld_shadow = (int64_t)l.out;
                }
                ZN_TRY(update(part == 1));
            }
            ZN_CUDA(ctx, cudaEventRecord(l.stepped, s_opt));
            ZN_CUDA(ctx, cudaStreamWaitEvent(s_comm, l.stepped, 0));
            if (l.gather_bf16) {
                // What the next forward pass needs is the bf16 operand copy and the fp32 bias: gather the first (half
                // the bytes of the fp32 weights, and no conversion pass afterwards), broadcast the second from the
                // rank(s) that own it.  The fp32 weights of the other ranks' pieces are brought up to date only when
                // somebody asks for them (zn_net_get_weights, zn_net_save).
                ZN_TRY(zn_dp_all_gather_bf16(ctx, l.w_op, l.shard, s_comm));
                const size_t b0 = l.b_off, b1 = l.b_off + l.out;
                for (size_t r = b0 / l.shard; r <= (b1 - 1) / l.shard; ++r) {
                    const size_t c0 = b0 > r * l.shard ? b0 : r * l.shard;
                    const size_t c1 = b1 < (r + 1) * l.shard ? b1 : (r + 1) * l.shard;
                    if (c0 < c1) ZN_TRY(zn_dp_broadcast(ctx, l.params + c0, c1 - c0, (int)r, s_comm));
                }
                n->params_stale = true;
            } else {
                ZN_TRY(zn_dp_all_gather(ctx, l.params, l.shard, s_comm));
                zn_lane_guard lane(ctx, ZN_LANE_COMM);
                ZN_TRY(refresh_operand_copy(n, l));
            }
            ZN_CUDA(ctx, cudaEventRecord(l.updated, s_comm));
            l.update_pending = true;
            continue;
        }
        // weights
        a.w = l.params; a.g = l.grads; a.m = l.m; a.v = l.v; a.count = l.in * l.out;
        a.shadow = l.w_op; a.shadow_bf16 = n->bf16; a.cols = (int64_t)l.out; a.ld_shadow = l.ld_w;
        ZN_TRY(update(false));
        // bias
        a.w = l.params + l.b_off; a.g = l.grads + l.b_off; a.count = l.out; a.shadow = nullptr;
        if (l.m) a.m = l.m + l.b_off;
        if (l.v) a.v = l.v + l.b_off;
        ZN_TRY(update(true));
        if (compact) continue;        // everything runs on the main stream: the next step is ordered after it anyway
        if (pair_update) {
            ZN_TRY(zn_k_multi_update(ctx, multi_args, multi_kind, multi_bias, multi_n));
            multi_n = 0;
        }
        ZN_CUDA(ctx, cudaEventRecord(l.updated, s_opt));
        l.update_pending = true;
    }
    if (compact && multi_n > 0) ZN_TRY(zn_k_multi_update(ctx, multi_args, multi_kind, multi_bias, multi_n));
    return ZN_OK;
}

// Sharded update with the bf16 hand-over: every rank gathers the fp32 weights of the other ranks' pieces.  Collective:
// every rank has to come here (zn_net_get_weights, zn_net_save and switching the sharding off do).
zn_status gather_stale_params(zn_net *n) {
    if (!n->params_stale) return ZN_OK;
    zn_ctx *ctx = n->ctx;
    ZN_TRY(zn_sync_all_lanes(ctx));
    for (Layer &l : n->layers)
        if (l.gather_bf16) ZN_TRY(zn_dp_all_gather(ctx, l.params, l.shard, ctx->lanes[ZN_LANE_COMM].stream));
    ZN_TRY(zn_sync_all_lanes(ctx));
    n->params_stale = false;
    return ZN_OK;
}

// A device operand of a network call must live on the network's own GPU: its kernels (and the tensor maps built
// over it) must never be handed another device's memory.
zn_status same_device(zn_net *n, const void *p, const char *what) {
    const int owner = zn_ptr_device(p);
    if (owner >= 0 && owner != n->ctx->device)
        return zn_fail(n->ctx, ZN_ERR_INVALID_DEVICE, "%s lives on device %d, the network on device %d", what, owner, n->ctx->device);
    return ZN_OK;
}

// kl_divergence (src/loss.zig:62-92) splits ONE output vector into [mu | log_var] and has no batched meaning.
bool loss_supported(int loss) { return loss >= ZN_LOSS_MSE && loss <= ZN_LOSS_BINARY_CROSS_ENTROPY; }

float loss_from_sum(const zn_net *n, float sum, size_t rows, int loss) {
    const size_t total_rows = (n->global_rows > 0 && zn_dp_active(n->ctx)) ? n->global_rows : rows;
    const size_t cols = n->layers.back().out;
    if (loss == ZN_LOSS_MSE || loss == ZN_LOSS_BINARY_CROSS_ENTROPY) return sum / (float)(total_rows * cols);
    return total_rows > 1 ? sum / (float)total_rows : sum;
}

// Entry checks.  Unless `keep_running`, the host also waits for everything the last step left running on the
// side lanes (parameter updates), so that whatever the caller reads or replaces next is final.
zn_status check_net(zn_net *n, bool need_layers, bool keep_running = false) {
    if (!n || !n->ctx) return ZN_ERR_NOT_INITIALIZED;
    if (need_layers && n->layers.empty()) return zn_fail(n->ctx, ZN_ERR_NOT_AVAILABLE, "network has no layers");
    cudaSetDevice(n->ctx->device);
    if (!keep_running) {
        bool pending = false;
        for (Layer &l : n->layers) pending = pending || l.update_pending;
        if (pending) {
            ZN_TRY(zn_sync_all_lanes(n->ctx));
            for (Layer &l : n->layers) l.update_pending = false;
        }
    }
    return ZN_OK;
}

zn_status ensure_slot(zn_net *n, Slot &s, size_t x_floats, size_t t_floats) {
    zn_ctx *ctx = n->ctx;
    if (!s.copied) {
        ZN_CUDA(ctx, cudaEventCreateWithFlags(&s.copied, cudaEventDisableTiming));
        ZN_CUDA(ctx, cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
        ZN_CUDA(ctx, cudaHostAlloc((void **)&s.loss_host, 4 * sizeof(float), cudaHostAllocDefault));
    }
    if (s.x_cap < x_floats) {
        ZN_TRY(zn_sync_all_lanes(ctx));
        cudaFree(s.x); s.x = nullptr; s.x_cap = 0;
        ZN_CUDA(ctx, cudaMalloc((void **)&s.x, x_floats * sizeof(float)));
        s.x_cap = x_floats;
    }
    if (s.t_cap < t_floats) {
        ZN_TRY(zn_sync_all_lanes(ctx));
        cudaFree(s.t); s.t = nullptr; s.t_cap = 0;
        ZN_CUDA(ctx, cudaMalloc((void **)&s.t, t_floats * sizeof(float)));
        s.t_cap = t_floats;
    }
    return ZN_OK;
}

uint64_t splitmix(uint64_t &s) {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

}   // namespace

extern "C" zn_status zn_net_create(zn_ctx *ctx, zn_precision precision, zn_net **out) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!out) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "net_create: null output");
    if (precision < ZN_FP32_SIMT || precision > ZN_BF16_TC) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "unknown precision");
    cudaSetDevice(ctx->device);
    zn_net *n = new zn_net();
    n->ctx = ctx;
    n->prec = precision;
    n->tc = precision == ZN_TF32_TC || precision == ZN_BF16_TC;
    n->bf16 = precision == ZN_BF16_TC;
    cudaError_t e = cudaMalloc((void **)&n->scalars, 16 * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc((void **)&n->sumsq, 64 * sizeof(double));
    if (e != cudaSuccess) { cudaFree(n->scalars); delete n; return zn_cuda_status(ctx, e, "cudaMalloc"); }
    cudaMemsetAsync(n->scalars, 0, 16 * sizeof(float), ctx->stream);
    cudaMemsetAsync(n->sumsq, 0, 64 * sizeof(double), ctx->stream);
    *out = n;
    return ZN_OK;
}

extern "C" void zn_net_destroy(zn_net *n) {
    if (!n) return;
    if (n->ctx) {
        cudaSetDevice(n->ctx->device);
        zn_sync_all_lanes(n->ctx);
        cudaStreamSynchronize(n->ctx->copy_stream);
    }
    free_acts(n);
    for (Layer &l : n->layers) {
        if (l.grads_nccl) zn_dp_free_registered(n->ctx, l.grads, l.grads_reg);
        else cudaFree(l.grads);
        if (l.params_nccl) zn_dp_free_registered(n->ctx, l.params, l.params_reg);
        else cudaFree(l.params);
        cudaFree(l.m); cudaFree(l.v); cudaFree(l.w_op);
        for (cudaEvent_t ev : {l.g_ready, l.bias_done, l.grads_ready, l.reduced, l.updated, l.stepped})
            if (ev) cudaEventDestroy(ev);
    }
    cudaFree(n->sumsq);
    if (n->norm_ready) cudaEventDestroy(n->norm_ready);
    for (Slot &s : n->slots) {
        cudaFree(s.x); cudaFree(s.t);
        if (s.copied) cudaEventDestroy(s.copied);
        if (s.done) cudaEventDestroy(s.done);
        if (s.loss_host) cudaFreeHost(s.loss_host);
    }
    cudaFree(n->scalars);
    delete n;
}

extern "C" zn_status zn_net_add_dense(zn_net *n, size_t input_size, size_t output_size, zn_activation act,
                                      int32_t *layer_index_out) {
    ZN_TRY(check_net(n, false));
    zn_ctx *ctx = n->ctx;
    if (input_size == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "InvalidInputSize: input_size is 0");     // src/layer.zig:307
    if (output_size == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "InvalidOutputSize: output_size is 0");  // src/layer.zig:308
    if (act < ZN_ACT_RELU || act > ZN_ACT_ELU) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "unknown activation %d", (int)act);
    if (!n->layers.empty() && n->layers.back().out != input_size)
        return zn_fail(ctx, ZN_ERR_SHAPE, "layer input %zu does not match previous output %zu", input_size, n->layers.back().out);
    if (n->inflight) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "steps in flight");
    if (n->shard_update) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "add every layer before zn_net_set_update_sharding");
    if (n->layers.size() >= 16) return zn_fail(ctx, ZN_ERR_UNSUPPORTED, "at most 16 Dense layers per network");
    Layer l;
    l.in = input_size; l.out = output_size; l.act = act;
    l.b_off = (size_t)round_up((int64_t)(input_size * output_size), 4);
    l.len = l.b_off + output_size;
    l.blk = (size_t)round_up((int64_t)l.len, 4);
    l.cap = l.blk + 4;
    const size_t alloc = l.cap * sizeof(float);
    ZN_CUDA(ctx, cudaMalloc((void **)&l.params, alloc));
    ZN_CUDA(ctx, cudaMalloc((void **)&l.grads, alloc));
    ZN_CUDA(ctx, cudaMemsetAsync(l.params, 0, alloc, ctx->stream));
    ZN_CUDA(ctx, cudaMemsetAsync(l.grads, 0, alloc, ctx->stream));
    for (cudaEvent_t *ev : {&l.g_ready, &l.bias_done, &l.grads_ready, &l.reduced, &l.updated, &l.stepped})
        ZN_CUDA(ctx, cudaEventCreateWithFlags(ev, cudaEventDisableTiming));
    if (n->tc) {
        const bool direct = !n->bf16 && output_size % 4 == 0;   // tf32 can read W itself when its pitch is TMA-legal
        if (!direct) {
            l.ld_w = round_up((int64_t)output_size, 8);
            const size_t bytes = input_size * (size_t)l.ld_w * esize(n);
            ZN_CUDA(ctx, cudaMalloc(&l.w_op, bytes));
            ZN_CUDA(ctx, cudaMemsetAsync(l.w_op, 0, bytes, ctx->stream));
        }
    }
    // Dense.init, src/layer.zig:326-339: U(-1,1) * scale(act), bias 0.  The generator is seeded by a
    // counter 1,2,3,... like the reference's, but is splitmix64, not Zig's PRNG.
    {
        const float scale = (act == ZN_ACT_RELU || act == ZN_ACT_LEAKY_RELU) ? sqrtf(2.0f / (float)input_size)
                            : (act == ZN_ACT_LINEAR) ? sqrtf(1.0f / (float)input_size)
                                                     : sqrtf(2.0f / (float)(input_size + output_size));
        uint64_t s = ++n->seed_counter;
        std::vector<float> w(input_size * output_size);
        for (float &x : w) {
            const float u = (float)(splitmix(s) >> 40) * (1.0f / 16777216.0f);   // [0,1)
            x = (u * 2.0f - 1.0f) * scale;
        }
        ZN_CUDA(ctx, cudaMemcpyAsync(l.params, w.data(), w.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
        ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    n->layers.push_back(l);
    ZN_TRY(refresh_operand_copy(n, n->layers.back()));
    if (n->cap_rows) { ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream)); free_acts(n); }
    if (layer_index_out) *layer_index_out = (int32_t)n->layers.size() - 1;
    return ZN_OK;
}

extern "C" zn_status zn_net_layer_count(const zn_net *n, size_t *out) {
    if (!n || !out) return ZN_ERR_INVALID_VALUE;
    *out = n->layers.size();
    return ZN_OK;
}

extern "C" zn_status zn_net_set_weights(zn_net *n, size_t layer, const float *weights, const float *bias) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (layer >= n->layers.size()) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "layer %zu out of range", layer);
    Layer &l = n->layers[layer];
    if (weights) ZN_CUDA(ctx, cudaMemcpyAsync(l.params, weights, l.in * l.out * sizeof(float), cudaMemcpyDefault, ctx->stream));
    if (bias) ZN_CUDA(ctx, cudaMemcpyAsync(l.params + l.b_off, bias, l.out * sizeof(float), cudaMemcpyDefault, ctx->stream));
    if (weights) ZN_TRY(refresh_operand_copy(n, l));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ZN_OK;
}

extern "C" zn_status zn_net_get_weights(zn_net *n, size_t layer, float *weights, float *bias) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    ZN_TRY(gather_stale_params(n));
    if (layer >= n->layers.size()) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "layer %zu out of range", layer);
    Layer &l = n->layers[layer];
    if (weights) ZN_CUDA(ctx, cudaMemcpyAsync(weights, l.params, l.in * l.out * sizeof(float), cudaMemcpyDefault, ctx->stream));
    if (bias) ZN_CUDA(ctx, cudaMemcpyAsync(bias, l.params + l.b_off, l.out * sizeof(float), cudaMemcpyDefault, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_net_get_grads(zn_net *n, size_t layer, float *gw, float *gb) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (layer >= n->layers.size()) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "layer %zu out of range", layer);
    Layer &l = n->layers[layer];
    if (n->shard_update && n->global_rows > 0 && zn_dp_active(ctx))
        return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "with the update sharded each rank holds the summed gradients of its own piece only");
    if (gw) ZN_CUDA(ctx, cudaMemcpyAsync(gw, l.grads, l.in * l.out * sizeof(float), cudaMemcpyDefault, ctx->stream));
    if (gb) ZN_CUDA(ctx, cudaMemcpyAsync(gb, l.grads + l.b_off, l.out * sizeof(float), cudaMemcpyDefault, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_net_get_input_grad(zn_net *n, float *grad_input, size_t count) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (!grad_input) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "null output");
    if (!n->last_input_grad) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "no training step has run");
    const size_t in = n->layers[0].in, rows = n->last_rows;
    if (count != rows * in) return zn_fail(ctx, ZN_ERR_SHAPE, "input gradient has %zu elements", rows * in);
    const int64_t ld = n->lds[0];
    std::vector<uint8_t> raw(rows * (size_t)ld * esize(n));
    ZN_CUDA(ctx, cudaMemcpyAsync(raw.data(), n->last_input_grad, raw.size(), cudaMemcpyDeviceToHost, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < in; ++c) {
            if (n->bf16) {
                const uint16_t h = reinterpret_cast<const uint16_t *>(raw.data())[r * ld + c];
                const uint32_t u = (uint32_t)h << 16;
                memcpy(&grad_input[r * in + c], &u, 4);
            } else {
                grad_input[r * in + c] = reinterpret_cast<const float *>(raw.data())[r * ld + c];
            }
        }
    return ZN_OK;
}

static zn_status for_layers(zn_net *n, int32_t layer, size_t *lo, size_t *hi) {
    if (layer < 0) { *lo = 0; *hi = n->layers.size(); return ZN_OK; }
    if ((size_t)layer >= n->layers.size()) return zn_fail(n->ctx, ZN_ERR_INVALID_VALUE, "layer %d out of range", layer);
    *lo = (size_t)layer; *hi = (size_t)layer + 1;
    return ZN_OK;
}

extern "C" zn_status zn_net_set_sgd(zn_net *n, int32_t layer, float weight_decay) {
    ZN_TRY(check_net(n, true));
    size_t lo, hi;
    ZN_TRY(for_layers(n, layer, &lo, &hi));
    for (size_t i = lo; i < hi; ++i) { n->layers[i].opt = OPT_SGD; n->layers[i].wd = weight_decay; }
    return ZN_OK;
}

// Optimizer state blocks have the shape of the parameter block; `two` asks for the second one (Adam's v).
static zn_status reset_state(zn_net *n, Layer &l, bool two) {
    zn_ctx *ctx = n->ctx;
    const size_t bytes = l.cap * sizeof(float);
    if (!l.m) ZN_CUDA(ctx, cudaMalloc((void **)&l.m, bytes));
    ZN_CUDA(ctx, cudaMemsetAsync(l.m, 0, bytes, ctx->stream));
    if (two) {
        if (!l.v) ZN_CUDA(ctx, cudaMalloc((void **)&l.v, bytes));
        ZN_CUDA(ctx, cudaMemsetAsync(l.v, 0, bytes, ctx->stream));
    }
    return ZN_OK;
}

static zn_status set_adam_kind(zn_net *n, int32_t layer, int kind, float beta1, float beta2, float eps, float weight_decay) {
    ZN_TRY(check_net(n, true));
    size_t lo, hi;
    ZN_TRY(for_layers(n, layer, &lo, &hi));
    for (size_t i = lo; i < hi; ++i) {
        Layer &l = n->layers[i];
        l.opt = kind; l.beta1 = beta1; l.beta2 = beta2; l.eps = eps; l.wd = weight_decay; l.t = 0;
        ZN_TRY(reset_state(n, l, true));
    }
    return ZN_OK;
}

extern "C" zn_status zn_net_set_adam(zn_net *n, int32_t layer, float beta1, float beta2, float eps, float weight_decay) {
    return set_adam_kind(n, layer, OPT_ADAM, beta1, beta2, eps, weight_decay);
}

extern "C" zn_status zn_net_set_adamw(zn_net *n, int32_t layer, float beta1, float beta2, float eps, float weight_decay) {
    return set_adam_kind(n, layer, OPT_ADAMW, beta1, beta2, eps, weight_decay);
}

extern "C" zn_status zn_net_set_sgd_momentum(zn_net *n, int32_t layer, float momentum) {
    ZN_TRY(check_net(n, true));
    size_t lo, hi;
    ZN_TRY(for_layers(n, layer, &lo, &hi));
    for (size_t i = lo; i < hi; ++i) {
        Layer &l = n->layers[i];
        l.opt = OPT_MOMENTUM; l.momentum = momentum; l.wd = 0.0f;
        ZN_TRY(reset_state(n, l, false));
    }
    return ZN_OK;
}

extern "C" zn_status zn_net_set_rmsprop(zn_net *n, int32_t layer, float rho, float eps, float weight_decay) {
    ZN_TRY(check_net(n, true));
    size_t lo, hi;
    ZN_TRY(for_layers(n, layer, &lo, &hi));
    for (size_t i = lo; i < hi; ++i) {
        Layer &l = n->layers[i];
        l.opt = OPT_RMSPROP; l.rho = rho; l.eps = eps; l.wd = weight_decay;
        ZN_TRY(reset_state(n, l, false));
    }
    return ZN_OK;
}

extern "C" zn_status zn_net_forward(zn_net *n, const float *input, size_t rows, float *output) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (!input || !output) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "forward: null operand");
    if (rows == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "forward: zero rows");
    ZN_TRY(same_device(n, input, "forward: input"));
    ZN_TRY(same_device(n, output, "forward: output"));
    const size_t in = n->layers[0].in, out = n->layers.back().out;
    const float *x_dev = input;
    if (!zn_is_device_ptr(input)) {
        ZN_TRY(ensure_slot(n, n->slots[0], rows * in, 1));
        ZN_CUDA(ctx, cudaMemcpyAsync(n->slots[0].x, input, rows * in * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
        x_dev = n->slots[0].x;
    }
    ZN_TRY(forward_dev(n, x_dev, rows));
    ZN_CUDA(ctx, cudaMemcpyAsync(output, final_output(n), rows * out * sizeof(float), cudaMemcpyDefault, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_net_evaluate_classification(zn_net *n, const float *input, const float *target, size_t rows,
                                                    size_t num_classes, uint64_t *confusion, float *metrics4) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (rows == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "EmptyInput: no samples to evaluate");
    if (!input || !target) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "evaluate_classification: null operand");
    if (n->inflight) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "pipelined steps in flight; wait for them first");
    ZN_TRY(same_device(n, input, "evaluate_classification: input"));
    ZN_TRY(same_device(n, target, "evaluate_classification: target"));
    const size_t in = n->layers[0].in, out = n->layers.back().out;
    Slot &s = n->slots[0];
    ZN_TRY(ensure_slot(n, s, rows * in, rows * out));
    const float *x_dev = input, *t_dev = target;
    if (!zn_is_device_ptr(input)) {
        ZN_CUDA(ctx, cudaMemcpyAsync(s.x, input, rows * in * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
        x_dev = s.x;
    }
    if (!zn_is_device_ptr(target)) {
        ZN_CUDA(ctx, cudaMemcpyAsync(s.t, target, rows * out * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
        t_dev = s.t;
    }
    ZN_TRY(forward_dev(n, x_dev, rows));
    const int64_t ld_o = n->tc ? (int64_t)out : n->lds[n->layers.size()];
    return zn_k_classification_metrics(ctx, final_output(n), ld_o, t_dev, (int64_t)out, rows, out, num_classes, confusion, metrics4);
}

extern "C" zn_status zn_net_train_step(zn_net *n, const float *input, const float *target, size_t rows, float lr,
                                       zn_loss loss, float *loss_out) {
    ZN_TRY(check_net(n, true, true));
    zn_ctx *ctx = n->ctx;
    if (!input || !target) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "train_step: null operand");
    if (rows == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "train_step: zero rows");
    ZN_TRY(same_device(n, input, "train_step: input"));
    ZN_TRY(same_device(n, target, "train_step: target"));
    if (!loss_supported(loss)) return zn_fail(ctx, ZN_ERR_UNSUPPORTED, "loss %d is not on the Dense path", (int)loss);
    if (n->inflight) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "pipelined steps in flight; wait for them first");
    const size_t in = n->layers[0].in, out = n->layers.back().out;
    Slot &s = n->slots[0];
    ZN_TRY(ensure_slot(n, s, rows * in, rows * out));
    const float *x_dev = input, *t_dev = target;
    if (!zn_is_device_ptr(input)) {
        ZN_CUDA(ctx, cudaMemcpyAsync(s.x, input, rows * in * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
        x_dev = s.x;
    }
    if (!zn_is_device_ptr(target)) {
        ZN_CUDA(ctx, cudaMemcpyAsync(s.t, target, rows * out * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
        t_dev = s.t;
    }
    ZN_TRY(step_dev(n, x_dev, t_dev, rows, lr, (int)loss, s.loss_host, s.done));
    // The loss and the norm are final once every layer is reduced; the parameter updates keep running on
    // the optimizer lane and the next step (or any getter) orders itself after them.
    ZN_TRY(zn_wait_event(ctx, s.done));
    n->last_norm = s.loss_host[1];
    n->last_factor = s.loss_host[2];
    if (loss_out) *loss_out = loss_from_sum(n, s.loss_host[0], rows, (int)loss);
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_net_submit_step(zn_net *n, const float *host_input, const float *host_target, size_t rows,
                                        float lr, zn_loss loss) {
    ZN_TRY(check_net(n, true, true));
    zn_ctx *ctx = n->ctx;
    if (!host_input || !host_target) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "submit_step: null operand");
    if (rows == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "submit_step: zero rows");
    if (!loss_supported(loss)) return zn_fail(ctx, ZN_ERR_UNSUPPORTED, "loss %d is not on the Dense path", (int)loss);
    if (n->inflight >= 2) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "two steps already in flight");
    const size_t in = n->layers[0].in, out = n->layers.back().out;
    const int idx = (n->head + n->inflight) & 1;
    Slot &s = n->slots[idx];
    ZN_TRY(ensure_slot(n, s, rows * in, rows * out));
    ZN_TRY(ensure_rows(n, rows));
    // The slot's previous step (two submits ago) has been waited for, so its buffers are free:
    // copy on the copy stream while the other slot's step computes.
    ZN_CUDA(ctx, cudaMemcpyAsync(s.x, host_input, rows * in * sizeof(float), cudaMemcpyHostToDevice, ctx->copy_stream));
    ZN_CUDA(ctx, cudaMemcpyAsync(s.t, host_target, rows * out * sizeof(float), cudaMemcpyHostToDevice, ctx->copy_stream));
    ZN_CUDA(ctx, cudaEventRecord(s.copied, ctx->copy_stream));
    ZN_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, s.copied, 0));
    ZN_TRY(step_dev(n, s.x, s.t, rows, lr, (int)loss, s.loss_host, s.done));
    s.rows = rows; s.loss = (int)loss; s.busy = true;
    n->inflight += 1;
    return ZN_OK;
}

extern "C" zn_status zn_net_wait_step(zn_net *n, float *loss_out) {
    ZN_TRY(check_net(n, true, true));
    zn_ctx *ctx = n->ctx;
    if (n->inflight == 0) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "no step in flight");
    Slot &s = n->slots[n->head];
    ZN_TRY(zn_wait_event(ctx, s.done));
    s.busy = false;
    n->head ^= 1;
    n->inflight -= 1;
    n->last_norm = s.loss_host[1];
    n->last_factor = s.loss_host[2];
    if (loss_out) *loss_out = loss_from_sum(n, s.loss_host[0], s.rows, s.loss);
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_net_train(zn_net *n, const float *inputs, const float *targets, size_t samples, size_t epochs,
                                  float lr, zn_loss loss, float *epoch_loss) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (!inputs || !targets) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "train: null operand");
    if (samples == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "train: no samples");
    if (!loss_supported(loss)) return zn_fail(ctx, ZN_ERR_UNSUPPORTED, "loss %d is not on the Dense path", (int)loss);
    if (n->inflight) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "pipelined steps in flight");
    const size_t in = n->layers[0].in, out = n->layers.back().out;
    Slot &s = n->slots[0];
    ZN_TRY(ensure_slot(n, s, samples * in, samples * out));
    ZN_CUDA(ctx, cudaMemcpyAsync(s.x, inputs, samples * in * sizeof(float), cudaMemcpyDefault, ctx->stream));
    ZN_CUDA(ctx, cudaMemcpyAsync(s.t, targets, samples * out * sizeof(float), cudaMemcpyDefault, ctx->stream));
    float *losses_dev = nullptr;
    ZN_CUDA(ctx, cudaMalloc((void **)&losses_dev, samples * sizeof(float)));
    std::vector<float> losses(samples);
    zn_status st = ZN_OK;
    for (size_t e = 0; e < epochs && st == ZN_OK; ++e) {
        // one trainStep per sample, in order (src/network.zig:613-614)
        for (size_t i = 0; i < samples && st == ZN_OK; ++i) {
            st = step_dev(n, s.x + i * in, s.t + i * out, 1, lr, (int)loss, losses_dev + i, nullptr);
        }
        if (st != ZN_OK) break;
        if (zn_sync_all_lanes(ctx) != ZN_OK ||
            cudaMemcpyAsync(losses.data(), losses_dev, samples * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess ||
            cudaStreamSynchronize(ctx->stream) != cudaSuccess) { st = zn_fail(ctx, ZN_ERR_CUDA, "loss read-back failed"); break; }
        float total = 0.f;
        for (size_t i = 0; i < samples; ++i) total += loss_from_sum(n, losses[i], 1, (int)loss);
        if (epoch_loss) epoch_loss[e] = total / (float)samples;   // src/network.zig:615
    }
    zn_sync_all_lanes(ctx);
    cudaFree(losses_dev);
    if (st != ZN_OK) return st;
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_net_last_clip(zn_net *n, float *norm_out, float *factor_out) {
    if (!n) return ZN_ERR_NOT_INITIALIZED;
    if (norm_out) *norm_out = n->last_norm;
    if (factor_out) *factor_out = n->last_factor;
    return ZN_OK;
}

// ---- .znn files: Network.save / Network.load (src/network.zig:692-745) -> saveModel / loadModel
// (src/serialization.zig:78-147).  Little-endian: "ZNN\0", u32 version = 1, u32 layer count; per Dense layer
// u32 type = 1, u32 input size, u32 output size, u32 activation tag, f32 weights[in*out], f32 bias[out]
// (writeLayer, :165-183).  As in the reference, optimizer state is not part of the file.
namespace {
constexpr uint32_t ZNN_VERSION = 1, ZNN_LAYER_DENSE = 1;
bool put_u32(FILE *f, uint32_t v) { return fwrite(&v, 4, 1, f) == 1; }
bool get_u32(FILE *f, uint32_t *v) { return fread(v, 4, 1, f) == 1; }
}   // namespace

extern "C" zn_status zn_net_save(zn_net *n, const char *path) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    ZN_TRY(gather_stale_params(n));
    if (!path) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "save: null path");
    FILE *f = fopen(path, "wb");
    if (!f) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "save: cannot create %s", path);
    bool ok = fwrite("ZNN\0", 1, 4, f) == 4 && put_u32(f, ZNN_VERSION) && put_u32(f, (uint32_t)n->layers.size());
    std::vector<float> host;
    for (size_t i = 0; i < n->layers.size() && ok; ++i) {
        Layer &l = n->layers[i];
        if (l.in > UINT32_MAX || l.out > UINT32_MAX) { ok = false; break; }
        host.resize(l.len);
        if (cudaMemcpyAsync(host.data(), l.params, l.len * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess ||
            cudaStreamSynchronize(ctx->stream) != cudaSuccess) { ok = false; break; }
        ok = put_u32(f, ZNN_LAYER_DENSE) && put_u32(f, (uint32_t)l.in) && put_u32(f, (uint32_t)l.out) && put_u32(f, (uint32_t)l.act) &&
             fwrite(host.data(), sizeof(float), l.in * l.out, f) == l.in * l.out &&
             fwrite(host.data() + l.b_off, sizeof(float), l.out, f) == l.out;
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) return zn_fail(ctx, ZN_ERR_CUDA, "save: writing %s failed", path);
    return ZN_OK;
}

extern "C" zn_status zn_net_load(zn_ctx *ctx, zn_precision precision, const char *path, zn_net **out) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!path || !out) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "load: null argument");
    *out = nullptr;
    FILE *f = fopen(path, "rb");
    if (!f) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "load: cannot open %s", path);
    char magic[4];
    uint32_t version = 0, count = 0;
    zn_status st = ZN_OK;
    zn_net *n = nullptr;
    if (fread(magic, 1, 4, f) != 4 || memcmp(magic, "ZNN\0", 4) != 0) st = zn_fail(ctx, ZN_ERR_INVALID_VALUE, "InvalidMagic: %s is not a .znn file", path);
    else if (!get_u32(f, &version) || version != ZNN_VERSION) st = zn_fail(ctx, ZN_ERR_UNSUPPORTED, "UnsupportedVersion %u", version);
    else if (!get_u32(f, &count) || count == 0 || count > 16) st = zn_fail(ctx, ZN_ERR_UNSUPPORTED, "layer count %u outside 1..16", count);
    if (st == ZN_OK) st = zn_net_create(ctx, precision, &n);
    std::vector<float> w, b;
    for (uint32_t i = 0; i < count && st == ZN_OK; ++i) {
        uint32_t type = 0, in = 0, o = 0, act = 0;
        if (!get_u32(f, &type) || !get_u32(f, &in) || !get_u32(f, &o) || !get_u32(f, &act)) { st = zn_fail(ctx, ZN_ERR_INVALID_VALUE, "load: truncated layer header"); break; }
        if (type != ZNN_LAYER_DENSE) { st = zn_fail(ctx, ZN_ERR_UNSUPPORTED, "layer type %u is not Dense", type); break; }
        if (in == 0 || o == 0 || (uint64_t)in * o > (1ull << 32)) { st = zn_fail(ctx, ZN_ERR_SHAPE, "load: layer %u has size %u x %u", i, in, o); break; }
        w.resize((size_t)in * o);
        b.resize(o);
        if (fread(w.data(), sizeof(float), w.size(), f) != w.size() || fread(b.data(), sizeof(float), o, f) != o) { st = zn_fail(ctx, ZN_ERR_INVALID_VALUE, "load: truncated layer data"); break; }
        st = zn_net_add_dense(n, in, o, (zn_activation)act, nullptr);
        if (st == ZN_OK) st = zn_net_set_weights(n, i, w.data(), b.data());
    }
    fclose(f);
    if (st != ZN_OK) { zn_net_destroy(n); return st; }
    *out = n;
    return ZN_OK;
}

namespace {

// Moves one parameter-shaped block into an allocation of `floats` floats (zero-filled beyond what is copied).
// `from_nccl`: try memory NCCL allocates and registers first.  The old block is released by its own kind.
zn_status regrow_block(zn_net *n, float **blk, bool *is_nccl, void **reg, size_t old_floats, size_t floats, bool from_nccl, bool keep) {
    zn_ctx *ctx = n->ctx;
    void *p = nullptr, *h = nullptr;
    bool nccl = false;
    if (from_nccl && zn_dp_alloc_registered(ctx, floats * sizeof(float), &p, &h) == ZN_OK) nccl = true;
    else ZN_CUDA(ctx, cudaMalloc(&p, floats * sizeof(float)));
    ZN_CUDA(ctx, cudaMemsetAsync(p, 0, floats * sizeof(float), ctx->stream));
    if (keep && *blk)
        ZN_CUDA(ctx, cudaMemcpyAsync(p, *blk, (old_floats < floats ? old_floats : floats) * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*blk) {
        if (is_nccl && *is_nccl) zn_dp_free_registered(ctx, *blk, reg ? *reg : nullptr);
        else cudaFree(*blk);
    }
    *blk = (float *)p;
    if (is_nccl) *is_nccl = nccl;
    if (reg) *reg = h;
    return ZN_OK;
}

}   // namespace

// Data parallel with the update split over the ranks: per layer a reduce-scatter instead of the all-reduce, each
// rank squares and updates only its own 1/world piece of the block, one exchange of L + 1 doubles carries the
// global sums of squares and the loss, and an all-gather of the updated fp32 weights replaces the second half of
// the all-reduce.  The bytes on NVLink are the same; the update's pass over the parameters and both optimizer
// states, which does not shrink with the batch, is divided by the number of ranks.  Same results up to the order
// in which NCCL adds the ranks' gradients.
extern "C" zn_status zn_net_set_update_sharding(zn_net *n, int32_t on) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (!on) {
        ZN_TRY(gather_stale_params(n));
        n->shard_update = false;
        return ZN_OK;
    }
    if (n->global_rows == 0 || !zn_dp_active(ctx)) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "call zn_net_set_data_parallel first");
    if (!zn_dp_can_shard(ctx)) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "this NCCL has no reduce-scatter / all-gather");
    if (n->prec == ZN_FP32_EXACT) return zn_fail(ctx, ZN_ERR_UNSUPPORTED, "FP32_EXACT sums every gradient in the reference's order on one rank; it cannot be sharded");
    if (n->inflight) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "steps in flight");
    const size_t world = (size_t)zn_dp_world(ctx);
    if (!n->norm_ready) ZN_CUDA(ctx, cudaEventCreateWithFlags(&n->norm_ready, cudaEventDisableTiming));
    for (Layer &l : n->layers) {
        l.shard = (size_t)round_up((int64_t)((l.blk + world - 1) / world), 4);
        const size_t need = world * l.shard + 4;
        if (need <= l.cap && l.params_nccl) continue;
        const size_t cap = need > l.cap ? need : l.cap;
        ZN_TRY(regrow_block(n, &l.params, &l.params_nccl, &l.params_reg, l.cap, cap, true, true));
        ZN_TRY(regrow_block(n, &l.grads, &l.grads_nccl, &l.grads_reg, l.cap, cap, true, false));
        if (l.m) ZN_TRY(regrow_block(n, &l.m, nullptr, nullptr, l.cap, cap, false, true));
        if (l.v) ZN_TRY(regrow_block(n, &l.v, nullptr, nullptr, l.cap, cap, false, true));
        l.cap = cap;
    }
    // The ranks exchange the updated fp32 weights.  With ZN_DP_GATHER_BF16=1 in the environment, bf16 networks whose
    // operand copy of W has W's own flat layout hand that copy over instead (half the bytes; the copy then needs
    // room for world * shard values): measured level with the fp32 form on 2 and 4 GPUs (15.13-15.16 against
    // 15.13 ms per 8192-wide step on 4) and not measured on 8, so it stays an option.
    static const bool fp32_gather = [] { const char *e = getenv("ZN_DP_GATHER_BF16"); return !(e && atoi(e) != 0); }();
    for (Layer &l : n->layers) {
        l.gather_bf16 = false;
        if (fp32_gather || !n->bf16 || !l.w_op || l.ld_w != (int64_t)l.out || !zn_dp_can_gather_bf16(ctx)) continue;
        const size_t elems = world * l.shard > l.in * l.out ? world * l.shard : l.in * l.out;
        void *grown = nullptr;
        ZN_CUDA(ctx, cudaMalloc(&grown, elems * sizeof(__nv_bfloat16)));
        ZN_CUDA(ctx, cudaMemsetAsync(grown, 0, elems * sizeof(__nv_bfloat16), ctx->stream));
        ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(l.w_op);
        l.w_op = grown;
        ZN_TRY(refresh_operand_copy(n, l));
        l.gather_bf16 = true;
    }
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    n->shard_update = true;
    return ZN_OK;
}

// Optimizer state beside a .znn file.  The reference's format holds weights and biases only
// (src/serialization.zig:165-183), so a run resumed from it restarts Adam's moments and step count; this
// second file carries what Optimizer keeps per layer (src/optimizer.zig:81-88, :169-184, :236-250, :311-320):
//   "ZNO\0", u32 version = 1, u32 layer count, then per layer
//   u32 kind (0 sgd, 1 adam, 2 momentum sgd, 3 adamw, 4 rmsprop), u32 input size, u32 output size, u64 t,
//   f32 beta1, beta2, eps, weight_decay, momentum, rho, u32 state tensors S (0, 1 or 2),
//   S x { f32 [in*out] weight-shaped part, f32 [out] bias-shaped part }     (m then v; velocity; g_avg)
namespace {
constexpr uint32_t ZNO_VERSION = 1;
int state_tensors(int opt) { return opt == OPT_SGD ? 0 : (opt == OPT_ADAM || opt == OPT_ADAMW) ? 2 : 1; }
}   // namespace

extern "C" zn_status zn_net_save_optimizer(zn_net *n, const char *path) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (!path) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "save_optimizer: null path");
    if (n->shard_update && n->global_rows > 0 && zn_dp_active(ctx))
        return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "with the update sharded each rank holds the optimizer state of its own piece only");
    FILE *f = fopen(path, "wb");
    if (!f) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "save_optimizer: cannot open %s", path);
    bool ok = fwrite("ZNO\0", 1, 4, f) == 4 && put_u32(f, ZNO_VERSION) && put_u32(f, (uint32_t)n->layers.size());
    std::vector<float> host;
    for (size_t i = 0; i < n->layers.size() && ok; ++i) {
        const Layer &l = n->layers[i];
        const uint64_t t = l.t;
        const float hp[6] = {l.beta1, l.beta2, l.eps, l.wd, l.momentum, l.rho};
        const int S = state_tensors(l.opt);
        ok = put_u32(f, (uint32_t)l.opt) && put_u32(f, (uint32_t)l.in) && put_u32(f, (uint32_t)l.out) &&
             fwrite(&t, 8, 1, f) == 1 && fwrite(hp, 4, 6, f) == 6 && put_u32(f, (uint32_t)S);
        for (int k = 0; k < S && ok; ++k) {
            const float *src = k == 0 ? l.m : l.v;
            host.resize(l.len);
            if (!src || cudaMemcpyAsync(host.data(), src, l.len * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess ||
                cudaStreamSynchronize(ctx->stream) != cudaSuccess) { ok = false; break; }
            ok = fwrite(host.data(), sizeof(float), l.in * l.out, f) == l.in * l.out &&
                 fwrite(host.data() + l.b_off, sizeof(float), l.out, f) == l.out;
        }
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) return zn_fail(ctx, ZN_ERR_CUDA, "save_optimizer: writing %s failed", path);
    return ZN_OK;
}

extern "C" zn_status zn_net_load_optimizer(zn_net *n, const char *path) {
    ZN_TRY(check_net(n, true));
    zn_ctx *ctx = n->ctx;
    if (!path) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "load_optimizer: null path");
    FILE *f = fopen(path, "rb");
    if (!f) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "load_optimizer: cannot open %s", path);
    char magic[4];
    uint32_t version = 0, count = 0;
    zn_status st = ZN_OK;
    if (fread(magic, 1, 4, f) != 4 || memcmp(magic, "ZNO\0", 4) != 0) st = zn_fail(ctx, ZN_ERR_INVALID_VALUE, "InvalidMagic: %s is not an optimizer-state file", path);
    else if (!get_u32(f, &version) || version != ZNO_VERSION) st = zn_fail(ctx, ZN_ERR_UNSUPPORTED, "UnsupportedVersion %u", version);
    else if (!get_u32(f, &count) || count != n->layers.size()) st = zn_fail(ctx, ZN_ERR_SHAPE, "load_optimizer: file has %u layers, the network %zu", count, n->layers.size());
    std::vector<float> host;
    for (uint32_t i = 0; i < count && st == ZN_OK; ++i) {
        Layer &l = n->layers[i];
        uint32_t kind = 0, in = 0, o = 0, S = 0;
        uint64_t t = 0;
        float hp[6];
        if (!get_u32(f, &kind) || !get_u32(f, &in) || !get_u32(f, &o) || fread(&t, 8, 1, f) != 1 || fread(hp, 4, 6, f) != 6 || !get_u32(f, &S)) {
            st = zn_fail(ctx, ZN_ERR_INVALID_VALUE, "load_optimizer: truncated layer header"); break;
        }
        if (kind > OPT_RMSPROP || (int)S != state_tensors((int)kind)) { st = zn_fail(ctx, ZN_ERR_INVALID_VALUE, "load_optimizer: layer %u has kind %u with %u state tensors", i, kind, S); break; }
        if (in != l.in || o != l.out) { st = zn_fail(ctx, ZN_ERR_SHAPE, "load_optimizer: layer %u is %u x %u in the file, %zu x %zu in the network", i, in, o, l.in, l.out); break; }
        l.opt = (int)kind; l.t = (size_t)t;
        l.beta1 = hp[0]; l.beta2 = hp[1]; l.eps = hp[2]; l.wd = hp[3]; l.momentum = hp[4]; l.rho = hp[5];
        if (S > 0) st = reset_state(n, l, S == 2);
        for (uint32_t k = 0; k < S && st == ZN_OK; ++k) {
            host.assign(l.cap, 0.0f);
            if (fread(host.data(), sizeof(float), l.in * l.out, f) != l.in * l.out || fread(host.data() + l.b_off, sizeof(float), l.out, f) != l.out) {
                st = zn_fail(ctx, ZN_ERR_INVALID_VALUE, "load_optimizer: truncated state of layer %u", i); break;
            }
            float *dst = k == 0 ? l.m : l.v;
            if (cudaMemcpyAsync(dst, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
                cudaStreamSynchronize(ctx->stream) != cudaSuccess) st = zn_fail(ctx, ZN_ERR_CUDA, "load_optimizer: upload failed");
        }
    }
    fclose(f);
    return st;
}

extern "C" zn_status zn_net_set_data_parallel(zn_net *n, size_t global_rows) {
    ZN_TRY(check_net(n, true));
    if (global_rows > 0 && !zn_dp_active(n->ctx))
        return zn_fail(n->ctx, ZN_ERR_NOT_AVAILABLE, "call zn_dp_init on the context first");
    n->global_rows = global_rows;
    if (global_rows > 0) {
        // Move the gradient blocks into memory NCCL allocates and registers, so that the per-layer all-reduce
        // works on them in place.  Every rank does this in the same order; without the interface the blocks stay.
        zn_ctx *ctx = n->ctx;
        for (Layer &l : n->layers) {
            if (l.grads_nccl) continue;
            const size_t bytes = l.cap * sizeof(float);
            void *p = nullptr, *h = nullptr;
            if (zn_dp_alloc_registered(ctx, bytes, &p, &h) != ZN_OK) break;
            ZN_CUDA(ctx, cudaMemsetAsync(p, 0, bytes, ctx->stream));
            ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(l.grads);
            l.grads = (float *)p;
            l.grads_reg = h;
            l.grads_nccl = true;
        }
    }
    return ZN_OK;
}
