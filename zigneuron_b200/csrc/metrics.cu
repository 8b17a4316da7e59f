// Classification metrics of a block of outputs on the device: metrics.evaluateClassification
// (src/metrics.zig:239-264) = getPredictedClass / getTrueClass per sample (:213-235), the confusion
// matrix and the macro-averaged figures of computeClassificationMetrics (:85-163).
//
// The per-sample class indices and the confusion matrix are integer work done on the GPU (one warp per
// sample, counters in shared memory when the matrix is small); only classes^2 counters come back to
// the host, where the four ratios are formed in f32 in the reference's order.
#include "zn_internal.h"

namespace {

constexpr int TPB = 256;
constexpr int LOCAL_CLASSES = 32;          // up to 32 x 32 counters per block in shared memory
constexpr long long NONE = 0x7fffffffffffffffLL;

__global__ void confusion_kernel(const float *__restrict__ out, int64_t ld_o, const float *__restrict__ tgt, int64_t ld_t,
                                 int64_t rows, int64_t cols, int classes, unsigned long long *__restrict__ cm,
                                 int *__restrict__ invalid) {
    __shared__ unsigned int local[LOCAL_CLASSES * LOCAL_CLASSES];
    const bool use_local = classes <= LOCAL_CLASSES;
    if (use_local) {
        for (int i = threadIdx.x; i < classes * classes; i += blockDim.x) local[i] = 0u;
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const float *o = out + r * ld_o, *t = tgt + r * ld_t;
        // getPredictedClass keeps the first maximum (it replaces only on a strict >).  A NaN never wins a
        // comparison, so: class 0 when output[0] is NaN, else the lowest index of the largest non-NaN value.
        float bv = -INFINITY;
        long long bi = NONE;
        for (int64_t c = lane; c < cols; c += 32) {
            const float v = o[c];
            if (!isnan(v) && (bi == NONE || v > bv)) { bv = v; bi = c; }
        }
        // getTrueClass: the first target above 0.5, else class 0
        long long ti = NONE;
        for (int64_t c = lane; c < cols; c += 32)
            if (t[c] > 0.5f) { ti = c; break; }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const long long oi = __shfl_xor_sync(0xffffffffu, bi, off);
            const long long ot = __shfl_xor_sync(0xffffffffu, ti, off);
            if (oi != NONE && (bi == NONE || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
            if (ot < ti) ti = ot;
        }
        if (lane == 0) {
            const long long pred = (isnan(o[0]) || bi == NONE) ? 0 : bi;
            const long long truth = ti == NONE ? 0 : ti;
            if (pred >= classes || truth >= classes) atomicExch(invalid, 1);          // error.InvalidClass
            else if (use_local) atomicAdd(&local[truth * classes + pred], 1u);
            else atomicAdd(&cm[truth * classes + pred], 1ull);
        }
    }
    if (use_local) {
        __syncthreads();
        for (int i = threadIdx.x; i < classes * classes; i += blockDim.x)
            if (local[i]) atomicAdd(&cm[i], (unsigned long long)local[i]);
    }
}

}   // namespace

// outputs / targets: fp32 device blocks of `rows` samples with pitches ld_o / ld_t.  confusion
// (num_classes^2 counters, [target][predicted]) and metrics4 (accuracy, macro precision, macro recall, F1)
// are host memory.  Synchronizes the current stream.
zn_status zn_k_classification_metrics(zn_ctx *ctx, const float *out_dev, int64_t ld_o, const float *tgt_dev, int64_t ld_t,
                                      size_t rows, size_t cols, size_t num_classes, uint64_t *confusion, float *metrics4) {
    if (rows == 0) return zn_fail(ctx, ZN_ERR_SHAPE, "EmptyInput: no samples to evaluate");               // src/metrics.zig:92
    if (num_classes == 0 || num_classes > 4096)
        return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "evaluate: num_classes %zu outside 1..4096", num_classes);
    const size_t cells = num_classes * num_classes;
    ZN_TRY(zn_scratch_reserve(ctx, cells * 2 + 2));
    unsigned long long *cm_dev = reinterpret_cast<unsigned long long *>(ctx->scratch);
    int *flag_dev = reinterpret_cast<int *>(cm_dev + cells);
    ZN_CUDA(ctx, cudaMemsetAsync(cm_dev, 0, cells * 8 + 8, ctx->stream));
    {
        zn_launch_scope scope(ctx, ZN_PROF_ELEMENTWISE, 0, 8.0 * rows * cols);
        int64_t blocks = ((int64_t)rows + TPB / 32 - 1) / (TPB / 32);
        const int64_t cap = (int64_t)ctx->sm_count * 8;
        if (blocks > cap) blocks = cap;
        confusion_kernel<<<(int)blocks, TPB, 0, ctx->stream>>>(out_dev, ld_o, tgt_dev, ld_t, (int64_t)rows, (int64_t)cols,
                                                                (int)num_classes, cm_dev, flag_dev);
        ZN_CUDA(ctx, cudaGetLastError());
    }
    std::vector<unsigned long long> cm(cells + 1);
    ZN_CUDA(ctx, cudaMemcpyAsync(cm.data(), cm_dev, cells * 8 + 8, cudaMemcpyDeviceToHost, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ZN_TRY(zn_check_device_status(ctx));
    if ((int)(cm[cells] & 0xffffffffull) != 0)
        return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "InvalidClass: a predicted or true class is >= num_classes %zu", num_classes);   // :105-110
    if (confusion)
        for (size_t i = 0; i < cells; ++i) confusion[i] = (uint64_t)cm[i];
    if (metrics4) {      // src/metrics.zig:114-160
        const size_t C = num_classes;
        size_t correct = 0;
        float total_precision = 0.f, total_recall = 0.f;
        for (size_t c = 0; c < C; ++c) {
            const size_t tp = (size_t)cm[c * C + c];
            size_t fp = 0, fn = 0;
            for (size_t i = 0; i < C; ++i)
                if (i != c) { fp += (size_t)cm[i * C + c]; fn += (size_t)cm[c * C + i]; }
            correct += tp;
            total_precision += (tp + fp > 0) ? (float)tp / (float)(tp + fp) : 0.0f;
            total_recall += (tp + fn > 0) ? (float)tp / (float)(tp + fn) : 0.0f;
        }
        const float precision = total_precision / (float)C, recall = total_recall / (float)C;
        metrics4[0] = (float)correct / (float)rows;
        metrics4[1] = precision;
        metrics4[2] = recall;
        metrics4[3] = (precision + recall > 0) ? 2.0f * precision * recall / (precision + recall) : 0.0f;
    }
    return ZN_OK;
}
