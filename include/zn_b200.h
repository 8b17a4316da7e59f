/*
 * zn_b200.h -- C ABI of libzn_b200.so: ZigNeuron's Dense-layer training path on
 * NVIDIA B200 (sm_100a).
 *
 * The library slots in below ZigNeuron's `Backend` (src/backend.zig): every
 * entry point names the reference function whose CUDA arm it provides.  The
 * interface is plain C: opaque handles, float pointers and sizes.  Slices
 * (`[]f32`) of the reference become `pointer, element count` or explicit
 * dimensions.
 *
 * Pointers: every `float*` argument of an op may be either a HOST pointer or a
 * DEVICE pointer obtained from zn_tensor_alloc().  A host pointer reproduces
 * the call shape of the reference (operands are copied in, the result copied
 * out, the call returns when the result is in host memory).  A device pointer
 * fills the role of the reference's `?*const metal.MTLBuffer` handle slot next
 * to each slice: the operand stays resident and the call only enqueues work
 * on the context's stream.
 *
 * Threading: like the reference's Backend ("NOT thread-safe, use separate
 * instances per thread", src/backend.zig:103-104) a zn_ctx and the objects
 * made from it belong to one thread at a time.
 *
 * Errors: every function returns a zn_status, never aborts or traps.
 * zn_last_error_string() gives the detail of the last failure on a context.
 *
 * There is no CPU path in this library: without a CUDA device every compute
 * entry point fails with ZN_ERR_NO_DEVICE.
 */
#ifndef ZN_B200_H
#define ZN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZN_API __attribute__((visibility("default")))

typedef int32_t zn_status;

/* Mirrors the reference's CudaError set (src/cuda_driver.zig:1119-1142) plus
 * the shape errors of src/layer.zig:307-308,382 and src/network.zig:491. */
enum {
    ZN_OK = 0,
    ZN_ERR_INVALID_VALUE = 1,      /* CudaInvalidValue / null or misaligned argument     */
    ZN_ERR_OUT_OF_MEMORY = 2,      /* CudaOutOfMemory                                    */
    ZN_ERR_NOT_INITIALIZED = 3,    /* CudaNotInitialized / ContextNotInitialized         */
    ZN_ERR_NO_DEVICE = 4,          /* CudaNoDevice / CudaDriverNotFound                  */
    ZN_ERR_INVALID_DEVICE = 5,     /* CudaInvalidDevice                                  */
    ZN_ERR_CUDA = 6,               /* CudaUnknownError: any other CUDA runtime failure   */
    ZN_ERR_SHAPE = 7,              /* InvalidInputSize / InvalidOutputSize / ShapeMismatch / OutputSizeMismatch */
    ZN_ERR_UNSUPPORTED = 8,        /* activation, loss or optimizer outside the Dense path */
    ZN_ERR_TIMEOUT = 9,            /* a bounded device-side wait gave up; context still usable */
    ZN_ERR_NCCL = 10,              /* NCCL missing or a collective failed                */
    ZN_ERR_NOT_AVAILABLE = 11      /* error.NotAvailable: object not in the needed state */
};

/* How the three GEMMs compute.  The API is f32 at the boundary in every mode. */
typedef enum {
    ZN_FP32_SIMT = 0,   /* fp32 FMA on CUDA cores, k summed in ascending order per element */
    ZN_FP32_EXACT = 1,  /* as above with a separate multiply and add: the reference's arithmetic */
    ZN_TF32_TC = 2,     /* tcgen05 kind::tf32, fp32 operands, fp32 accumulation in TMEM */
    ZN_BF16_TC = 3      /* tcgen05 kind::f16 on bf16 operands, fp32 accumulation, fp32 master weights */
} zn_precision;

/* Same order as `Activation` in src/activation.zig:14-22. */
typedef enum {
    ZN_ACT_RELU = 0, ZN_ACT_SIGMOID = 1, ZN_ACT_TANH = 2, ZN_ACT_SOFTMAX = 3,
    ZN_ACT_LINEAR = 4, ZN_ACT_GELU = 5, ZN_ACT_LEAKY_RELU = 6, ZN_ACT_ELU = 7
} zn_activation;

/* Same order as `Loss` in src/loss.zig:12-22.  All but KL_DIVERGENCE are taken (that one splits a single
 * output vector into [mu | log_var], src/loss.zig:62-92, and has no batched form): ZN_ERR_UNSUPPORTED. */
typedef enum {
    ZN_LOSS_MSE = 0, ZN_LOSS_CROSS_ENTROPY = 1, ZN_LOSS_CROSS_ENTROPY_LOGITS = 2,
    ZN_LOSS_BINARY_CROSS_ENTROPY = 3, ZN_LOSS_KL_DIVERGENCE = 4
} zn_loss;

typedef struct zn_ctx zn_ctx;   /* replaces CudaBackend + CudaContext + CudaDriver (src/cuda.zig:163, src/cuda_context.zig:382) */
typedef struct zn_net zn_net;   /* device-resident Network (src/network.zig:38-60) */

/* ---- context: Backend.init / Backend.deinit, src/backend.zig:43-82 -------- */

/* Number of CUDA devices (0 without a driver); CudaBackend.isAvailable, src/cuda.zig:317-328. */
ZN_API int32_t zn_device_count(void);
/* Creates a context with its own compute, copy and communication streams on `device`. */
ZN_API zn_status zn_ctx_create(int32_t device, zn_ctx **out);
ZN_API void zn_ctx_destroy(zn_ctx *ctx);                 /* NULL allowed */
ZN_API const char *zn_last_error_string(const zn_ctx *ctx);
ZN_API const char *zn_status_string(zn_status s);
/* Precision used by the op-level GEMM calls below (default ZN_FP32_SIMT). */
ZN_API zn_status zn_ctx_set_precision(zn_ctx *ctx, zn_precision p);
/* Backend.beginCommandBatch / endCommandBatch, src/backend.zig:105-125: ops on
 * device pointers only enqueue; end waits for the stream and reports any
 * device-side timeout flag. */
ZN_API zn_status zn_begin_command_batch(zn_ctx *ctx);
ZN_API zn_status zn_end_command_batch(zn_ctx *ctx);

/* ---- device tensors: Tensor.init/deinit + the mtl_buffer slot, src/tensor.zig:17-118 */
ZN_API zn_status zn_tensor_alloc(zn_ctx *ctx, size_t count, float **out_dev);   /* zero-filled */
ZN_API zn_status zn_tensor_free(zn_ctx *ctx, float *dev);
ZN_API zn_status zn_tensor_upload(zn_ctx *ctx, float *dev, const float *host, size_t count);
ZN_API zn_status zn_tensor_download(zn_ctx *ctx, float *host, const float *dev, size_t count);
/* Backend.copyData, src/backend.zig:128-136: any mix of host and device pointers. */
ZN_API zn_status zn_copy_data(zn_ctx *ctx, const float *src, float *dst, size_t count);

/* ---- GEMMs ------------------------------------------------------------------ */
/* Backend.matMul / matMulBatch, src/backend.zig:169-195: C[m x n] (+)= A[m x k] . B[k x n]. */
ZN_API zn_status zn_matmul(zn_ctx *ctx, const float *a, const float *b, float *c,
                           size_t m, size_t n, size_t k, int32_t accumulate);
/* Backend.matMulTransposeA, src/backend.zig:298-307: C[m x n] (+)= A[k x m]^T . B[k x n]. */
ZN_API zn_status zn_matmul_transpose_a(zn_ctx *ctx, const float *a, const float *b, float *c,
                                       size_t m, size_t n, size_t k, int32_t accumulate);
/* Backend.matMulTransposeB, src/backend.zig:310-325: C[m x n] (+)= A[m x k] . B[n x k]^T. */
ZN_API zn_status zn_matmul_transpose_b(zn_ctx *ctx, const float *a, const float *b, float *c,
                                       size_t m, size_t n, size_t k, int32_t accumulate);
/* Backend.matMulBias / matMulBiasRelu / matMulBiasSigmoid / matMulBiasTanh,
 * src/backend.zig:200-295: C[batch x n] = act(A[batch x k] . B[k x n] + bias[n]),
 * one kernel (act = ZN_ACT_LINEAR for plain matMulBias).  The other activations are taken too:
 * gelu / leaky_relu / elu in the same kernel, softmax by a second kernel over the rows of C
 * (the way Dense.forward applies it sample by sample, src/layer.zig:398-406). */
ZN_API zn_status zn_matmul_bias_act(zn_ctx *ctx, const float *a, const float *b, const float *bias, float *c,
                                    size_t batch, size_t n, size_t k, zn_activation act);

/* ---- bias and activations ----------------------------------------------------- */
/* Backend.addBias, src/backend.zig:658-671: out[r][i] += bias[i], rows = out_len / bias_len. */
ZN_API zn_status zn_add_bias(zn_ctx *ctx, float *out, size_t out_len, const float *bias, size_t bias_len);
/* Backend.accumulateBias, src/backend.zig:649-655 -> :706-713: grad_bias[i] += sum over rows of g[r][i]. */
ZN_API zn_status zn_accumulate_bias(zn_ctx *ctx, float *grad_bias, size_t bias_len, const float *g, size_t g_len);
/* No counterpart in the reference.  The same accumulation as zn_accumulate_bias, with the same order of
 * additions in every precision mode of the context, for callers that must not trigger a device allocation:
 * programs whose own pool already owns all device memory, and loops that cannot take the device-wide stall of
 * cudaMalloc/cudaFree.  It calls no allocator: the per-split partial sums live in a fixed 4 MiB block
 * (1,048,576 floats) that is part of the library image on every GPU that loads it.  Both pointers must be
 * DEVICE pointers.  A problem whose partial sums do not fit (row splits x bias_len > 1,048,576; the split
 * count shrinks as bias_len grows, so this means a bias_len of roughly a million or more) is rejected with
 * ZN_ERR_INVALID_VALUE and a message giving the sizes.  On a ZN_FP32_EXACT context the sums run in the
 * reference's order (one running sum per column), which needs no scratch at all and has no size limit.  The
 * first call on each device looks up the block's device address; make that call before starting any stream
 * capture.  All calls on a GPU share the block: calls that overlap in time on one GPU race and must be ordered
 * by the caller; nothing in the block needs clearing between calls.  The call makes the context's device the
 * calling thread's current device. */
ZN_API zn_status zn_accumulate_bias_noalloc(zn_ctx *ctx, float *grad_bias, size_t bias_len, const float *g, size_t g_len);
/* Backend.activationForward, src/backend.zig:367-386 (in == out allowed).  With softmax the
 * whole slice is one vector, as in the reference (:377-379); likewise in the backward. */
ZN_API zn_status zn_activation_forward(zn_ctx *ctx, zn_activation act, const float *in, float *out, size_t count);
/* Backend.activationBackward, src/backend.zig:390-399 -> :2649-2669; `y` is the ACTIVATED output. */
ZN_API zn_status zn_activation_backward(zn_ctx *ctx, zn_activation act, const float *y, const float *grad_out,
                                        float *grad_in, size_t count);

/* ---- loss ---------------------------------------------------------------------- */
/* Loss.forward, src/loss.zig:34-46.  rows > 1 takes cross-entropy per row and
 * returns the mean over rows; MSE is over all rows*cols elements. */
ZN_API zn_status zn_loss_forward(zn_ctx *ctx, zn_loss loss, const float *output, const float *target,
                                 size_t rows, size_t cols, float *loss_out /* host */);
/* Backend.lossBackward, src/backend.zig:403-417 -> Loss.backward, src/loss.zig:48-60. */
ZN_API zn_status zn_loss_backward(zn_ctx *ctx, zn_loss loss, const float *output, const float *target,
                                  float *grad_out, size_t rows, size_t cols);

/* metrics.evaluateClassification, src/metrics.zig:239-264: per sample getPredictedClass
 * (first maximum, :213-227) and getTrueClass (first target > 0.5, else 0, :230-235), then
 * computeClassificationMetrics (:85-163).  outputs / targets: rows x cols, host or device.
 * confusion (host, num_classes^2 counters, [true][predicted]) and metrics4 (host: accuracy,
 * macro precision, macro recall, F1) may each be null.  rows = 0 fails with ZN_ERR_SHAPE
 * (error.EmptyInput), a class index >= num_classes with ZN_ERR_INVALID_VALUE (error.InvalidClass). */
ZN_API zn_status zn_evaluate_classification(zn_ctx *ctx, const float *outputs, const float *targets, size_t rows,
                                            size_t cols, size_t num_classes, uint64_t *confusion, float *metrics4);

/* ---- optimizers ------------------------------------------------------------------ */
/* Backend.sgdUpdate, src/backend.zig:420-430 -> cpuSgdUpdate :2722-2739 (clamps included). */
ZN_API zn_status zn_sgd_update(zn_ctx *ctx, float *weights, const float *grads, size_t count,
                               float learning_rate, float weight_decay);
/* Backend.sgdUpdateBias, src/backend.zig:640-646 -> :2741-2758. */
ZN_API zn_status zn_sgd_update_bias(zn_ctx *ctx, float *bias, const float *grads, size_t count, float learning_rate);
/* Backend.adamUpdate, src/backend.zig:433-443 -> cpuAdamUpdate :2760-2772; the
 * bias corrections are the caller's, as in Adam.step (src/optimizer.zig:210-213). */
ZN_API zn_status zn_adam_update(zn_ctx *ctx, float *weights, const float *grads, float *m, float *v, size_t count,
                                float lr, float beta1, float beta2, float eps, float bias_corr1, float bias_corr2);
/* Backend.rmspropUpdate, src/backend.zig:446-456 -> cpuRmspropUpdate :2774-2783. */
ZN_API zn_status zn_rmsprop_update(zn_ctx *ctx, float *weights, const float *grads, float *g_avg, size_t count,
                                   float lr, float rho, float eps);
/* The global gradient-norm clip of Network.trainStep, src/network.zig:513-535,
 * over `tensor_count` gradient tensors in the order given (device or host
 * pointers, all of one kind).  norm_out / factor_out are host floats (may be NULL). */
ZN_API zn_status zn_clip_grad_norm(zn_ctx *ctx, float *const *grads, const size_t *counts, size_t tensor_count,
                                   float *norm_out, float *factor_out);

/* ---- network: Network + Dense + Optimizer, resident on the device -------------- */
/* Network.init, src/network.zig:62-76. */
ZN_API zn_status zn_net_create(zn_ctx *ctx, zn_precision precision, zn_net **out);
ZN_API void zn_net_destroy(zn_net *net);                 /* Network.deinit :78-102; NULL allowed */
/* Network.addDense -> Dense.init, src/layer.zig:306-348.  Weights are drawn as
 * the reference draws them, U(-1,1) * scale(act), from a counter-seeded
 * generator; the VALUES differ from Zig's PRNG, so callers that need known
 * weights set them with zn_net_set_weights.  Returns the layer index. */
ZN_API zn_status zn_net_add_dense(zn_net *net, size_t input_size, size_t output_size, zn_activation act,
                                  int32_t *layer_index_out /* may be NULL */);
ZN_API zn_status zn_net_layer_count(const zn_net *net, size_t *out);
/* Layer.getWeights / getBias / getGradWeights / getGradBias, src/layer.zig:170-248 (host copies). */
ZN_API zn_status zn_net_set_weights(zn_net *net, size_t layer, const float *weights, const float *bias);
ZN_API zn_status zn_net_get_weights(zn_net *net, size_t layer, float *weights, float *bias);
ZN_API zn_status zn_net_get_grads(zn_net *net, size_t layer, float *grad_weights, float *grad_bias);
/* Gradient of the loss with respect to the network input of the last step
 * (the reference computes it for layer 0 as well, src/layer.zig:448). */
ZN_API zn_status zn_net_get_input_grad(zn_net *net, float *grad_input, size_t count);
/* Network.optimizers[layer] = Sgd{momentum 0} / Adam, src/network.zig:44,117;
 * layer = -1 sets every layer.  Sgd.step :160-164, Adam.step :209-233. */
ZN_API zn_status zn_net_set_sgd(zn_net *net, int32_t layer, float weight_decay);
ZN_API zn_status zn_net_set_adam(zn_net *net, int32_t layer, float beta1, float beta2, float eps, float weight_decay);
/* Sgd{ .momentum > 0 }, src/optimizer.zig:96-104 (velocity tensors) and Sgd.step :114-159:
 * v = momentum*v - lr*g; w = w + v, without the clamps of the plain SGD path. */
ZN_API zn_status zn_net_set_sgd_momentum(zn_net *net, int32_t layer, float momentum);
/* AdamW, src/optimizer.zig:236-297: Adam.step's update without the L2 term, then the
 * decoupled decay w *= 1 - lr*weight_decay on weights and bias. */
ZN_API zn_status zn_net_set_adamw(zn_net *net, int32_t layer, float beta1, float beta2, float eps, float weight_decay);
/* Rmsprop, src/optimizer.zig:300-359: optional L2 term added to the gradients, then
 * Backend.rmspropUpdate on weights and bias. */
ZN_API zn_status zn_net_set_rmsprop(zn_net *net, int32_t layer, float rho, float eps, float weight_decay);
/* Network.forward, src/network.zig:309-386, on a block of `rows` samples. */
ZN_API zn_status zn_net_forward(zn_net *net, const float *input, size_t rows, float *output);
/* Network.forward on the block, then metrics.evaluateClassification (below) on its output
 * and `target` (rows x output size, one-hot), all on the device. */
ZN_API zn_status zn_net_evaluate_classification(zn_net *net, const float *input, const float *target, size_t rows,
                                                size_t num_classes, uint64_t *confusion, float *metrics4);
/* Network.trainStep, src/network.zig:481-579, on a block of `rows` samples:
 * clear gradients, forward, loss gradient, backward, global norm clip,
 * optimizer, and the loss of the pre-update output in *loss_out (host).
 * rows == 1 is the literal reference step; for rows > 1 cross-entropy is taken
 * per row (gradient softmax - target per row, loss = mean over rows). */
ZN_API zn_status zn_net_train_step(zn_net *net, const float *input, const float *target, size_t rows,
                                   float learning_rate, zn_loss loss, float *loss_out);
/* Pipelined form of the step for host inputs: submit copies the block from
 * (pinned) host memory on the copy stream into one of two device slots and
 * enqueues the step; wait returns the loss of the OLDEST submitted step.  At
 * most two steps may be in flight. */
ZN_API zn_status zn_net_submit_step(zn_net *net, const float *host_input, const float *host_target, size_t rows,
                                    float learning_rate, zn_loss loss);
ZN_API zn_status zn_net_wait_step(zn_net *net, float *loss_out);
/* Network.train, src/network.zig:596-616 with the constant scheduler and no
 * early stopping: for each epoch one trainStep per sample in order;
 * epoch_loss[e] (host, may be NULL) = mean of the per-sample losses. */
ZN_API zn_status zn_net_train(zn_net *net, const float *inputs, const float *targets, size_t samples,
                              size_t epochs, float learning_rate, zn_loss loss, float *epoch_loss);
/* Norm and clip factor of the last step (host floats, may be NULL). */
ZN_API zn_status zn_net_last_clip(zn_net *net, float *norm_out, float *factor_out);
/* Network.save / Network.load, src/network.zig:692-745 -> saveModel / loadModel, src/serialization.zig:78-147:
 * the reference's .znn file ("ZNN\0", version 1, layer count, then per Dense layer type 1, input size, output
 * size, activation tag, weights, bias; little-endian; no optimizer state).  Files written by either side load
 * in the other as long as every layer is Dense. */
ZN_API zn_status zn_net_save(zn_net *net, const char *path);
ZN_API zn_status zn_net_load(zn_ctx *ctx, zn_precision precision, const char *path, zn_net **out);
/* Optimizer state beside the .znn file: per layer the optimizer kind, its hyper-parameters, the
 * step count t and the state tensors (Adam / AdamW m and v, momentum velocity, RMSprop g_avg;
 * src/optimizer.zig:81-88,169-184,236-250,311-320).  The reference's file format has no place
 * for them (src/serialization.zig:165-183 writes weights and bias only), so a run restarted from
 * a .znn alone restarts the moments; with this file it continues exactly.  The layout is this
 * library's own ("ZNO\0", version 1).  Loading needs a network of the same layer shapes. */
ZN_API zn_status zn_net_save_optimizer(zn_net *net, const char *path);
ZN_API zn_status zn_net_load_optimizer(zn_net *net, const char *path);
/* Pinned host memory for the pipelined step's inputs. */
ZN_API zn_status zn_host_alloc(zn_ctx *ctx, size_t count, float **out_host);
ZN_API zn_status zn_host_free(zn_ctx *ctx, float *host);

/* ---- data parallel: replaces MultiCudaContext / MultiGpuCompute ----------------- */
/* MultiCudaContext.distributeWorkload(.round_robin), src/cuda_multi_gpu.zig:247-265:
 * contiguous shard `index` of `total` rows over `parts`. */
ZN_API zn_status zn_distribute_workload(size_t total, size_t parts, size_t index, size_t *start, size_t *end);
/* One rank per GPU.  Rank 0 makes the 128-byte id and hands it to the others
 * by any host channel; every rank then joins.  After zn_net_set_data_parallel
 * a step takes the rank's shard: gradients (and the loss sum) are summed over
 * ranks with one NCCL all-reduce per layer, issued on the communication
 * stream as soon as that layer's gradients exist, and every rank applies the
 * same clip and update.  `global_rows` fixes the MSE divisor. */
ZN_API zn_status zn_dp_unique_id(uint8_t id_out[128]);
ZN_API zn_status zn_dp_init(zn_ctx *ctx, int32_t rank, int32_t world, const uint8_t id[128]);
ZN_API zn_status zn_dp_destroy(zn_ctx *ctx);
ZN_API zn_status zn_net_set_data_parallel(zn_net *net, size_t global_rows);
/* Optional, after zn_net_set_data_parallel: split the parameter update over the ranks.  Per layer a
 * reduce-scatter of the gradients, each rank clips and updates its own 1/world piece, then an all-gather of the
 * updated fp32 weights; results as before up to the order NCCL adds in.  While it is on, zn_net_get_grads and
 * zn_net_save_optimizer fail with ZN_ERR_NOT_AVAILABLE (a rank holds its own piece only) and FP32_EXACT is
 * refused.  Option, ZN_DP_GATHER_BF16=1 in the environment of this call: bf16 networks whose layer widths are
 * multiples of 8 exchange the bf16 operand copy of the weights instead (half the bytes); a rank's fp32 copy of the
 * other ranks' pieces is then brought up to date only by zn_net_get_weights / zn_net_save, which become
 * COLLECTIVE (an all-gather every rank has to take part in: call them on all ranks, in the same order).  No
 * counterpart in the reference, whose multi-GPU layer has no collective at all (src/cuda_multi_gpu.zig). */
ZN_API zn_status zn_net_set_update_sharding(zn_net *net, int32_t on);

/* ---- failure detection ------------------------------------------------------------ */
/* The reference maps driver failures to errors and never waits on another GPU (src/cuda_driver.zig:1119-1159;
 * its multi-GPU layer has no collective, src/cuda_multi_gpu.zig:424-498), so what follows has no counterpart
 * there.  On a data-parallel context every host wait that can sit behind a collective (zn_net_train_step,
 * zn_net_wait_step, zn_end_command_batch, the getters, zn_timer_stop) polls: work done, asynchronous error of
 * the communicator (ncclCommGetAsyncError), deadline.  On an error or a missed deadline the communicator is
 * aborted (ncclCommAbort), the call returns ZN_ERR_NCCL, and every later step fails with ZN_ERR_NCCL until
 * zn_dp_destroy + zn_dp_init.  The deadline defaults to 120 s (ZN_DP_TIMEOUT_MS in the environment of
 * zn_dp_init overrides the default). */
ZN_API zn_status zn_dp_set_timeout_ms(zn_ctx *ctx, int64_t ms);
/* The polling loop itself, free of CUDA and NCCL so that its decisions can be checked anywhere: calls
 * ready(user) (> 0 done, 0 not yet, < 0 the query failed) continuously and, once a millisecond,
 * comm_error(user) (0 = healthy, otherwise the communicator's error code, stored in *comm_error_out) and the
 * deadline (deadline_ms < 0: none).  comm_error and comm_error_out may be NULL. */
enum { ZN_WAIT_READY = 0, ZN_WAIT_COMM_ERROR = 1, ZN_WAIT_DEADLINE = 2, ZN_WAIT_QUERY_FAILED = 3 };
typedef int (*zn_poll_ready_fn)(void *user);
typedef int (*zn_poll_error_fn)(void *user);
ZN_API int32_t zn_wait_poll(zn_poll_ready_fn ready, zn_poll_error_fn comm_error, void *user, int64_t deadline_ms,
                            int32_t *comm_error_out);
/* Bounded device-side waits: every mbarrier wait of the tensor-core GEMMs gives up after about a second,
 * writes a code into a status word the host can read, and lets the kernel return (tensor memory released);
 * the next synchronising call returns ZN_ERR_TIMEOUT with that code and clears the word.  Two probes make
 * that path observable without a hung kernel (no counterpart in the reference): the first launches one small
 * CTA that waits, with the GEMMs' own wait routine and a limit of `limit_cycles` clock cycles, on a barrier
 * nothing ever arrives at, and reports code 99; the second writes `code` into the status word from the host. */
ZN_API zn_status zn_debug_bounded_wait_probe(zn_ctx *ctx, int64_t limit_cycles);
ZN_API zn_status zn_debug_set_device_status(zn_ctx *ctx, int32_t code);
/* Which tensor-core GEMM form a product of this shape would get on a GPU of `sm_count` SMs with `reserve_sms` of
 * them left free (elem_type 0 = bf16, 1 = tf32; `stageable` = C is a single, only-written block with 16-byte
 * aligned base and pitch).  Host arithmetic only, no device needed; no counterpart in the reference.
 * out[0] kernel (0 one-CTA, 1 two-CTA), out[1] tile columns, out[2] results staged through shared memory,
 * out[3] epilogue warps per CTA, out[4] rows of tiles per band, out[5] k-blocks of the main loop. */
ZN_API zn_status zn_debug_tc_route(int32_t elem_type, int64_t m, int64_t n, int64_t k, int32_t sm_count,
                                   int32_t reserve_sms, int32_t stageable, int32_t out[6]);

/* ---- measurement ------------------------------------------------------------------ */
/* Per-kernel-family CUDA-event timing on the compute stream. */
typedef enum {
    ZN_PROF_GEMM_TC = 0, ZN_PROF_GEMM_SIMT = 1, ZN_PROF_LOSS = 2, ZN_PROF_BIAS_REDUCE = 3,
    ZN_PROF_GRAD_NORM = 4, ZN_PROF_OPTIMIZER = 5, ZN_PROF_CONVERT = 6, ZN_PROF_ELEMENTWISE = 7,
    ZN_PROF_FAMILY_COUNT = 8
} zn_prof_family;
ZN_API zn_status zn_profile_enable(zn_ctx *ctx, int32_t on);
ZN_API zn_status zn_profile_reset(zn_ctx *ctx);
/* Totals since the last reset: device milliseconds, launches, algorithmic
 * flops and algorithmic bytes of that family (synchronizes the stream). */
ZN_API zn_status zn_profile_get(zn_ctx *ctx, zn_prof_family family, double *ms, uint64_t *launches,
                                double *flops, double *bytes);
/* CUDA-event stopwatch on the context's compute stream: stop waits for the stream and returns the
 * device time between the two records. */
ZN_API zn_status zn_timer_start(zn_ctx *ctx);
ZN_API zn_status zn_timer_stop(zn_ctx *ctx, float *ms_out);
/* Kernels this library launched on the context since creation. */
ZN_API zn_status zn_launch_count(zn_ctx *ctx, uint64_t *out);

#ifdef __cplusplus
}
#endif
#endif /* ZN_B200_H */
