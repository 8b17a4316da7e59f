// Context, device tensors, copies, error reporting and event-based profiling.
// Replaces CudaBackend.init / CudaContext.init / the dlopen'd driver table of the
// reference (src/cuda.zig:163, src/cuda_context.zig:382-497, src/cuda_driver.zig:710).
#include <cstdarg>
#include <cstdlib>
#include <cstring>

#include "zn_internal.h"

zn_status zn_fail(zn_ctx *ctx, zn_status s, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, ZN_MAX_ERR, fmt, ap);
        va_end(ap);
    }
    return s;
}

zn_status zn_cuda_status(zn_ctx *ctx, cudaError_t e, const char *what) {
    zn_status s = ZN_ERR_CUDA;
    switch (e) {
    case cudaErrorMemoryAllocation: s = ZN_ERR_OUT_OF_MEMORY; break;
    case cudaErrorInvalidValue: s = ZN_ERR_INVALID_VALUE; break;
    case cudaErrorInvalidDevice: s = ZN_ERR_INVALID_DEVICE; break;
    case cudaErrorNoDevice:
    case cudaErrorInsufficientDriver: s = ZN_ERR_NO_DEVICE; break;
    case cudaErrorInitializationError: s = ZN_ERR_NOT_INITIALIZED; break;
    default: break;
    }
    return zn_fail(ctx, s, "%s: %s", what, cudaGetErrorString(e));
}

extern "C" const char *zn_status_string(zn_status s) {
    switch (s) {
    case ZN_OK: return "ok";
    case ZN_ERR_INVALID_VALUE: return "invalid value";
    case ZN_ERR_OUT_OF_MEMORY: return "out of memory";
    case ZN_ERR_NOT_INITIALIZED: return "not initialized";
    case ZN_ERR_NO_DEVICE: return "no CUDA device";
    case ZN_ERR_INVALID_DEVICE: return "invalid device";
    case ZN_ERR_CUDA: return "CUDA error";
    case ZN_ERR_SHAPE: return "shape mismatch";
    case ZN_ERR_UNSUPPORTED: return "unsupported on the Dense path";
    case ZN_ERR_TIMEOUT: return "device-side wait timed out";
    case ZN_ERR_NCCL: return "NCCL error";
    case ZN_ERR_NOT_AVAILABLE: return "not available";
    default: return "unknown status";
    }
}

extern "C" const char *zn_last_error_string(const zn_ctx *ctx) { return ctx ? ctx->err : "null context"; }

extern "C" int32_t zn_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

extern "C" zn_status zn_ctx_create(int32_t device, zn_ctx **out) {
    if (!out) return ZN_ERR_INVALID_VALUE;
    *out = nullptr;
    int n = zn_device_count();
    if (n == 0) return ZN_ERR_NO_DEVICE;
    if (device < 0 || device >= n) return ZN_ERR_INVALID_DEVICE;
    zn_ctx *ctx = new zn_ctx();
    ctx->device = device;
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking);
    // The side lanes carry short kernels on the step's critical chain (exchange of the last gradients, their
    // norm, the update the next forward waits for).  At the highest priority their blocks are placed before
    // those of the next persistent GEMM whenever SMs fall free.  ZN_FLAT_PRIORITIES: all lanes equal (diagnostic).
    int prio_least = 0, prio_greatest = 0;
    if (e == cudaSuccess) e = cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest);
    const int side = getenv("ZN_FLAT_PRIORITIES") ? prio_least : prio_greatest;
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&ctx->comm_stream, cudaStreamNonBlocking, side);
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&ctx->opt_stream, cudaStreamNonBlocking, side);
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&ctx->aux_stream, cudaStreamNonBlocking, side);
    for (int i = 0; i < 4 && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&ctx->lane_join[i], cudaEventDisableTiming);
    ctx->lanes[ZN_LANE_MAIN].stream = ctx->stream;
    ctx->lanes[ZN_LANE_COMM].stream = ctx->comm_stream;
    ctx->lanes[ZN_LANE_OPT].stream = ctx->opt_stream;
    ctx->lanes[ZN_LANE_AUX].stream = ctx->aux_stream;
    if (getenv("ZN_SERIAL_LANES")) {   // diagnostic: reductions and updates back on the main stream, in program order
        ctx->lanes[ZN_LANE_OPT].stream = ctx->stream;
        ctx->lanes[ZN_LANE_AUX].stream = ctx->stream;
    }
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaHostAlloc((void **)&ctx->status_host, sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) {
        *ctx->status_host = 0;
        e = cudaHostGetDevicePointer((void **)&ctx->status_dev, ctx->status_host, 0);
    }
    if (e == cudaSuccess) e = cudaHostAlloc((void **)&ctx->pinned_scalar, 16 * sizeof(float), cudaHostAllocDefault);
    if (e != cudaSuccess) {
        zn_ctx_destroy(ctx);
        cudaGetLastError();
        return e == cudaErrorMemoryAllocation ? ZN_ERR_OUT_OF_MEMORY : ZN_ERR_CUDA;
    }
    *out = ctx;
    return ZN_OK;
}

extern "C" zn_status zn_dp_destroy(zn_ctx *ctx);

extern "C" void zn_ctx_destroy(zn_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    zn_lane_switch(ctx, ZN_LANE_MAIN);
    for (int i = 0; i < 4; ++i)
        if (ctx->lanes[i].stream) cudaStreamSynchronize(ctx->lanes[i].stream);
    if (ctx->dp) zn_dp_destroy(ctx);
    for (auto &kv : ctx->tensors) cudaFree(kv.first);
    for (int i = 0; i < 6; ++i) cudaFree(ctx->stage[i]);
    cudaFree(ctx->scratch);
    cudaFree(ctx->tile_counters);
    cudaFree(ctx->block_counters);
    for (int i = 1; i < 4; ++i) cudaFree(ctx->lanes[i].scratch);
    for (int i = 0; i < 4; ++i)
        if (ctx->lane_join[i]) cudaEventDestroy(ctx->lane_join[i]);
    if (ctx->opt_stream) cudaStreamDestroy(ctx->opt_stream);
    if (ctx->aux_stream) cudaStreamDestroy(ctx->aux_stream);
    for (auto &slot : ctx->prof)
        for (auto &p : slot.pending) { cudaEventDestroy(p.first); cudaEventDestroy(p.second); }
    for (auto ev : ctx->event_pool) cudaEventDestroy(ev);
    if (ctx->trace_origin) cudaEventDestroy(ctx->trace_origin);
    if (ctx->timer0) cudaEventDestroy(ctx->timer0);
    if (ctx->timer1) cudaEventDestroy(ctx->timer1);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->pinned_scalar) cudaFreeHost(ctx->pinned_scalar);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
    if (ctx->comm_stream) cudaStreamDestroy(ctx->comm_stream);
    delete ctx;
}

extern "C" zn_status zn_ctx_set_precision(zn_ctx *ctx, zn_precision p) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (p < ZN_FP32_SIMT || p > ZN_BF16_TC) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "unknown precision %d", (int)p);
    ctx->precision = p;
    return ZN_OK;
}

zn_status zn_check_device_status(zn_ctx *ctx) {
    if (ctx->status_host && *ctx->status_host != 0) {
        int code = *ctx->status_host;
        *ctx->status_host = 0;
        return zn_fail(ctx, ZN_ERR_TIMEOUT, "a bounded device-side wait gave up (code %d)", code);
    }
    return ZN_OK;
}

extern "C" zn_status zn_debug_set_device_status(zn_ctx *ctx, int32_t code) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!ctx->status_host) return zn_fail(ctx, ZN_ERR_NOT_INITIALIZED, "context has no status word");
    *ctx->status_host = code;
    return ZN_OK;
}

void zn_lane_switch(zn_ctx *ctx, int lane) {
    if (lane == ctx->lane) return;
    zn_ctx::lane_state &cur = ctx->lanes[ctx->lane];
    cur.stream = ctx->stream;
    cur.scratch = ctx->scratch;
    cur.scratch_floats = ctx->scratch_floats;
    const zn_ctx::lane_state &next = ctx->lanes[lane];
    ctx->stream = next.stream;
    ctx->scratch = next.scratch;
    ctx->scratch_floats = next.scratch_floats;
    ctx->lane = lane;
}

zn_status zn_sync_all_lanes(zn_ctx *ctx) {
    zn_lane_switch(ctx, ZN_LANE_MAIN);
    for (int i = 0; i < 4; ++i) {
        cudaStream_t s = i == ZN_LANE_MAIN ? ctx->stream : ctx->lanes[i].stream;
        if (s) ZN_TRY(zn_wait_stream(ctx, s));
    }
    return ZN_OK;
}

zn_status zn_join_lanes_into_main(zn_ctx *ctx) {
    zn_lane_switch(ctx, ZN_LANE_MAIN);
    for (int i = 1; i < 4; ++i) {
        ZN_CUDA(ctx, cudaEventRecord(ctx->lane_join[i], ctx->lanes[i].stream));
        ZN_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->lane_join[i], 0));
    }
    return ZN_OK;
}

extern "C" zn_status zn_begin_command_batch(zn_ctx *ctx) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    ctx->batch_depth += 1;
    return ZN_OK;
}

extern "C" zn_status zn_end_command_batch(zn_ctx *ctx) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (ctx->batch_depth > 0) ctx->batch_depth -= 1;
    ZN_TRY(zn_sync_all_lanes(ctx));
    return zn_check_device_status(ctx);
}

bool zn_is_device_ptr(const void *p) {
    if (!p) return false;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

zn_status zn_lane_counters(zn_ctx *ctx, unsigned int **out) {
    if (!ctx->block_counters) {
        const size_t bytes = 4 * ZN_COUNTERS_PER_LANE * sizeof(unsigned int);
        ZN_CUDA(ctx, cudaMalloc((void **)&ctx->block_counters, bytes));
        ZN_CUDA(ctx, cudaMemset(ctx->block_counters, 0, bytes));      // synchronous: cleared before any lane uses it
    }
    *out = ctx->block_counters + ctx->lane * ZN_COUNTERS_PER_LANE;
    return ZN_OK;
}

// Device that owns a device pointer, or -1 for host memory and unknown addresses.
int zn_ptr_device(const void *p) {
    if (!p) return -1;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return (a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged) ? a.device : -1;
}

zn_status zn_scratch_reserve(zn_ctx *ctx, size_t floats) {
    if (ctx->scratch_floats >= floats) return ZN_OK;
    // Work already queued may still use the old block: drain before replacing it.
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(ctx->scratch);
    ctx->scratch = nullptr;
    ctx->scratch_floats = 0;
    size_t want = floats < (1u << 16) ? (1u << 16) : floats;
    ZN_CUDA(ctx, cudaMalloc((void **)&ctx->scratch, want * sizeof(float)));
    ctx->scratch_floats = want;
    return ZN_OK;
}

// ---- tensors ----------------------------------------------------------------------

extern "C" zn_status zn_tensor_alloc(zn_ctx *ctx, size_t count, float **out_dev) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!out_dev || count == 0) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "zn_tensor_alloc: null output or zero size");
    if (count > (SIZE_MAX / sizeof(float))) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "zn_tensor_alloc: size overflow");
    cudaSetDevice(ctx->device);
    float *p = nullptr;
    ZN_CUDA(ctx, cudaMalloc((void **)&p, count * sizeof(float)));
    cudaError_t e = cudaMemsetAsync(p, 0, count * sizeof(float), ctx->stream);
    if (e != cudaSuccess) { cudaFree(p); return zn_cuda_status(ctx, e, "cudaMemsetAsync"); }
    ctx->tensors[p] = count;
    *out_dev = p;
    return ZN_OK;
}

extern "C" zn_status zn_tensor_free(zn_ctx *ctx, float *dev) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!dev) return ZN_OK;
    auto it = ctx->tensors.find(dev);
    if (it == ctx->tensors.end()) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "zn_tensor_free: not a tensor of this context");
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ZN_CUDA(ctx, cudaFree(dev));
    ctx->tensors.erase(it);
    return ZN_OK;
}

extern "C" zn_status zn_tensor_upload(zn_ctx *ctx, float *dev, const float *host, size_t count) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!dev || !host) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "zn_tensor_upload: null pointer");
    ZN_CUDA(ctx, cudaMemcpyAsync(dev, host, count * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ZN_OK;
}

extern "C" zn_status zn_tensor_download(zn_ctx *ctx, float *host, const float *dev, size_t count) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!dev || !host) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "zn_tensor_download: null pointer");
    ZN_CUDA(ctx, cudaMemcpyAsync(host, dev, count * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_copy_data(zn_ctx *ctx, const float *src, float *dst, size_t count) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!src || !dst) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "zn_copy_data: null pointer");
    if (src == dst || count == 0) return ZN_OK;
    ZN_CUDA(ctx, cudaMemcpyAsync(dst, src, count * sizeof(float), cudaMemcpyDefault, ctx->stream));
    if (!(zn_is_device_ptr(src) && zn_is_device_ptr(dst))) ZN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ZN_OK;
}

extern "C" zn_status zn_host_alloc(zn_ctx *ctx, size_t count, float **out_host) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!out_host || count == 0) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "zn_host_alloc: null output or zero size");
    ZN_CUDA(ctx, cudaHostAlloc((void **)out_host, count * sizeof(float), cudaHostAllocDefault));
    return ZN_OK;
}

extern "C" zn_status zn_host_free(zn_ctx *ctx, float *host) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (host) ZN_CUDA(ctx, cudaFreeHost(host));
    return ZN_OK;
}

// ---- profiling ----------------------------------------------------------------------

static cudaEvent_t take_event(zn_ctx *ctx) {
    if (!ctx->event_pool.empty()) {
        cudaEvent_t e = ctx->event_pool.back();
        ctx->event_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

zn_launch_scope::zn_launch_scope(zn_ctx *c, int fam, double flops, double bytes, int n_launches) : ctx(c), family(fam) {
    ctx->launches += (uint64_t)n_launches;
    if (!ctx->profiling) return;
    zn_prof_slot &s = ctx->prof[family];
    s.launches += (uint64_t)n_launches;
    s.flops += flops;
    s.bytes += bytes;
    e0 = take_event(ctx);
    e1 = take_event(ctx);
    cudaEventRecord(e0, ctx->stream);
}

zn_launch_scope::~zn_launch_scope() {
    if (!e0) return;
    cudaEventRecord(e1, ctx->stream);
    ctx->prof[family].pending.emplace_back(e0, e1);
    if (ctx->trace_origin) ctx->trace.push_back({family, ctx->lane, e0, e1});
}

static void drain_profile(zn_ctx *ctx) {
    zn_sync_all_lanes(ctx);
    if (ctx->trace_origin && !ctx->trace.empty()) {
        if (FILE *f = fopen(ctx->trace_path, "a")) {
            for (const zn_trace_rec &r : ctx->trace) {
                float t0 = 0, t1 = 0;
                if (cudaEventElapsedTime(&t0, ctx->trace_origin, r.e0) == cudaSuccess &&
                    cudaEventElapsedTime(&t1, ctx->trace_origin, r.e1) == cudaSuccess)
                    fprintf(f, "%d %d %.4f %.4f\n", r.family, r.lane, t0, t1);
            }
            fclose(f);
        }
        ctx->trace.clear();
    }
    for (auto &slot : ctx->prof) {
        for (auto &p : slot.pending) {
            float ms = 0;
            if (cudaEventElapsedTime(&ms, p.first, p.second) == cudaSuccess) slot.ms += ms;
            ctx->event_pool.push_back(p.first);
            ctx->event_pool.push_back(p.second);
        }
        slot.pending.clear();
    }
}

extern "C" zn_status zn_profile_enable(zn_ctx *ctx, int32_t on) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!on && ctx->profiling) drain_profile(ctx);
    ctx->profiling = on != 0;
    if (on && !ctx->trace_origin && (ctx->trace_path = getenv("ZN_TRACE_FILE")) != nullptr) {
        ZN_CUDA(ctx, cudaEventCreate(&ctx->trace_origin));
        ZN_CUDA(ctx, cudaEventRecord(ctx->trace_origin, ctx->stream));
    }
    return ZN_OK;
}

extern "C" zn_status zn_profile_reset(zn_ctx *ctx) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    drain_profile(ctx);
    for (auto &slot : ctx->prof) { slot.ms = slot.flops = slot.bytes = 0; slot.launches = 0; }
    return ZN_OK;
}

extern "C" zn_status zn_profile_get(zn_ctx *ctx, zn_prof_family family, double *ms, uint64_t *launches, double *flops,
                                    double *bytes) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (family < 0 || family >= ZN_PROF_FAMILY_COUNT) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "unknown kernel family");
    drain_profile(ctx);
    const zn_prof_slot &s = ctx->prof[family];
    if (ms) *ms = s.ms;
    if (launches) *launches = s.launches;
    if (flops) *flops = s.flops;
    if (bytes) *bytes = s.bytes;
    return ZN_OK;
}

extern "C" zn_status zn_timer_start(zn_ctx *ctx) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!ctx->timer0) {
        ZN_CUDA(ctx, cudaEventCreate(&ctx->timer0));
        ZN_CUDA(ctx, cudaEventCreate(&ctx->timer1));
    }
    ZN_CUDA(ctx, cudaEventRecord(ctx->timer0, ctx->stream));
    return ZN_OK;
}

extern "C" zn_status zn_timer_stop(zn_ctx *ctx, float *ms_out) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!ctx->timer0 || !ms_out) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "timer not started or null output");
    ZN_TRY(zn_join_lanes_into_main(ctx));   // work still running on the other lanes belongs to the timed region
    ZN_CUDA(ctx, cudaEventRecord(ctx->timer1, ctx->stream));
    ZN_TRY(zn_wait_event(ctx, ctx->timer1));
    ZN_CUDA(ctx, cudaEventElapsedTime(ms_out, ctx->timer0, ctx->timer1));
    return zn_check_device_status(ctx);
}

extern "C" zn_status zn_launch_count(zn_ctx *ctx, uint64_t *out) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!out) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "null output");
    *out = ctx->launches;
    return ZN_OK;
}

extern "C" zn_status zn_distribute_workload(size_t total, size_t parts, size_t index, size_t *start, size_t *end) {
    if (!start || !end || parts == 0 || index >= parts) return ZN_ERR_INVALID_VALUE;
    const size_t base = total / parts, rem = total % parts;
    const size_t lo = index * base + (index < rem ? index : rem);
    *start = lo;
    *end = lo + base + (index < rem ? 1 : 0);
    return ZN_OK;
}
