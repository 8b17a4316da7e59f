// Data-parallel plumbing: one rank per GPU, gradients summed with NCCL.
//
// The reference's multi-GPU layer (src/cuda_multi_gpu.zig) plans a contiguous
// batch split and nothing else; there is no collective anywhere in it.  Here the
// split keeps its semantics (zn_distribute_workload) and the missing exchange is
// one ncclAllReduce(sum, fp32) per layer on the context's communication stream.
//
// NCCL is bound at run time with dlopen, the way the reference binds libcuda
// (src/cuda_driver.zig:786-816), so the library loads on machines without it and
// shares the copy of NCCL a host process may already have loaded.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>

#include "zn_internal.h"

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    // optional (NCCL >= 2.19): memory the collectives can work on in place
    ncclResult_t (*MemAlloc)(void **, size_t) = nullptr;
    ncclResult_t (*MemFree)(void *) = nullptr;
    ncclResult_t (*CommRegister)(const ncclComm_t, void *, size_t, void **) = nullptr;
    ncclResult_t (*CommDeregister)(const ncclComm_t, void *) = nullptr;
    bool ok = false;
};

NcclApi &api() {
    static NcclApi a;
    static bool tried = false;
    if (tried) return a;
    tried = true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *nm : names) {
        a.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    if (!a.handle) return a;
#define ZN_SYM(field, name) *(void **)(&a.field) = dlsym(a.handle, name)
    ZN_SYM(GetUniqueId, "ncclGetUniqueId");
    ZN_SYM(CommInitRank, "ncclCommInitRank");
    ZN_SYM(CommDestroy, "ncclCommDestroy");
    ZN_SYM(CommAbort, "ncclCommAbort");
    ZN_SYM(AllReduce, "ncclAllReduce");
    ZN_SYM(ReduceScatter, "ncclReduceScatter");
    ZN_SYM(AllGather, "ncclAllGather");
    ZN_SYM(Broadcast, "ncclBroadcast");
    ZN_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    ZN_SYM(GetErrorString, "ncclGetErrorString");
    ZN_SYM(MemAlloc, "ncclMemAlloc");
    ZN_SYM(MemFree, "ncclMemFree");
    ZN_SYM(CommRegister, "ncclCommRegister");
    ZN_SYM(CommDeregister, "ncclCommDeregister");
#undef ZN_SYM
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.GetErrorString;
    return a;
}

}   // namespace

struct zn_dp_state {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    int64_t timeout_ms = 120000;   // deadline of every host wait that may sit behind a collective
    bool failed = false;           // the communicator reported an error or missed the deadline and was aborted
};

bool zn_dp_active(const zn_ctx *ctx) { return ctx && ctx->dp && ctx->dp->world > 1; }

// ---- failure detection ---------------------------------------------------------------------------
//
// A rank that dies or falls out of step leaves the others inside a collective that never completes.  Every
// host wait that can sit behind a collective therefore polls instead of blocking: is the work done, has the
// communicator reported an asynchronous error, has the deadline passed.  The loop itself knows nothing of
// CUDA or NCCL (it takes the three questions as callbacks), so its decisions can be tested on a machine
// without either.
extern "C" int32_t zn_wait_poll(zn_poll_ready_fn ready, zn_poll_error_fn comm_error, void *user, int64_t deadline_ms,
                                int32_t *comm_error_out) {
    using clock = std::chrono::steady_clock;
    if (comm_error_out) *comm_error_out = 0;
    if (!ready) return ZN_WAIT_QUERY_FAILED;
    const clock::time_point t0 = clock::now();
    clock::time_point next_check = t0;
    for (;;) {
        const int r = ready(user);
        if (r > 0) return ZN_WAIT_READY;
        if (r < 0) return ZN_WAIT_QUERY_FAILED;
        const clock::time_point now = clock::now();
        if (now < next_check) continue;                      // spin on `ready`; the other questions once a millisecond
        next_check = now + std::chrono::milliseconds(1);
        if (comm_error) {
            const int e = comm_error(user);
            if (e != 0) {
                if (comm_error_out) *comm_error_out = e;
                return ZN_WAIT_COMM_ERROR;
            }
        }
        if (deadline_ms >= 0 && now - t0 > std::chrono::milliseconds(deadline_ms)) return ZN_WAIT_DEADLINE;
    }
}

namespace {

struct WaitTarget { zn_ctx *ctx; cudaEvent_t event; cudaStream_t stream; cudaError_t cuda_error; };

int target_ready(void *user) {
    WaitTarget *w = static_cast<WaitTarget *>(user);
    const cudaError_t e = w->event ? cudaEventQuery(w->event) : cudaStreamQuery(w->stream);
    if (e == cudaSuccess) return 1;
    if (e == cudaErrorNotReady) { cudaGetLastError(); return 0; }
    w->cuda_error = e;
    return -1;
}

int target_comm_error(void *user) {
    WaitTarget *w = static_cast<WaitTarget *>(user);
    zn_dp_state *dp = w->ctx->dp;
    if (!dp || !dp->comm || !api().CommGetAsyncError) return 0;
    ncclResult_t async = ncclSuccess;
    const ncclResult_t r = api().CommGetAsyncError(dp->comm, &async);
    if (r != ncclSuccess) return (int)r;
    return (async == ncclSuccess || async == ncclInProgress) ? 0 : (int)async;
}

// Ends the communicator: its kernels in flight give up, the streams drain, later collectives are refused.
void abort_comm(zn_ctx *ctx) {
    zn_dp_state *dp = ctx->dp;
    if (!dp || !dp->comm) return;
    if (api().CommAbort) api().CommAbort(dp->comm);
    dp->comm = nullptr;
    dp->failed = true;
}

zn_status wait_target(zn_ctx *ctx, WaitTarget &w, const char *what) {
    int32_t comm_err = 0;
    const int32_t r = zn_wait_poll(target_ready, target_comm_error, &w, ctx->dp->timeout_ms, &comm_err);
    if (r == ZN_WAIT_READY) return ZN_OK;
    if (r == ZN_WAIT_QUERY_FAILED) return zn_cuda_status(ctx, w.cuda_error, what);
    abort_comm(ctx);
    // what the aborted collective held back can finish now; give it a bounded time to do so
    WaitTarget drain = w;
    zn_wait_poll(target_ready, nullptr, &drain, 5000, nullptr);
    if (r == ZN_WAIT_COMM_ERROR)
        return zn_fail(ctx, ZN_ERR_NCCL, "%s: the communicator reported '%s'; it has been aborted", what,
                       api().GetErrorString ? api().GetErrorString((ncclResult_t)comm_err) : "an error");
    return zn_fail(ctx, ZN_ERR_NCCL, "%s: no completion within %lld ms (a peer rank is missing or stuck); the communicator "
                   "has been aborted", what, (long long)ctx->dp->timeout_ms);
}

}   // namespace

// Host waits of a data-parallel context.  Without a live communicator they are the plain blocking calls.
zn_status zn_wait_event(zn_ctx *ctx, cudaEvent_t ev) {
    if (!zn_dp_active(ctx) || !ctx->dp->comm) { ZN_CUDA(ctx, cudaEventSynchronize(ev)); return ZN_OK; }
    WaitTarget w{ctx, ev, nullptr, cudaSuccess};
    return wait_target(ctx, w, "waiting for a training step");
}

zn_status zn_wait_stream(zn_ctx *ctx, cudaStream_t s) {
    if (!zn_dp_active(ctx) || !ctx->dp->comm) { ZN_CUDA(ctx, cudaStreamSynchronize(s)); return ZN_OK; }
    WaitTarget w{ctx, nullptr, s, cudaSuccess};
    return wait_target(ctx, w, "waiting for a stream");
}

static zn_status comm_gone(zn_ctx *ctx) {
    return zn_fail(ctx, ZN_ERR_NCCL, "the communicator was aborted after an error or a missed deadline; "
                                     "call zn_dp_destroy and zn_dp_init to rejoin");
}

extern "C" zn_status zn_dp_set_timeout_ms(zn_ctx *ctx, int64_t ms) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!ctx->dp) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "call zn_dp_init first");
    if (ms <= 0) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "dp_set_timeout_ms: %lld is not a positive time", (long long)ms);
    ctx->dp->timeout_ms = ms;
    return ZN_OK;
}

zn_status zn_dp_allreduce(zn_ctx *ctx, float *buf, size_t count, cudaStream_t stream) {
    if (!zn_dp_active(ctx)) return ZN_OK;
    if (!ctx->dp->comm) return comm_gone(ctx);
#ifdef ZN_DIAG
    // diagnostic builds only (-DZN_DIAG): time a step without its exchange (the ranks then diverge; never for results)
    static const bool skip = getenv("ZN_DP_SKIP_ALLREDUCE") != nullptr;
    if (skip) return ZN_OK;
#endif
    ncclResult_t r = api().AllReduce(buf, buf, count, ncclFloat32, ncclSum, ctx->dp->comm, stream);
    if (r != ncclSuccess) return zn_fail(ctx, ZN_ERR_NCCL, "ncclAllReduce: %s", api().GetErrorString(r));
    return ZN_OK;
}

int zn_dp_rank(const zn_ctx *ctx) { return zn_dp_active(ctx) ? ctx->dp->rank : 0; }
int zn_dp_world(const zn_ctx *ctx) { return zn_dp_active(ctx) ? ctx->dp->world : 1; }
bool zn_dp_can_shard(const zn_ctx *ctx) { return zn_dp_active(ctx) && api().ReduceScatter && api().AllGather; }

zn_status zn_dp_allreduce_f64(zn_ctx *ctx, double *buf, size_t count, cudaStream_t stream) {
    if (!zn_dp_active(ctx)) return ZN_OK;
    if (!ctx->dp->comm) return comm_gone(ctx);
    ncclResult_t r = api().AllReduce(buf, buf, count, ncclFloat64, ncclSum, ctx->dp->comm, stream);
    if (r != ncclSuccess) return zn_fail(ctx, ZN_ERR_NCCL, "ncclAllReduce(f64): %s", api().GetErrorString(r));
    return ZN_OK;
}

// In place on a block of world * shard floats: afterwards rank r holds the sum over ranks of its own piece
// [r * shard, (r + 1) * shard); the other pieces keep this rank's partial values.
zn_status zn_dp_reduce_scatter(zn_ctx *ctx, float *buf, size_t shard, cudaStream_t stream) {
    if (!zn_dp_can_shard(ctx)) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "reduce-scatter needs an initialised communicator");
    if (!ctx->dp->comm) return comm_gone(ctx);
    ncclResult_t r = api().ReduceScatter(buf, buf + (size_t)ctx->dp->rank * shard, shard, ncclFloat32, ncclSum, ctx->dp->comm, stream);
    if (r != ncclSuccess) return zn_fail(ctx, ZN_ERR_NCCL, "ncclReduceScatter: %s", api().GetErrorString(r));
    return ZN_OK;
}

// In place: every rank contributes its own piece [r * shard, (r + 1) * shard) and ends with all of them.
zn_status zn_dp_all_gather(zn_ctx *ctx, float *buf, size_t shard, cudaStream_t stream) {
    if (!zn_dp_can_shard(ctx)) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "all-gather needs an initialised communicator");
    if (!ctx->dp->comm) return comm_gone(ctx);
    ncclResult_t r = api().AllGather(buf + (size_t)ctx->dp->rank * shard, buf, shard, ncclFloat32, ctx->dp->comm, stream);
    if (r != ncclSuccess) return zn_fail(ctx, ZN_ERR_NCCL, "ncclAllGather: %s", api().GetErrorString(r));
    return ZN_OK;
}

bool zn_dp_can_gather_bf16(const zn_ctx *ctx) { return zn_dp_can_shard(ctx) && api().Broadcast; }

// In place on world * shard bf16 values: every rank contributes its own piece and ends with all of them.
zn_status zn_dp_all_gather_bf16(zn_ctx *ctx, void *buf, size_t shard, cudaStream_t stream) {
    if (!zn_dp_can_shard(ctx)) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "all-gather needs an initialised communicator");
    if (!ctx->dp->comm) return comm_gone(ctx);
    __nv_bfloat16 *b = static_cast<__nv_bfloat16 *>(buf);
    ncclResult_t r = api().AllGather(b + (size_t)ctx->dp->rank * shard, b, shard, ncclBfloat16, ctx->dp->comm, stream);
    if (r != ncclSuccess) return zn_fail(ctx, ZN_ERR_NCCL, "ncclAllGather(bf16): %s", api().GetErrorString(r));
    return ZN_OK;
}

// In place: `count` floats at buf go from rank `root` to every rank.
zn_status zn_dp_broadcast(zn_ctx *ctx, float *buf, size_t count, int root, cudaStream_t stream) {
    if (!zn_dp_can_gather_bf16(ctx)) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "broadcast needs an initialised communicator");
    if (!ctx->dp->comm) return comm_gone(ctx);
    ncclResult_t r = api().Broadcast(buf, buf, count, ncclFloat32, root, ctx->dp->comm, stream);
    if (r != ncclSuccess) return zn_fail(ctx, ZN_ERR_NCCL, "ncclBroadcast: %s", api().GetErrorString(r));
    return ZN_OK;
}

// A gradient block allocated by NCCL and registered with the communicator.  On NVSwitch machines NCCL can
// then reduce it in place through the switch (NVLS) instead of staging it through its own buffers, which takes
// fewer SMs and less HBM traffic away from the GEMMs the exchange runs under.  Returns ZN_ERR_NOT_AVAILABLE
// (nothing allocated, nothing reported) when this NCCL has no such interface or registration is switched
// off with ZN_DP_NO_REGISTER; the caller then keeps its ordinary allocation.
zn_status zn_dp_alloc_registered(zn_ctx *ctx, size_t bytes, void **ptr_out, void **handle_out) {
    *ptr_out = nullptr;
    *handle_out = nullptr;
    static const bool off = getenv("ZN_DP_NO_REGISTER") != nullptr;
    if (off || !zn_dp_active(ctx) || !ctx->dp->comm || !api().MemAlloc || !api().MemFree || !api().CommRegister || !api().CommDeregister)
        return ZN_ERR_NOT_AVAILABLE;
    void *p = nullptr, *h = nullptr;
    if (api().MemAlloc(&p, bytes) != ncclSuccess || !p) { cudaGetLastError(); return ZN_ERR_NOT_AVAILABLE; }
    if (api().CommRegister(ctx->dp->comm, p, bytes, &h) != ncclSuccess) {
        api().MemFree(p);
        cudaGetLastError();
        return ZN_ERR_NOT_AVAILABLE;
    }
    *ptr_out = p;
    *handle_out = h;
    return ZN_OK;
}

void zn_dp_free_registered(zn_ctx *ctx, void *ptr, void *handle) {
    if (!ptr) return;
    // after zn_dp_destroy the communicator, and with it the registration, is gone already
    if (handle && ctx && ctx->dp && ctx->dp->comm && api().CommDeregister) api().CommDeregister(ctx->dp->comm, handle);
    if (api().MemFree) api().MemFree(ptr);
}

static_assert(sizeof(ncclUniqueId) == 128, "the C ABI carries the NCCL id as 128 bytes");

extern "C" zn_status zn_dp_unique_id(uint8_t id_out[128]) {
    if (!id_out) return ZN_ERR_INVALID_VALUE;
    if (!api().ok) return ZN_ERR_NCCL;
    ncclUniqueId id;
    if (api().GetUniqueId(&id) != ncclSuccess) return ZN_ERR_NCCL;
    memcpy(id_out, &id, 128);
    return ZN_OK;
}

extern "C" zn_status zn_dp_init(zn_ctx *ctx, int32_t rank, int32_t world, const uint8_t id_bytes[128]) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (world < 1 || rank < 0 || rank >= world) return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "dp_init: rank %d of %d", rank, world);
    if (ctx->dp) return zn_fail(ctx, ZN_ERR_NOT_AVAILABLE, "dp_init: already initialised");
    zn_dp_state *st = new zn_dp_state();
    st->rank = rank;
    st->world = world;
    if (world > 1) {
        if (!id_bytes) { delete st; return zn_fail(ctx, ZN_ERR_INVALID_VALUE, "dp_init: null id"); }
        if (!api().ok) { delete st; return zn_fail(ctx, ZN_ERR_NCCL, "libnccl.so.2 could not be loaded"); }
        cudaSetDevice(ctx->device);
        ncclUniqueId id;
        memcpy(&id, id_bytes, 128);
        ncclResult_t r = api().CommInitRank(&st->comm, world, id, rank);
        if (r != ncclSuccess) {
            delete st;
            return zn_fail(ctx, ZN_ERR_NCCL, "ncclCommInitRank: %s", api().GetErrorString(r));
        }
    }
    if (const char *e = getenv("ZN_DP_TIMEOUT_MS")) {
        const long long v = atoll(e);
        if (v > 0) st->timeout_ms = v;
    }
    ctx->dp = st;
    return ZN_OK;
}

extern "C" zn_status zn_dp_destroy(zn_ctx *ctx) {
    if (!ctx) return ZN_ERR_NOT_INITIALIZED;
    if (!ctx->dp) return ZN_OK;
    if (ctx->dp->comm) {
        zn_wait_stream(ctx, ctx->comm_stream);                 // may abort the communicator and clear the pointer
        if (ctx->dp->comm) api().CommDestroy(ctx->dp->comm);
    }
    delete ctx->dp;
    ctx->dp = nullptr;
    return ZN_OK;
}
