// Gradient / cross-shard combine: NCCL all-reduce over NVLink.
//
// The reference has no collectives at all (single device, no rank concept).  The realize path shards along the
// batch (row) axis, so the only exchange a step needs is a sum of the parameter gradients (or of column / global
// sums of a sharded input) over the ranks: one ncclAllReduce(sum, fp32) per bucket.  One process drives one GPU;
// the 128-byte NCCL unique id travels between the processes by whatever the host already has
// (torch.distributed, MPI, a file).
//
// Streams: the all-reduce can be queued on the compute stream (in order with the kernels) or on a second
// "comm" stream that first waits for everything queued on the compute stream so far — so a bucket whose gradient is
// ready goes out while the remaining backward kernels run; ormi_b200_comm_join makes the compute stream wait for it.
//
// Failure detection.  The communicator is created non-blocking (ncclCommInitRankConfig, blocking = 0): no NCCL call
// can then hold the host for ever.  Every call that returns ncclInProgress is polled, together with
// ncclCommGetAsyncError, against a wall-clock deadline ("comm_timeout_ms", default ten minutes), and so is every
// host-side wait for a stream that a collective may be queued on (ormi_b200_sync, the device-to-host copies,
// ormi_b200_comm_destroy).  When the deadline passes — a rank has left, or never joined — or NCCL reports an
// asynchronous error, the communicator is aborted (ncclCommAbort ends the collective kernels still spinning on
// this GPU), the call returns a non-zero status with a message, and the context stays usable for everything that
// is not a collective.  Survivors are meant to learn of a missing rank on the host, before they launch
// (ormi_b200/guard.py); this is the net under that.
//
// NCCL is loaded with dlopen at first use, so the library itself has no link-time dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstring>
#include <thread>

#include "context.h"

namespace ormi_b200 {

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
};

NcclApi& api() {
    static NcclApi a;
    if (a.handle) return a;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) { a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (a.handle) break; }
    if (!a.handle) throw Error(std::string("NCCL Error: cannot load libnccl: ") + dlerror());
    auto sym = [&](const char* name) { void* p = dlsym(a.handle, name); if (!p) throw Error(std::string("NCCL Error: missing symbol ") + name); return p; };
    a.GetUniqueId = (decltype(a.GetUniqueId))sym("ncclGetUniqueId");
    a.CommInitRankConfig = (decltype(a.CommInitRankConfig))sym("ncclCommInitRankConfig");
    a.CommGetAsyncError = (decltype(a.CommGetAsyncError))sym("ncclCommGetAsyncError");
    a.CommDestroy = (decltype(a.CommDestroy))sym("ncclCommDestroy");
    a.CommAbort = (decltype(a.CommAbort))sym("ncclCommAbort");
    a.AllReduce = (decltype(a.AllReduce))sym("ncclAllReduce");
    a.GetErrorString = (decltype(a.GetErrorString))sym("ncclGetErrorString");
    a.GroupStart = (decltype(a.GroupStart))sym("ncclGroupStart");
    a.GroupEnd = (decltype(a.GroupEnd))sym("ncclGroupEnd");
    return a;
}

void nccl_check(ncclResult_t r, const char* what) {
    if (r != ncclSuccess) throw Error(std::string("NCCL Error: ") + api().GetErrorString(r) + " (" + what + ")");
}

constexpr int kCommMarks = 8;

struct CommState {
    ncclComm_t comm = nullptr;
    bool dead = false;                 // aborted after a deadline or an asynchronous error: no more collectives
    int rank = 0, world = 1;
    cudaStream_t stream = nullptr;     // second stream for overlapped buckets
    cudaEvent_t ready = nullptr, done = nullptr;
    cudaEvent_t marks[kCommMarks] = {};   // ormi_b200_comm_mark / ormi_b200_comm_wait
};

CommState* state(ormi_b200_ctx* ctx) {
    if (!ctx->nccl) throw Error("NCCL Error: ormi_b200_comm_init has not been called on this context");
    CommState* st = static_cast<CommState*>(ctx->nccl);
    if (st->dead) throw Error("NCCL Error: the communicator was aborted (a collective ran past its deadline or failed); create a new one");
    return st;
}

using Clock = std::chrono::steady_clock;

Clock::time_point deadline_of(const ormi_b200_ctx* ctx) {
    return Clock::now() + std::chrono::milliseconds(ctx->comm_timeout_ms > 0 ? ctx->comm_timeout_ms : 600000);
}

// Ends the collectives of this communicator that are still in flight on the GPU and marks it unusable.
void abort_comm(CommState* st) {
    if (st->comm) api().CommAbort(st->comm);
    st->comm = nullptr;
    st->dead = true;
}

void pause_briefly(int spins) {
    if (spins < 2000) std::this_thread::yield();
    else std::this_thread::sleep_for(std::chrono::microseconds(100));
}

// Waits until the last non-blocking NCCL call on this communicator has been carried out (its kernels are queued),
// failed, or the deadline passed.
void settle(ormi_b200_ctx* ctx, CommState* st, ncclResult_t r, const char* what) {
    const auto deadline = deadline_of(ctx);
    for (int spins = 0; r == ncclInProgress; ++spins) {
        ncclResult_t q = api().CommGetAsyncError(st->comm, &r);
        if (q != ncclSuccess) { r = q; break; }
        if (r != ncclInProgress) break;
        if (Clock::now() > deadline) {
            abort_comm(st);
            throw Error(std::string("NCCL Error: ") + what + " did not complete within the collective deadline; communicator aborted");
        }
        pause_briefly(spins);
    }
    if (r != ncclSuccess) {
        const std::string msg = api().GetErrorString(r);
        abort_comm(st);
        throw Error("NCCL Error: " + msg + " (" + what + "); communicator aborted");
    }
}

}  // namespace

void comm_unique_id(char* out128) {
    static_assert(sizeof(ncclUniqueId) == 128, "unexpected ncclUniqueId size");
    ncclUniqueId id;
    nccl_check(api().GetUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(out128, &id, 128);
}

void comm_init(ormi_b200_ctx* ctx, const char* id128, int rank, int world) {
    if (ctx->nccl) throw Error("NCCL Error: communicator already initialised");
    if (world < 1 || rank < 0 || rank >= world) throw Error("NCCL Error: bad rank / world size");
    ORMI_CUDA(cudaSetDevice(ctx->device));
    auto st = std::make_unique<CommState>();
    st->rank = rank; st->world = world;
    ncclUniqueId id;
    std::memcpy(&id, id128, 128);
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 0;
    ncclResult_t r = api().CommInitRankConfig(&st->comm, world, id, rank, &config);
    if (r != ncclSuccess && r != ncclInProgress) nccl_check(r, "ncclCommInitRankConfig");
    settle(ctx, st.get(), ncclInProgress, "ncclCommInitRankConfig (some rank never joined?)");
    try {
        ORMI_CUDA(cudaStreamCreateWithFlags(&st->stream, cudaStreamNonBlocking));
        ORMI_CUDA(cudaEventCreateWithFlags(&st->ready, cudaEventDisableTiming));
        ORMI_CUDA(cudaEventCreateWithFlags(&st->done, cudaEventDisableTiming));
        for (auto& e : st->marks) ORMI_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    } catch (...) {
        abort_comm(st.get());          // do not leak a communicator the peers would wait on
        if (st->stream) cudaStreamDestroy(st->stream);
        if (st->ready) cudaEventDestroy(st->ready);
        if (st->done) cudaEventDestroy(st->done);
        for (auto& e : st->marks) if (e) cudaEventDestroy(e);
        throw;
    }
    ctx->nccl = st.release();
}

void comm_allreduce(ormi_b200_ctx* ctx, void* const* bufs, const size_t* counts, int n, int overlap) {
    CommState* st = state(ctx);
    cudaStream_t s = ctx->stream;
    if (overlap) {   // run behind everything queued on the compute stream so far, but not in its way
        ORMI_CUDA(cudaEventRecord(st->ready, ctx->stream));
        ORMI_CUDA(cudaStreamWaitEvent(st->stream, st->ready, 0));
        s = st->stream;
    }
    nccl_check(api().GroupStart(), "ncclGroupStart");
    for (int i = 0; i < n; ++i) {
        ncclResult_t r = api().AllReduce(bufs[i], bufs[i], counts[i], ncclFloat32, ncclSum, st->comm, s);
        if (r != ncclSuccess && r != ncclInProgress) { api().GroupEnd(); nccl_check(r, "ncclAllReduce"); }
    }
    // non-blocking communicator: the group may still be on its way to the stream when ncclGroupEnd returns; events
    // recorded behind it (ormi_b200_comm_mark / join) must come after its kernels, so wait until it is queued
    settle(ctx, st, api().GroupEnd(), "ncclGroupEnd (all-reduce)");
    if (overlap) ctx->comm_inflight++;
    ctx->counters["allreduce_calls"] += n;
    for (int i = 0; i < n; ++i) ctx->counters["allreduce_bytes"] += (int64_t)counts[i] * 4;
}

void comm_join(ormi_b200_ctx* ctx) {
    CommState* st = state(ctx);
    ORMI_CUDA(cudaEventRecord(st->done, st->stream));
    ORMI_CUDA(cudaStreamWaitEvent(ctx->stream, st->done, 0));
    ctx->comm_inflight = 0;            // everything queued on the second stream so far is now ahead of the compute stream
}

void comm_mark(ormi_b200_ctx* ctx, int slot) {
    CommState* st = state(ctx);
    if (slot < 0 || slot >= kCommMarks) throw Error("NCCL Error: mark slot out of range");
    ORMI_CUDA(cudaEventRecord(st->marks[slot], st->stream));
    ctx->comm_last_mark = slot;
}

void comm_wait(ormi_b200_ctx* ctx, int slot) {
    CommState* st = state(ctx);
    if (slot < 0 || slot >= kCommMarks) throw Error("NCCL Error: mark slot out of range");
    ORMI_CUDA(cudaStreamWaitEvent(ctx->stream, st->marks[slot], 0));   // a slot never marked is already complete
    if (slot == ctx->comm_last_mark) ctx->comm_inflight = 0;           // the latest bucket: nothing of the second stream is left beside us
}

// Host-side wait for `stream` that cannot outlast the collective deadline while a communicator exists: polls the
// stream and NCCL's asynchronous error state.  Returns normally when the stream has drained.
void comm_guarded_sync(ormi_b200_ctx* ctx, cudaStream_t stream) {
    CommState* st = static_cast<CommState*>(ctx->nccl);
    if (!st || st->dead || !st->comm) { ORMI_CUDA(cudaStreamSynchronize(stream)); return; }
    const auto deadline = deadline_of(ctx);
    for (int spins = 0;; ++spins) {
        cudaError_t q = cudaStreamQuery(stream);
        if (q == cudaSuccess) return;
        if (q != cudaErrorNotReady) ORMI_CUDA(q);
        ncclResult_t async = ncclSuccess;
        ncclResult_t r = (spins & 63) == 63 ? api().CommGetAsyncError(st->comm, &async) : ncclSuccess;
        const bool failed = r != ncclSuccess || (async != ncclSuccess && async != ncclInProgress);
        if (failed || Clock::now() > deadline) {
            const std::string why = failed ? std::string("NCCL reported ") + api().GetErrorString(r != ncclSuccess ? r : async)
                                           : std::string("a collective did not finish within the deadline (a rank left or never joined?)");
            abort_comm(st);
            cudaStreamSynchronize(stream);        // the aborted kernels leave the stream
            throw Error("NCCL Error: " + why + "; communicator aborted");
        }
        pause_briefly(spins);
    }
}

void comm_destroy(ormi_b200_ctx* ctx) {
    if (!ctx->nccl) return;
    CommState* st = static_cast<CommState*>(ctx->nccl);
    try { comm_guarded_sync(ctx, st->stream); comm_guarded_sync(ctx, ctx->stream); } catch (const Error&) { /* aborted: carry on tearing down */ }
    if (st->comm) api().CommDestroy(st->comm);
    cudaEventDestroy(st->ready);
    cudaEventDestroy(st->done);
    for (auto& e : st->marks) cudaEventDestroy(e);
    cudaStreamDestroy(st->stream);
    delete st;
    ctx->nccl = nullptr;
}

}  // namespace ormi_b200
