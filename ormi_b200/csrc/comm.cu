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
// NCCL is loaded with dlopen at first use, so the library itself has no link-time dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "context.h"

namespace ormi_b200 {

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
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
    a.CommInitRank = (decltype(a.CommInitRank))sym("ncclCommInitRank");
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
    int rank = 0, world = 1;
    cudaStream_t stream = nullptr;     // second stream for overlapped buckets
    cudaEvent_t ready = nullptr, done = nullptr;
    cudaEvent_t marks[kCommMarks] = {};   // ormi_b200_comm_mark / ormi_b200_comm_wait
};

CommState* state(ormi_b200_ctx* ctx) {
    if (!ctx->nccl) throw Error("NCCL Error: ormi_b200_comm_init has not been called on this context");
    return static_cast<CommState*>(ctx->nccl);
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
    nccl_check(api().CommInitRank(&st->comm, world, id, rank), "ncclCommInitRank");
    ORMI_CUDA(cudaStreamCreateWithFlags(&st->stream, cudaStreamNonBlocking));
    ORMI_CUDA(cudaEventCreateWithFlags(&st->ready, cudaEventDisableTiming));
    ORMI_CUDA(cudaEventCreateWithFlags(&st->done, cudaEventDisableTiming));
    for (auto& e : st->marks) ORMI_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
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
    for (int i = 0; i < n; ++i)
        nccl_check(api().AllReduce(bufs[i], bufs[i], counts[i], ncclFloat32, ncclSum, st->comm, s), "ncclAllReduce");
    nccl_check(api().GroupEnd(), "ncclGroupEnd");
    ctx->counters["allreduce_calls"] += n;
    for (int i = 0; i < n; ++i) ctx->counters["allreduce_bytes"] += (int64_t)counts[i] * 4;
}

void comm_join(ormi_b200_ctx* ctx) {
    CommState* st = state(ctx);
    ORMI_CUDA(cudaEventRecord(st->done, st->stream));
    ORMI_CUDA(cudaStreamWaitEvent(ctx->stream, st->done, 0));
}

void comm_mark(ormi_b200_ctx* ctx, int slot) {
    CommState* st = state(ctx);
    if (slot < 0 || slot >= kCommMarks) throw Error("NCCL Error: mark slot out of range");
    ORMI_CUDA(cudaEventRecord(st->marks[slot], st->stream));
}

void comm_wait(ormi_b200_ctx* ctx, int slot) {
    CommState* st = state(ctx);
    if (slot < 0 || slot >= kCommMarks) throw Error("NCCL Error: mark slot out of range");
    ORMI_CUDA(cudaStreamWaitEvent(ctx->stream, st->marks[slot], 0));   // a slot never marked is already complete
}

void comm_destroy(ormi_b200_ctx* ctx) {
    if (!ctx->nccl) return;
    CommState* st = static_cast<CommState*>(ctx->nccl);
    cudaStreamSynchronize(st->stream);
    cudaStreamSynchronize(ctx->stream);
    if (st->comm) api().CommDestroy(st->comm);
    cudaEventDestroy(st->ready);
    cudaEventDestroy(st->done);
    for (auto& e : st->marks) cudaEventDestroy(e);
    cudaStreamDestroy(st->stream);
    delete st;
    ctx->nccl = nullptr;
}

}  // namespace ormi_b200
