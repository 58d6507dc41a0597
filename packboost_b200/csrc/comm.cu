// Cross-device exchange of the feature-sharded training path on NCCL, for hosts that do not bring
// their own collective library: the per-depth merge of the candidate tables and of the go-left
// bit masks, enqueued on the caller's stream behind the kernels that produce them.
//
// NCCL is not linked: it is looked up at run time (dlopen of libnccl.so.2, which resolves to the
// copy already loaded into the process when there is one, e.g. the one a framework ships), so the
// library loads and every other entry point works where NCCL is absent.

#include <dlfcn.h>

#include <mutex>

#include "common.cuh"

namespace pb {
namespace {

// the few NCCL declarations used, restated from its public header (nccl.h)
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;      // ncclSuccess == 0
typedef int ncclDataType_t;    // ncclInt32 == 2
typedef int ncclRedOp_t;       // ncclSum == 0
constexpr int kNcclInt32 = 2;
constexpr int kNcclSum = 0;

struct Nccl {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    const char* why = "not tried";
};

Nccl& nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* nm : names) {
            n.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
            if (n.handle) break;
        }
        if (!n.handle) {
            n.why = "libnccl.so.2 could not be loaded";
            return;
        }
#define PB_SYM(field, name)                                                   \
        n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.handle, name)); \
        if (!n.field) { n.why = "NCCL lacks " name; n.handle = nullptr; return; }
        PB_SYM(GetUniqueId, "ncclGetUniqueId")
        PB_SYM(CommInitRank, "ncclCommInitRank")
        PB_SYM(AllReduce, "ncclAllReduce")
        PB_SYM(CommDestroy, "ncclCommDestroy")
        PB_SYM(CommAbort, "ncclCommAbort")
        PB_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
        PB_SYM(GetErrorString, "ncclGetErrorString")
#undef PB_SYM
        n.why = "";
    });
    return n;
}

struct Comm {
    ncclComm_t comm = nullptr;
    int n_ranks = 0, rank = 0;
};

int fail_nccl(ncclResult_t r, const char* what) {
    set_error("NCCL error: %s in %s", nccl().GetErrorString ? nccl().GetErrorString(r) : "?", what);
    return PB_ERR_CUDA;
}

int need_nccl() {
    if (!nccl().handle) return fail_arg("NCCL is unavailable: %s", nccl().why);
    return PB_OK;
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_comm_unique_id(void* id_out) {
    PB_REQUIRE(id_out != nullptr, "id_out is null");
    int rc = need_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    ncclResult_t r = nccl().GetUniqueId(&id);
    if (r != 0) return fail_nccl(r, "ncclGetUniqueId");
    memcpy(id_out, &id, sizeof(id));
    return PB_OK;
}

extern "C" int pb_comm_init(void** comm_out, const void* unique_id, int64_t n_ranks, int64_t rank) {
    PB_REQUIRE(comm_out && unique_id, "null argument");
    PB_REQUIRE(n_ranks >= 1 && n_ranks <= 4096 && rank >= 0 && rank < n_ranks, "rank %lld of %lld is out of range",
               (long long)rank, (long long)n_ranks);
    int rc = need_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    Comm* c = new (std::nothrow) Comm();
    PB_REQUIRE(c != nullptr, "out of host memory");
    ncclResult_t r = nccl().CommInitRank(&c->comm, (int)n_ranks, id, (int)rank);
    if (r != 0) {
        delete c;
        return fail_nccl(r, "ncclCommInitRank");
    }
    c->n_ranks = (int)n_ranks;
    c->rank = (int)rank;
    *comm_out = c;
    return PB_OK;
}

static int all_reduce_words(void* comm_, void* words, int64_t n_words, void* stream, const char* what) {
    PB_REQUIRE(comm_ != nullptr, "communicator is null");
    PB_REQUIRE(words != nullptr && n_words >= 0 && ((uintptr_t)words % 4) == 0, "%s: bad buffer", what);
    Comm* c = static_cast<Comm*>(comm_);
    if (n_words == 0 || c->n_ranks == 1) return PB_OK;
    // an asynchronous failure of an earlier collective (a peer that went away) surfaces here as an
    // error code instead of a wait that never ends
    ncclResult_t async = 0;
    ncclResult_t r = nccl().CommGetAsyncError(c->comm, &async);
    if (r != 0) return fail_nccl(r, "ncclCommGetAsyncError");
    if (async != 0) return fail_nccl(async, "an earlier collective of this communicator");
    r = nccl().AllReduce(words, words, (size_t)n_words, kNcclInt32, kNcclSum, c->comm, (cudaStream_t)stream);
    if (r != 0) return fail_nccl(r, what);
    return PB_OK;
}

extern "C" int pb_comm_allreduce_candidates(void* comm, const pb_train_state* st, int64_t depth, int64_t n_sampled,
                                            void* stream) {
    PB_REQUIRE(comm != nullptr, "communicator is null");
    void* ptr = nullptr;
    int64_t bytes = 0;
    int rc = pb_candidates_buffer(st, depth, n_sampled, &ptr, &bytes);
    if (rc) return rc;
    return all_reduce_words(comm, ptr, bytes / 4, stream, "ncclAllReduce (candidate table)");
}

extern "C" int pb_comm_allreduce_mask(void* comm, uint32_t* bits, int64_t n_words, void* stream) {
    return all_reduce_words(comm, bits, n_words, stream, "ncclAllReduce (go-left bits)");
}

extern "C" int pb_comm_destroy(void* comm_) {
    if (!comm_) return PB_OK;
    Comm* c = static_cast<Comm*>(comm_);
    int rc = PB_OK;
    if (c->comm && nccl().handle) {
        ncclResult_t r = nccl().CommDestroy(c->comm);
        if (r != 0) rc = fail_nccl(r, "ncclCommDestroy");
    }
    delete c;
    return rc;
}
