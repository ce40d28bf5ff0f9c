#include "comm.hpp"

#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "cn_types.hpp"

namespace cn {

namespace {

// The few NCCL declarations used here, spelled out so that no NCCL header is needed to
// build.  Values follow the public nccl.h (ncclDataType_t / ncclRedOp_t enumerations).
typedef void* ncclComm_t;
struct ncclUniqueId_ {
    char internal[128];
};
enum { kNcclInt32 = 2, kNcclInt64 = 4, kNcclFloat32 = 7, kNcclFloat64 = 8, kNcclSum = 0 };

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(ncclUniqueId_*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId_, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*Send)(const void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    std::string error;
};

NcclApi* load_nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* env = getenv("CN_NCCL_LIB");
        const char* candidates[] = {env, "libnccl.so.2", "libnccl.so"};
        for (const char* c : candidates) {
            if (!c || !*c) continue;
            api.handle = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) {
            api.error = "libnccl.so.2 not found (set CN_NCCL_LIB to its path)";
            return;
        }
#define CN_SYM(name)                                                                   \
    api.name = reinterpret_cast<decltype(api.name)>(dlsym(api.handle, "nccl" #name)); \
    if (!api.name) api.error = "libnccl lacks nccl" #name;
        CN_SYM(GetUniqueId)
        CN_SYM(CommInitRank)
        CN_SYM(CommDestroy)
        CN_SYM(GroupStart)
        CN_SYM(GroupEnd)
        CN_SYM(Send)
        CN_SYM(Recv)
        CN_SYM(AllReduce)
        CN_SYM(Broadcast)
        CN_SYM(GetErrorString)
#undef CN_SYM
    });
    return &api;
}

int nccl_type(int dtype) {
    switch (dtype) {
        case DT_F32: return kNcclFloat32;
        case DT_F64: return kNcclFloat64;
        case DT_I32: return kNcclInt32;
        default: return kNcclInt64;
    }
}

int check(NcclApi* api, int rc, const char* what, std::string* err) {
    if (rc == 0) return CN_OK;
    if (err) *err = std::string(what) + ": " + (api->GetErrorString ? api->GetErrorString(rc) : "?");
    return CN_ERR_COMM;
}

NcclApi* api_or_error(std::string* err) {
    NcclApi* api = load_nccl();
    if (!api->handle || !api->error.empty()) {
        if (err) *err = api->error;
        return nullptr;
    }
    return api;
}

}  // namespace

int comm_unique_id(char id[128], std::string* err) {
    NcclApi* api = api_or_error(err);
    if (!api) return CN_ERR_COMM;
    ncclUniqueId_ u;
    int rc = check(api, api->GetUniqueId(&u), "ncclGetUniqueId", err);
    if (rc) return rc;
    memcpy(id, u.internal, 128);
    return CN_OK;
}

int comm_init(Comm* c, const char id[128], int rank, int nranks, std::string* err) {
    NcclApi* api = api_or_error(err);
    if (!api) return CN_ERR_COMM;
    ncclUniqueId_ u;
    memcpy(u.internal, id, 128);
    ncclComm_t comm = nullptr;
    int rc = check(api, api->CommInitRank(&comm, nranks, u, rank), "ncclCommInitRank", err);
    if (rc) return rc;
    c->comm = comm;
    c->rank = rank;
    c->nranks = nranks;
    c->ready = true;
    return CN_OK;
}

void comm_destroy(Comm* c) {
    if (!c->ready) return;
    NcclApi* api = load_nccl();
    if (api->handle && api->CommDestroy) api->CommDestroy((ncclComm_t)c->comm);
    c->comm = nullptr;
    c->ready = false;
}

int comm_group_start(std::string* err) {
    NcclApi* api = api_or_error(err);
    if (!api) return CN_ERR_COMM;
    return check(api, api->GroupStart(), "ncclGroupStart", err);
}

int comm_group_end(std::string* err) {
    NcclApi* api = api_or_error(err);
    if (!api) return CN_ERR_COMM;
    return check(api, api->GroupEnd(), "ncclGroupEnd", err);
}

int comm_send(Comm* c, const void* buf, int64_t count, int dtype, int peer, cudaStream_t s,
              std::string* err) {
    NcclApi* api = api_or_error(err);
    if (!api) return CN_ERR_COMM;
    return check(api, api->Send(buf, (size_t)count, nccl_type(dtype), peer, (ncclComm_t)c->comm, s),
                 "ncclSend", err);
}

int comm_recv(Comm* c, void* buf, int64_t count, int dtype, int peer, cudaStream_t s,
              std::string* err) {
    NcclApi* api = api_or_error(err);
    if (!api) return CN_ERR_COMM;
    return check(api, api->Recv(buf, (size_t)count, nccl_type(dtype), peer, (ncclComm_t)c->comm, s),
                 "ncclRecv", err);
}

int comm_allreduce_sum(Comm* c, void* buf, int64_t count, int dtype, cudaStream_t s,
                       std::string* err) {
    NcclApi* api = api_or_error(err);
    if (!api) return CN_ERR_COMM;
    return check(api,
                 api->AllReduce(buf, buf, (size_t)count, nccl_type(dtype), kNcclSum,
                                (ncclComm_t)c->comm, s),
                 "ncclAllReduce", err);
}

int comm_broadcast(Comm* c, const void* send, void* recv, int64_t count, int dtype, int root,
                   cudaStream_t s, std::string* err) {
    NcclApi* api = api_or_error(err);
    if (!api) return CN_ERR_COMM;
    return check(api,
                 api->Broadcast(send, recv, (size_t)count, nccl_type(dtype), root,
                                (ncclComm_t)c->comm, s),
                 "ncclBroadcast", err);
}

}  // namespace cn
