// Cross-GPU communication: one NCCL communicator per context (one process per GPU).
// Replaces the Charm++ entry-method messages, `contribute` reductions and the PE-0 gather
// of the reference (src/backend.ci:24-40, src/executor_reduce.cpp:102-110,
// src/partition_get.cpp:54).  libnccl is opened with dlopen on first use, so a single-GPU
// context needs no NCCL at all.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

namespace cn {

struct Comm {
    void* comm = nullptr;  // ncclComm_t
    int rank = 0;
    int nranks = 1;
    bool ready = false;
};

int comm_unique_id(char id[128], std::string* err);
int comm_init(Comm* c, const char id[128], int rank, int nranks, std::string* err);
void comm_destroy(Comm* c);

int comm_group_start(std::string* err);
int comm_group_end(std::string* err);
int comm_send(Comm* c, const void* buf, int64_t count, int dtype, int peer, cudaStream_t s,
              std::string* err);
int comm_recv(Comm* c, void* buf, int64_t count, int dtype, int peer, cudaStream_t s,
              std::string* err);
int comm_allreduce_sum(Comm* c, void* buf, int64_t count, int dtype, cudaStream_t s,
                       std::string* err);
int comm_broadcast(Comm* c, const void* send, void* recv, int64_t count, int dtype, int root,
                   cudaStream_t s, std::string* err);

// Scope of one NCCL group call.  The group is always closed: by end() on the normal path, by
// the destructor when an error return leaves the scope early (an open group would swallow
// every later call of this rank).
class CommGroup {
public:
    explicit CommGroup(std::string* err) : err_(err), rc_(comm_group_start(err)), open_(rc_ == 0) {}
    ~CommGroup() {
        std::string ignored;
        if (open_) comm_group_end(&ignored);
    }
    CommGroup(const CommGroup&) = delete;
    CommGroup& operator=(const CommGroup&) = delete;
    int started() const { return rc_; }  // status of the group start
    int end() {
        if (!open_) return rc_;
        open_ = false;
        return comm_group_end(err_);
    }

private:
    std::string* err_;
    int rc_;
    bool open_;
};

}  // namespace cn
