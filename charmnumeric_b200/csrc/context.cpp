#include "context.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "kernels.hpp"
#include "regions.hpp"

namespace cn {

namespace {

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Mailboxes that outlived their context.  A mailbox is exported over CUDA IPC and another rank
// may still hold a mapping of it when this rank's context goes away, so it is never freed; the
// next context created on the same device in this process takes it over instead of allocating
// another 64 MiB.
std::mutex g_box_mutex;
std::map<int, std::vector<void*>> g_spare_boxes;  // device -> mailboxes ready for reuse

}  // namespace

Context::Context(int device, int rank, int nranks)
    : device_(device), rank_(rank), nranks_(nranks), failed_(nranks > 0 ? nranks : 1, false) {
    if (const char* t = getenv("CN_TILE")) {
        int tx = 0, r = 0;
        if (sscanf(t, "%d,%d", &tx, &r) == 2 && tx >= 8 && tx <= 256 && (256 % tx) == 0 && r >= 1 &&
            r <= 16) {
            tile_.tx = tx;
            tile_.r = r;
            tile_set_ = true;
        }
    }
    if (const char* f = getenv("CN_FUSE_REDUCTIONS")) fuse_reductions_ = atoi(f) != 0;
    if (const char* f = getenv("CN_FLAT_PREFETCH")) flat_prefetch_ = std::max(-1, std::min(2, atoi(f)));
    if (const char* f = getenv("CN_PUSH_HALO")) push_halo_ = atoi(f) != 0;
    if (const char* f = getenv("CN_FUSE_PRODUCERS")) fuse_producers_ = std::max(0, std::min(2, atoi(f)));
    if (const char* f = getenv("CN_STENCIL_SHFL")) stencil_shfl_ = atoi(f) != 0;
    if (const char* f = getenv("CN_DEPENDENT_LAUNCH")) dependent_launch_ = atoi(f) != 0;
    if (const char* f = getenv("CN_FUSE_SCALAR_TAIL")) fuse_scalar_tail_ = atoi(f) != 0;
    if (const char* f = getenv("CN_STENCIL_BLOCKS")) shifted_minb_ = std::max(1, std::min(8, atoi(f)));
    if (const char* f = getenv("CN_FLAT_BLOCKS")) flat_minb_ = std::max(1, std::min(8, atoi(f)));
    if (const char* f = getenv("CN_PLAN_CACHE")) plan_cache_ = atoi(f) != 0;
    if (const char* f = getenv("CN_OVERLAP_HALO")) overlap_halo_ = atoi(f) != 0;
    if (const char* f = getenv("CN_DEEP_HALO")) deep_halo_ = atoi(f) != 0;
    if (const char* f = getenv("CN_HALO")) {
        int v = atoi(f);
        if (v >= 0 && v <= 64) halo_ = v;
    }
    staged_tile_.tx = 64;
    staged_tile_.r = 4;
    if (const char* n = getenv("CN_STAGED_NS")) {
        int v = atoi(n);
        if (v >= 4 && v <= 12) staged_ns_ = v;
    }
    if (const char* t = getenv("CN_STAGED_TILE")) {
        int tx = 0, r = 0;
        if (sscanf(t, "%d,%d", &tx, &r) == 2 && tx >= 8 && tx <= 64 && (256 % tx) == 0 && r >= 1 && r <= 16) {
            staged_tile_.tx = tx;
            staged_tile_.r = r;
            staged_tile_set_ = true;
        }
    }
}

Context::~Context() {
    if (!initialised_) return;
    cudaSetDevice(device_);
    cudaStreamSynchronize(stream_);
    comm_destroy(&comm_);
    for (auto& kv : arrays_) {
        free_buffer(&kv.second.buf);
        free_buffer(&kv.second.shadow);
    }
    for (auto& kv : kernels_)
        if (kv.second.module && drv_.ModuleUnload) drv_.ModuleUnload(kv.second.module);
    if (partials_) cudaFree(partials_);
    if (counter_) cudaFree(counter_);
    if (pinned_) cudaFreeHost(pinned_);
    if (scratch_) cudaFree(scratch_);
    if (peer_.ready) {
        for (int p = 0; p < nranks_; ++p)
            if (p != rank_ && peer_.box[p]) cudaIpcCloseMemHandle(peer_.box[p]);
        cudaFree(peer_.ticket);
        // peer_.mine is not freed: another rank may still hold a mapping of it, and freeing
        // exported memory under a live mapping is undefined; the next context on this device reuses it
        std::lock_guard<std::mutex> lock(g_box_mutex);
        g_spare_boxes[device_].push_back(peer_.mine);
    }
    if (stream2_) {
        cudaStreamSynchronize(stream2_);
        cudaStreamDestroy(stream2_);
        cudaEventDestroy(ev_fork_);
        cudaEventDestroy(ev_join_);
    }
    if (ev_start_) cudaEventDestroy(ev_start_);
    if (ev_stop_) cudaEventDestroy(ev_stop_);
    cudaStreamSynchronize(stream_);
    cudaStreamDestroy(stream_);
}

int Context::fail(int code, const std::string& msg) {
    err_ = msg;
    return code;
}

int Context::cuda_fail(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return CN_OK;
    err_ = std::string(what) + ": " + cudaGetErrorString(e);
    if (e == cudaErrorMemoryAllocation) return CN_ERR_OUT_OF_MEMORY;
    return CN_ERR_CUDA;
}

int Context::driver_fail(CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return CN_OK;
    const char* s = nullptr;
    if (drv_.GetErrorString) drv_.GetErrorString(r, &s);
    err_ = std::string(what) + ": " + (s ? s : "driver error");
    return CN_ERR_CUDA;
}

int Context::init() {
    if (rank_ < 0 || nranks_ < 1 || rank_ >= nranks_)
        return fail(CN_ERR_INVALID_ARGUMENT, "rank / nranks out of range");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(CN_ERR_NO_DEVICE, "no CUDA device is visible; this backend has no CPU path");
    }
    if (device_ < 0 || device_ >= count) return fail(CN_ERR_INVALID_ARGUMENT, "device index out of range");
    int rc;
    if ((rc = cuda_fail(cudaSetDevice(device_), "cudaSetDevice"))) return rc;
    if ((rc = cuda_fail(cudaFree(0), "context creation"))) return rc;
    cudaDeviceProp prop;
    if ((rc = cuda_fail(cudaGetDeviceProperties(&prop, device_), "cudaGetDeviceProperties"))) return rc;
    if (prop.major < 10)
        return fail(CN_ERR_NO_DEVICE, "kernels are built for sm_100a; device is older");
    sm_count_ = prop.multiProcessorCount;
    if ((rc = cuda_fail(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "stream"))) return rc;
    if ((rc = cuda_fail(cudaEventCreate(&ev_start_), "event"))) return rc;
    if ((rc = cuda_fail(cudaEventCreate(&ev_stop_), "event"))) return rc;
    // keep freed blocks in the stream-ordered pool: array lifetimes recycle memory
    // (the reference keeps a 4-deep free list per shape, src/backend.hpp:366-468)
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device_) == cudaSuccess) {
        unsigned long long thr = ~0ULL;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thr);
    }
    max_grid_ = sm_count_ * 16;
    if ((rc = cuda_fail(cudaMalloc(&partials_, sizeof(double) * CN_MAX_RED * max_grid_), "scratch"))) return rc;
    if ((rc = cuda_fail(cudaMalloc(&counter_, 256), "scratch"))) return rc;
    if ((rc = cuda_fail(cudaMemset(counter_, 0, 256), "scratch"))) return rc;
#define CN_DRV(field, sym)                                                                    \
    {                                                                                         \
        void* fp = nullptr;                                                                   \
        cudaDriverEntryPointQueryResult q;                                                    \
        cudaError_t de = cudaGetDriverEntryPoint(sym, &fp, cudaEnableDefault, &q);            \
        if (de != cudaSuccess || !fp || q != cudaDriverEntryPointSuccess)                     \
            return fail(CN_ERR_CUDA, std::string("driver entry point missing: ") + sym);      \
        drv_.field = reinterpret_cast<decltype(drv_.field)>(fp);                              \
    }
    CN_DRV(ModuleLoadData, "cuModuleLoadData")
    CN_DRV(ModuleGetFunction, "cuModuleGetFunction")
    CN_DRV(ModuleUnload, "cuModuleUnload")
    CN_DRV(LaunchKernel, "cuLaunchKernel")
    CN_DRV(LaunchKernelEx, "cuLaunchKernelEx")
    CN_DRV(GetErrorString, "cuGetErrorString")
    CN_DRV(OccupancyMaxActiveBlocksPerMultiprocessor, "cuOccupancyMaxActiveBlocksPerMultiprocessor")
    CN_DRV(FuncSetAttribute, "cuFuncSetAttribute")
    CN_DRV(FuncGetAttribute, "cuFuncGetAttribute")
    CN_DRV(TensorMapEncodeTiled, "cuTensorMapEncodeTiled")
    error_word_ = counter_ + 16;  // second cache line of the zeroed 256-byte scratch block
    if (cudaHostAlloc((void**)&pinned_, kPinnedBytes, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        pinned_ = nullptr;  // small results then take the pageable path
    }
#undef CN_DRV
    initialised_ = true;
    return CN_OK;
}

// ---- arrays -----------------------------------------------------------------------------

Array* Context::find(int name) {
    auto it = arrays_.find(name);
    return it == arrays_.end() ? nullptr : &it->second;
}

// Slab partition of dimension 0: ceil(n0 / nranks) consecutive rows per rank, the last
// non-empty rank takes the remainder, ranks beyond it own nothing.
void slab_partition(int64_t n0, int nranks, int rank, int64_t* begin, int64_t* end) {
    slab_rows(n0, nranks, rank, begin, end);
}

void Context::partition(int64_t n0, int64_t* begin, int64_t* end, int r) const {
    slab_partition(n0, nranks_, r, begin, end);
}

int Context::alloc_buffer(const Array& a, Buffer* b) {
    const size_t esz = dtype_size(a.dtype);
    const size_t halo_bytes = (size_t)a.halo * a.unit * esz;
    const size_t front = round_up(halo_bytes + 64, 256);
    const size_t total = front + (size_t)a.local_elems() * esz + halo_bytes + 256;
    void* p = nullptr;
    cudaError_t e = cudaMallocAsync(&p, total, stream_);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMallocAsync");
    b->alloc = p;
    b->data = (char*)p + front;
    b->bytes = total;
    return CN_OK;
}

void Context::free_buffer(Buffer* b) {
    if (b->alloc) cudaFreeAsync(b->alloc, stream_);
    b->alloc = nullptr;
    b->data = nullptr;
    b->bytes = 0;
}

int Context::create_array(int name, int ndims, const int64_t* shape, int dtype, bool zero,
                          Array** out) {
    if (ndims < 1 || ndims > kMaxDims) return fail(CN_ERR_INVALID_ARGUMENT, "array rank must be 1..3");
    if (!dtype_valid(dtype)) return fail(CN_ERR_BAD_DTYPE, "bad dtype code");
    for (int d = 0; d < ndims; ++d)
        if (shape[d] < 0) return fail(CN_ERR_INVALID_ARGUMENT, "negative extent");
    Array* old = find(name);
    if (old) {
        bool same = old->ndims == ndims && old->dtype == dtype;
        for (int d = 0; same && d < ndims; ++d) same = old->shape[d] == shape[d];
        if (same) {
            if (zero) {
                int rc = cuda_fail(cudaMemsetAsync(old->buf.alloc, 0, old->buf.bytes, stream_), "memset");
                if (rc) return rc;
                old->mark_written();
            }
            if (out) *out = old;
            return CN_OK;
        }
        free_buffer(&old->buf);
        free_buffer(&old->shadow);
        arrays_.erase(name);
    }
    Array a;
    a.name = name;
    a.ndims = ndims;
    a.dtype = dtype;
    for (int d = 0; d < ndims; ++d) a.shape[d] = shape[d];
    a.unit = 1;
    for (int d = 1; d < ndims; ++d) a.unit *= shape[d];
    a.replicated = a.global_elems() == 1;
    if (a.replicated || nranks_ == 1) {
        a.row_begin = 0;
        a.row_end = shape[0];
        a.halo = 0;
    } else {
        partition(shape[0], &a.row_begin, &a.row_end, rank_);
        a.halo = halo_;
    }
    int rc = alloc_buffer(a, &a.buf);
    if (rc) return rc;
    if (zero) {
        rc = cuda_fail(cudaMemsetAsync(a.buf.alloc, 0, a.buf.bytes, stream_), "memset");
        if (rc) return rc;
    }
    auto ins = arrays_.emplace(name, a);
    if (out) *out = &ins.first->second;
    return CN_OK;
}

int Context::ensure_shadow(Array* a) {
    if (a->shadow.alloc) return CN_OK;
    return alloc_buffer(*a, &a->shadow);
}

int Context::check_leaf(const Array* a, int ndims, const int64_t* shape, const char* what) {
    if (a->ndims != ndims) return fail(CN_ERR_SHAPE_MISMATCH, std::string(what) + ": rank differs from the stored array");
    for (int d = 0; d < ndims; ++d)
        if (a->shape[d] != shape[d])
            return fail(CN_ERR_SHAPE_MISMATCH, std::string(what) + ": shape differs from the stored array");
    return CN_OK;
}

int Context::delete_array(int name) {
    Array* a = find(name);
    if (!a) return fail(CN_ERR_UNKNOWN_ARRAY, "delete_array: unknown array " + std::to_string(name));
    free_buffer(&a->buf);
    free_buffer(&a->shadow);
    arrays_.erase(name);
    return CN_OK;
}

int Context::array_info(int name, int* ndims, int64_t* shape, int* dtype, int64_t* row_begin,
                        int64_t* row_end) {
    Array* a = find(name);
    if (!a) return fail(CN_ERR_UNKNOWN_ARRAY, "unknown array " + std::to_string(name));
    if (ndims) *ndims = a->ndims;
    if (shape)
        for (int d = 0; d < a->ndims; ++d) shape[d] = a->shape[d];
    if (dtype) *dtype = a->dtype;
    if (row_begin) *row_begin = a->row_begin;
    if (row_end) *row_end = a->row_end;
    return CN_OK;
}

// ---- communication ----------------------------------------------------------------------

int Context::comm_init_id(const char id[128]) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    if (nranks_ == 1) return CN_OK;
    cudaSetDevice(device_);
    int rc = comm_init(&comm_, id, rank_, nranks_, &err_);
    if (rc) return rc;
    return setup_peer_boxes();
}

// Allocate this rank's mailbox, hand its IPC handle to every other rank (through the NCCL
// communicator that already exists) and map theirs.  All ranks then agree, by an allreduce
// of a success flag, whether the peer path is used; any failure leaves NCCL in charge.
int Context::setup_peer_boxes() {
    peer_.ready = false;
    if (const char* e = getenv("CN_P2P")) p2p_wanted_ = atoi(e) != 0;
    int ok = (p2p_wanted_ && nranks_ <= CN_MAX_PEERS) ? 1 : 0;
    const size_t box_bytes = sizeof(CnPeerBox) + 4ull * CN_PEER_HALO_SLOT;
    cudaIpcMemHandle_t mine_h;
    memset(&mine_h, 0, sizeof(mine_h));
    if (ok) {
        {
            std::lock_guard<std::mutex> lock(g_box_mutex);
            std::vector<void*>& spare = g_spare_boxes[device_];
            if (!spare.empty()) {
                peer_.mine = spare.back();
                spare.pop_back();
            }
        }
        if ((!peer_.mine && cudaMalloc(&peer_.mine, box_bytes) != cudaSuccess) ||
            cudaMemset(peer_.mine, 0, sizeof(CnPeerBox)) != cudaSuccess ||
            cudaIpcGetMemHandle(&mine_h, peer_.mine) != cudaSuccess) {
            cudaGetLastError();
            ok = 0;
        }
    }
    // staging area: nranks handles + one flag word
    const size_t hs = sizeof(cudaIpcMemHandle_t);
    int rc = ensure_scratch(hs * nranks_ + 256);
    if (rc) return rc;
    char* stage = (char*)scratch_;
    if ((rc = cuda_fail(cudaMemcpyAsync(stage + hs * rank_, &mine_h, hs, cudaMemcpyHostToDevice, stream_), "peer handle"))) return rc;
    CommGroup group(&err_);
    if ((rc = group.started())) return rc;
    for (int p = 0; p < nranks_; ++p)
        if ((rc = comm_broadcast(&comm_, stage + hs * p, stage + hs * p, (int64_t)(hs / 4), DT_I32, p, stream_, &err_))) return rc;
    if ((rc = group.end())) return rc;
    std::vector<cudaIpcMemHandle_t> handles(nranks_);
    if ((rc = cuda_fail(cudaMemcpyAsync(handles.data(), stage, hs * nranks_, cudaMemcpyDeviceToHost, stream_), "peer handles"))) return rc;
    if ((rc = cuda_fail(cudaStreamSynchronize(stream_), "peer handles"))) return rc;
    if (ok) {
        for (int p = 0; p < nranks_ && ok; ++p) {
            if (p == rank_) {
                peer_.box[p] = peer_.mine;
                continue;
            }
            void* ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, handles[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();
                ok = 0;
            } else {
                peer_.box[p] = ptr;
            }
        }
    }
    if (ok && cudaMalloc((void**)&peer_.ticket, 256) == cudaSuccess) cudaMemset(peer_.ticket, 0, 256);
    else ok = 0;
    // unanimous or not at all
    int* flag = (int*)(stage + hs * nranks_);
    if ((rc = cuda_fail(cudaMemcpyAsync(flag, &ok, sizeof(int), cudaMemcpyHostToDevice, stream_), "peer flag"))) return rc;
    if ((rc = comm_allreduce_sum(&comm_, flag, 1, DT_I32, stream_, &err_))) return rc;
    int total = 0;
    if ((rc = cuda_fail(cudaMemcpyAsync(&total, flag, sizeof(int), cudaMemcpyDeviceToHost, stream_), "peer flag"))) return rc;
    if ((rc = cuda_fail(cudaStreamSynchronize(stream_), "peer flag"))) return rc;
    peer_.ready = total == nranks_;
    if (!peer_.ready) {
        for (int p = 0; p < nranks_; ++p)
            if (p != rank_ && peer_.box[p]) cudaIpcCloseMemHandle(peer_.box[p]);
        // another rank may have mapped this rank's mailbox before the vote failed; freeing
        // exported memory under a live mapping is undefined, so it is kept for the next context
        if (peer_.ticket) cudaFree(peer_.ticket);
        if (peer_.mine) {
            std::lock_guard<std::mutex> lock(g_box_mutex);
            g_spare_boxes[device_].push_back(peer_.mine);
        }
        peer_ = PeerState();
    }
    return CN_OK;
}

void Context::bind_peers(CnGroupArgs* a) {
    a->peer_n = 0;
    if (!peer_.ready) return;
    for (int p = 0; p < nranks_; ++p) a->peer_box[p] = peer_.box[p];
    a->peer_rank = rank_;
    a->peer_n = nranks_;
    a->peer_epoch = ++peer_.red_epoch;
    a->error = error_word_;
    waiting_launches_++;
    stats_.peer_exchanges++;
}

int Context::mark_rank_failed(int r) {
    if (r < 0 || r >= nranks_) return fail(CN_ERR_INVALID_ARGUMENT, "rank out of range");
    failed_[r] = true;
    return CN_OK;
}

int Context::ensure_second_stream() {
    if (stream2_) return CN_OK;
    int rc;
    // highest priority: its few blocks (halo rows, edge rows) should get the first free SM slots
    int least = 0, greatest = 0;
    cudaDeviceGetStreamPriorityRange(&least, &greatest);
    if ((rc = cuda_fail(cudaStreamCreateWithPriority(&stream2_, cudaStreamNonBlocking, greatest), "second stream"))) return rc;
    if ((rc = cuda_fail(cudaEventCreateWithFlags(&ev_fork_, cudaEventDisableTiming), "event"))) return rc;
    return cuda_fail(cudaEventCreateWithFlags(&ev_join_, cudaEventDisableTiming), "event");
}

int Context::exchange_halo(Array* a, cudaStream_t st) {
    if (nranks_ == 1 || a->replicated || (a->halo > 0 && a->halo_fresh == a->halo)) return CN_OK;
    if (!comm_.ready) return fail(CN_ERR_COMM, "halo exchange needs cn_comm_init first");
    const int H = a->halo;
    const int64_t nl = a->local_rows();
    int64_t nb, ne, pb, pe;
    bool has_prev = false, has_next = false;
    if (nl > 0 && rank_ > 0) {
        partition(a->shape[0], &pb, &pe, rank_ - 1);
        has_prev = pe > pb;
        if (has_prev && (pe - pb < H || nl < H))
            return fail(CN_ERR_UNSUPPORTED, "a slab is thinner than the halo depth");
    }
    if (nl > 0 && rank_ + 1 < nranks_) {
        partition(a->shape[0], &nb, &ne, rank_ + 1);
        has_next = ne > nb;
        if (has_next && (ne - nb < H || nl < H))
            return fail(CN_ERR_UNSUPPORTED, "a slab is thinner than the halo depth");
    }
    const int64_t cnt = (int64_t)H * a->unit;
    const size_t esz = dtype_size(a->dtype);
    int rc;
    if (peer_.ready) {
        if ((size_t)cnt * esz <= CN_PEER_HALO_SLOT && (cnt * esz) % 8 == 0) {
            if (has_prev || has_next) {
                const std::vector<Array*> one{a};
                rc = exchange_halo_p2p(one, has_prev, has_next, st);
                if (rc) return rc;
            }
            a->halo_fresh = a->halo;
            stats_.halo_exchanges++;
            return CN_OK;
        }
    }
    prof_start("halo exchange (nccl)", (double)cnt * esz * ((has_prev ? 2 : 0) + (has_next ? 2 : 0)), st);
    CommGroup group(&err_);
    if ((rc = group.started())) return rc;
    if (has_prev) {
        if ((rc = comm_send(&comm_, a->buf.data, cnt, a->dtype, rank_ - 1, st, &err_))) return rc;
        if ((rc = comm_recv(&comm_, a->buf.data - cnt * esz, cnt, a->dtype, rank_ - 1, st, &err_))) return rc;
    }
    if (has_next) {
        if ((rc = comm_send(&comm_, a->buf.data + (nl * a->unit - cnt) * esz, cnt, a->dtype, rank_ + 1, st, &err_))) return rc;
        if ((rc = comm_recv(&comm_, a->buf.data + nl * a->unit * esz, cnt, a->dtype, rank_ + 1, st, &err_))) return rc;
    }
    if ((rc = group.end())) return rc;
    prof_stop();
    a->halo_fresh = a->halo;
    stats_.halo_exchanges++;
    return CN_OK;
}

// The halo rows of several arrays at once.  Arrays of one row partition whose rows fit the
// payload slot together travel in ONE peer-store launch (CG's fused kernel needs r and p: one
// exchange latency instead of two); anything else goes array by array.
int Context::exchange_halos(const std::vector<Array*>& arrays, cudaStream_t st) {
    // remember who asks together: the kernels that produce these arrays next will push their
    // edge rows themselves, into one payload slot
    if (!arrays.empty() && arrays.size() <= CN_HALO_PARTS) {
        std::vector<int> names;
        for (Array* a : arrays) {
            a->halo_wanted = true;
            names.push_back(a->name);
        }
        if (names != halo_group_) halo_group_ = names;
    }
    // rows that the producing kernels pushed already: publish, wait, copy in
    if (pending_.active) {
        int rc = pull_pending(st);
        if (rc) return rc;
    }
    std::vector<Array*> todo;
    for (Array* a : arrays)
        if (!(nranks_ == 1 || a->replicated || (a->halo > 0 && a->halo_fresh == a->halo))) todo.push_back(a);
    bool batch = peer_.ready && todo.size() > 1 && todo.size() <= CN_HALO_PARTS && comm_.ready;
    size_t total = 0;
    for (Array* a : todo) {
        const size_t bytes = (size_t)a->halo * a->unit * dtype_size(a->dtype);
        if (a->shape[0] != todo[0]->shape[0] || a->halo != todo[0]->halo || bytes % 8 || a->local_rows() < a->halo) batch = false;
        total += (bytes + 15) & ~(size_t)15;
    }
    if (batch && total <= CN_PEER_HALO_SLOT) {
        Array* a = todo[0];
        const int H = a->halo;
        const int64_t nl = a->local_rows();
        int64_t b, e;
        bool has_prev = false, has_next = false, thin = false;
        if (nl > 0 && rank_ > 0) {
            partition(a->shape[0], &b, &e, rank_ - 1);
            has_prev = e > b;
            thin = thin || (has_prev && e - b < H);
        }
        if (nl > 0 && rank_ + 1 < nranks_) {
            partition(a->shape[0], &b, &e, rank_ + 1);
            has_next = e > b;
            thin = thin || (has_next && e - b < H);
        }
        if (!thin) {
            int rc = CN_OK;
            if (has_prev || has_next)
                if ((rc = exchange_halo_p2p(todo, has_prev, has_next, st))) return rc;
            for (Array* x : todo) x->halo_fresh = x->halo;
            stats_.halo_exchanges++;
            return CN_OK;
        }
    }
    for (Array* a : todo) {
        int rc = exchange_halo(a, st);
        if (rc) return rc;
    }
    return CN_OK;
}

// The second half of an exchange whose first half (this rank's edge rows into the neighbours'
// mailboxes) was done by the kernels that produced the rows: publish them with the epoch,
// wait (bounded) for the neighbours' rows of the same epoch and copy those into the halo rows
// of every array whose pushed version is still the current one.
int Context::pull_pending(cudaStream_t st) {
    if (!pending_.active) return CN_OK;
    pending_.active = false;
    HaloArgs h;
    h.pull_only = true;
    h.nparts = (int)pending_.names.size();
    std::vector<Array*> installed;
    double total = 0;
    for (size_t q = 0; q < pending_.names.size(); ++q) {
        h.bytes[q] = pending_.bytes[q];
        Array* a = find(pending_.names[q]);
        const size_t esz = a ? dtype_size(a->dtype) : 8;
        if (!a || !a->halo_pushed || (size_t)a->halo * a->unit * esz != pending_.bytes[q]) continue;  // overwritten since
        const int64_t nl = a->local_rows();
        h.halo_below[q] = a->buf.data - pending_.bytes[q];
        h.halo_above[q] = a->buf.data + (size_t)nl * a->unit * esz;
        installed.push_back(a);
        total += (double)pending_.bytes[q];
    }
    h.epoch_prev = pending_.epoch_prev;
    h.epoch_next = pending_.epoch_next;
    h.me = peer_.mine;
    h.box_prev = pending_.has_prev ? peer_.box[rank_ - 1] : nullptr;
    h.box_next = pending_.has_next ? peer_.box[rank_ + 1] : nullptr;
    h.ticket = peer_.ticket;
    h.error = error_word_;
    if (h.box_prev || h.box_next) {
        prof_start("halo pull (rows pushed by their producers)", total * ((h.box_prev ? 1 : 0) + (h.box_next ? 1 : 0)), st);
        int rc = cuda_fail(launch_halo_exchange(h, sm_count_, st), "halo pull");
        prof_stop();
        if (rc) return rc;
        stats_.kernel_launches++;
        waiting_launches_++;
        stats_.peer_exchanges++;
    }
    for (Array* a : installed) {
        a->halo_fresh = a->halo;
        a->halo_pushed = false;
    }
    stats_.halo_exchanges++;
    return CN_OK;
}

// Halo rows as peer stores: one small kernel pushes this rank's boundary rows into the
// neighbours' mailboxes, publishes them with a flag, waits (bounded) for the neighbours' rows
// and copies them into the local halo.
int Context::exchange_halo_p2p(const std::vector<Array*>& arrays, bool has_prev, bool has_next, cudaStream_t st) {
    HaloArgs h;
    h.nparts = (int)arrays.size();
    double total = 0;
    for (size_t q = 0; q < arrays.size(); ++q) {
        Array* a = arrays[q];
        const size_t esz = dtype_size(a->dtype);
        const size_t bytes = (size_t)a->halo * a->unit * esz;
        const int64_t nl = a->local_rows();
        h.bytes[q] = bytes;
        h.first_rows[q] = a->buf.data;
        h.last_rows[q] = a->buf.data + ((size_t)nl * a->unit * esz - bytes);
        h.halo_below[q] = a->buf.data - bytes;
        h.halo_above[q] = a->buf.data + (size_t)nl * a->unit * esz;
        total += (double)bytes;
    }
    if (has_prev) h.epoch_prev = ++peer_.epoch_prev;
    if (has_next) h.epoch_next = ++peer_.epoch_next;
    h.me = peer_.mine;
    h.box_prev = has_prev ? peer_.box[rank_ - 1] : nullptr;
    h.box_next = has_next ? peer_.box[rank_ + 1] : nullptr;
    h.ticket = peer_.ticket;
    h.error = error_word_;
    prof_start("halo exchange (peer stores)", total * ((has_prev ? 2 : 0) + (has_next ? 2 : 0)), st);
    int rc = cuda_fail(launch_halo_exchange(h, sm_count_, st), "halo exchange");
    prof_stop();
    if (rc) return rc;
    stats_.kernel_launches++;
    waiting_launches_++;
    stats_.peer_exchanges++;
    return CN_OK;
}

// Test hook for the failure path of the peer transport, without a second GPU and without
// hanging anything: one halo exchange against a scratch mailbox that plays both this rank and
// its neighbour.  The kernel publishes its rows, then waits for rows that nobody sends; the
// short bound runs out, the kernel sets the error word and returns, and the next synchronise
// reports it as a status code.
int Context::debug_peer_wait() {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    cudaSetDevice(device_);
    const size_t box_bytes = sizeof(CnPeerBox) + 4ull * CN_PEER_HALO_SLOT;
    void* box = nullptr;
    unsigned int* ticket = nullptr;
    int rc = cuda_fail(cudaMalloc(&box, box_bytes), "scratch mailbox");
    if (rc) return rc;
    if ((rc = cuda_fail(cudaMalloc((void**)&ticket, 256), "scratch mailbox"))) return rc;
    cudaMemsetAsync(box, 0, sizeof(CnPeerBox) + 64, stream_);
    cudaMemsetAsync(ticket, 0, 256, stream_);
    HaloArgs h;
    h.bytes[0] = 64;
    h.epoch_prev = 2;
    h.me = box;
    h.box_prev = box;
    h.first_rows[0] = (const char*)box + sizeof(CnPeerBox);      // any 64 readable bytes
    h.halo_below[0] = (char*)box + sizeof(CnPeerBox) + 256;
    h.ticket = ticket;
    h.error = error_word_;
    h.wait_limit = 20000;
    rc = cuda_fail(launch_halo_exchange(h, sm_count_, stream_), "halo exchange");
    waiting_launches_++;
    stats_.kernel_launches++;
    cudaStreamSynchronize(stream_);
    cudaFree(box);
    cudaFree(ticket);
    return rc;
}

int Context::ensure_scratch(size_t bytes) {
    if (scratch_bytes_ >= bytes) return CN_OK;
    if (scratch_) {
        cudaStreamSynchronize(stream_);
        cudaFree(scratch_);
        scratch_ = nullptr;
        scratch_bytes_ = 0;
    }
    int rc = cuda_fail(cudaMalloc(&scratch_, bytes), "scratch allocation");
    if (rc) return rc;
    scratch_bytes_ = bytes;
    return CN_OK;
}

// ---- DAG execution ----------------------------------------------------------------------

int Context::receive_dag(int epoch, int64_t size, const char* msg) {
    (void)epoch;
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    for (int r = 0; r < nranks_; ++r)
        if (failed_[r]) return fail(CN_ERR_RANK_FAILED, "rank " + std::to_string(r) + " was marked failed");
    cudaSetDevice(device_);
    // the epoch (bytes 4..8) is the only field that differs between two runs of one step
    uint64_t h = 1469598103934665603ULL;
    const bool cacheable = plan_cache_ && msg && size >= 8;
    if (cacheable) {
        int64_t b = 0;
        for (; b + 8 <= size; b += 8) {
            uint64_t w;
            memcpy(&w, msg + b, 8);
            if (b == 0) w &= 0xffffffffULL;  // little-endian: the magic stays, the epoch goes
            h = (h ^ w) * 0x9E3779B97F4A7C15ULL;
            h ^= h >> 29;
        }
        for (; b < size; ++b) h = (h ^ (unsigned char)msg[b]) * 1099511628211ULL;
        auto it = plans_.find(h);
        if (it != plans_.end()) {
            Plan& p = it->second;
            if ((int64_t)p.blob.size() == size && p.staged_level == staged_level() &&
                memcmp(p.blob.data(), msg, 4) == 0 && memcmp(p.blob.data() + 8, msg + 8, (size_t)size - 8) == 0) {
                stats_.plan_hits++;
                return run_plan(p);
            }
        }
    }
    Plan plan;
    int rc = parse_dag(msg, size, &plan.dag, &err_);
    if (rc) return rc;
    plan.staged_level = staged_level();
    recording_ = cacheable ? &plan : nullptr;
    size_t i = 0;
    while (i < plan.dag.nodes.size()) {
        const size_t start = i, had = plan.steps.size();
        rc = execute_node(plan.dag, &i);
        if (rc) {
            recording_ = nullptr;
            return rc;
        }
        if (recording_ && plan.steps.size() == had) {
            PlanStep st;  // a node that is not a lowered group: replayed through execute_node
            st.index = start;
            plan.steps.push_back(std::move(st));
        }
    }
    recording_ = nullptr;
    for (int name : plan.dag.deletes)
        if (find(name)) delete_array(name);
    if (cacheable) {
        if (plans_.size() >= 256) plans_.clear();
        plan.blob.assign(msg, (size_t)size);
        plans_[h] = std::move(plan);
    }
    return CN_OK;
}

int Context::run_plan(Plan& plan) {
    for (PlanStep& st : plan.steps) {
        int rc;
        if (st.group) {
            stats_.nodes += 1 + (long long)(st.fused + st.tails);
            rc = run_lowered(st.g, st.k);
            if (rc == CN_OK) {
                stats_.fused_reductions += (long long)st.fused;
                stats_.scalar_tails += (long long)st.tails;
            }
        } else {
            size_t i = st.index;
            rc = execute_node(plan.dag, &i);
        }
        if (rc) return rc;
    }
    for (int name : plan.dag.deletes)
        if (find(name)) delete_array(name);
    return CN_OK;
}

static bool is_group_node(const DagNode& n) {
    if (n.roots.empty()) return false;
    bool any = false;
    for (auto& r : n.roots) {
        int op = r->opcode;
        if (op == OP_NOOP) continue;
        if (is_elementwise(op) || op == OP_SET_REGION || op == OP_COPY) any = true;
        else if ((op == OP_SUM || op == OP_REDUCE) && n.fusible && n.roots.size() > 1)
            continue;  // terminal reduction inside a fusible group
        else return false;
    }
    return any;
}

int Context::execute_node(const Dag& dag, size_t* index) {
    const DagNode& node = dag.nodes[*index];
    stats_.nodes++;
    if (node.roots.empty()) {
        ++*index;
        return CN_OK;
    }
    // an assignment whose source has another rank (or its singleton dimensions elsewhere)
    if (node.roots.size() == 1 && node.roots[0]->opcode == OP_SET_REGION && node.roots[0]->operands.size() == 2) {
        const AstNode& r = *node.roots[0];
        const Operand& rhs = r.operands[1];
        if (!rhs.is_ref && rhs.leaf && r.operands[0].leaf && !rhs.leaf->is_scalar && !rhs.leaf->is_broadcast) {
            const AstNode& tl = *r.operands[0].leaf;
            const Region sreg = rhs.region.is_global ? Region::full(rhs.leaf->ndims, rhs.leaf->shape) : rhs.region;
            const Region treg = r.region.is_global ? Region::full(tl.ndims, tl.shape) : r.region;
            bool same = sreg.ndims == treg.ndims;
            for (int d = 0; same && d < sreg.ndims; ++d) same = sreg.extent(d) == treg.extent(d);
            if (!same && sreg.size() > 1) {
                ++*index;
                return execute_cross_set_region(r);
            }
        }
    }
    if (is_group_node(node)) {
        // REDUCE / SUM nodes that directly follow a group may be folded into its kernel
        auto scan_reductions = [&](size_t from, size_t* end) {
            std::vector<const AstNode*> found;
            size_t j = from;
            while (fuse_reductions_ && j < dag.nodes.size() && (int)found.size() < CN_MAX_RED) {
                const DagNode& nx = dag.nodes[j];
                if (nx.roots.size() != 1) break;
                const AstNode* r = nx.roots[0].get();
                if (r->opcode != OP_REDUCE && r->opcode != OP_SUM) break;
                bool ok = true;
                for (auto& op : r->operands)
                    if (op.is_ref || !op.leaf || op.leaf->is_scalar) ok = false;
                if (!ok) break;
                found.push_back(r);
                ++j;
            }
            *end = j;
            return found;
        };
        // A whole-array assignment followed by a stencil over the array it assigns runs as one
        // kernel: staged (the assigned values are computed tile by tile in shared memory) where
        // that form fits, otherwise recomputed at every stencil point.
        DagNode merged, consumer, producer;
        const DagNode* gnode = &node;
        size_t after = *index + 1;
        GroupIR probe;
        bool lowered = false;
        std::vector<const AstNode*> fused;
        size_t j = after;
        int rc = CN_OK;
        if (fuse_producers_ > 0 && after < dag.nodes.size() && is_group_node(dag.nodes[after])) {
            int pseudo = 0, target = 0;
            if (fuse_producers_ >= 2 && stage_producer(node, dag.nodes[after], &consumer, &producer, &pseudo, &target)) {
                size_t end = after + 1;
                std::vector<const AstNode*> behind = scan_reductions(after + 1, &end);
                std::string terr;
                if (lower_staged_producer(consumer, producer, pseudo, target, behind, &probe, &terr) == CN_OK) {
                    lowered = true;
                    fused = behind;
                    j = end;
                } else if (!behind.empty() &&
                           lower_staged_producer(consumer, producer, pseudo, target, {}, &probe, &terr) == CN_OK) {
                    lowered = true;
                    j = after + 1;
                }
                if (lowered) {
                    gnode = &consumer;
                    stats_.nodes++;
                    stats_.inlined_producers++;
                }
            }
            if (!lowered && inline_producer(node, dag.nodes[after], &merged)) {
                GroupIR trial;
                std::string terr;
                if (lower_group(merged, {}, &trial, &terr) == CN_OK && trial.cls == GroupIR::SHIFTED && !trial.flat) {
                    gnode = &merged;
                    ++after;
                    stats_.nodes++;
                    stats_.inlined_producers++;
                }
            }
        }
        if (!lowered) {
            bool done = false;
            rc = gnode == &node ? try_plain_fill(node, &done) : CN_OK;
            if (rc) return rc;
            if (done) {
                ++*index;
                return CN_OK;
            }
            fused = scan_reductions(after, &j);
            if (!fused.empty()) {
                std::string perr;
                int lrc = lower_group(*gnode, fused, &probe, &perr);
                bool related = false;
                if (lrc == CN_OK && probe.cls == GroupIR::SHIFTED) {
                    // only worth fusing when a reduction operand is produced or read by the group
                    for (auto& rd : probe.reds)
                        for (const ValRef* v : {&rd.a, &rd.b}) {
                            if (v->kind == ValRef::OUTVAL || v->kind == ValRef::ROOT) related = true;
                            if (v->kind == ValRef::LEAF)
                                for (auto& l : probe.leaves)
                                    if (&l != &probe.leaves[v->idx] && l.name == probe.leaves[v->idx].name)
                                        related = true;
                        }
                }
                if (lrc != CN_OK || probe.cls != GroupIR::SHIFTED || !related) {
                    fused.clear();
                    j = after;
                } else {
                    lowered = true;  // the probe is the group as it will run
                }
            }
            if (!lowered) {
                probe = GroupIR();
                if ((rc = lower_group(*gnode, fused, &probe, &err_))) return rc;
            }
        }
        // A scalar-only node behind the fused reductions (beta = r.r / rtr; res = sum) is
        // evaluated by the thread that finishes the reductions.  On several ranks that needs
        // the reductions finished inside the kernel (peer mailboxes), not by a collective
        // behind it.
        size_t tail_nodes = 0;
        if (fuse_scalar_tail_ && probe.cls == GroupIR::SHIFTED && !probe.reds.empty() && probe.tail.empty() &&
            j < dag.nodes.size() && is_group_node(dag.nodes[j]) && (nranks_ == 1 || peer_.ready)) {
            GroupIR t;
            std::string terr;
            if (lower_group(dag.nodes[j], {}, &t, &terr) == CN_OK && t.cls == GroupIR::SCALAR_ONLY &&
                t.dtype == probe.dtype && !t.souts.empty()) {
                size_t sc = probe.scalars.size() + t.scalars.size(), bc = probe.bcast_names.size() + t.bcast_names.size();
                if (!probe.producer.empty()) {
                    sc += probe.producer[0].scalars.size();
                    bc += probe.producer[0].bcast_names.size();
                }
                bool fits = sc <= CN_MAX_SC && bc <= CN_MAX_BC && probe.souts.size() + t.souts.size() <= CN_MAX_SOUT;
                // a size-1 result of the group itself goes to a fresh buffer that is swapped in
                // after the launch: the tail could not read it, nor write the same array
                for (auto& so : probe.souts) {
                    for (int name : t.bcast_names) fits = fits && name != so.name;
                    for (auto& ts : t.souts) fits = fits && ts.name != so.name;
                }
                if (fits) {
                    probe.tail.push_back(t);
                    tail_nodes = 1;
                    ++j;
                }
            }
        }
        CompiledGroup* k = nullptr;
        if ((rc = get_kernel(probe, &k))) return rc;
        if (recording_) {
            PlanStep st;
            st.index = *index;
            st.group = true;
            st.fused = fused.size();
            st.tails = tail_nodes;
            st.g = probe;
            st.k = k;
            recording_->steps.push_back(std::move(st));
        }
        int rc2 = run_lowered(probe, k);
        if (rc2) return rc2;
        stats_.fused_reductions += (long long)fused.size();
        stats_.nodes += (long long)(fused.size() + tail_nodes);
        stats_.scalar_tails += (long long)tail_nodes;
        *index = j;
        return CN_OK;
    }
    ++*index;
    int last = CN_OK;
    for (auto& r : node.roots) {
        switch (r->opcode) {
            case OP_NOOP: break;
            case OP_CREATE: last = execute_create(*r); break;
            case OP_REDUCE:
            case OP_SUM: last = execute_reduce(*r); break;
            case OP_MATMUL: last = execute_matmul(*r); break;
            case OP_RANDU: last = execute_randu(*r); break;
            case OP_DIAG: last = execute_diag(*r); break;
            case OP_TILE: last = execute_tile(*r); break;
            case OP_MATMATMUL:
            case OP_GET_REGION:
                return fail(CN_ERR_UNSUPPORTED, "opcode " + std::to_string(r->opcode) +
                                                    " is outside this backend's scope");
            default:
                return fail(CN_ERR_BAD_OPCODE, "unknown opcode " + std::to_string(r->opcode));
        }
        if (last) return last;
    }
    return CN_OK;
}

int Context::execute_create(const AstNode& r) {
    if (r.ndims < 1) return fail(CN_ERR_INVALID_ARGUMENT, "CREATE without a shape");
    return create_array(r.result_name, r.ndims, r.shape, r.dtype, true, nullptr);
}

// A group that is nothing but SET_REGION(target, literal) nodes needs no generated kernel
// (the reference routes these to its interpreter too, src/execute_node.cpp:108-110).
int Context::try_plain_fill(const DagNode& node, bool* done) {
    *done = false;
    for (auto& r : node.roots) {
        if (r->opcode != OP_SET_REGION || r->operands.size() != 2) return CN_OK;
        const Operand& rhs = r->operands[1];
        if (rhs.is_ref || !rhs.leaf || !rhs.leaf->is_scalar) return CN_OK;
        if (!r->operands[0].leaf) return CN_OK;
    }
    for (auto& r : node.roots) {
        const AstNode* t = r->operands[0].leaf.get();
        Array* a = find(t->result_name);
        if (!a) return fail(CN_ERR_UNKNOWN_ARRAY, "SET_REGION target " + std::to_string(t->result_name) + " does not exist");
        int rc = check_leaf(a, t->ndims, t->shape, "SET_REGION target");
        if (rc) return rc;
        Region reg = r->region.is_global ? Region::full(a->ndims, a->shape) : r->region;
        if (reg.ndims != a->ndims) return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION region rank differs from target");
        for (int d = 0; d < a->ndims; ++d)
            if (reg.stop[d] > a->shape[d]) return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION region outside its target");
        // rows of the region that live on this rank
        int64_t s0 = reg.start[0], st0 = reg.step[0];
        int64_t first = s0;
        if (first < a->row_begin) first = s0 + (a->row_begin - s0 + st0 - 1) / st0 * st0;
        int64_t stop0 = std::min<int64_t>(reg.stop[0], a->row_end);
        int64_t n0 = first < stop0 ? (stop0 - first + st0 - 1) / st0 : 0;
        StridedView v;
        int64_t ext[3] = {1, 1, 1};
        int64_t strides[3] = {0, 0, 0};
        strides[a->ndims - 1] = 1;
        for (int d = a->ndims - 2; d >= 0; --d) strides[d] = strides[d + 1] * a->shape[d + 1];
        // iteration dims are right-aligned into 3 slots
        int shift = 3 - a->ndims;
        v.off = (first - a->row_begin) * strides[0];
        for (int d = 0; d < a->ndims; ++d) {
            ext[shift + d] = d == 0 ? n0 : reg.extent(d);
            v.str[shift + d] = reg.step[d] * strides[d];
            if (d > 0) v.off += reg.start[d] * strides[d];
        }
        if (n0 > 0 && ext[1] > 0 && ext[2] > 0 && ext[0] > 0) {
            rc = cuda_fail(launch_fill_region(a->buf.data, a->dtype, v, ext, r->operands[1].leaf->scalar, stream_), "fill");
            if (rc) return rc;
            stats_.kernel_launches++;
        }
        a->mark_written();
    }
    *done = true;
    return CN_OK;
}

}  // namespace cn
