// The per-GPU execution context: array table, slab partition, DAG executor, kernel cache.
//
// One context = one rank = one GPU.  It takes the place of the reference's
// ArrayDAGGroup + PartitionImpl<N> + ArrayDAGExecutorND<N> trio (src/backend.hpp:239-582):
// instead of over-decomposed chare tiles there is exactly one slab per array per GPU,
// split along dimension 0, with `halo` extra rows (planes) on each side when more than
// one rank takes part.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "cn_device.cuh"
#include "cn_types.hpp"
#include "comm.hpp"
#include "group_ir.hpp"
#include "jit.hpp"

namespace cn {

struct Lattice;

struct Buffer {
    void* alloc = nullptr;  // start of the allocation
    char* data = nullptr;   // address of local element (0,0,0)
    size_t bytes = 0;
};

struct Array {
    int name = -1;
    int ndims = 0;
    int64_t shape[kMaxDims] = {0, 0, 0};
    int dtype = DT_F64;
    bool replicated = false;  // size-1 arrays live on every rank
    int64_t row_begin = 0, row_end = 0;  // local range of dimension 0
    int64_t unit = 1;                    // elements per index of dimension 0
    int halo = 0;                        // halo rows allocated on each side
    Buffer buf, shadow;
    int halo_fresh = 0;  // halo rows (per side) that hold the neighbours' current values, 0..halo
    bool halo_pushed = false;  // the producing kernel stored the current edge rows into the neighbours' mailboxes
    bool halo_wanted = false;  // a stencil has asked for this array's halo before: worth pushing

    // the array's own rows changed by a path that neither widens nor pushes: the halo is stale
    void mark_written() {
        halo_fresh = 0;
        halo_pushed = false;
    }

    int64_t local_rows() const { return row_end - row_begin; }
    int64_t local_elems() const { return local_rows() * unit; }
    int64_t global_elems() const {
        int64_t n = 1;
        for (int d = 0; d < ndims; ++d) n *= shape[d];
        return n;
    }
};

struct CompiledGroup {
    CUmodule module = nullptr;
    CUfunction func = nullptr;
    int blocks_per_sm = 1;  // resident 256-thread blocks per SM, from the occupancy query
    std::string label;      // short description used by the profile report
    TileConfig tile;        // tile shape the kernel was compiled for
    size_t smem_bytes = 0;  // dynamic shared memory (staged kernels)
    std::string source;
    std::string log;
};

// A DAG blob that has run once keeps what was derived from its bytes alone: the parsed
// nodes, which reductions were folded into which group, each group's lowered form and its
// compiled kernel.  Running the same bytes again skips parsing, lowering and the kernel
// cache's string keys; everything that depends on the array table (existence, shapes,
// buffers, halos) is still resolved per run.
struct PlanStep {
    size_t index = 0;     // node this step starts at
    bool group = false;   // a lowered group (g, k valid); otherwise the node runs generically
    size_t fused = 0;     // REDUCE / SUM nodes folded into the group
    size_t tails = 0;     // scalar-only nodes folded in behind them
    GroupIR g;
    CompiledGroup* k = nullptr;
};

struct Plan {
    std::string blob;
    int staged_level = 0;  // process-wide staging level the groups were lowered under
    Dag dag;
    std::vector<PlanStep> steps;
};

struct Stats {
    long long kernel_launches = 0;   // kernels of this library launched (AOT + generated)
    long long group_launches = 0;    // of which generated group kernels
    long long staged_launches = 0;   // of which TMA-staged stencil kernels
    long long compiles = 0;          // NVRTC compilations (cache misses)
    long long halo_exchanges = 0;
    long long allreduces = 0;
    long long fused_reductions = 0;  // REDUCE/SUM nodes folded into a group kernel
    long long nodes = 0;             // DAG nodes executed
    long long bytes_h2d = 0, bytes_d2h = 0;
    long long plan_hits = 0;         // DAGs served from the plan cache
    long long peer_exchanges = 0;    // reductions finished / halos moved through the peer mailboxes
    long long overlapped_sweeps = 0; // stencil sweeps whose interior ran beside the halo exchange
    long long deep_halo_sweeps = 0;  // stencil sweeps that also updated halo rows (no exchange needed next)
    long long halo_pushes = 0;       // kernels that stored their edge rows into the neighbours' mailboxes themselves
    long long row_fetches = 0;       // operands whose rows were fetched from other ranks for a strided group
    long long inlined_producers = 0; // whole-array assignments folded into the stencil kernel that reads them
    long long scalar_tails = 0;      // scalar-only nodes evaluated inside the kernel that finished the reductions they read
};

struct DriverApi {
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                             unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*OccupancyMaxActiveBlocksPerMultiprocessor)(int*, CUfunction, int, size_t) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*FuncGetAttribute)(int*, CUfunction_attribute, CUfunction) = nullptr;
    CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                     CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                     CUtensorMapFloatOOBfill) = nullptr;
};

void slab_partition(int64_t n0, int nranks, int rank, int64_t* begin, int64_t* end);

class Context {
public:
    Context(int device, int rank, int nranks);
    ~Context();
    int init();  // binds the device, creates streams and scratch; CN_ERR_NO_DEVICE without a GPU

    // ---- boundary entry points (see include/cnb200.h) ----
    int comm_init_id(const char id[128]);
    int receive_dag(int epoch, int64_t size, const char* msg);
    int get(int name, int64_t count, int dtype, void* out);
    int get_local(int name, int64_t* row_begin, int64_t* row_end, int64_t capacity, void* out);
    int get_root(int name, int64_t count, int dtype, int root, void* out);
    int put_local(int name, int ndims, const int64_t* shape, int dtype, int64_t capacity, const void* host_slab);
    int execute_single_node(const char* blob, int64_t size);
    int put(int name, int ndims, const int64_t* shape, int dtype, const void* host);
    int delete_array(int name);
    int synchronize();
    int compile_group(const char* blob, int64_t size, uint64_t* handle);
    int group_source(uint64_t handle, const char** src);
    int launch_group(uint64_t handle, int n_in, void* const* in_ptrs, const int64_t* in_off,
                     const int64_t* in_str, int n_bc, void* const* bc_ptrs, int n_out,
                     void* const* out_ptrs, const int64_t* out_off, const int64_t* out_str,
                     const int64_t* ext);
    int timer_start();
    int timer_stop(float* ms);
    void set_profile(bool on) { profile_ = on; }
    int profile_report(char* buf, int64_t cap);
    int mark_rank_failed(int r);
    int debug_peer_wait();  // test hook: a halo exchange whose partner never answers
    int array_info(int name, int* ndims, int64_t* shape, int* dtype, int64_t* row_begin,
                   int64_t* row_end);

    const std::string& last_error() const { return err_; }
    const Stats& stats() const { return stats_; }
    int rank() const { return rank_; }
    int nranks() const { return nranks_; }
    // every option that lowering or kernel selection looks at drops the cached plans
    void set_halo(int h) { halo_ = h; plans_.clear(); }
    void set_fuse_reductions(bool f) { fuse_reductions_ = f; plans_.clear(); }
    void set_tile(int tx, int r) {
        if (tx > 0) tile_.tx = tx;
        if (r > 0) tile_.r = r;
        tile_set_ = true;
        plans_.clear();
    }
    void set_staged_tile(int tx, int r) {
        if (tx > 0) staged_tile_.tx = tx;
        if (r > 0) staged_tile_.r = r;
        staged_tile_set_ = true;
        plans_.clear();
    }
    void set_debug_drop_copies(bool on) { debug_drop_copies_ = on; plans_.clear(); }
    void set_flat_prefetch(int mode) { flat_prefetch_ = mode; plans_.clear(); }
    void set_fuse_producers(int mode) { fuse_producers_ = mode; plans_.clear(); }
    void set_fuse_scalar_tail(bool on) { fuse_scalar_tail_ = on; plans_.clear(); }
    void set_stencil_shfl(bool on) { stencil_shfl_ = on; plans_.clear(); }
    void set_dependent_launch(bool on) { dependent_launch_ = on; }
    void set_plan_cache(bool on) { plan_cache_ = on; plans_.clear(); }
    void set_overlap_halo(bool on) { overlap_halo_ = on; }
    void set_deep_halo(bool on) { deep_halo_ = on; }
    void set_p2p(bool on) { p2p_wanted_ = on; }
    void set_push_halo(bool on) { push_halo_ = on; plans_.clear(); }  // takes effect at cn_comm_init
    bool p2p_ready() const { return peer_.ready; }

private:
    int fail(int code, const std::string& msg);
    int cuda_fail(cudaError_t e, const char* what);
    int driver_fail(CUresult r, const char* what);

    // arrays
    Array* find(int name);
    int create_array(int name, int ndims, const int64_t* shape, int dtype, bool zero, Array** out);
    int alloc_buffer(const Array& a, Buffer* b);
    void free_buffer(Buffer* b);
    int ensure_shadow(Array* a);
    int check_leaf(const Array* a, int ndims, const int64_t* shape, const char* what);
    void partition(int64_t n0, int64_t* begin, int64_t* end, int r) const;

    // execution
    int execute_node(const Dag& dag, size_t* index);
    int run_plan(Plan& plan);
    int run_lowered(const GroupIR& g, CompiledGroup* k);
    int report_error_word(unsigned int word);
    int bind_tail(const GroupIR& g, CnGroupArgs* a);
    int run_shifted(const GroupIR& g, CompiledGroup* k);
    int run_strided(const GroupIR& g, CompiledGroup* k);
    int run_scalar_only(const GroupIR& g, CompiledGroup* k);
    int bind_scalars(const GroupIR& g, CnGroupArgs* a, std::vector<std::pair<Array*, Buffer>>* swaps);
    int bind_reductions(const GroupIR& g, CnGroupArgs* a, int grid, std::vector<Array*>* results);
    int finish_reductions(const std::vector<Array*>& results, bool in_kernel);
    int launch(CompiledGroup* k, const CnGroupArgs& a, int grid, int block, double bytes, cudaStream_t st = nullptr);
    void prof_start(const std::string& label, double bytes, cudaStream_t st = nullptr);
    void prof_stop();
    int get_kernel(const GroupIR& g, CompiledGroup** out);
    int execute_reduce(const AstNode& root);
    int execute_matmul(const AstNode& root);
    int execute_randu(const AstNode& root);
    int execute_diag(const AstNode& root);
    int execute_cross_set_region(const AstNode& root);
    int execute_tile(const AstNode& root);
    int execute_create(const AstNode& root);
    int try_plain_fill(const DagNode& node, bool* done);
    int exchange_halo(Array* a, cudaStream_t st);
    int fetch_operand_rows(Array* x, const struct Lattice& anchor, int64_t anchor_n0, const struct Lattice& lv, char** data,
                           int64_t* base_row, std::vector<void*>* fetched);
    int exchange_halos(const std::vector<Array*>& arrays, cudaStream_t st);
    int pull_pending(cudaStream_t st);
    void plan_push(const GroupIR& g, const std::vector<Array*>& outs, int64_t ext, CnGroupArgs* a,
                   std::vector<Array*>* pushed);
    int exchange_halo_p2p(const std::vector<Array*>& arrays, bool has_prev, bool has_next, cudaStream_t st);
    int ensure_second_stream();
    int setup_peer_boxes();
    void bind_peers(CnGroupArgs* a);
    int ensure_scratch(size_t bytes);
    int encode_tensor_map(const Array& x, const CompiledGroup& k, const GroupIR& g, CnGroupArgs* a);
    int check_device_error();
    int operand_array(const Operand& op, Array** out, Region* region);

    int device_, rank_, nranks_;
    int halo_ = 1;
    bool fuse_reductions_ = true;
    bool debug_drop_copies_ = false;  // test hook: staged kernels issue no tile copies
    int flat_prefetch_ = -1;          // flat kernels' load placement (TileConfig::prefetch); -1: chosen per group
    int staged_ns_ = 0;               // ring depth of staged 3-D kernels (0: default)
    bool staged_tile_set_ = false;    // the staged tile shape was chosen by the caller
    bool tile_set_ = false;           // the tile shape of the other kernels was chosen by the caller
    // a scalar-only node behind fused reductions runs inside their kernel.  One launch fewer per
    // CG iteration and per residual sweep, but no time: with dependent launches the size-1 kernel
    // costs nothing measurable (CG 8192^2 890.6 against 891.4 us, Jacobi2D 10.27 against
    // 10.21 us per step), so the option is off
    bool fuse_scalar_tail_ = false;
    int fuse_producers_ = 2;          // a whole-array assignment + the stencil that reads it as one kernel:
                                      // 0 never, 1 recomputed per stencil point, 2 staged in shared memory where it fits
    // generated kernels are launched with programmatic stream serialisation: a kernel's launch
    // is released when the blocks of the kernel before it have exited, without waiting for that
    // kernel to drain (each kernel waits for its predecessor's completion before it touches
    // memory).  Measured: Jacobi2D 2048^2 14.2 -> 12.1 us per sweep, CG 8192^2 888 -> 882 us
    bool dependent_launch_ = true;
    // resident blocks per SM the cache-served stencil kernels are compiled for (a register cap);
    // measured on the 5-point sweep, 1 (no cap) / 6 / 8: 12.2 / 10.6 / 10.7 us at 2048^2,
    // 195 / 178 us at 8192^2, 875 / 750 us at 16384^2; larger groups spill at 7 and 8
    int shifted_minb_ = 6;
    // the same cap for flat kernels (1: none).  Measured without effect: the CG update kernel
    // at 40 registers / 6 blocks takes 522 us against 519 us at 48 / 5
    int flat_minb_ = 1;
    bool stencil_shfl_ = false;       // cache-served stencil kernels take x-neighbours by warp shuffle
    bool plan_cache_ = true;
    std::unordered_map<uint64_t, Plan> plans_;  // keyed by a hash of the blob bytes
    Plan* recording_ = nullptr;                 // plan being recorded by the running receive_dag
    bool initialised_ = false;
    int sm_count_ = 148;
    cudaStream_t stream_ = nullptr;
    // second stream of the overlapped sweeps: halo exchange and the slab's edge rows run here
    // while the interior runs on stream_; it is always joined back before anything else happens
    cudaStream_t stream2_ = nullptr;
    cudaEvent_t ev_fork_ = nullptr, ev_join_ = nullptr;
    cudaStream_t prof_stream_ = nullptr;
    bool deep_halo_ = true;      // with halo > 1: sweeps also update halo rows, fewer exchanges
    bool overlap_halo_ = false;  // measured: no gain at 2048^2, a loss at 1024^3 (the halo kernel's
                                 // blocks queue behind the persistent interior blocks)
    cudaEvent_t ev_start_ = nullptr, ev_stop_ = nullptr;
    Comm comm_;
    // Peer mailboxes (one per rank, mapped into every rank of the box through CUDA IPC):
    // reductions finish inside the producing kernel and halos travel as peer stores, with
    // NCCL as the fallback when the mapping cannot be set up.
    struct PeerState {
        bool ready = false;
        void* mine = nullptr;                 // this rank's CnPeerBox + payload slots
        void* box[CN_MAX_PEERS] = {nullptr};  // every rank's box as mapped here (box[rank_] == mine)
        unsigned long long red_epoch = 0;             // fused reductions so far (all ranks take part in each)
        unsigned long long epoch_prev = 0, epoch_next = 0;  // halo exchanges with rank - 1 / rank + 1
        unsigned int* ticket = nullptr;       // block counter of the halo kernel
    } peer_;
    // Edge rows pushed by the kernels that produced them (one exchange epoch, up to CN_HALO_PARTS
    // arrays), waiting for the small kernel that publishes them, waits for the neighbours' and
    // copies those into the local halo rows.
    struct PendingPush {
        bool active = false;
        std::vector<int> names;     // arrays of the group, in payload order
        std::vector<size_t> bytes;  // halo bytes per direction of each
        bool has_prev = false, has_next = false;
        unsigned long long epoch_prev = 0, epoch_next = 0;
    } pending_;
    std::vector<int> halo_group_;   // arrays whose halos were last asked for together
    bool push_halo_ = false;        // option "push_halo": measured slower than the stand-alone exchange, off
    bool p2p_wanted_ = true;
    long long waiting_launches_ = 0;          // launches that contain a bounded wait (TMA, peers)
    long long checked_launches_ = 0;          // of which already covered by an error-word check
    std::vector<bool> failed_;
    DriverApi drv_;
    TileConfig tile_;
    TileConfig staged_tile_;   // tile shape of the TMA-staged stencil kernels
    unsigned int* error_word_ = nullptr;  // set by a kernel whose bounded wait ran out
    // 4 KiB of pinned host memory: small results (cn_get of a size-1 array) and the error word
    // come back through it as truly asynchronous copies behind one synchronisation, instead
    // of one staged copy into pageable memory each
    unsigned char* pinned_ = nullptr;
    enum { kPinnedBytes = 4096, kPinnedWord = 4096 - 64 };

    std::unordered_map<int, Array> arrays_;
    std::unordered_map<std::string, CompiledGroup> kernels_;
    std::vector<std::pair<std::string, GroupIR>> handles_;  // cn_compile_group handles

    double* partials_ = nullptr;  // CN_MAX_RED * max_grid_ accumulators
    unsigned int* counter_ = nullptr;
    int max_grid_ = 0;
    void* scratch_ = nullptr;  // matvec x gather / get staging
    size_t scratch_bytes_ = 0;

    // per-kernel CUDA-event timing (off by default; see cn_profile_report)
    struct ProfEntry {
        long long launches = 0;
        double bytes = 0;
        std::vector<std::pair<cudaEvent_t, cudaEvent_t>> events;
    };
    bool profile_ = false;
    std::map<std::string, ProfEntry> prof_;
    ProfEntry* prof_open_ = nullptr;

    std::string err_;
    Stats stats_;
};

}  // namespace cn
