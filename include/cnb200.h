/*
 * cnb200 -- C ABI of the B200 execution backend for charmnumeric's data-parallel hot path
 * (fused elementwise / stencil groups, dot and sum reductions, row-partitioned matvec over
 * slab-partitioned arrays).  Plain pointers and sizes only; every function returns a status
 * code (0 = ok) and never aborts the process.  One context drives one GPU; with N GPUs there
 * are N processes, each with one context of rank r in [0, N).
 *
 * Each entry point names the reference interface it stands in for (paths are relative to
 * the reference tree).
 */
#ifndef CNB200_H
#define CNB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cn_context cn_context;

/* status codes */
enum {
    CN_STATUS_OK = 0,
    CN_STATUS_INVALID_ARGUMENT = 1,
    CN_STATUS_BAD_BLOB = 2,
    CN_STATUS_UNKNOWN_ARRAY = 3,
    CN_STATUS_SHAPE_MISMATCH = 4,
    CN_STATUS_UNSUPPORTED = 5,
    CN_STATUS_BAD_OPCODE = 6,
    CN_STATUS_BAD_DTYPE = 7,
    CN_STATUS_CUDA = 8,
    CN_STATUS_COMPILE = 9,
    CN_STATUS_COMM = 10,
    CN_STATUS_HAZARD = 11,
    CN_STATUS_OUT_OF_MEMORY = 12,
    CN_STATUS_LIMIT = 13,
    CN_STATUS_RANK_FAILED = 14,
    CN_STATUS_NO_DEVICE = 15
};

/* opcode numbering: src/opcodes.hpp:3-20 == charmnumeric/charmnumeric.py:139-150;
 * values >= 11 are additions of this backend. */
enum {
    CN_OP_COPY = -5, CN_OP_SET_REGION = -4, CN_OP_GET_REGION = -3, CN_OP_CREATE = -2,
    CN_OP_NOOP = -1, CN_OP_ADD = 0, CN_OP_SUB = 1, CN_OP_MUL = 2, CN_OP_DIV = 3,
    CN_OP_MATMUL = 4, CN_OP_TANH = 5, CN_OP_EXP = 6, CN_OP_TILE = 7, CN_OP_REDUCE = 8,
    CN_OP_MATMATMUL = 9, CN_OP_DIAG = 10,
    CN_OP_SQRT = 11, CN_OP_ABS = 12, CN_OP_SUM = 13, CN_OP_RANDU = 14
};

/* dtype codes: charmnumeric/charmnumeric.py:37-40 */
enum { CN_DTYPE_F32 = 0, CN_DTYPE_F64 = 1, CN_DTYPE_I32 = 2, CN_DTYPE_I64 = 3 };

int cn_version(void);
const char* cn_status_string(int status);

/* Context life cycle.  Stands in for Main / ArrayDAGGroup construction and the chare
 * arrays it creates (src/server.cpp:7-20, src/dag_group_runtime.cpp:7-32).  Fails with
 * CN_STATUS_NO_DEVICE when no sm_100 GPU is visible: there is no CPU path. */
int cn_context_create(int device, int rank, int nranks, cn_context** out);
int cn_context_destroy(cn_context* ctx);
const char* cn_last_error(cn_context* ctx);

/* Multi-GPU wiring.  Stands in for `charmrun +pN` start-up and proxy broadcast
 * (charmnumeric/interface.py:74-92, src/dag_group_runtime.cpp:18-28).  Rank 0 obtains an
 * id, the host program hands the 128 bytes to every rank by any means, every rank calls
 * cn_comm_init with it. */
int cn_comm_unique_id(char id[128]);
int cn_comm_init(cn_context* ctx, const char id[128]);
/* Host-side failure notice: after a rank is marked failed every call that would need a
 * collective returns CN_STATUS_RANK_FAILED instead of starting it. */
int cn_mark_rank_failed(cn_context* ctx, int rank);

/* Execute one DAG.  Stands in for the entry method
 * ArrayDAGGroup::receive_dag(int epoch, int size, char msg[size]) (src/backend.ci:15,
 * src/dag_group_receive.cpp:191-575).  `msg` is a CNB1 blob (grammar: csrc/wire.cpp).
 * Work is enqueued on the context's stream; the call does not wait for the GPU. */
int cn_receive_dag(cn_context* ctx, int epoch, int64_t size, const char* msg);

/* Fetch a whole array as a row-major host buffer on every calling rank.  Stands in for
 * receive_get_request(int ndims, int epoch, int name, int size, int dtype) + gather +
 * send_reply (src/backend.ci:16-17, src/dag_group_runtime.cpp:55-118,
 * src/partition_get.cpp:3-67).  Waits for all enqueued work. */
int cn_get(cn_context* ctx, int ndims, int epoch, int name, int64_t count, int dtype, void* out);
/* The same gather onto ONE rank, as the reference does it (process_get sends every tile to
 * PE 0, which replies to the client: src/partition_get.cpp:3-67,
 * src/dag_group_runtime.cpp:99-118).  Every rank calls it; only `root` receives the array
 * (`out` may be NULL elsewhere): the other ranks send their slab to the root and hold no copy
 * of the whole array, on the device or on the host. */
int cn_get_root(cn_context* ctx, int ndims, int epoch, int name, int64_t count, int dtype,
                int root, void* out);
/* This rank's slab only (rows [*row_begin, *row_end) of dimension 0); out may be NULL to
 * query the range.  No counterpart in the reference (its chares are gathered on PE 0). */
int cn_get_local(cn_context* ctx, int name, int64_t* row_begin, int64_t* row_end,
                 int64_t capacity, void* out);
/* Bulk upload of a whole row-major host array; each rank copies its own slab.  No
 * counterpart in the reference, which assigns host data one SET_REGION per element
 * (charmnumeric/charmnumeric.py:863-878). */
int cn_put(cn_context* ctx, int name, int ndims, const int64_t* shape, int dtype,
           const void* host);

/* The slab-wise counterpart of cn_put: `host_slab` holds only the rows this rank owns
 * (cn_partition of shape[0]), `capacity` its length in elements.  No counterpart in the
 * reference. */
int cn_put_local(cn_context* ctx, int name, int ndims, const int64_t* shape, int dtype,
                 int64_t capacity, const void* host_slab);

/* Execute one DAG node at once.  Stands in for DAGExecutor::execute_dag_node(DAGNode*)
 * (src/backend.hpp:322-347, src/executor_core.cpp:194), which the reference's scheduler calls
 * once per ready node on every chare; `node_blob` is one `node` production of the CNB1 format
 * (what cn_compile_group takes).  Completion is stream-ordered (the reference reports
 * node_finished(node_id)); the status code is the result.  A one-node cn_receive_dag does
 * the same work plus the plan cache and the delete list. */
int cn_execute_node(cn_context* ctx, const char* node_blob, int64_t size);

/* DAGExecutor::delete_array(int name) (src/backend.hpp:334, src/executor_core.cpp:184-192). */
int cn_delete_array(cn_context* ctx, int name);
int cn_array_info(cn_context* ctx, int name, int* ndims, int64_t shape[3], int* dtype,
                  int64_t* row_begin, int64_t* row_end);
int cn_synchronize(cn_context* ctx);

/* Kernel-ABI level.  cn_compile_group stands in for ArrayDAGGroup::compile_node
 * (src/dag_group_compile.cpp:6-41): it takes one serialized group (the `node` production
 * of the CNB1 format) and returns a handle to the compiled kernel.  cn_launch_group stands
 * in for dispatch_kernel (src/dispatch.hpp:137-265): inputs in leaf discovery order, then
 * size-1 arrays, then outputs, each array argument as (device pointer, element offset,
 * element stride per dimension) -- the fields of the reference's MemRef descriptor
 * (src/array_region.hpp:406-415).  in_str / out_str hold ndims entries per argument. */
int cn_compile_group(cn_context* ctx, const char* node_blob, int64_t size, uint64_t* handle);
int cn_group_source(cn_context* ctx, uint64_t handle, const char** source);
int cn_launch_group(cn_context* ctx, uint64_t handle, int n_in, void* const* in_ptrs,
                    const int64_t* in_off, const int64_t* in_str, int n_bc,
                    void* const* bc_ptrs, int n_out, void* const* out_ptrs,
                    const int64_t* out_off, const int64_t* out_str, const int64_t* ext);

/* Host-only checks (no GPU needed): parse a DAG blob; lower + generate + compile one group
 * for sm_100a and return its CUDA source (truncated to cap-1 bytes) and cubin size. */
int cn_dag_check(const char* msg, int64_t size, int* n_nodes, int* n_roots, char* err, int errcap);
int cn_group_compile_check(const char* node_blob, int64_t size, char* source, int64_t cap,
                           int64_t* cubin_bytes, char* err, int errcap);

/* Host-only: would node_a (a whole-array elementwise assignment) and node_b (a stencil group
 * over the assigned array) run as one kernel?  *fused = 1 and the kernel's CUDA source when the
 * pair fits the pattern, lowers and compiles for sm_100a; *fused = 0 otherwise. */
int cn_fuse_check(const char* node_a, int64_t size_a, const char* node_b, int64_t size_b,
                  char* source, int64_t cap, int* fused, char* err, int errcap);

/* Host-only: a DAG of one group node, one or more REDUCE / SUM nodes the group's kernel can take
 * in, and a last node of size-1 arithmetic (CG's beta = r.r / rtr; rtr = r.r).  *fused = 1 and the
 * CUDA source of the single kernel when the last node runs as that kernel's scalar tail (see
 * option "fuse_scalar_tail") and the kernel compiles for sm_100a; *fused = 0 otherwise. */
int cn_tail_check(const char* dag_blob, int64_t size, char* source, int64_t cap, int* fused,
                  char* err, int errcap);

/* Host-only region algebra of the slab planner, on (start, stop, step) triples of row indices.
 * cn_region_intersect: common rows of two stepped regions (ArrayRegion intersect,
 * src/array_region.hpp:136-222).  cn_region_map: `part` is a piece of view `from`; the result is
 * the piece of view `to` at the same positions (map, src/array_region.hpp:461-536, pinned by
 * tests/test_jit.cpp:301-326).  cn_plan_row_transfers: a group iterates over `anchor` (the view
 * of its first output, an array of anchor_n0 rows) and reads `leaf` (a view of an array of
 * leaf_n0 rows); rank q executes the iteration rows whose anchor row it owns
 * (iteration_rows[2q], [2q+1], optional) and every (src, dst, row_lo, row_hi) quadruple in
 * `transfers` is a block of operand rows that has to travel (local_inputs /
 * send_remote_inputs, src/array_region.hpp:553-663). */
int cn_region_intersect(const int64_t a[3], const int64_t b[3], int64_t out[3]);
int cn_region_map(const int64_t part[3], const int64_t from[3], const int64_t to[3], int64_t out[3]);
int cn_plan_row_transfers(const int64_t anchor[3], int64_t anchor_n0, const int64_t leaf[3],
                          int64_t leaf_n0, int nranks, int64_t* transfers, int64_t cap,
                          int64_t* count, int64_t* iteration_rows);

/* Host-only: tile sizes and alignment offsets for the arrays a DAG creates, so that their tiles
 * line up with the tiles of the arrays they are computed from or stored into.  Stands in for
 * decomposition_solver::compute_decompositions(array_meta, dag, odf, num_pes)
 * (src/decomposition_solver.hpp:95; known answers: tests/test_compute_decompositions.cpp:128-396).
 * `arrays` is read and updated in place: entries with decomp_final != 0 are fixed, the others
 * receive a tile, an offset per dimension and decomp_final = 1 when the DAG relates them to a
 * fixed array.  `dag_blob` is a CNB1 blob (may be NULL: tiles only); `min_tile` gives the
 * minimum tile of 1-D / 2-D / 3-D arrays (NULL: 262144 / 512 / 64, src/backend.hpp:15-17).
 * The slab executor itself needs no per-array offsets; this is for hosts that keep tile grids. */
typedef struct cn_array_meta {
    int32_t name;
    int32_t ndims;
    int64_t shape[3];
    int64_t offset[3];
    int64_t tile;
    int32_t decomp_final;
    int32_t reserved;
} cn_array_meta;
int cn_compute_decompositions(cn_array_meta* arrays, int n_arrays, const char* dag_blob,
                              int64_t size, int odf, int num_pes, const int64_t min_tile[3]);

/* Rows [*begin, *end) of dimension 0 that `rank` of `nranks` owns for an array with n0 rows
 * (host-only).  Takes the place of the reference's tile -> chare map
 * (ArrayDecomp::owning_chare / chare_region_global, src/array_region.hpp:357-368): here one
 * slab of ceil(n0 / nranks) consecutive rows per rank. */
int cn_partition(int64_t n0, int nranks, int rank, int64_t* begin, int64_t* end);

/* Device timing with CUDA events on the context's own stream. */
int cn_timer_start(cn_context* ctx);
int cn_timer_stop(cn_context* ctx, float* milliseconds);

/* Per-kernel timing.  After cn_set_option(ctx, "profile", 1) every kernel launch of the
 * library is bracketed by CUDA events on the context's stream; cn_profile_report waits for
 * the stream, writes one line per kernel -- label <tab> launches <tab> total milliseconds
 * <tab> algorithmic bytes moved -- and clears the records.  No counterpart in the reference
 * (it has no timers at all). */
int cn_profile_report(cn_context* ctx, char* buf, int64_t cap);

/* Dot product that allocates nothing: result[0] = sum_i a[i] * b[i] for two float64 device
 * arrays of n elements, result a device pointer, launched on `stream` (a cudaStream_t, NULL
 * for the default stream) of the current device.  No counterpart in the reference.
 * For callers that cannot allocate device memory -- inside another runtime's callback, after
 * the application has claimed all memory as its own arena, on an out-of-memory error path,
 * or where touching the allocator is ruled out for latency or determinism.  The per-block
 * partial sums of the deterministic two-pass reduction live in a fixed 256 KiB array inside
 * the library image instead of an allocated buffer; this call makes no allocation or free of
 * its own.  Limit: n <= CN_NOALLOC_MAX_ELEMS (one partial per 8192 elements), otherwise
 * CN_STATUS_LIMIT and nothing is launched.  The first call on a device resolves the array's
 * device address, and with CUDA's lazy module loading it is also the moment the driver puts
 * the library's device image (this array included) into device memory: make that first call
 * as a warm-up (n = 0 is enough) while memory is still available and outside stream capture;
 * only the calls after it are allocation-free.  All calls on a device share the
 * array (the ticket counter is cleared on the stream before each launch); calls whose
 * kernels may overlap on the GPU race on it and must be ordered by the caller.  Needs no
 * context. */
#define CN_NOALLOC_MAX_ELEMS 268435456LL
int cn_dot_noalloc(const double* a, const double* b, int64_t n, double* result, void* stream);

/* Counters since context creation. */
typedef struct cn_stats {
    int64_t kernel_launches;   /* kernels of this library launched */
    int64_t group_launches;    /* of which generated group kernels */
    int64_t compiles;          /* run-time compilations (cache misses) */
    int64_t halo_exchanges;
    int64_t allreduces;
    int64_t fused_reductions;  /* REDUCE / SUM nodes folded into a group kernel */
    int64_t nodes;             /* DAG nodes executed */
    int64_t bytes_h2d;
    int64_t bytes_d2h;
    int64_t plan_hits;         /* DAGs whose bytes had run before (parsing and lowering skipped) */
    int64_t peer_exchanges;    /* reductions finished in-kernel / halos moved through peer mailboxes */
    int64_t overlapped_sweeps; /* stencil sweeps whose interior ran beside the halo exchange */
    int64_t deep_halo_sweeps;  /* stencil sweeps that also updated halo rows (see option "halo") */
    int64_t inlined_producers; /* whole-array assignments folded into the stencil kernel behind them */
    int64_t row_fetches;       /* operands of strided groups whose rows were fetched from other ranks */
    int64_t halo_pushes;       /* outputs whose edge rows the producing kernel stored into the neighbours' mailboxes */
    int64_t scalar_tails;      /* scalar-only nodes evaluated inside the kernel that finished the reductions they read */
} cn_stats;
int cn_get_stats(cn_context* ctx, cn_stats* out);

/* Options: "halo" depth (rows per side, 0..64, default 1; set before creating arrays; with a depth
 * above the stencil's reach, sweeps without a fused reduction also update the halo rows they can
 * (the neighbour computes the same values), so one exchange serves several sweeps; "deep_halo" 0
 * switches that off),
 * "fuse_reductions" 0/1, "tile_tx" / "tile_rows" (shape of generated kernels: threads along
 * the last dimension, rows per thread), "staged" 0/1/2 (TMA / shared-memory staging of stencil
 * tiles: never / 3-D groups only (default) / 2-D groups too; process-wide), "staged_tile_tx" /
 * "staged_tile_rows", "profile" 0/1, "plan_cache" 0/1 (default 1: a DAG blob whose bytes,
 * epoch aside, have run before skips parsing and lowering), "flat_prefetch" -1/0/1/2 (where flat
 * kernels place their loads: 0 next to their use, 1 the next tile's inputs are requested before
 * the arithmetic of the current one, 2 all loads of a tile ahead of its arithmetic; default -1:
 * 2 for groups heavy in exp / tanh / sqrt / division, 0 otherwise),
 * "p2p" 0/1 (default 1; read by cn_comm_init: map every rank's mailbox into every other rank
 * with CUDA IPC, finish reductions inside the producing kernel and move halo rows as NVLink
 * peer stores; when the mapping cannot be set up on all ranks, NCCL does both),
 * "overlap_halo" 0/1 (default 0: a stencil sweep without a fused reduction is cut along
 * dimension 0; the halo exchange and the rows next to the slab edges run on a second stream
 * beside the interior), "fuse_producers" 0/1/2 (a whole-array elementwise assignment
 * directly followed by a stencil group over the assigned array runs as one kernel instead of
 * writing the array and reading it back: 1 the assigned values are recomputed at every stencil
 * point, 2 (default) they are computed tile by tile, halo ring included, into shared memory
 * where that form fits (2-D float64), recomputed otherwise; 0 two kernels),
 * "push_halo" 0/1 (default 0, with "p2p": a kernel that rewrites an array whose halo a stencil
 * has asked for before stores the slab's edge rows into the neighbours' mailboxes itself; a small
 * kernel publishes them, waits for the neighbours' rows and copies those in when the stencil
 * asks.  Measured slower than the stand-alone exchange kernel -- the peer stores and their
 * registers cost the sweep more than the exchange launch they save -- so it is off),
 * "stencil_shfl" 0/1 (default 0, measured slower: cache-served stencil kernels take the
 * neighbours along the last dimension from neighbour lanes by warp shuffle),
 * "fuse_scalar_tail" 0/1 (default 0, measured without effect on time: a scalar-only node that directly follows a group with fused
 * reductions -- CG's beta = r.r / rtr, rtr = r.r; a Jacobi sweep's res = sum -- is evaluated by
 * the thread that has just finished those reductions instead of by a kernel of its own; on
 * several ranks only with "p2p"),
 * "dependent_launch" 0/1 (default 1: generated kernels are launched with programmatic stream
 * serialisation: a kernel's launch is released when the blocks of the kernel before it have
 * exited instead of after that kernel has drained, and every kernel waits for its
 * predecessor's completion before it touches memory; 15 % on 13 us sweeps, under 1 % on
 * kernels of hundreds of microseconds). */
int cn_set_option(cn_context* ctx, const char* key, int64_t value);

#ifdef __cplusplus
}
#endif
#endif /* CNB200_H */
