// extern "C" surface declared in include/cnb200.h.
#include <cstdlib>
#include <cstring>
#include <new>

#include "../../include/cnb200.h"
#include "context.hpp"
#include "regions.hpp"

struct cn_context {
    cn::Context impl;
    cn_context(int d, int r, int n) : impl(d, r, n) {}
};

namespace {
thread_local std::string g_create_error;

void copy_err(const std::string& s, char* err, int cap) {
    if (!err || cap <= 0) return;
    size_t n = std::min<size_t>(s.size(), (size_t)cap - 1);
    memcpy(err, s.data(), n);
    err[n] = 0;
}
}  // namespace

extern "C" {

int cn_version(void) { return 100; }

const char* cn_status_string(int status) { return cn::status_string(status); }

int cn_context_create(int device, int rank, int nranks, cn_context** out) {
    if (!out) return cn::CN_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    cn_context* c = new (std::nothrow) cn_context(device, rank, nranks);
    if (!c) return cn::CN_ERR_OUT_OF_MEMORY;
    int rc = c->impl.init();
    if (rc) {
        g_create_error = c->impl.last_error();
        delete c;
        return rc;
    }
    *out = c;
    return cn::CN_OK;
}

int cn_context_destroy(cn_context* ctx) {
    delete ctx;
    return cn::CN_OK;
}

const char* cn_last_error(cn_context* ctx) {
    if (!ctx) return g_create_error.c_str();
    return ctx->impl.last_error().c_str();
}

int cn_comm_unique_id(char id[128]) {
    std::string err;
    int rc = cn::comm_unique_id(id, &err);
    if (rc) g_create_error = err;
    return rc;
}

int cn_comm_init(cn_context* ctx, const char id[128]) {
    if (!ctx || !id) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.comm_init_id(id);
}

int cn_mark_rank_failed(cn_context* ctx, int rank) {
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.mark_rank_failed(rank);
}

int cn_receive_dag(cn_context* ctx, int epoch, int64_t size, const char* msg) {
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.receive_dag(epoch, size, msg);
}

int cn_get(cn_context* ctx, int ndims, int epoch, int name, int64_t count, int dtype, void* out) {
    (void)ndims;
    (void)epoch;
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.get(name, count, dtype, out);
}

int cn_get_local(cn_context* ctx, int name, int64_t* row_begin, int64_t* row_end, int64_t capacity,
                 void* out) {
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.get_local(name, row_begin, row_end, capacity, out);
}

int cn_put(cn_context* ctx, int name, int ndims, const int64_t* shape, int dtype, const void* host) {
    if (!ctx || !shape) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.put(name, ndims, shape, dtype, host);
}

int cn_get_root(cn_context* ctx, int ndims, int epoch, int name, int64_t count, int dtype, int root,
                void* out) {
    (void)ndims;
    (void)epoch;
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.get_root(name, count, dtype, root, out);
}

int cn_put_local(cn_context* ctx, int name, int ndims, const int64_t* shape, int dtype,
                 int64_t capacity, const void* host_slab) {
    if (!ctx || !shape) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.put_local(name, ndims, shape, dtype, capacity, host_slab);
}

int cn_execute_node(cn_context* ctx, const char* node_blob, int64_t size) {
    if (!ctx || !node_blob) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.execute_single_node(node_blob, size);
}

int cn_delete_array(cn_context* ctx, int name) {
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.delete_array(name);
}

int cn_array_info(cn_context* ctx, int name, int* ndims, int64_t shape[3], int* dtype,
                  int64_t* row_begin, int64_t* row_end) {
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.array_info(name, ndims, shape, dtype, row_begin, row_end);
}

int cn_synchronize(cn_context* ctx) {
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.synchronize();
}

int cn_compile_group(cn_context* ctx, const char* node_blob, int64_t size, uint64_t* handle) {
    if (!ctx || !handle) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.compile_group(node_blob, size, handle);
}

int cn_group_source(cn_context* ctx, uint64_t handle, const char** source) {
    if (!ctx || !source) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.group_source(handle, source);
}

int cn_launch_group(cn_context* ctx, uint64_t handle, int n_in, void* const* in_ptrs,
                    const int64_t* in_off, const int64_t* in_str, int n_bc, void* const* bc_ptrs,
                    int n_out, void* const* out_ptrs, const int64_t* out_off,
                    const int64_t* out_str, const int64_t* ext) {
    if (!ctx || !ext) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.launch_group(handle, n_in, in_ptrs, in_off, in_str, n_bc, bc_ptrs, n_out,
                                  out_ptrs, out_off, out_str, ext);
}

int cn_dag_check(const char* msg, int64_t size, int* n_nodes, int* n_roots, char* err, int errcap) {
    cn::Dag dag;
    std::string e;
    int rc = cn::parse_dag(msg, size, &dag, &e);
    copy_err(e, err, errcap);
    if (rc) return rc;
    if (n_nodes) *n_nodes = (int)dag.nodes.size();
    if (n_roots) {
        int n = 0;
        for (auto& nd : dag.nodes) n += (int)nd.roots.size();
        *n_roots = n;
    }
    return cn::CN_OK;
}

int cn_group_compile_check(const char* node_blob, int64_t size, char* source, int64_t cap,
                           int64_t* cubin_bytes, char* err, int errcap) {
    cn::DagNode node;
    std::string e;
    int rc = cn::parse_node(node_blob, size, &node, &e);
    if (rc) {
        copy_err(e, err, errcap);
        return rc;
    }
    // trailing REDUCE / SUM roots of a fusible group are its fused reductions
    cn::GroupIR g;
    rc = cn::lower_group(node, {}, &g, &e);
    if (rc) {
        copy_err(e, err, errcap);
        return rc;
    }
    std::string src;
    rc = cn::generate_source(g, &src, &e);
    if (rc) {
        copy_err(e, err, errcap);
        return rc;
    }
    if (source && cap > 0) {
        size_t n = std::min<size_t>(src.size(), (size_t)cap - 1);
        memcpy(source, src.data(), n);
        source[n] = 0;
    }
    std::vector<char> cubin;
    std::string log;
    cn::TileConfig tile;
    if (g.staged) {  // a staged tile is one TMA box
        tile.tx = 64;
        tile.r = 4;
    }
    if (const char* sh = getenv("CN_STENCIL_SHFL")) tile.shfl = atoi(sh) != 0 && !g.flat && !g.staged;
    if (const char* pf = getenv("CN_FLAT_PREFETCH")) tile.prefetch = g.flat ? std::max(0, std::min(2, atoi(pf))) : 0;
    rc = cn::nvrtc_compile(src, tile, &cubin, &log);
    if (rc) {
        copy_err(log, err, errcap);
        return rc;
    }
    if (cubin_bytes) *cubin_bytes = (int64_t)cubin.size();
    return cn::CN_OK;
}

int cn_fuse_check(const char* node_a, int64_t size_a, const char* node_b, int64_t size_b, char* source,
                  int64_t cap, int* fused, char* err, int errcap) {
    if (fused) *fused = 0;
    cn::DagNode a, b, m;
    std::string e;
    int rc = cn::parse_node(node_a, size_a, &a, &e);
    if (!rc) rc = cn::parse_node(node_b, size_b, &b, &e);
    if (rc) {
        copy_err(e, err, errcap);
        return rc;
    }
    cn::GroupIR g;
    cn::DagNode cons, prod;
    int pseudo = 0, target = 0;
    bool staged = false;
    if (!(getenv("CN_FUSE_PRODUCERS") && atoi(getenv("CN_FUSE_PRODUCERS")) < 2) &&
        cn::stage_producer(a, b, &cons, &prod, &pseudo, &target))
        staged = cn::lower_staged_producer(cons, prod, pseudo, target, {}, &g, &e) == cn::CN_OK;
    if (!staged && getenv("CN_DEBUG_FUSE")) fprintf(stderr, "[cnb200] staged form not used: %s\n", e.c_str());
    if (!staged) {
        if (!cn::inline_producer(a, b, &m)) return cn::CN_OK;
        g = cn::GroupIR();
        rc = cn::lower_group(m, {}, &g, &e);
        if (rc || g.cls != cn::GroupIR::SHIFTED || g.flat) {
            copy_err(e, err, errcap);
            return cn::CN_OK;  // the pair would run as two kernels
        }
    }
    std::string src;
    if ((rc = cn::generate_source(g, &src, &e))) {
        copy_err(e, err, errcap);
        return rc;
    }
    std::vector<char> cubin;
    std::string log;
    cn::TileConfig tile;
    if (g.staged) {
        tile.tx = 64;
        tile.r = g.producer.empty() ? 4 : 8;
    }
    if ((rc = cn::nvrtc_compile(src, tile, &cubin, &log))) {
        copy_err(log, err, errcap);
        return rc;
    }
    if (source && cap > 0) {
        size_t n = std::min<size_t>(src.size(), (size_t)cap - 1);
        memcpy(source, src.data(), n);
        source[n] = 0;
    }
    if (fused) *fused = 1;
    return cn::CN_OK;
}

int cn_tail_check(const char* dag_blob, int64_t size, char* source, int64_t cap, int* fused, char* err,
                  int errcap) {
    if (fused) *fused = 0;
    cn::Dag dag;
    std::string e;
    int rc = cn::parse_dag(dag_blob, size, &dag, &e);
    if (rc) {
        copy_err(e, err, errcap);
        return rc;
    }
    if (dag.nodes.size() < 3) return cn::CN_ERR_INVALID_ARGUMENT;
    std::vector<const cn::AstNode*> reds;
    for (size_t i = 1; i + 1 < dag.nodes.size(); ++i) {
        const cn::DagNode& n = dag.nodes[i];
        if (n.roots.size() != 1 || (n.roots[0]->opcode != cn::OP_REDUCE && n.roots[0]->opcode != cn::OP_SUM))
            return cn::CN_ERR_INVALID_ARGUMENT;
        reds.push_back(n.roots[0].get());
    }
    cn::GroupIR g, t;
    if ((rc = cn::lower_group(dag.nodes[0], reds, &g, &e))) {
        copy_err(e, err, errcap);
        return rc;
    }
    if (g.cls != cn::GroupIR::SHIFTED || g.reds.empty()) return cn::CN_OK;
    if (cn::lower_group(dag.nodes.back(), {}, &t, &e) != cn::CN_OK || t.cls != cn::GroupIR::SCALAR_ONLY ||
        t.dtype != g.dtype || t.souts.empty()) {
        copy_err(e, err, errcap);
        return cn::CN_OK;
    }
    g.tail.push_back(t);
    std::string src;
    if ((rc = cn::generate_source(g, &src, &e))) {
        copy_err(e, err, errcap);
        return rc;
    }
    std::vector<char> cubin;
    std::string log;
    cn::TileConfig tile;
    if (g.staged) {
        tile.tx = 64;
        tile.r = 4;
    }
    if ((rc = cn::nvrtc_compile(src, tile, &cubin, &log))) {
        copy_err(log, err, errcap);
        return rc;
    }
    if (source && cap > 0) {
        size_t n = std::min<size_t>(src.size(), (size_t)cap - 1);
        memcpy(source, src.data(), n);
        source[n] = 0;
    }
    if (fused) *fused = 1;
    return cn::CN_OK;
}

static cn::Lattice lat(const int64_t* r) { return cn::Lattice{r[0], r[1], r[2]}; }

int cn_region_intersect(const int64_t a[3], const int64_t b[3], int64_t out[3]) {
    if (!a || !b || !out || a[2] < 1 || b[2] < 1) return cn::CN_ERR_INVALID_ARGUMENT;
    const cn::Lattice r = cn::lattice_intersect(lat(a), lat(b));
    out[0] = r.start;
    out[1] = r.stop;
    out[2] = r.step;
    return cn::CN_OK;
}

int cn_region_map(const int64_t part[3], const int64_t from[3], const int64_t to[3], int64_t out[3]) {
    if (!part || !from || !to || !out || part[2] < 1 || from[2] < 1 || to[2] < 1) return cn::CN_ERR_INVALID_ARGUMENT;
    if (part[2] % from[2] != 0 || (part[0] - from[0]) % from[2] != 0 || part[0] < from[0])
        return cn::CN_ERR_INVALID_ARGUMENT;  // not a sub-lattice of `from`
    const cn::Lattice r = cn::lattice_map(lat(part), lat(from), lat(to));
    out[0] = r.start;
    out[1] = r.stop;
    out[2] = r.step;
    return cn::CN_OK;
}

int cn_plan_row_transfers(const int64_t anchor[3], int64_t anchor_n0, const int64_t leaf[3], int64_t leaf_n0,
                          int nranks, int64_t* transfers, int64_t cap, int64_t* count, int64_t* iteration_rows) {
    if (!anchor || !leaf || !count || nranks < 1 || anchor[2] < 1 || leaf[2] < 1 || anchor_n0 < 0 || leaf_n0 < 0)
        return cn::CN_ERR_INVALID_ARGUMENT;
    const std::vector<cn::RowTransfer> moves = cn::plan_transfers(lat(anchor), anchor_n0, lat(leaf), leaf_n0, nranks);
    *count = (int64_t)moves.size();
    for (int64_t i = 0; transfers && i < *count && i < cap; ++i) {
        transfers[4 * i + 0] = moves[i].src;
        transfers[4 * i + 1] = moves[i].dst;
        transfers[4 * i + 2] = moves[i].lo;
        transfers[4 * i + 3] = moves[i].hi;
    }
    for (int q = 0; iteration_rows && q < nranks; ++q)
        cn::iteration_rows(lat(anchor), anchor_n0, nranks, q, &iteration_rows[2 * q], &iteration_rows[2 * q + 1]);
    return cn::CN_OK;
}

int cn_partition(int64_t n0, int nranks, int rank, int64_t* begin, int64_t* end) {
    if (n0 < 0 || nranks < 1 || rank < 0 || rank >= nranks || !begin || !end)
        return cn::CN_ERR_INVALID_ARGUMENT;
    cn::slab_partition(n0, nranks, rank, begin, end);
    return cn::CN_OK;
}

int cn_timer_start(cn_context* ctx) {
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.timer_start();
}

int cn_timer_stop(cn_context* ctx, float* milliseconds) {
    if (!ctx || !milliseconds) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.timer_stop(milliseconds);
}

int cn_profile_report(cn_context* ctx, char* buf, int64_t cap) {
    if (!ctx) return cn::CN_ERR_INVALID_ARGUMENT;
    return ctx->impl.profile_report(buf, cap);
}

int cn_get_stats(cn_context* ctx, cn_stats* out) {
    if (!ctx || !out) return cn::CN_ERR_INVALID_ARGUMENT;
    const cn::Stats& s = ctx->impl.stats();
    out->kernel_launches = s.kernel_launches;
    out->group_launches = s.group_launches;
    out->compiles = s.compiles;
    out->halo_exchanges = s.halo_exchanges;
    out->allreduces = s.allreduces;
    out->fused_reductions = s.fused_reductions;
    out->nodes = s.nodes;
    out->bytes_h2d = s.bytes_h2d;
    out->bytes_d2h = s.bytes_d2h;
    out->plan_hits = s.plan_hits;
    out->peer_exchanges = s.peer_exchanges;
    out->overlapped_sweeps = s.overlapped_sweeps;
    out->deep_halo_sweeps = s.deep_halo_sweeps;
    out->inlined_producers = s.inlined_producers;
    out->row_fetches = s.row_fetches;
    out->halo_pushes = s.halo_pushes;
    out->scalar_tails = s.scalar_tails;
    return cn::CN_OK;
}

int cn_set_option(cn_context* ctx, const char* key, int64_t value) {
    if (!ctx || !key) return cn::CN_ERR_INVALID_ARGUMENT;
    std::string k(key);
    if (k == "halo") {
        if (value < 0 || value > 64) return cn::CN_ERR_INVALID_ARGUMENT;
        ctx->impl.set_halo((int)value);
    } else if (k == "staged") {
        cn::set_staged_level((int)value);
    } else if (k == "staged_tile_tx") {
        if (value < 8 || value > 64 || 256 % value) return cn::CN_ERR_INVALID_ARGUMENT;
        ctx->impl.set_staged_tile((int)value, -1);
    } else if (k == "staged_tile_rows") {
        if (value < 1 || value > 16) return cn::CN_ERR_INVALID_ARGUMENT;
        ctx->impl.set_staged_tile(-1, (int)value);
    } else if (k == "debug_drop_copies") {
        ctx->impl.set_debug_drop_copies(value != 0);
    } else if (k == "deep_halo") {
        ctx->impl.set_deep_halo(value != 0);
    } else if (k == "overlap_halo") {
        ctx->impl.set_overlap_halo(value != 0);
    } else if (k == "debug_peer_wait") {
        return ctx->impl.debug_peer_wait();
    } else if (k == "p2p") {
        ctx->impl.set_p2p(value != 0);
    } else if (k == "push_halo") {
        ctx->impl.set_push_halo(value != 0);
    } else if (k == "fuse_producers") {
        if (value < 0 || value > 2) return cn::CN_ERR_INVALID_ARGUMENT;
        ctx->impl.set_fuse_producers((int)value);
    } else if (k == "fuse_scalar_tail") {
        ctx->impl.set_fuse_scalar_tail(value != 0);
    } else if (k == "dependent_launch") {
        ctx->impl.set_dependent_launch(value != 0);
    } else if (k == "stencil_shfl") {
        ctx->impl.set_stencil_shfl(value != 0);
    } else if (k == "plan_cache") {
        ctx->impl.set_plan_cache(value != 0);
    } else if (k == "flat_prefetch") {
        if (value < -1 || value > 2) return cn::CN_ERR_INVALID_ARGUMENT;
        ctx->impl.set_flat_prefetch((int)value);
    } else if (k == "profile") {
        ctx->impl.set_profile(value != 0);
    } else if (k == "fuse_reductions") {
        ctx->impl.set_fuse_reductions(value != 0);
    } else if (k == "tile_tx") {
        if (value < 8 || value > 256 || 256 % value) return cn::CN_ERR_INVALID_ARGUMENT;
        ctx->impl.set_tile((int)value, -1);
    } else if (k == "tile_rows") {
        if (value < 1 || value > 16) return cn::CN_ERR_INVALID_ARGUMENT;
        ctx->impl.set_tile(-1, (int)value);
    } else {
        return cn::CN_ERR_INVALID_ARGUMENT;
    }
    return cn::CN_OK;
}

}  // extern "C"
