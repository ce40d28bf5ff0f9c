// Node execution: fused groups (generated kernels), dot / sum, matvec, seeded fill, and the
// host-facing get / put / timer entry points.
//
// Reference counterparts: execute_node_nd JIT paths (src/execute_node.cpp:1195-1585),
// execute_reduce_node (src/executor_reduce.cpp:7-119), execute_matmul_node
// (src/executor_matmul.cpp:149-498), process_get + gather (src/partition_get.cpp:3-67,
// src/dag_group_runtime.cpp:99-118).
#include <algorithm>
#include <cstring>

#include "context.hpp"
#include "kernels.hpp"
#include "regions.hpp"

namespace cn {

namespace {

void array_strides(const Array& a, int64_t* s) {
    s[0] = s[1] = s[2] = 0;
    s[a.ndims - 1] = 1;
    for (int d = a.ndims - 2; d >= 0; --d) s[d] = s[d + 1] * a.shape[d + 1];
}

}  // namespace

int Context::get_kernel(const GroupIR& g, CompiledGroup** out) {
    TileConfig tile = tile_;
    bool heavy_flat = false;
    if (g.flat && !tile_set_) {
        // exp, tanh, sqrt and division are long dependent chains in double precision: four
        // rows per thread give the scheduler eight independent elements to interleave
        int heavy = 0;
        for (auto& r : g.roots)
            if (r.opcode == OP_EXP || r.opcode == OP_TANH || r.opcode == OP_SQRT || r.opcode == OP_DIV) ++heavy;
        if (heavy >= 2) tile.r = 4;
        heavy_flat = heavy >= 2;
        // one block of 1024 threads per SM: measured 6 % faster on the 2^28 chain than four
        // blocks of 256 (0.93 against 0.99 ms on a stand-alone copy of the kernel)
        if (heavy_flat) tile.block = 1024;
        if (const char* e = getenv("CN_FLAT_BLOCK")) {
            const int v = atoi(e);
            if (heavy_flat && (v == 128 || v == 256 || v == 512 || v == 1024)) tile.block = v;
        }
    }
    if (g.staged) {
        // a staged tile is one TMA box: at most 256 elements per side
        tile = staged_tile_;
        // measured best: 3-D march 128 columns x 8 rows per plane tile with a 4-deep ring
        // (42 KB of shared memory per block, four blocks per SM); 2-D tiles 128 x 16
        if (g.ndims == 3 && !staged_tile_set_) tile.r = 2;
        // computed tiles carry a halo ring of redundant work: 128 x 32 points keep it below 10 %
        if (!g.producer.empty() && !staged_tile_set_) tile.r = 8;
        if (tile.tx > 64) tile.tx = 64;
        while ((tile.block / tile.tx) * tile.r + 2 * g.hy > 256) tile.r /= 2;
    }
    if (g.cls == GroupIR::SHIFTED && !g.flat && g.ndims >= 2) {
        // specialise on the element strides of the (common) array shape
        tile.s0 = g.ndims == 2 ? g.array_shape[1] : g.array_shape[1] * g.array_shape[2];
        tile.s1 = g.ndims == 3 ? g.array_shape[2] : 0;
    }
    if (!g.producer.empty()) {
        if (const char* e = getenv("CN_PRODUCER_MINB")) tile.minb = std::max(1, std::min(8, atoi(e)));
        if (const char* e = getenv("CN_PRODUCER_FILL_U")) tile.fill_u = std::max(1, std::min(9, atoi(e)));
    }
    tile.drop_copies = g.staged && debug_drop_copies_;
    if (const char* e = getenv("CN_LAUNCH_TRIGGER")) tile.trigger = atoi(e) != 0;
    tile.shfl = stencil_shfl_ && g.cls == GroupIR::SHIFTED && !g.flat && !g.staged;
    tile.push = push_halo_ && nranks_ > 1 && peer_.ready && g.cls == GroupIR::SHIFTED && !overlap_halo_;
    // heavy flat groups issue the loads of all their rows before the arithmetic: between the
    // out-of-line slow paths of exp / sqrt / division the compiler leaves each row's loads
    // next to their use, and the memory system idles while a row is computed (measured on the
    // 2^28 chain: 1.18 -> 1.0 ms)
    tile.prefetch = !g.flat ? 0 : (flat_prefetch_ >= 0 ? flat_prefetch_ : (heavy_flat ? 2 : 0));
    if (g.staged && g.ndims == 3) tile.ns = staged_ns_ ? staged_ns_ : (g.hz == 1 ? 4 : 0);
    std::string key = g.key() + "|T" + std::to_string(tile.tx) + "," + std::to_string(tile.r) + "/" + std::to_string(tile.block) + "|S" +
                      std::to_string(tile.s0) + "," + std::to_string(tile.s1) + (tile.drop_copies ? "|drop" : "") + "|N" + std::to_string(tile.ns) +
                      "|mb" + std::to_string(tile.minb) + "|fu" + std::to_string(tile.fill_u) +
                      "|pf" + std::to_string(tile.prefetch) + (tile.shfl ? "|sh" : "") + (tile.push ? "|push" : "") +
                      (tile.trigger ? "|trig" : "") + "|sb" + std::to_string(shifted_minb_) + "," + std::to_string(flat_minb_);
    auto it = kernels_.find(key);
    if (it != kernels_.end()) {
        *out = &it->second;
        return CN_OK;
    }
    CompiledGroup k;
    int rc = generate_source(g, &k.source, &err_);
    if (rc) return rc;
    std::vector<char> cubin;
    // Cache-served stencil kernels are bound by the latency of their loads: with the registers
    // capped for six resident blocks per SM (30 instead of 44 registers for a 5-point sweep,
    // which then runs eight blocks) more warps are in flight.  A group too large for the cap
    // would spill, and is compiled again without it.
    const int cap_blocks = (g.cls == GroupIR::SHIFTED && !g.staged && tile.block == 256 && tile.minb == 1)
                               ? (g.flat ? flat_minb_ : shifted_minb_) : 1;
    const bool cap_registers = cap_blocks > 1;
    if (cap_registers) {
        TileConfig tight = tile;
        tight.minb = cap_blocks;
        std::string log;
        if (nvrtc_compile(k.source, tight, &cubin, &log) == CN_OK && spill_bytes(log) == 0) {
            tile = tight;
            k.log = log;
        } else {
            cubin.clear();
        }
    }
    k.tile = tile;
    if (cubin.empty()) {
        rc = nvrtc_compile(k.source, tile, &cubin, &k.log);
        if (rc) return fail(rc, "group kernel failed to compile:\n" + k.log);
    }
    stats_.compiles++;
    if ((rc = driver_fail(drv_.ModuleLoadData(&k.module, cubin.data()), "cuModuleLoadData"))) return rc;
    rc = driver_fail(drv_.ModuleGetFunction(&k.func, k.module, g.entry_name().c_str()), "cuModuleGetFunction");
    if (rc) return rc;
    {
        const char* cls = g.cls == GroupIR::SHIFTED ? (g.flat ? "flat" : "shifted")
                          : (g.cls == GroupIR::STRIDED ? "strided" : "scalar");
        char lbl[160];
        const size_t n_in = g.producer.empty() ? g.input_arrays().size()
                                               : g.input_arrays().size() - 1 + g.producer[0].input_arrays().size();
        snprintf(lbl, sizeof(lbl), "group%zu[%s %dd vec%d in%zu out%zu red%zu%s]", kernels_.size(), cls,
                 g.ndims, g.vec, n_in, g.outs.size(), g.reds.size(),
                 g.copy_through ? " copy-through" : "");
        k.label = lbl;
    }
    if (g.staged) {
        const int ns = tile.ns ? tile.ns : (g.ndims == 3 ? 2 * g.hz + 3 : 3);
        const size_t sw = (size_t)tile.tx * 2 + 4, sh = (size_t)(tile.block / tile.tx) * tile.r + 2 * g.hy;
        const size_t slot = (sh * sw + 15) / 16 * 16;
        k.smem_bytes = ns * slot * sizeof(double) + ns * sizeof(unsigned long long);
        if (!g.producer.empty()) k.smem_bytes = slot * sizeof(double) + sizeof(unsigned long long);
        k.label += g.producer.empty() ? " tma" : " staged-producer";
        if ((rc = driver_fail(drv_.FuncSetAttribute(k.func, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                                    (int)k.smem_bytes), "cuFuncSetAttribute")))
            return rc;
    }
    {
        char tag[16];
        snprintf(tag, sizeof(tag), " #%08x", code_digest(k.source, tile));
        k.label += tag;
    }
    int occ = 0;
    if (drv_.OccupancyMaxActiveBlocksPerMultiprocessor(&occ, k.func, tile.block, k.smem_bytes) == CUDA_SUCCESS && occ > 0)
        k.blocks_per_sm = occ;
    if (g.staged && g.ndims == 3) {
        // measured on the 1024^3 sweep: four marching blocks per SM saturate HBM; a fifth only
        // adds planes in flight and costs 14 %
        int cap = 4;
        if (const char* c = getenv("CN_STAGED_BLOCKS")) cap = std::max(1, atoi(c));
        k.blocks_per_sm = std::min(k.blocks_per_sm, cap);
    }
    if (getenv("CN_KERNEL_INFO")) {  // one line per compiled kernel on stderr
        int regs = 0;
        drv_.FuncGetAttribute(&regs, CU_FUNC_ATTRIBUTE_NUM_REGS, k.func);
        fprintf(stderr, "[cnb200] %s %s: %d registers, %zu B dynamic smem, %d blocks/SM, tile %dx%d\n",
                g.entry_name().c_str(), k.label.c_str(), regs, k.smem_bytes, k.blocks_per_sm, tile.tx, tile.r);
    }
    auto ins = kernels_.emplace(key, std::move(k));
    *out = &ins.first->second;
    return CN_OK;
}

void Context::prof_start(const std::string& label, double bytes, cudaStream_t st) {
    if (!st) st = stream_;
    if (!profile_) return;
    ProfEntry& e = prof_[label];
    e.launches++;
    e.bytes += bytes;
    cudaEvent_t a = nullptr, b = nullptr;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    cudaEventRecord(a, st);
    e.events.push_back({a, b});
    prof_open_ = &e;
    prof_stream_ = st;
}

void Context::prof_stop() {
    if (!profile_ || !prof_open_) return;
    cudaEventRecord(prof_open_->events.back().second, prof_stream_);
    prof_open_ = nullptr;
}

// One line per kernel: label <tab> launches <tab> total_ms <tab> algorithmic_bytes
int Context::profile_report(char* buf, int64_t cap) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    int rc = synchronize();
    if (rc) return rc;
    std::string out;
    for (auto& kv : prof_) {
        double ms = 0;
        for (auto& ev : kv.second.events) {
            float t = 0;
            if (cudaEventElapsedTime(&t, ev.first, ev.second) == cudaSuccess) ms += t;
            cudaEventDestroy(ev.first);
            cudaEventDestroy(ev.second);
        }
        char line[512];
        snprintf(line, sizeof(line), "%s\t%lld\t%.6f\t%.0f\n", kv.first.c_str(), kv.second.launches, ms,
                 kv.second.bytes);
        out += line;
    }
    prof_.clear();
    if (buf && cap > 0) {
        size_t n = std::min<size_t>(out.size(), (size_t)cap - 1);
        memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return CN_OK;
}

int Context::launch(CompiledGroup* k, const CnGroupArgs& a, int grid, int block, double bytes, cudaStream_t st) {
    if (!st) st = stream_;
    void* params[] = {(void*)&a};
    prof_start(k->label, bytes, st);
    int rc;
    if (dependent_launch_) {
        CUlaunchAttribute attr;
        memset(&attr, 0, sizeof(attr));
        attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr.value.programmaticStreamSerializationAllowed = 1;
        CUlaunchConfig cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDimX = (unsigned)grid;
        cfg.gridDimY = cfg.gridDimZ = 1;
        cfg.blockDimX = (unsigned)block;
        cfg.blockDimY = cfg.blockDimZ = 1;
        cfg.sharedMemBytes = (unsigned)k->smem_bytes;
        cfg.hStream = (CUstream)st;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        rc = driver_fail(drv_.LaunchKernelEx(&cfg, k->func, params, nullptr), "cuLaunchKernelEx");
    } else {
        rc = driver_fail(drv_.LaunchKernel(k->func, (unsigned)grid, 1, 1, (unsigned)block, 1, 1,
                                           (unsigned)k->smem_bytes, (CUstream)st, params, nullptr),
                         "cuLaunchKernel");
    }
    prof_stop();
    if (rc) return rc;
    stats_.kernel_launches++;
    stats_.group_launches++;
    if (k->smem_bytes) {
        stats_.staged_launches++;
        waiting_launches_++;
    }
    return CN_OK;
}

int Context::run_lowered(const GroupIR& g, CompiledGroup* k) {
    switch (g.cls) {
        case GroupIR::SCALAR_ONLY: return run_scalar_only(g, k);
        case GroupIR::SHIFTED: return run_shifted(g, k);
        case GroupIR::STRIDED: return run_strided(g, k);
    }
    return fail(CN_ERR_UNSUPPORTED, "unknown group class");
}

// TMA descriptor of the stencil array's local slab (halo rows included), box = one tile.
int Context::encode_tensor_map(const Array& x, const CompiledGroup& k, const GroupIR& g, CnGroupArgs* a) {
    const int nd = x.ndims;
    const size_t esz = sizeof(double);
    cuuint64_t dims[3] = {1, 1, 1};
    cuuint64_t strides[2] = {0, 0};
    cuuint32_t box[3] = {1, 1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const cuuint64_t rows0 = (cuuint64_t)(x.local_rows() + 2 * x.halo);
    const cuuint32_t sw = (cuuint32_t)k.tile.tx * 2 + 4;
    const cuuint32_t sh = (cuuint32_t)(k.tile.block / k.tile.tx) * k.tile.r + 2 * g.hy;
    if (nd == 2) {
        dims[0] = (cuuint64_t)x.shape[1];
        dims[1] = rows0;
        strides[0] = (cuuint64_t)x.shape[1] * esz;
        box[0] = sw;
        box[1] = sh;
    } else {
        dims[0] = (cuuint64_t)x.shape[2];
        dims[1] = (cuuint64_t)x.shape[1];
        dims[2] = rows0;
        strides[0] = (cuuint64_t)x.shape[2] * esz;
        strides[1] = (cuuint64_t)x.shape[2] * x.shape[1] * esz;
        box[0] = sw;
        box[1] = sh;
        box[2] = 1;
    }
    if (rows0 == 0) dims[nd - 1] = 1;
    char* base = x.buf.data - (size_t)x.halo * x.unit * esz;
    CUtensorMap tm;
    CUresult r = drv_.TensorMapEncodeTiled(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, (cuuint32_t)nd, base, dims, strides,
                                           box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    int rc = driver_fail(r, "cuTensorMapEncodeTiled");
    if (rc) return rc;
    static_assert(sizeof(CUtensorMap) == 128, "descriptor size");
    memcpy(a->tmap, &tm, sizeof(tm));
    a->tm_off[0] = x.halo;
    a->tm_off[1] = 0;
    a->tm_off[2] = 0;
    return CN_OK;
}

// Size-1 inputs and outputs.  An output whose array is also read as an input of the same
// launch gets a fresh buffer (other blocks may still be reading the old one).
int Context::bind_scalars(const GroupIR& g, CnGroupArgs* a,
                          std::vector<std::pair<Array*, Buffer>>* swaps) {
    for (size_t i = 0; i < g.scalars.size(); ++i) a->sc[i] = g.scalars[i];
    for (size_t i = 0; i < g.bcast_names.size(); ++i) {
        Array* s = find(g.bcast_names[i]);
        if (!s) return fail(CN_ERR_UNKNOWN_ARRAY, "size-1 array " + std::to_string(g.bcast_names[i]) + " does not exist");
        if (s->global_elems() != 1) return fail(CN_ERR_SHAPE_MISMATCH, "broadcast operand is not a size-1 array");
        if (s->dtype != g.dtype) return fail(CN_ERR_BAD_DTYPE, "size-1 operand dtype differs from the group dtype");
        a->bc[i] = s->buf.data;
    }
    for (size_t i = 0; i < g.souts.size(); ++i) {
        const ScalarOutIR& so = g.souts[i];
        Array* s = find(so.name);
        if (!s) {
            if (so.is_set) return fail(CN_ERR_UNKNOWN_ARRAY, "SET_REGION target " + std::to_string(so.name) + " does not exist");
            int64_t one[1] = {1};
            int rc = create_array(so.name, 1, one, g.dtype, false, &s);
            if (rc) return rc;
        }
        if (s->global_elems() != 1) return fail(CN_ERR_SHAPE_MISMATCH, "scalar result stored into a larger array");
        if (s->dtype != g.dtype) return fail(CN_ERR_BAD_DTYPE, "scalar result dtype differs from the group dtype");
        bool read_too = std::find(g.bcast_names.begin(), g.bcast_names.end(), so.name) != g.bcast_names.end();
        if (read_too && g.cls != GroupIR::SCALAR_ONLY) {
            Buffer nb;
            int rc = alloc_buffer(*s, &nb);
            if (rc) return rc;
            a->sout[i] = nb.data;
            swaps->push_back({s, nb});
        } else {
            a->sout[i] = s->buf.data;
        }
    }
    return CN_OK;
}

int Context::bind_reductions(const GroupIR& g, CnGroupArgs* a, int grid, std::vector<Array*>* results) {
    if (g.reds.empty()) return CN_OK;
    if (grid > max_grid_) return fail(CN_ERR_LIMIT, "grid larger than the reduction scratch");
    a->partials = partials_;
    a->counter = counter_;
    for (size_t q = 0; q < g.reds.size(); ++q) {
        Array* r = nullptr;
        int64_t one[1] = {1};
        int rc = create_array(g.reds[q].result_name, 1, one, g.dtype, false, &r);
        if (rc) return rc;
        a->red[q] = r->buf.data;
        results->push_back(r);
    }
    // with peer mailboxes the kernel's last block also adds up the other ranks' totals
    if (nranks_ > 1) bind_peers(a);
    return CN_OK;
}

// Launch arguments of a group's scalar tail: literal scalars, size-1 operands and size-1
// results behind the group's (and its producer's) own.  Runs after bind_reductions, so that a
// reduction result the tail reads exists.  Results are written in place: the tail runs after
// every block of the launch has finished.
int Context::bind_tail(const GroupIR& g, CnGroupArgs* a) {
    const GroupIR& t = g.tail[0];
    size_t sc_base = g.scalars.size(), bc_base = g.bcast_names.size();
    if (!g.producer.empty()) {
        sc_base += g.producer[0].scalars.size();
        bc_base += g.producer[0].bcast_names.size();
    }
    const size_t so_base = g.souts.size();
    if (sc_base + t.scalars.size() > CN_MAX_SC || bc_base + t.bcast_names.size() > CN_MAX_BC ||
        so_base + t.souts.size() > CN_MAX_SOUT)
        return fail(CN_ERR_LIMIT, "scalar tail does not fit the launch arguments");
    for (size_t i = 0; i < t.scalars.size(); ++i) a->sc[sc_base + i] = t.scalars[i];
    // results first: creating one may move the table, and operand pointers are taken after
    for (size_t i = 0; i < t.souts.size(); ++i) {
        const ScalarOutIR& so = t.souts[i];
        Array* s = find(so.name);
        if (!s) {
            if (so.is_set) return fail(CN_ERR_UNKNOWN_ARRAY, "SET_REGION target " + std::to_string(so.name) + " does not exist");
            int64_t one[1] = {1};
            int rc = create_array(so.name, 1, one, t.dtype, false, &s);
            if (rc) return rc;
        }
        if (s->global_elems() != 1) return fail(CN_ERR_SHAPE_MISMATCH, "scalar result stored into a larger array");
        if (s->dtype != t.dtype) return fail(CN_ERR_BAD_DTYPE, "scalar result dtype differs from the group dtype");
    }
    for (size_t i = 0; i < t.souts.size(); ++i) {
        Array* s = find(t.souts[i].name);
        a->sout[so_base + i] = s->buf.data;
        s->mark_written();
    }
    for (size_t i = 0; i < t.bcast_names.size(); ++i) {
        Array* s = find(t.bcast_names[i]);
        if (!s) return fail(CN_ERR_UNKNOWN_ARRAY, "size-1 array " + std::to_string(t.bcast_names[i]) + " does not exist");
        if (s->global_elems() != 1) return fail(CN_ERR_SHAPE_MISMATCH, "broadcast operand is not a size-1 array");
        if (s->dtype != t.dtype) return fail(CN_ERR_BAD_DTYPE, "size-1 operand dtype differs from the group dtype");
        a->bc[bc_base + i] = s->buf.data;
    }
    return CN_OK;
}

int Context::finish_reductions(const std::vector<Array*>& results, bool in_kernel) {
    if (nranks_ == 1) return CN_OK;
    if (in_kernel && peer_.ready) {  // already summed over the ranks inside the kernel
        stats_.allreduces += (long long)results.size();
        return CN_OK;
    }
    if (!comm_.ready && !results.empty()) return fail(CN_ERR_COMM, "reduction across ranks needs cn_comm_init first");
    for (Array* r : results) {
        int rc = comm_allreduce_sum(&comm_, r->buf.data, 1, r->dtype, stream_, &err_);
        if (rc) return rc;
        stats_.allreduces++;
    }
    return CN_OK;
}

int Context::run_scalar_only(const GroupIR& g, CompiledGroup* k) {
    CnGroupArgs a;
    memset(&a, 0, sizeof(a));
    std::vector<std::pair<Array*, Buffer>> swaps;
    int rc = bind_scalars(g, &a, &swaps);
    if (rc) return rc;
    return launch(k, a, 1, 32, 0.0);
}

int Context::run_shifted(const GroupIR& g, CompiledGroup* k) {
    const int nd = g.ndims;
    CnGroupArgs a;
    memset(&a, 0, sizeof(a));
    std::vector<std::pair<Array*, Buffer>> swaps;
    int rc = bind_scalars(g, &a, &swaps);
    if (rc) return rc;

    // inputs
    std::vector<int> in_names = g.input_arrays();
    if ((int)in_names.size() > CN_MAX_IN) return fail(CN_ERR_LIMIT, "too many input arrays in one group");
    Array* ref = nullptr;
    std::vector<Array*> ins;
    const bool prod = !g.producer.empty();  // the stage array is a stand-in computed in the kernel
    for (size_t i = 0; i < in_names.size(); ++i) {
        if (prod && in_names[i] == g.stage_array) {
            ins.push_back(nullptr);
            continue;
        }
        Array* x = find(in_names[i]);
        if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "operand array " + std::to_string(in_names[i]) + " does not exist");
        if ((rc = check_leaf(x, nd, g.array_shape, "group operand"))) return rc;
        if (x->dtype != g.dtype) return fail(CN_ERR_BAD_DTYPE, "operand dtype differs from the group dtype");
        ins.push_back(x);
        ref = x;
    }
    // outputs
    std::vector<Array*> outs;
    for (size_t m = 0; m < g.outs.size(); ++m) {
        const OutIR& o = g.outs[m];
        Array* x = find(o.name);
        if (o.is_set) {
            if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "SET_REGION target " + std::to_string(o.name) + " does not exist");
            if ((rc = check_leaf(x, nd, g.array_shape, "SET_REGION target"))) return rc;
            if (x->dtype != g.dtype) return fail(CN_ERR_BAD_DTYPE, "target dtype differs from the group dtype");
        } else {
            if ((rc = create_array(o.name, nd, g.array_shape, g.dtype, false, &x))) return rc;
            // create_array may have re-hashed the table: refresh the input pointers
            for (size_t i = 0; i < in_names.size(); ++i)
                if (ins[i]) ins[i] = find(in_names[i]);
            for (size_t j = 0; j < outs.size(); ++j) outs[j] = find(g.outs[j].name);
        }
        outs.push_back(x);
        ref = x;
    }
    if (!ref) return fail(CN_ERR_UNSUPPORTED, "group touches no array");
    // staged producer: its inputs, literal scalars and size-1 operands follow the group's own
    std::vector<Array*> pins;
    if (prod) {
        const GroupIR& gp = g.producer[0];
        const std::vector<int> pnames = gp.input_arrays();
        if (in_names.size() + pnames.size() > CN_MAX_IN) return fail(CN_ERR_LIMIT, "too many input arrays in one group");
        for (size_t kx = 0; kx < pnames.size(); ++kx) {
            Array* x = find(pnames[kx]);
            if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "operand array " + std::to_string(pnames[kx]) + " does not exist");
            if ((rc = check_leaf(x, nd, g.array_shape, "group operand"))) return rc;
            if (x->dtype != g.dtype) return fail(CN_ERR_BAD_DTYPE, "operand dtype differs from the group dtype");
            pins.push_back(x);
        }
        for (size_t i = 0; i < gp.scalars.size(); ++i) a.sc[g.scalars.size() + i] = gp.scalars[i];
        for (size_t i = 0; i < gp.bcast_names.size(); ++i) {
            Array* sarr = find(gp.bcast_names[i]);
            if (!sarr) return fail(CN_ERR_UNKNOWN_ARRAY, "size-1 array " + std::to_string(gp.bcast_names[i]) + " does not exist");
            if (sarr->global_elems() != 1) return fail(CN_ERR_SHAPE_MISMATCH, "broadcast operand is not a size-1 array");
            if (sarr->dtype != g.dtype) return fail(CN_ERR_BAD_DTYPE, "size-1 operand dtype differs from the group dtype");
            a.bc[g.bcast_names.size() + i] = sarr->buf.data;
        }
    }

    // halos: a leaf shifted along dimension 0 reads rows owned by a neighbour.  Every array
    // keeps count of how many of its halo rows still hold the neighbours' current values
    // (halo_fresh); an exchange refreshes all `halo` rows at once.
    std::vector<Array*> stale;
    int64_t ext = 0;  // rows beyond each slab edge that this sweep computes redundantly
    if (nranks_ > 1 && !ref->replicated) {
        if (g.max_halo > halo_) return fail(CN_ERR_UNSUPPORTED, "stencil reaches further along dimension 0 than the halo depth");
        std::vector<int64_t> reach(ins.size(), 0);  // how far each input is read along dimension 0
        for (auto& l : g.leaves) {
            const int64_t r = l.delta[0] < 0 ? -l.delta[0] : l.delta[0];
            for (size_t i = 0; i < in_names.size(); ++i)
                if (in_names[i] == l.name) reach[i] = std::max(reach[i], r);
        }
        for (size_t i = 0; i < ins.size(); ++i) {
            // what the stencil reads of the stand-in, the producer reads of each of its inputs
            std::vector<Array*> readers = ins[i] ? std::vector<Array*>{ins[i]} : pins;
            for (Array* x : readers) {
                if (reach[i] > x->halo)
                    return fail(CN_ERR_UNSUPPORTED, "array " + std::to_string(x->name) + " was created with a halo of " +
                                                        std::to_string(x->halo) + " rows, the stencil reaches " + std::to_string(reach[i]));
                if (reach[i] > 0 && x->halo_fresh < reach[i] && std::find(stale.begin(), stale.end(), x) == stale.end())
                    stale.push_back(x);
            }
        }
        // With a halo deeper than the stencil's reach a sweep can also update rows of the halo
        // itself (the neighbour computes the same values for its own rows), so that the next
        // sweeps need no exchange: one exchange of `halo` rows serves up to halo / reach sweeps.
        // (a fused reduction does not stand in the way: it counts the rank's own rows only)
        if (deep_halo_ && halo_ > 1 && g.souts.empty() && !g.flat && !prod && ref->row_end > ref->row_begin) {
            int64_t e = halo_;
            for (size_t i = 0; i < ins.size(); ++i) {
                const bool refreshed = std::find(stale.begin(), stale.end(), ins[i]) != stale.end();
                const int64_t fresh = refreshed ? ins[i]->halo : ins[i]->halo_fresh;
                e = std::min<int64_t>(e, std::min<int64_t>(fresh, ins[i]->halo) - reach[i]);
            }
            for (Array* x : outs) e = std::min<int64_t>(e, x->halo);
            ext = std::max<int64_t>(e, 0);
        }
    }
    // Without a fused reduction the sweep can be cut along dimension 0: the rows next to the
    // slab edges wait for the neighbours' halo rows on a second stream while the interior,
    // which needs none of them, runs on the main stream.
    const bool overlap = overlap_halo_ && !stale.empty() && g.reds.empty() && g.souts.empty() && !g.flat && !prod && ext == 0;
    if (!overlap)
        if ((rc = exchange_halos(stale, stream_))) return rc;

    for (size_t i = 0; i < ins.size(); ++i) a.in[i] = ins[i] ? ins[i]->buf.data : nullptr;
    for (size_t kx = 0; kx < pins.size(); ++kx) a.in[ins.size() + kx] = pins[kx]->buf.data;
    for (size_t m = 0; m < outs.size(); ++m) {
        Array* x = outs[m];
        a.old[m] = x->buf.data;
        if (g.copy_through && g.outs[m].hazard) {
            if ((rc = ensure_shadow(x))) return rc;
            a.out[m] = x->shadow.data;
        } else {
            a.out[m] = x->buf.data;
        }
    }

    // iteration box in local coordinates
    const int64_t rb = ref->row_begin, re = ref->row_end;
    int64_t lo[3] = {0, 0, 0}, hi[3] = {0, 0, 0}, rlo[3] = {0, 0, 0}, rhi[3] = {0, 0, 0};
    for (int d = 0; d < nd; ++d) {
        lo[d] = g.box_lo[d];
        hi[d] = g.box_hi[d];
        rlo[d] = g.reg_lo[d];
        rhi[d] = g.reg_hi[d];
    }
    // local rows, widened by `ext` towards every neighbour that exists (the global box clips at
    // the physical edges of the array by itself)
    const int64_t wb = rb - (rb > 0 ? ext : 0), we = re + (re < ref->shape[0] ? ext : 0);
    a.own_lo = 0;
    a.own_hi = re - rb;
    lo[0] = std::max(lo[0], wb) - rb;
    hi[0] = std::min(hi[0], we) - rb;
    rlo[0] = std::max(rlo[0], wb) - rb;
    rhi[0] = std::min(rhi[0], we) - rb;
    int64_t strides[3];
    array_strides(*ref, strides);
    const int V = g.vec;
    // Tiles and grid of one launch over the box [lo, hi) (local coordinates).
    auto plan = [&](const int64_t* lo, const int64_t* hi, CnGroupArgs& a, int* grid_out, int64_t* ntiles_out,
                    bool* empty_out) -> int {
    bool empty = false;
    for (int d = 0; d < nd; ++d)
        if (hi[d] <= lo[d]) empty = true;
    int64_t ntiles = 0;
    if (g.flat) {
        int64_t n = ref->local_elems();
        a.lo[0] = 0;
        a.hi[0] = n;
        a.rlo[0] = 0;
        a.rhi[0] = n;
        int64_t per = (int64_t)k->tile.r * k->tile.block * V;
        ntiles = (n + per - 1) / per;
    } else {
        for (int d = 0; d < nd; ++d) {
            a.lo[d] = lo[d];
            a.hi[d] = hi[d];
            a.rlo[d] = rlo[d];
            a.rhi[d] = rhi[d];
        }
        a.stride[0] = strides[0];
        a.stride[1] = strides[1];
        a.stride[2] = strides[2];
        if (!empty) {
            const int L = nd - 1;
            int64_t xbase = V == 2 ? (lo[L] & ~1LL) : lo[L];
            if (nd == 1) {
                int64_t per = (int64_t)k->tile.r * k->tile.block * V;
                ntiles = (hi[0] - xbase + per - 1) / per;
            } else {
                int64_t ntx = (hi[L] - xbase + (int64_t)k->tile.tx * V - 1) / ((int64_t)k->tile.tx * V);
                int64_t rows_per = (int64_t)(k->tile.block / k->tile.tx) * k->tile.r;
                int64_t nty = (hi[nd - 2] - lo[nd - 2] + rows_per - 1) / rows_per;
                int64_t nz = nd == 3 ? hi[0] - lo[0] : 1;
                a.ntx = ntx;
                a.nty = nty;
                if (g.staged && nd == 3) {
                    // chunks of dimension 0: enough tiles to balance the persistent blocks,
                    // long enough that the 2*hz planes of run-in stay cheap
                    // The persistent blocks take chunks round-robin, so the launch lasts as long
                    // as the block with the most chunks: pick the chunk count whose load balance
                    // (mean / maximum chunks per block) times run-in efficiency is best.
                    const int64_t blocks = (int64_t)sm_count_ * k->blocks_per_sm;
                    const int64_t cols = ntx * nty;
                    int64_t nzc = 1, zchunk = nz;
                    double best = -1.0;
                    for (int64_t c = 1; c <= 64 && c <= nz; ++c) {
                        const int64_t zc = (nz + c - 1) / c;
                        if (c > 1 && zc < 16) break;
                        const int64_t cc = (nz + zc - 1) / zc;
                        const int64_t tiles = cols * cc;
                        const double per = (double)tiles / (double)blocks;
                        const double balance = tiles >= blocks ? per / (double)((tiles + blocks - 1) / blocks)
                                                               : (double)tiles / (double)blocks;
                        const double eff = balance * (double)zc / (double)(zc + 2 * g.hz);
                        if (eff > best + 1e-9) {
                            best = eff;
                            nzc = cc;
                            zchunk = zc;
                        }
                    }
                    a.nzc = nzc;
                    a.zchunk = zchunk;
                    ntiles = ntx * nty * nzc;
                } else {
                    ntiles = ntx * nty * nz;
                }
            }
        }
    }
        if (ntiles >= (1LL << 31)) return fail(CN_ERR_LIMIT, "too many tiles for one launch");
    if (g.staged && prod) {
        // rows and columns of the producer's inputs that hold data: the slab plus the halo
        // rows towards every neighbour that exists
        int64_t h = 0;
        if (nranks_ > 1 && !ref->replicated) {
            h = ref->halo;
            for (Array* x : pins) h = std::min<int64_t>(h, x->halo);
        }
        a.fill_lo[0] = rb > 0 ? -h : 0;
        a.fill_hi[0] = (re - rb) + (re < ref->shape[0] ? h : 0);
        a.fill_lo[1] = 0;
        a.fill_hi[1] = ref->shape[nd - 1];
    } else if (g.staged) {
        Array* sx = find(g.stage_array);
        if (!sx) return fail(CN_ERR_UNKNOWN_ARRAY, "stencil array vanished");
        if ((rc = encode_tensor_map(*sx, *k, g, &a))) return rc;
        a.error = error_word_;
    }
    a.ntiles = ntiles;
    // Grid: persistent blocks (one wave) when there are many tiles per block; with only a few
    // tiles per resident block a static split leaves a long tail, so small problems get one
    // block per tile and the hardware scheduler balances them.  Kernels with a fused
    // reduction stay within the partial-sum scratch; staged 3-D kernels always march.
    const int64_t resident = (int64_t)sm_count_ * k->blocks_per_sm;
    int64_t grid64 = std::min<int64_t>(std::max<int64_t>(ntiles, 1), resident);
    if (ntiles > resident && ntiles <= 16 * resident && !(g.staged && nd == 3)) {
        const int64_t cap = g.reds.empty() ? (int64_t)1 << 20 : (int64_t)max_grid_;
        if (ntiles <= cap) grid64 = ntiles;
    }
    int grid = (int)grid64;

    *grid_out = grid;
    *ntiles_out = ntiles;
    *empty_out = empty;
    return CN_OK;
    };
    int grid = 1;
    int64_t ntiles = 0;
    bool empty = false;
    if ((rc = plan(lo, hi, a, &grid, &ntiles, &empty))) return rc;

    std::vector<Array*> results;
    if ((rc = bind_reductions(g, &a, grid, &results))) return rc;
    // binding may have created arrays: the table can re-hash, so refresh raw pointers
    if (!results.empty()) {
        for (size_t q = 0; q < results.size(); ++q) {
            results[q] = find(g.reds[q].result_name);
            a.red[q] = results[q]->buf.data;
        }
        for (size_t m = 0; m < outs.size(); ++m) outs[m] = find(g.outs[m].name);
    }

    // (elements of the array table keep their addresses when the table grows)
    if (!g.tail.empty() && (rc = bind_tail(g, &a))) return rc;

    std::vector<Array*> pushed;
    if (k->tile.push && ntiles > 0 && !overlap) plan_push(g, outs, ext, &a, &pushed);
    if (ntiles > 0 || !g.reds.empty() || !g.souts.empty()) {
        // algorithmic bytes: every distinct array read once, every output written once
        double vol = 1;
        if (g.flat) vol = (double)ref->local_elems();
        else for (int d = 0; d < nd; ++d) vol *= (double)std::max<int64_t>(0, hi[d] - lo[d]);
        if (empty) vol = 0;
        const size_t n_arrays = in_names.size() + g.outs.size() + (prod ? pins.size() - 1 : 0);
        double bytes = vol * (double)n_arrays * dtype_size(g.dtype);
        bool done = false;
        if (overlap && !empty) {
            // rows [0, H) and [nl - H, nl) of the slab read halo rows; everything between does not
            // (H is the stencil's own reach along dimension 0, whatever depth the option holds now)
            const int64_t H = std::max<int64_t>(g.max_halo, 1), nl = re - rb;
            const int64_t i0 = std::max<int64_t>(lo[0], H), i1 = std::min<int64_t>(hi[0], nl - H);
            if (i1 - i0 >= 4 * H && (rc = ensure_second_stream()) == CN_OK) {
                const double row_bytes = bytes / (double)(hi[0] - lo[0]);
                cudaEventRecord(ev_fork_, stream_);
                cudaStreamWaitEvent(stream2_, ev_fork_, 0);
                for (Array* x : stale)
                    if ((rc = exchange_halo(x, stream2_))) return rc;
                int64_t blo[3] = {lo[0], lo[1], lo[2]}, bhi[3] = {hi[0], hi[1], hi[2]};
                const int64_t parts[3][2] = {{lo[0], i0}, {i1, hi[0]}, {i0, i1}};
                for (int part = 0; part < 3; ++part) {
                    blo[0] = parts[part][0];
                    bhi[0] = parts[part][1];
                    if (bhi[0] <= blo[0]) continue;
                    CnGroupArgs b = a;
                    int bgrid = 1;
                    int64_t bt = 0;
                    bool be = false;
                    if ((rc = plan(blo, bhi, b, &bgrid, &bt, &be))) return rc;
                    if (bt > 0 && (rc = launch(k, b, bgrid, k->tile.block, row_bytes * (double)(bhi[0] - blo[0]),
                                               part == 2 ? stream_ : stream2_)))
                        return rc;
                }
                cudaEventRecord(ev_join_, stream2_);
                cudaStreamWaitEvent(stream_, ev_join_, 0);
                stats_.overlapped_sweeps++;
                done = true;
            } else if (rc) {
                return rc;
            }
        }
        if (!done) {
            if (overlap)
                for (Array* x : stale)
                    if ((rc = exchange_halo(x, stream_))) return rc;
            if ((rc = launch(k, a, grid, k->tile.block, bytes))) return rc;
        }
    } else if (overlap) {
        for (Array* x : stale)
            if ((rc = exchange_halo(x, stream_))) return rc;
    }
    for (size_t m = 0; m < outs.size(); ++m) {
        Array* x = outs[m];
        const bool through = g.copy_through && g.outs[m].hazard;
        if (through) std::swap(x->buf, x->shadow);
        // The widened sweep left `ext` halo rows up to date where it wrote them.  An assignment
        // that is not copied through writes the region only: halo cells outside it (the side
        // columns of a two-array ping-pong sweep, a physical edge row inside the halo) keep
        // what they held, so they are only as fresh as the halo was before.
        int fresh = (int)ext;
        if (g.outs[m].is_set && !through) {
            bool whole = g.reg_lo[0] <= 0 && g.reg_hi[0] >= x->shape[0];
            for (int d = 1; d < nd; ++d) whole = whole && g.reg_lo[d] <= 0 && g.reg_hi[d] >= x->shape[d];
            if (!whole) fresh = std::min(fresh, x->halo_fresh);
        }
        x->halo_fresh = fresh;
        x->halo_pushed = std::find(pushed.begin(), pushed.end(), x) != pushed.end();
    }
    if (ext > 0) stats_.deep_halo_sweeps++;
    for (auto& sw : swaps) {
        free_buffer(&sw.first->buf);
        sw.first->buf = sw.second;
    }
    return finish_reductions(results, true);
}

// Which outputs of this launch store their edge rows into the neighbours' mailboxes
// themselves.  An output qualifies when a stencil has asked for its halo before, the launch
// leaves its halo stale (no widening), it writes whole rows, and it belongs to the group of
// arrays whose halos were last asked for together (their rows share one exchange epoch and lie
// one behind the other in the payload slot).  The rows are published and the neighbours'
// copied in by pull_pending(), when a stencil asks for them.
void Context::plan_push(const GroupIR& g, const std::vector<Array*>& outs, int64_t ext, CnGroupArgs* a,
                        std::vector<Array*>* pushed) {
    if (ext != 0 || !peer_.ready || halo_group_.empty()) return;
    for (size_t m = 0; m < outs.size() && m < CN_MAX_OUT; ++m) {
        Array* x = outs[m];
        const OutIR& o = g.outs[m];
        if (!x->halo_wanted || x->replicated || x->halo <= 0) continue;
        const auto part = std::find(halo_group_.begin(), halo_group_.end(), x->name);
        if (part == halo_group_.end()) continue;
        // every element of the edge rows has to come out of this kernel
        const bool through = g.copy_through && o.hazard;
        bool whole_rows = g.flat || through;
        if (!whole_rows) {
            whole_rows = !(g.two_domains && o.domain == DOM_REGION);
            for (int d = 1; d < g.ndims; ++d) whole_rows = whole_rows && g.box_lo[d] <= 0 && g.box_hi[d] >= x->shape[d];
            whole_rows = whole_rows && g.box_lo[0] <= x->row_begin && g.box_hi[0] >= x->row_end;
        }
        if (!whole_rows) continue;
        const size_t esz = dtype_size(x->dtype);
        const int64_t nl = x->local_rows();
        const size_t bytes = (size_t)x->halo * x->unit * esz;
        if (nl < x->halo || bytes % 8) continue;
        int64_t b, e;
        bool has_prev = false, has_next = false, thin = false;
        if (nl > 0 && rank_ > 0) {
            partition(x->shape[0], &b, &e, rank_ - 1);
            has_prev = e > b;
            thin = thin || (has_prev && e - b < x->halo);
        }
        if (nl > 0 && rank_ + 1 < nranks_) {
            partition(x->shape[0], &b, &e, rank_ + 1);
            has_next = e > b;
            thin = thin || (has_next && e - b < x->halo);
        }
        // every rank has to come to the same decision: no slab anywhere may be thinner than the halo
        for (int q = 0; q < nranks_ && !thin; ++q) {
            partition(x->shape[0], &b, &e, q);
            thin = e > b && e - b < x->halo;
        }
        if (thin) continue;
        // payload layout of the group: every member's rows, 16-byte aligned, in group order
        std::vector<size_t> sizes;
        size_t total = 0, offset = 0;
        bool fits = true;
        for (int name : halo_group_) {
            Array* y = find(name);
            if (!y || y->shape[0] != x->shape[0] || y->halo != x->halo || y->replicated) {
                fits = false;
                break;
            }
            const size_t sz = (size_t)y->halo * y->unit * dtype_size(y->dtype);
            if (name == x->name) offset = total;
            sizes.push_back(sz);
            total += (sz + 15) & ~(size_t)15;
        }
        if (!fits || total > CN_PEER_HALO_SLOT) continue;
        // one epoch at a time: rows of another group, or an earlier version of this array,
        // are published and pulled first
        if (pending_.active && (pending_.names != halo_group_ || x->halo_pushed)) {
            if (pull_pending(stream_) != CN_OK) return;
        }
        if (!pending_.active) {
            pending_ = PendingPush();
            pending_.active = true;
            pending_.names = halo_group_;
            pending_.bytes = sizes;
            pending_.has_prev = has_prev;
            pending_.has_next = has_next;
            if (has_prev) pending_.epoch_prev = ++peer_.epoch_prev;
            if (has_next) pending_.epoch_next = ++peer_.epoch_next;
        } else if (pending_.has_prev != has_prev || pending_.has_next != has_next) {
            continue;
        }
        const int bp = (int)(pending_.epoch_prev & 1ULL), bn = (int)(pending_.epoch_next & 1ULL);
        char* const base_prev = has_prev ? (char*)peer_.box[rank_ - 1] + sizeof(CnPeerBox) + (size_t)(bp * 2 + 1) * CN_PEER_HALO_SLOT : nullptr;
        char* const base_next = has_next ? (char*)peer_.box[rank_ + 1] + sizeof(CnPeerBox) + (size_t)(bn * 2 + 0) * CN_PEER_HALO_SLOT : nullptr;
        a->push_prev[m] = base_prev ? base_prev + offset : nullptr;
        a->push_next[m] = base_next ? base_next + offset : nullptr;
        a->push_elems = (long long)x->halo * x->unit;
        a->push_last = (long long)(nl - x->halo) * x->unit;
        a->push_mask |= 1u << m;
        pushed->push_back(x);
        stats_.halo_pushes++;
    }
}

// Rows of operand `x` (view rows `lv`) that this rank reads while it executes its iteration
// rows of `anchor`, when some of them live on other ranks: every rank takes part, receives what
// it reads from the others into a scratch copy and sends what the others read of its slab.
// *data stays null (and *base_row untouched) when every rank reads its own rows only.
int Context::fetch_operand_rows(Array* x, const Lattice& anchor, int64_t anchor_n0, const Lattice& lv, char** data,
                                int64_t* base_row, std::vector<void*>* fetched) {
    *data = nullptr;
    const std::vector<RowTransfer> moves = plan_transfers(anchor, anchor_n0, lv, x->shape[0], nranks_);
    if (moves.empty()) return CN_OK;
    if (!comm_.ready) return fail(CN_ERR_COMM, "moving operand rows between ranks needs cn_comm_init first");
    for (int r = 0; r < nranks_; ++r)
        if (failed_[r]) return fail(CN_ERR_RANK_FAILED, "rank " + std::to_string(r) + " was marked failed");
    const size_t esz = dtype_size(x->dtype);
    int rc;
    int64_t lo = 0, hi = 0;
    rows_read(anchor, anchor_n0, lv, nranks_, rank_, &lo, &hi);
    char* scratch = nullptr;
    if (hi > lo) {
        void* t = nullptr;
        if ((rc = cuda_fail(cudaMallocAsync(&t, (size_t)(hi - lo) * x->unit * esz + 256, stream_), "operand rows"))) return rc;
        fetched->push_back(t);
        scratch = (char*)t;
        const int64_t o0 = std::max(lo, x->row_begin), o1 = std::min(hi, x->row_end);  // rows this rank owns itself
        if (o1 > o0)
            if ((rc = cuda_fail(cudaMemcpyAsync(scratch + (size_t)(o0 - lo) * x->unit * esz,
                                                x->buf.data + (size_t)(o0 - x->row_begin) * x->unit * esz,
                                                (size_t)(o1 - o0) * x->unit * esz, cudaMemcpyDeviceToDevice, stream_),
                                "operand rows")))
                return rc;
    }
    {
        CommGroup group(&err_);
        if ((rc = group.started())) return rc;
        for (const RowTransfer& m : moves) {
            if (m.dst == rank_)
                if ((rc = comm_recv(&comm_, scratch + (size_t)(m.lo - lo) * x->unit * esz, (m.hi - m.lo) * x->unit, x->dtype,
                                    m.src, stream_, &err_)))
                    return rc;
            if (m.src == rank_)
                if ((rc = comm_send(&comm_, x->buf.data + (size_t)(m.lo - x->row_begin) * x->unit * esz,
                                    (m.hi - m.lo) * x->unit, x->dtype, m.dst, stream_, &err_)))
                    return rc;
        }
        if ((rc = group.end())) return rc;
    }
    stats_.row_fetches++;
    if (scratch) {
        *data = scratch;
        *base_row = lo;
    }
    return CN_OK;
}

int Context::run_strided(const GroupIR& g, CompiledGroup* k) {
    const int nd = g.ndims;
    CnGroupArgs a;
    memset(&a, 0, sizeof(a));
    std::vector<std::pair<Array*, Buffer>> swaps;
    int rc = bind_scalars(g, &a, &swaps);
    if (rc) return rc;
    if ((int)g.leaves.size() > CN_MAX_IN) return fail(CN_ERR_LIMIT, "too many operands in one group");

    // Iteration rows of this rank.  The anchor is the first output's view (the first operand's
    // for a group that only reduces): rank q executes the iteration rows whose anchor row lies
    // in its slab of the anchor array.  An operand whose view is stepped or offset against the
    // anchor may then read rows that live on other ranks; those rows are fetched into a scratch
    // copy first (the slab counterpart of send_remote_inputs, src/array_region.hpp:627-663).
    int64_t it_lo = 0, it_hi = g.extent[0];  // iteration rows executed on this rank
    Lattice anchor;
    int64_t anchor_n0 = 0;
    if (nranks_ > 1) {
        const Region* ar = nullptr;
        if (!g.outs.empty()) {
            ar = &g.outs[0].region;
            anchor_n0 = g.outs[0].shape[0];
        } else if (!g.leaves.empty()) {
            ar = &g.leaves[0].region;
            anchor_n0 = g.leaves[0].shape[0];
        }
        if (ar) {
            anchor = Lattice{ar->start[0], ar->stop[0], ar->step[0]};
            // further outputs have to walk their slabs exactly like the first one
            for (auto& o : g.outs)
                if (o.region.start[0] != ar->start[0] || o.region.step[0] != ar->step[0] || o.shape[0] != anchor_n0)
                    return fail(CN_ERR_UNSUPPORTED,
                                "outputs of one strided group that are offset against each other along "
                                "dimension 0 need a single rank");
            iteration_rows(anchor, anchor_n0, nranks_, rank_, &it_lo, &it_hi);
        }
    }
    std::vector<void*> fetched;  // scratch copies of operand rows, released after the launch
    std::vector<char*> leaf_scratch(g.leaves.size(), nullptr);

    // Address of iteration row it_lo of a view: `base_row` is the global row that `data` holds first.
    auto bind_view = [&](const Array& x, const Region& r, int64_t base_row, long long* off, long long* str) {
        int64_t s[3];
        array_strides(x, s);
        *off = (r.start[0] + it_lo * r.step[0] - base_row) * s[0];
        for (int d = 1; d < nd; ++d) *off += r.start[d] * s[d];
        for (int d = 0; d < nd; ++d) str[d] = r.step[d] * s[d];
    };
    for (size_t i = 0; i < g.leaves.size(); ++i) {
        const LeafIR& l = g.leaves[i];
        Array* x = find(l.name);
        if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "operand array " + std::to_string(l.name) + " does not exist");
        if ((rc = check_leaf(x, l.ndims, l.shape, "group operand"))) return rc;
        if (x->dtype != g.dtype) return fail(CN_ERR_BAD_DTYPE, "operand dtype differs from the group dtype");
        a.in[i] = x->buf.data;
        int64_t base_row = x->row_begin;
        if (nranks_ > 1 && !x->replicated) {
            const Lattice lv{l.region.start[0], l.region.stop[0], l.region.step[0]};
            char* scratch = nullptr;
            if ((rc = fetch_operand_rows(x, anchor, anchor_n0, lv, &scratch, &base_row, &fetched))) return rc;
            if (scratch) {
                a.in[i] = scratch;
                leaf_scratch[i] = scratch;
            }
        }
        bind_view(*x, l.region, base_row, &a.in_off[i], a.in_str[i]);
    }
    struct Pending {
        Array* target;
        Buffer temp;
        Region region;
    };
    std::vector<Pending> copy_back;
    int64_t ext[3] = {1, 1, 1};
    for (int d = 0; d < nd; ++d) ext[d] = g.extent[d];
    ext[0] = it_hi - it_lo;
    for (size_t m = 0; m < g.outs.size(); ++m) {
        const OutIR& o = g.outs[m];
        Array* x = find(o.name);
        if (o.is_set) {
            if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "SET_REGION target " + std::to_string(o.name) + " does not exist");
            if ((rc = check_leaf(x, o.ndims, o.shape, "SET_REGION target"))) return rc;
            if (x->dtype != g.dtype) return fail(CN_ERR_BAD_DTYPE, "target dtype differs from the group dtype");
        } else {
            if ((rc = create_array(o.name, o.ndims, o.shape, g.dtype, false, &x))) return rc;
            for (size_t i = 0; i < g.leaves.size(); ++i)
                a.in[i] = leaf_scratch[i] ? leaf_scratch[i] : find(g.leaves[i].name)->buf.data;
        }
        if (o.hazard) {
            // right-hand side reads the target elsewhere: evaluate into a dense temporary
            // first, then copy (what the reference always does, src/execute_node.cpp:1581-1584)
            Pending p;
            p.target = x;
            p.region = o.region;
            size_t bytes = (size_t)std::max<int64_t>(1, ext[0] * (nd > 1 ? ext[1] : 1) * (nd > 2 ? ext[2] : 1)) * dtype_size(g.dtype);
            void* t = nullptr;
            if ((rc = cuda_fail(cudaMallocAsync(&t, bytes + 256, stream_), "temporary"))) return rc;
            p.temp.alloc = t;
            p.temp.data = (char*)t;
            p.temp.bytes = bytes;
            a.out[m] = t;
            a.out_off[m] = 0;
            int64_t s = 1;
            for (int d = nd - 1; d >= 0; --d) {
                a.out_str[m][d] = s;
                s *= ext[d];
            }
            copy_back.push_back(p);
        } else {
            a.out[m] = x->buf.data;
            bind_view(*x, o.region, x->row_begin, &a.out_off[m], a.out_str[m]);
        }
        x->mark_written();
    }
    for (int d = 0; d < 3; ++d) a.ext[d] = d < nd ? ext[d] : 1;
    int64_t total = 1;
    for (int d = 0; d < nd; ++d) total *= ext[d];
    int grid = (int)std::min<int64_t>(std::max<int64_t>((total + k->tile.block - 1) / k->tile.block, 1), (int64_t)sm_count_ * k->blocks_per_sm);
    std::vector<Array*> results;
    if ((rc = bind_reductions(g, &a, grid, &results))) return rc;
    for (size_t q = 0; q < results.size(); ++q) {
        results[q] = find(g.reds[q].result_name);
        a.red[q] = results[q]->buf.data;
    }
    if (total > 0 || !g.reds.empty() || !g.souts.empty())
        if ((rc = launch(k, a, grid, k->tile.block,
                         (double)total * (double)(g.leaves.size() + g.outs.size()) * dtype_size(g.dtype))))
            return rc;
    for (auto& p : copy_back) {
        Array* x = find(p.target->name);
        StridedView dv, sv;
        int64_t e3[3] = {1, 1, 1};
        int64_t s[3];
        array_strides(*x, s);
        const int shift = 3 - nd;
        dv.off = (p.region.start[0] + it_lo * p.region.step[0] - x->row_begin) * s[0];
        for (int d = 1; d < nd; ++d) dv.off += p.region.start[d] * s[d];
        int64_t dense = 1;
        for (int d = nd - 1; d >= 0; --d) {
            e3[shift + d] = ext[d];
            dv.str[shift + d] = p.region.step[d] * s[d];
            sv.str[shift + d] = dense;
            dense *= ext[d];
        }
        if (total > 0) {
            if ((rc = cuda_fail(launch_copy_region(x->buf.data, dv, p.temp.data, sv, e3, g.dtype, stream_), "copy back"))) return rc;
            stats_.kernel_launches++;
        }
        cudaFreeAsync(p.temp.alloc, stream_);
    }
    for (void* t : fetched) cudaFreeAsync(t, stream_);
    for (auto& sw : swaps) {
        free_buffer(&sw.first->buf);
        sw.first->buf = sw.second;
    }
    return finish_reductions(results, true);
}

// ---- non-fusible nodes --------------------------------------------------------------------

int Context::operand_array(const Operand& op, Array** out, Region* region) {
    if (op.is_ref || !op.leaf) return fail(CN_ERR_BAD_BLOB, "operand must name an array");
    Array* x = find(op.leaf->result_name);
    if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "operand array " + std::to_string(op.leaf->result_name) + " does not exist");
    *out = x;
    *region = op.region.is_global ? Region::full(x->ndims, x->shape) : op.region;
    if (region->ndims != x->ndims) return fail(CN_ERR_SHAPE_MISMATCH, "operand region rank differs from its array");
    for (int d = 0; d < x->ndims; ++d)
        if (region->stop[d] > x->shape[d] || region->start[d] > region->stop[d])
            return fail(CN_ERR_SHAPE_MISMATCH, "operand region lies outside its array");
    return CN_OK;
}

// dot(lhs, rhs) / sum(x) -> size-1 array.  The reference accepts 1-D operands only
// (src/executor_reduce.cpp:9-12); any rank is accepted here as long as both operands are
// whole arrays of one shape (an addition to the protocol).
int Context::execute_reduce(const AstNode& r) {
    const bool is_dot = r.opcode == OP_REDUCE;
    if ((int)r.operands.size() != (is_dot ? 2 : 1)) return fail(CN_ERR_BAD_BLOB, "wrong operand count for a reduction");
    Array *x = nullptr, *y = nullptr;
    Region rx, ry;
    int rc = operand_array(r.operands[0], &x, &rx);
    if (rc) return rc;
    if (is_dot && (rc = operand_array(r.operands[1], &y, &ry))) return rc;
    auto whole = [](const Array& a, const Region& g) {
        for (int d = 0; d < a.ndims; ++d)
            if (g.start[d] != 0 || g.stop[d] != a.shape[d] || g.step[d] != 1) return false;
        return true;
    };
    if (!whole(*x, rx) || (y && !whole(*y, ry)))
        return fail(CN_ERR_UNSUPPORTED, "reductions over sub-regions are not supported; assign the view to an array first");
    if (y) {
        if (x->ndims != y->ndims) return fail(CN_ERR_SHAPE_MISMATCH, "dot operands have different ranks");
        for (int d = 0; d < x->ndims; ++d)
            if (x->shape[d] != y->shape[d]) return fail(CN_ERR_SHAPE_MISMATCH, "dot operands have different shapes");
        if (x->dtype != y->dtype) return fail(CN_ERR_BAD_DTYPE, "dot operands have different dtypes");
    }
    const int dtype = x->dtype;
    const int64_t n = x->local_elems();
    const void* px = x->buf.data;
    const void* py = y ? y->buf.data : nullptr;
    Array* res = nullptr;
    int64_t one[1] = {1};
    if ((rc = create_array(r.result_name, 1, one, dtype, false, &res))) return rc;
    int grid = dot_grid_size(n, sm_count_);
    if (grid > max_grid_) grid = max_grid_;
    prof_start(std::string(py ? "dot #" : "sum #") + kAotSourceDigest, (double)n * (py ? 2 : 1) * dtype_size(dtype));
    rc = cuda_fail(launch_dot(px, py, n, dtype, partials_, counter_, res->buf.data, grid, stream_), "dot");
    prof_stop();
    if (rc) return rc;
    stats_.kernel_launches++;
    std::vector<Array*> results{res};
    return finish_reductions(results, false);
}

// y = A @ x for a 2-D matrix and a 1-D vector; A is row-partitioned, x is gathered to every
// rank, each rank multiplies its row block (no partial sums cross ranks, unlike the
// reference's column-tile partials, src/execute_node.cpp:233-270, :550-578).
int Context::execute_matmul(const AstNode& r) {
    if (r.operands.size() != 2) return fail(CN_ERR_BAD_BLOB, "MATMUL needs (matrix, vector)");
    Array *A = nullptr, *x = nullptr;
    Region ra, rx;
    int rc = operand_array(r.operands[0], &A, &ra);
    if (rc) return rc;
    if ((rc = operand_array(r.operands[1], &x, &rx))) return rc;
    if (A->ndims != 2) return fail(CN_ERR_UNSUPPORTED, "only 2-D matrices are supported by matvec (3-D dim-drop and mat-mat are out of scope)");
    // an (n, 1) column vector is stored and partitioned exactly like a 1-D vector of n
    const bool column = x->ndims == 2 && x->shape[1] == 1;
    if (x->ndims != 1 && !column) return fail(CN_ERR_UNSUPPORTED, "matvec needs a 1-D vector or an (n, 1) column");
    if (A->dtype != x->dtype) return fail(CN_ERR_BAD_DTYPE, "matvec operands have different dtypes");
    if (!ra.unit_step() || !rx.unit_step()) return fail(CN_ERR_UNSUPPORTED, "matvec on stepped views is not supported");
    const int64_t rows = ra.extent(0), cols = ra.extent(1);
    if (cols != rx.extent(0)) return fail(CN_ERR_SHAPE_MISMATCH, "matrix columns differ from vector length");
    const size_t esz = dtype_size(A->dtype);
    const int dtype = A->dtype;
    const int aname = A->name, xname = x->name;
    int64_t yshape[2] = {rows, 1};
    Array* y = nullptr;
    if (r.result_name == aname || r.result_name == xname) return fail(CN_ERR_HAZARD, "matvec result aliases an operand");
    if ((rc = create_array(r.result_name, column ? 2 : 1, yshape, dtype, false, &y))) return rc;
    A = find(aname);
    x = find(xname);
    if (nranks_ == 1) {
        const char* pa = A->buf.data + (ra.start[0] * A->shape[1] + ra.start[1]) * esz;
        const char* px = x->buf.data + rx.start[0] * esz;
        prof_start(std::string("matvec #") + kAotSourceDigest, ((double)rows * cols + rows + cols) * esz);
        rc = cuda_fail(launch_matvec(pa, A->shape[1], px, y->buf.data, rows, cols, dtype, stream_), "matvec");
        prof_stop();
        if (rc) return rc;
        stats_.kernel_launches++;
        y->mark_written();
        return CN_OK;
    }
    // Several ranks: y is partitioned like any array of `rows` rows; each rank multiplies the
    // rows of A[rs:re, cs:ce] that belong to its rows of y.  For whole operands those are its
    // own rows of A; for a row slice they may live elsewhere and are fetched first (the
    // reference sends x slices and partial sums instead, src/executor_matmul.cpp:362-390).
    // x is gathered whole onto every rank.
    if (!comm_.ready) return fail(CN_ERR_COMM, "matvec across ranks needs cn_comm_init first");
    const int64_t xlen = x->shape[0];
    if ((rc = ensure_scratch((size_t)xlen * esz + 256))) return rc;
    A = find(aname);
    x = find(xname);
    y = find(r.result_name);
    {
        CommGroup group(&err_);
        if ((rc = group.started())) return rc;
        for (int p = 0; p < nranks_; ++p) {
            int64_t b, e;
            partition(xlen, &b, &e, p);
            if (e <= b) continue;
            if ((rc = comm_broadcast(&comm_, x->buf.data, (char*)scratch_ + b * esz, e - b, dtype, p, stream_, &err_))) return rc;
        }
        if ((rc = group.end())) return rc;
    }
    const Lattice anchor{0, rows, 1}, arows{ra.start[0], ra.stop[0], 1};
    std::vector<void*> fetched;
    char* moved = nullptr;
    int64_t base_row = A->row_begin;
    if ((rc = fetch_operand_rows(A, anchor, rows, arows, &moved, &base_row, &fetched))) return rc;
    const int64_t my_rows = y->local_rows();
    const char* pa = (moved ? moved : A->buf.data) + ((ra.start[0] + y->row_begin - base_row) * A->shape[1] + ra.start[1]) * esz;
    const char* px = (const char*)scratch_ + rx.start[0] * esz;
    prof_start(std::string("matvec #") + kAotSourceDigest, ((double)my_rows * cols + my_rows + cols) * esz);
    rc = cuda_fail(launch_matvec(pa, A->shape[1], px, y->buf.data, my_rows, cols, dtype, stream_), "matvec");
    prof_stop();
    for (void* t : fetched) cudaFreeAsync(t, stream_);
    if (rc) return rc;
    stats_.kernel_launches++;
    y->mark_written();
    return CN_OK;
}

// Cross-dimension SET_REGION (execute_cross_set_region_node, src/executor_transfer.cpp:66-177):
// the assigned region and the source view have different ranks, or carry their singleton
// dimensions in different places -- `A[i, :] = v`, `v[:] = A[:, j]`, `H[t, :, k:] = prev`.  The
// dimensions of extent > 1 of both sides are matched in order (the reference's dim_map); the
// assignment is then one strided copy.  With several ranks the source rows are either aligned
// with the target rows through the row lattices (both sides iterate over their dimension 0
// together), or the source region is gathered whole onto every rank first.
int Context::execute_cross_set_region(const AstNode& r) {
    if (r.operands.size() != 2 || !r.operands[0].leaf) return fail(CN_ERR_BAD_BLOB, "SET_REGION needs (target, rhs)");
    Array* t = find(r.operands[0].leaf->result_name);
    if (!t) return fail(CN_ERR_UNKNOWN_ARRAY, "SET_REGION target " + std::to_string(r.operands[0].leaf->result_name) + " does not exist");
    Array* src = nullptr;
    Region sreg;
    int rc = operand_array(r.operands[1], &src, &sreg);
    if (rc) return rc;
    if (src->dtype != t->dtype) return fail(CN_ERR_BAD_DTYPE, "SET_REGION source dtype differs from the target");
    if (src->name == t->name) return fail(CN_ERR_HAZARD, "cross-dimension SET_REGION of an array into itself");
    Region treg = r.region.is_global ? Region::full(t->ndims, t->shape) : r.region;
    if (treg.ndims != t->ndims) return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION region rank differs from target");
    for (int d = 0; d < t->ndims; ++d)
        if (treg.stop[d] > t->shape[d] || treg.start[d] > treg.stop[d]) return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION region outside its target");
    // dimensions of extent > 1, matched in order
    int map[kMaxDims] = {-1, -1, -1};  // target dim -> source dim
    std::vector<int> td, sd;
    for (int d = 0; d < t->ndims; ++d)
        if (treg.extent(d) > 1) td.push_back(d);
    for (int d = 0; d < src->ndims; ++d)
        if (sreg.extent(d) > 1) sd.push_back(d);
    if (td.size() != sd.size()) return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION source and region do not have the same non-singleton dimensions");
    for (size_t i = 0; i < td.size(); ++i) {
        if (treg.extent(td[i]) != sreg.extent(sd[i])) return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION source does not match the region shape");
        map[td[i]] = sd[i];
    }
    if (treg.size() == 0) return CN_OK;
    if (treg.size() != sreg.size()) return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION source does not match the region shape");
    const size_t esz = dtype_size(t->dtype);
    int64_t ts[3], ss[3];
    array_strides(*t, ts);
    array_strides(*src, ss);
    // target rows of the region on this rank: positions [i0, i1) along the region's dimension 0
    const Lattice trows{treg.start[0], treg.stop[0], treg.step[0]};
    int64_t i0 = 0, i1 = treg.extent(0);
    if (nranks_ > 1 && !t->replicated) iteration_rows(trows, t->shape[0], nranks_, rank_, &i0, &i1);
    const char* sdata = src->buf.data;
    int64_t sbase = src->row_begin;  // global row that sdata holds first
    std::vector<void*> fetched;
    const bool row_aligned = map[0] == 0;  // both sides walk their dimension 0 together
    if (nranks_ > 1 && !src->replicated) {
        if (!comm_.ready) return fail(CN_ERR_COMM, "SET_REGION across ranks needs cn_comm_init first");
        if (row_aligned && !t->replicated) {
            char* moved = nullptr;
            const Lattice srows{sreg.start[0], sreg.stop[0], sreg.step[0]};
            if ((rc = fetch_operand_rows(src, trows, t->shape[0], srows, &moved, &sbase, &fetched))) return rc;
            if (moved) sdata = moved;
        } else {
            // every rank gets the rows of the source region: [sreg.start[0], sreg.stop[0])
            const int64_t g0 = sreg.start[0], g1 = sreg.stop[0];
            if ((rc = ensure_scratch((size_t)(g1 - g0) * src->unit * esz + 256))) return rc;
            t = find(r.operands[0].leaf->result_name);
            src = find(r.operands[1].leaf->result_name);
            CommGroup group(&err_);
            if ((rc = group.started())) return rc;
            for (int p = 0; p < nranks_; ++p) {
                int64_t b, e;
                partition(src->shape[0], &b, &e, p);
                const int64_t o0 = std::max(b, g0), o1 = std::min(e, g1);
                if (o1 <= o0) continue;
                const char* mine = src->buf.data + (size_t)(o0 - src->row_begin) * src->unit * esz;
                char* const landing = (char*)scratch_ + (size_t)(o0 - g0) * src->unit * esz;
                if ((rc = comm_broadcast(&comm_, p == rank_ ? mine : landing, landing,
                                         (o1 - o0) * src->unit, src->dtype, p, stream_, &err_)))
                    return rc;
            }
            if ((rc = group.end())) return rc;
            sdata = (const char*)scratch_;
            sbase = g0;
        }
    }
    if (i1 > i0) {
        StridedView dv, sv;
        int64_t ext[3] = {1, 1, 1};
        const int shift = 3 - t->ndims;
        dv.off = (treg.start[0] + i0 * treg.step[0] - t->row_begin) * ts[0];
        for (int d = 1; d < t->ndims; ++d) dv.off += treg.start[d] * ts[d];
        // source element of region position 0 along every dimension, rows counted from sbase
        sv.off = (sreg.start[0] - sbase) * ss[0];
        for (int d = 1; d < src->ndims; ++d) sv.off += sreg.start[d] * ss[d];
        for (int d = 0; d < t->ndims; ++d) {
            ext[shift + d] = d == 0 ? i1 - i0 : treg.extent(d);
            dv.str[shift + d] = treg.step[d] * ts[d];
            sv.str[shift + d] = map[d] >= 0 ? sreg.step[map[d]] * ss[map[d]] : 0;
        }
        // the target's dimension 0 starts at position i0: advance the source along the dimension it maps to
        if (map[0] >= 0) sv.off += i0 * sreg.step[map[0]] * ss[map[0]];
        rc = cuda_fail(launch_copy_region(t->buf.data, dv, sdata, sv, ext, t->dtype, stream_), "cross-dimension copy");
        if (rc) return rc;
        stats_.kernel_launches++;
    }
    for (void* p : fetched) cudaFreeAsync(p, stream_);
    t->mark_written();
    return CN_OK;
}

// DIAG (src/execute_node.cpp:600-750): a vector becomes the k-th diagonal of a zeroed square
// matrix, or the k-th diagonal of a matrix becomes a vector.  Both are one strided copy.
// With k = 0 (and rows <= cols for the extraction) the row partition of the matrix and the
// partition of the vector coincide, so the copy is local on every rank; with an offset the
// rows behind a rank's part of the result are fetched from their owners first.
int Context::execute_diag(const AstNode& r) {
    if (r.operands.size() != 2) return fail(CN_ERR_BAD_BLOB, "DIAG needs (array, k)");
    const Operand& kop = r.operands[1];
    if (kop.is_ref || !kop.leaf || !kop.leaf->is_scalar) return fail(CN_ERR_BAD_BLOB, "DIAG offset must be a literal scalar");
    const int64_t k = (int64_t)kop.leaf->scalar;
    Array* v = nullptr;
    Region rv;
    int rc = operand_array(r.operands[0], &v, &rv);
    if (rc) return rc;
    for (int d = 0; d < v->ndims; ++d)
        if (rv.start[d] != 0 || rv.stop[d] != v->shape[d] || rv.step[d] != 1)
            return fail(CN_ERR_UNSUPPORTED, "DIAG of a view is not supported; assign the view to an array first");
    if (r.result_name == v->name) return fail(CN_ERR_HAZARD, "DIAG result aliases its operand");
    const int64_t roff = k < 0 ? -k : 0, coff = k > 0 ? k : 0;
    const int vname = v->name, dtype = v->dtype;
    const size_t esz = dtype_size(dtype);
    Array* out = nullptr;
    StridedView dv, sv;
    int64_t ext[3] = {1, 1, 0};
    const char* sdata = nullptr;
    std::vector<void*> fetched;
    if (v->ndims == 1) {
        // out[i + roff, i + coff] = v[i]: this rank fills the diagonal entries of its own rows
        const int64_t len = v->shape[0], n = len + roff + coff;
        int64_t shape[2] = {n, n};
        if ((rc = create_array(r.result_name, 2, shape, dtype, true, &out))) return rc;
        v = find(vname);
        int64_t i0 = 0, i1 = len;  // positions along the diagonal whose row this rank owns
        const Lattice orows{roff, roff + len, 1}, vrows{0, len, 1};
        int64_t vbase = v->row_begin;
        sdata = v->buf.data;
        if (nranks_ > 1) {
            iteration_rows(orows, n, nranks_, rank_, &i0, &i1);
            char* moved = nullptr;
            if ((rc = fetch_operand_rows(v, orows, n, vrows, &moved, &vbase, &fetched))) return rc;
            out = find(r.result_name);
            v = find(vname);
            if (moved) sdata = moved;
            else sdata = v->buf.data;
        }
        ext[2] = i1 - i0;
        sv.off = i0 - vbase;
        sv.str[2] = 1;
        dv.off = (i0 + roff - out->row_begin) * n + i0 + coff;
        dv.str[2] = n + 1;
    } else if (v->ndims == 2) {
        // d[i] = M[i + roff, i + coff]: this rank fills its own entries of d
        const int64_t rows = v->shape[0], cols = v->shape[1];
        const int64_t len = k >= 0 ? std::min(rows, cols - k) : std::min(rows + k, cols);
        if (len <= 0) return fail(CN_ERR_SHAPE_MISMATCH, "DIAG offset outside the matrix");
        int64_t shape[1] = {len};
        if ((rc = create_array(r.result_name, 1, shape, dtype, false, &out))) return rc;
        v = find(vname);
        const Lattice drows{0, len, 1}, mrows{roff, roff + len, 1};
        int64_t mbase = v->row_begin;
        sdata = v->buf.data;
        if (nranks_ > 1) {
            char* moved = nullptr;
            if ((rc = fetch_operand_rows(v, drows, len, mrows, &moved, &mbase, &fetched))) return rc;
            out = find(r.result_name);
            v = find(vname);
            sdata = moved ? moved : v->buf.data;
        }
        ext[2] = out->local_rows();
        dv.off = 0;
        dv.str[2] = 1;
        sv.off = (out->row_begin + roff - mbase) * cols + out->row_begin + coff;
        sv.str[2] = cols + 1;
    } else {
        return fail(CN_ERR_UNSUPPORTED, "DIAG needs a 1-D or 2-D array");
    }
    if (ext[2] > 0) {
        rc = cuda_fail(launch_copy_region(out->buf.data, dv, sdata, sv, ext, dtype, stream_), "diag");
        if (rc) return rc;
        stats_.kernel_launches++;
    }
    for (void* p : fetched) cudaFreeAsync(p, stream_);
    (void)esz;
    out->mark_written();
    return CN_OK;
}

// TILE (charmnumeric/operations.py:52-72, src/executor_transfer.cpp): the operand is repeated
// along every dimension, with leading dimensions added when there are more repeat counts than
// operand dimensions.  The operand is usually small: with several ranks it is gathered whole
// onto every rank first (the same grouped broadcasts cn_get uses), then every rank fills its
// own rows of the result.
int Context::execute_tile(const AstNode& r) {
    if (r.operands.size() < 2) return fail(CN_ERR_BAD_BLOB, "TILE needs (array, repeat counts...)");
    Array* x = nullptr;
    Region rx;
    int rc = operand_array(r.operands[0], &x, &rx);
    if (rc) return rc;
    for (int d = 0; d < x->ndims; ++d)
        if (rx.start[d] != 0 || rx.stop[d] != x->shape[d] || rx.step[d] != 1)
            return fail(CN_ERR_UNSUPPORTED, "TILE of a view is not supported; assign the view to an array first");
    const int nrep = (int)r.operands.size() - 1;
    const int ond = std::max(x->ndims, nrep);
    if (ond > kMaxDims) return fail(CN_ERR_UNSUPPORTED, "TILE result has more than three dimensions");
    if (r.result_name == x->name) return fail(CN_ERR_HAZARD, "TILE result aliases its operand");
    // shapes left-aligned on the result's dimensions: the operand gets leading 1s, the repeat
    // counts too; unused trailing slots are 1
    int64_t sshape[3] = {1, 1, 1}, oshape[3] = {1, 1, 1};
    for (int d = 0; d < x->ndims; ++d) sshape[ond - x->ndims + d] = x->shape[d];
    for (int d = 0; d < ond; ++d) oshape[d] = sshape[d];
    for (int i = 0; i < nrep; ++i) {
        const Operand& op = r.operands[1 + i];
        if (op.is_ref || !op.leaf || !op.leaf->is_scalar) return fail(CN_ERR_BAD_BLOB, "TILE repeat counts must be literal scalars");
        const int64_t rep = (int64_t)op.leaf->scalar;
        if (rep < 1) return fail(CN_ERR_INVALID_ARGUMENT, "TILE repeat counts must be positive");
        oshape[ond - nrep + i] *= rep;
    }
    const int dtype = x->dtype, xname = x->name;
    const size_t esz = dtype_size(dtype);
    Array* out = nullptr;
    if ((rc = create_array(r.result_name, ond, oshape, dtype, false, &out))) return rc;
    x = find(xname);
    const void* src = x->buf.data;
    if (nranks_ > 1 && !x->replicated) {
        if (!comm_.ready) return fail(CN_ERR_COMM, "TILE across ranks needs cn_comm_init first");
        if ((rc = ensure_scratch((size_t)x->global_elems() * esz + 256))) return rc;
        CommGroup group(&err_);
    if ((rc = group.started())) return rc;
        for (int p = 0; p < nranks_; ++p) {
            int64_t b, e;
            partition(x->shape[0], &b, &e, p);
            if (e <= b) continue;
            if ((rc = comm_broadcast(&comm_, x->buf.data, (char*)scratch_ + b * x->unit * esz, (e - b) * x->unit, dtype, p, stream_, &err_))) return rc;
        }
        if ((rc = group.end())) return rc;
        src = scratch_;
    }
    rc = cuda_fail(launch_tile(out->buf.data, oshape, out->row_begin, out->local_rows(), src, sshape, dtype, stream_), "tile");
    if (rc) return rc;
    stats_.kernel_launches++;
    out->mark_written();
    return CN_OK;
}

// Seeded uniform fill (an addition: the reference's random.randn returns zeros,
// charmnumeric/random.py:4-5).  Element with global linear index g depends on (seed, g)
// only, so the values do not change with the number of ranks.
int Context::execute_randu(const AstNode& r) {
    if (r.operands.size() != 3) return fail(CN_ERR_BAD_BLOB, "RANDU needs (seed, lo, hi)");
    double v[3];
    for (int i = 0; i < 3; ++i) {
        const Operand& op = r.operands[i];
        if (op.is_ref || !op.leaf || !op.leaf->is_scalar) return fail(CN_ERR_BAD_BLOB, "RANDU operands must be literal scalars");
        v[i] = op.leaf->scalar;
    }
    if (v[0] < 0 || v[0] > 9007199254740992.0) return fail(CN_ERR_INVALID_ARGUMENT, "RANDU seed must be an integer in [0, 2^53]");
    Array* x = nullptr;
    int rc = create_array(r.result_name, r.ndims, r.shape, r.dtype, false, &x);
    if (rc) return rc;
    rc = cuda_fail(launch_randu(x->buf.data, x->dtype, x->local_elems(), x->row_begin * x->unit,
                                (uint64_t)v[0], v[1], v[2], stream_), "randu");
    if (rc) return rc;
    stats_.kernel_launches++;
    x->mark_written();
    return CN_OK;
}

// ---- host-facing data movement -----------------------------------------------------------

int Context::synchronize() {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    int rc = cuda_fail(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    if (rc) return rc;
    return check_device_error();
}

// A staged kernel whose bounded wait on a tile ran out leaves 1 in the error word.
int Context::check_device_error() {
    if (waiting_launches_ == checked_launches_) return CN_OK;
    checked_launches_ = waiting_launches_;
    unsigned int word = 0;
    unsigned int* dst = pinned_ ? (unsigned int*)(pinned_ + kPinnedWord) : &word;
    int rc = cuda_fail(cudaMemcpyAsync(dst, error_word_, sizeof(word), cudaMemcpyDeviceToHost, stream_), "error word");
    if (rc) return rc;
    if ((rc = cuda_fail(cudaStreamSynchronize(stream_), "cudaStreamSynchronize"))) return rc;
    return report_error_word(*dst);
}

int Context::report_error_word(unsigned int word) {
    if (word) {
        cudaMemsetAsync(error_word_, 0, sizeof(word), stream_);
        return fail(CN_ERR_CUDA, word == 1 ? "a stencil kernel gave up waiting for a tile copy (results are incomplete)"
                                           : "a kernel gave up waiting for another GPU's data (results are incomplete)");
    }
    return CN_OK;
}

int Context::get(int name, int64_t count, int dtype, void* out) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    cudaSetDevice(device_);
    Array* x = find(name);
    if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "get: unknown array " + std::to_string(name));
    if (dtype != x->dtype) return fail(CN_ERR_BAD_DTYPE, "get: dtype differs from the stored array");
    if (count != x->global_elems()) return fail(CN_ERR_SHAPE_MISMATCH, "get: element count differs from the stored array");
    if (!out) return fail(CN_ERR_INVALID_ARGUMENT, "get: null output buffer");
    const size_t esz = dtype_size(dtype);
    int rc;
    if ((nranks_ == 1 || x->replicated) && pinned_ && count * esz <= (size_t)kPinnedWord) {
        // a small result (the scalar a solver reads every step): result and error word travel
        // as two asynchronous copies into pinned memory behind one synchronisation
        if ((rc = cuda_fail(cudaMemcpyAsync(pinned_, x->buf.data, count * esz, cudaMemcpyDeviceToHost, stream_), "get copy"))) return rc;
        const bool check = waiting_launches_ != checked_launches_;
        if (check) {
            checked_launches_ = waiting_launches_;
            if ((rc = cuda_fail(cudaMemcpyAsync(pinned_ + kPinnedWord, error_word_, sizeof(unsigned int),
                                                cudaMemcpyDeviceToHost, stream_), "error word"))) return rc;
        }
        if ((rc = cuda_fail(cudaStreamSynchronize(stream_), "cudaStreamSynchronize"))) return rc;
        memcpy(out, pinned_, count * esz);
        stats_.bytes_d2h += count * esz;
        return check ? report_error_word(*(unsigned int*)(pinned_ + kPinnedWord)) : CN_OK;
    }
    if (nranks_ == 1 || x->replicated) {
        if ((rc = cuda_fail(cudaMemcpyAsync(out, x->buf.data, count * esz, cudaMemcpyDeviceToHost, stream_), "get copy"))) return rc;
        stats_.bytes_d2h += count * esz;
        return synchronize();
    }
    if (!comm_.ready) return fail(CN_ERR_COMM, "get across ranks needs cn_comm_init first");
    if ((rc = ensure_scratch(count * esz + 256))) return rc;
    x = find(name);
    CommGroup group(&err_);
    if ((rc = group.started())) return rc;
    for (int p = 0; p < nranks_; ++p) {
        int64_t b, e;
        partition(x->shape[0], &b, &e, p);
        if (e <= b) continue;
        if ((rc = comm_broadcast(&comm_, x->buf.data, (char*)scratch_ + b * x->unit * esz, (e - b) * x->unit, dtype, p, stream_, &err_))) return rc;
    }
    if ((rc = group.end())) return rc;
    if ((rc = cuda_fail(cudaMemcpyAsync(out, scratch_, count * esz, cudaMemcpyDeviceToHost, stream_), "get copy"))) return rc;
    stats_.bytes_d2h += count * esz;
    return synchronize();
}

// The whole array on rank `root` only (the reference assembles it on PE 0,
// src/partition_get.cpp:3-67): every other rank sends its slab straight to the root, which
// receives the slabs side by side in a device staging buffer and copies it to the host once.
// Only the root holds the full array; NVLink carries every slab once.
int Context::get_root(int name, int64_t count, int dtype, int root, void* out) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    if (root < 0 || root >= nranks_) return fail(CN_ERR_INVALID_ARGUMENT, "get_root: root rank out of range");
    if (nranks_ == 1) return get(name, count, dtype, out);
    cudaSetDevice(device_);
    Array* x = find(name);
    if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "get_root: unknown array " + std::to_string(name));
    if (dtype != x->dtype) return fail(CN_ERR_BAD_DTYPE, "get_root: dtype differs from the stored array");
    if (count != x->global_elems()) return fail(CN_ERR_SHAPE_MISMATCH, "get_root: element count differs from the stored array");
    const bool is_root = rank_ == root;
    if (is_root && !out) return fail(CN_ERR_INVALID_ARGUMENT, "get_root: null output buffer on the root");
    const size_t esz = dtype_size(dtype);
    int rc;
    if (x->replicated) {
        if (is_root) {
            if ((rc = cuda_fail(cudaMemcpyAsync(out, x->buf.data, count * esz, cudaMemcpyDeviceToHost, stream_), "get copy"))) return rc;
            stats_.bytes_d2h += count * esz;
        }
        return synchronize();
    }
    for (int r = 0; r < nranks_; ++r)
        if (failed_[r]) return fail(CN_ERR_RANK_FAILED, "rank " + std::to_string(r) + " was marked failed");
    if (!comm_.ready) return fail(CN_ERR_COMM, "get across ranks needs cn_comm_init first");
    if (is_root) {
        if ((rc = ensure_scratch(count * esz + 256))) return rc;
        x = find(name);
    }
    {
        CommGroup group(&err_);
        if ((rc = group.started())) return rc;
        if (is_root) {
            for (int p = 0; p < nranks_; ++p) {
                int64_t b, e;
                partition(x->shape[0], &b, &e, p);
                if (e <= b || p == root) continue;
                if ((rc = comm_recv(&comm_, (char*)scratch_ + b * x->unit * esz, (e - b) * x->unit, dtype, p, stream_, &err_))) return rc;
            }
        } else if (x->local_elems() > 0) {
            if ((rc = comm_send(&comm_, x->buf.data, x->local_elems(), dtype, root, stream_, &err_))) return rc;
        }
        if ((rc = group.end())) return rc;
    }
    if (is_root) {
        // the root's own slab goes straight from the array to the host buffer
        const size_t own_off = (size_t)x->row_begin * x->unit * esz, own = (size_t)x->local_elems() * esz;
        if (own_off)
            if ((rc = cuda_fail(cudaMemcpyAsync(out, scratch_, own_off, cudaMemcpyDeviceToHost, stream_), "get copy"))) return rc;
        if (own)
            if ((rc = cuda_fail(cudaMemcpyAsync((char*)out + own_off, x->buf.data, own, cudaMemcpyDeviceToHost, stream_), "get copy"))) return rc;
        const size_t tail = own_off + own;
        if (count * esz > tail)
            if ((rc = cuda_fail(cudaMemcpyAsync((char*)out + tail, (char*)scratch_ + tail, count * esz - tail, cudaMemcpyDeviceToHost, stream_), "get copy"))) return rc;
        stats_.bytes_d2h += count * esz;
    }
    return synchronize();
}

int Context::get_local(int name, int64_t* row_begin, int64_t* row_end, int64_t capacity, void* out) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    cudaSetDevice(device_);
    Array* x = find(name);
    if (!x) return fail(CN_ERR_UNKNOWN_ARRAY, "get_local: unknown array " + std::to_string(name));
    if (row_begin) *row_begin = x->row_begin;
    if (row_end) *row_end = x->row_end;
    if (!out) return CN_OK;
    if (capacity < x->local_elems()) return fail(CN_ERR_INVALID_ARGUMENT, "get_local: buffer too small");
    const size_t bytes = (size_t)x->local_elems() * dtype_size(x->dtype);
    int rc = cuda_fail(cudaMemcpyAsync(out, x->buf.data, bytes, cudaMemcpyDeviceToHost, stream_), "get_local copy");
    if (rc) return rc;
    stats_.bytes_d2h += bytes;
    return synchronize();
}

int Context::put(int name, int ndims, const int64_t* shape, int dtype, const void* host) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    cudaSetDevice(device_);
    if (!host) return fail(CN_ERR_INVALID_ARGUMENT, "put: null host buffer");
    Array* x = nullptr;
    int rc = create_array(name, ndims, shape, dtype, false, &x);
    if (rc) return rc;
    const size_t esz = dtype_size(dtype);
    const size_t bytes = (size_t)x->local_elems() * esz;
    const char* src = (const char*)host + (size_t)x->row_begin * x->unit * esz;
    if (bytes) {
        if ((rc = cuda_fail(cudaMemcpyAsync(x->buf.data, src, bytes, cudaMemcpyHostToDevice, stream_), "put copy"))) return rc;
        stats_.bytes_h2d += bytes;
    }
    x->mark_written();
    return CN_OK;
}

// This rank's slab only, from a host buffer that holds just those rows.
int Context::put_local(int name, int ndims, const int64_t* shape, int dtype, int64_t capacity, const void* host_slab) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    cudaSetDevice(device_);
    Array* x = nullptr;
    int rc = create_array(name, ndims, shape, dtype, false, &x);
    if (rc) return rc;
    if (capacity < x->local_elems()) return fail(CN_ERR_INVALID_ARGUMENT, "put_local: buffer smaller than this rank's slab");
    const size_t bytes = (size_t)x->local_elems() * dtype_size(dtype);
    if (bytes) {
        if (!host_slab) return fail(CN_ERR_INVALID_ARGUMENT, "put_local: null host buffer");
        if ((rc = cuda_fail(cudaMemcpyAsync(x->buf.data, host_slab, bytes, cudaMemcpyHostToDevice, stream_), "put copy"))) return rc;
        stats_.bytes_h2d += bytes;
    }
    x->mark_written();
    return CN_OK;
}

// One serialized node (the `node` production of the blob format), executed at once: the
// executor-level entry point (DAGExecutor::execute_dag_node, src/backend.hpp:334).
int Context::execute_single_node(const char* blob, int64_t size) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    for (int r = 0; r < nranks_; ++r)
        if (failed_[r]) return fail(CN_ERR_RANK_FAILED, "rank " + std::to_string(r) + " was marked failed");
    cudaSetDevice(device_);
    Dag dag;
    dag.nodes.emplace_back();
    int rc = parse_node(blob, size, &dag.nodes[0], &err_);
    if (rc) return rc;
    size_t i = 0;
    return execute_node(dag, &i);
}

int Context::timer_start() {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    return cuda_fail(cudaEventRecord(ev_start_, stream_), "cudaEventRecord");
}

int Context::timer_stop(float* ms) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    int rc = cuda_fail(cudaEventRecord(ev_stop_, stream_), "cudaEventRecord");
    if (rc) return rc;
    if ((rc = cuda_fail(cudaEventSynchronize(ev_stop_), "cudaEventSynchronize"))) return rc;
    return cuda_fail(cudaEventElapsedTime(ms, ev_start_, ev_stop_), "cudaEventElapsedTime");
}

// ---- kernel-ABI level: compile a group, launch it on caller-provided strided views ----------

int Context::compile_group(const char* blob, int64_t size, uint64_t* handle) {
    DagNode node;
    int rc = parse_node(blob, size, &node, &err_);
    if (rc) return rc;
    GroupIR g;
    rc = lower_group(node, {}, &g, &err_, true);
    if (rc) return rc;
    std::string src;
    if ((rc = generate_source(g, &src, &err_))) return rc;
    if (initialised_) {
        cudaSetDevice(device_);
        CompiledGroup* k = nullptr;
        if ((rc = get_kernel(g, &k))) return rc;
    } else {
        // no device: still prove that the source compiles for sm_100a
        std::vector<char> cubin;
        std::string log;
        if ((rc = nvrtc_compile(src, tile_, &cubin, &log))) return fail(rc, "group kernel failed to compile:\n" + log);
    }
    handles_.push_back({src, g});
    *handle = handles_.size();
    return CN_OK;
}

int Context::group_source(uint64_t handle, const char** src) {
    if (handle == 0 || handle > handles_.size()) return fail(CN_ERR_INVALID_ARGUMENT, "bad group handle");
    *src = handles_[handle - 1].first.c_str();
    return CN_OK;
}

int Context::launch_group(uint64_t handle, int n_in, void* const* in_ptrs, const int64_t* in_off,
                          const int64_t* in_str, int n_bc, void* const* bc_ptrs, int n_out,
                          void* const* out_ptrs, const int64_t* out_off, const int64_t* out_str,
                          const int64_t* ext) {
    if (!initialised_) return fail(CN_ERR_NO_DEVICE, "context not initialised");
    if (handle == 0 || handle > handles_.size()) return fail(CN_ERR_INVALID_ARGUMENT, "bad group handle");
    cudaSetDevice(device_);
    const GroupIR& g = handles_[handle - 1].second;
    if (g.cls == GroupIR::SCALAR_ONLY || !g.reds.empty() || !g.souts.empty())
        return fail(CN_ERR_UNSUPPORTED, "raw launch supports array-valued groups without reductions");
    if (n_in != (int)g.leaves.size() || n_out != (int)g.outs.size() || n_bc != (int)g.bcast_names.size())
        return fail(CN_ERR_INVALID_ARGUMENT, "argument counts differ from the compiled group");
    CompiledGroup* k = nullptr;
    int rc = get_kernel(g, &k);
    if (rc) return rc;
    CnGroupArgs a;
    memset(&a, 0, sizeof(a));
    for (size_t i = 0; i < g.scalars.size(); ++i) a.sc[i] = g.scalars[i];
    for (int i = 0; i < n_bc; ++i) a.bc[i] = bc_ptrs[i];
    const int nd = g.ndims;
    for (int i = 0; i < n_in; ++i) {
        a.in[i] = in_ptrs[i];
        a.in_off[i] = in_off[i];
        for (int d = 0; d < nd; ++d) a.in_str[i][d] = in_str[i * nd + d];
    }
    for (int m = 0; m < n_out; ++m) {
        a.out[m] = out_ptrs[m];
        a.out_off[m] = out_off[m];
        for (int d = 0; d < nd; ++d) a.out_str[m][d] = out_str[m * nd + d];
    }
    int64_t total = 1;
    for (int d = 0; d < 3; ++d) {
        a.ext[d] = d < nd ? ext[d] : 1;
        total *= a.ext[d];
    }
    if (total <= 0) return CN_OK;
    int grid = (int)std::min<int64_t>((total + k->tile.block - 1) / k->tile.block, (int64_t)sm_count_ * 8);
    return launch(k, a, grid, k->tile.block, (double)total * (n_in + n_out) * dtype_size(g.dtype));
}

}  // namespace cn
