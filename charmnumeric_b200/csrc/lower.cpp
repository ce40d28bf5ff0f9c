// AST -> GroupIR lowering for one fused DAG group.
//
// Follows the reference's rules for what a group kernel sees (src/jit.cpp):
//   * roots are evaluated in flat list order (:119-120);
//   * an operand whose result_name is an earlier root is an internal value, not an input
//     (:226-243); SET_REGION's operand 0 is the destination, never an input (:245-248);
//   * literal scalars are cast to the element type (:108-116), size-1 arrays are passed as
//     scalars and de-duplicated by name (:254-256), every other leaf is one strided view per
//     (array, operand region) use (:257-259);
//   * the element type is the dtype of the first root that is not float32 (:48-69).
// What is added: classification into the "shifted" class (unit-step views of arrays of one
// common shape: stencils and plain elementwise chains) and the general "strided" class,
// hazard detection for in-place SET_REGION, and REDUCE / SUM roots fused behind the group.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <sstream>

#include "cn_device.cuh"
#include "group_ir.hpp"

namespace cn {

namespace {

struct Use {  // one array-leaf use before de-duplication
    int name;
    int ndims;
    int64_t shape[kMaxDims];
    Region region;
    int root;  // root index that consumes it (-1: reduction operand)
    int red;   // reduction index when root == -1
    int slot;  // 0 = operand a, 1 = operand b
};

bool same_shape(int nd, const int64_t* a, const int64_t* b) {
    for (int d = 0; d < nd; ++d)
        if (a[d] != b[d]) return false;
    return true;
}

bool region_equal(const Region& a, const Region& b) {
    if (a.ndims != b.ndims) return false;
    for (int d = 0; d < a.ndims; ++d)
        if (a.start[d] != b.start[d] || a.stop[d] != b.stop[d] || a.step[d] != b.step[d])
            return false;
    return true;
}

bool region_is_full(const Region& r, int nd, const int64_t* shape) {
    if (r.ndims != nd) return false;
    for (int d = 0; d < nd; ++d)
        if (r.start[d] != 0 || r.stop[d] != shape[d] || r.step[d] != 1) return false;
    return true;
}

int64_t shape_size(int nd, const int64_t* s) {
    int64_t n = 1;
    for (int d = 0; d < nd; ++d) n *= s[d];
    return n;
}

struct Lowering {
    const DagNode& node;
    GroupIR& g;
    std::string* err;
    std::vector<Use> uses;
    std::map<int, int> root_by_name;  // result_name -> root index
    std::map<int, int> out_by_name;   // array name -> outs index
    std::map<int, int> bc_by_name;
    bool force_strided = false;
    bool allow_staged = true;
    bool force_staged = false;  // stage whatever the process-wide level says (staged producers)

    int fail(int code, const std::string& m) {
        if (err) *err = m;
        return code;
    }

    // Resolve one operand of root `ri` (or of reduction `red`) to a ValRef.
    int resolve(const Operand& op, int ri, int red, int slot, ValRef* out, bool* scalar_valued,
                int* nd, int64_t* shape) {
        *scalar_valued = false;
        if (op.is_ref) {
            auto it = root_by_name.find(op.ref_name);
            if (it == root_by_name.end())
                return fail(CN_ERR_BAD_BLOB, "operand refers to an unknown earlier root");
            const RootIR& r = g.roots[it->second];
            out->kind = ValRef::ROOT;
            out->idx = it->second;
            if (r.domain == DOM_SCALAR) {
                *scalar_valued = true;
            } else {
                if (!op.region.is_global) {
                    Region full = Region::full(g.ndims, r.shape);
                    if (!region_equal(op.region, full))
                        return fail(CN_ERR_HAZARD,
                                    "a view of a value computed inside the same group cannot be fused");
                }
                *nd = g.ndims;
                for (int d = 0; d < g.ndims; ++d) shape[d] = r.shape[d];
            }
            return CN_OK;
        }
        const AstNode* leaf = op.leaf.get();
        if (!leaf) return fail(CN_ERR_BAD_BLOB, "operand without a leaf");
        if (leaf->opcode != OP_NOOP && leaf->opcode != OP_CREATE)
            return fail(CN_ERR_BAD_BLOB, "inline operand must be a NOOP/CREATE leaf");
        if (leaf->is_scalar) {
            if ((int)g.scalars.size() >= CN_MAX_SC)
                return fail(CN_ERR_LIMIT, "too many literal scalars in one group");
            out->kind = ValRef::CONST;
            out->idx = (int)g.scalars.size();
            g.scalars.push_back(leaf->scalar);
            *scalar_valued = true;
            return CN_OK;
        }
        int64_t lsize = shape_size(leaf->ndims, leaf->shape);
        if (leaf->is_broadcast || (leaf->ndims >= 1 && lsize == 1 && op.region.is_global)) {
            // a size-1 array written earlier in this group is forwarded from its root
            auto rit = root_by_name.find(leaf->result_name);
            if (rit != root_by_name.end() && g.roots[rit->second].domain == DOM_SCALAR) {
                out->kind = ValRef::ROOT;
                out->idx = rit->second;
                *scalar_valued = true;
                return CN_OK;
            }
            auto it = bc_by_name.find(leaf->result_name);
            if (it == bc_by_name.end()) {
                if ((int)g.bcast_names.size() >= CN_MAX_BC)
                    return fail(CN_ERR_LIMIT, "too many size-1 array operands in one group");
                bc_by_name[leaf->result_name] = (int)g.bcast_names.size();
                g.bcast_names.push_back(leaf->result_name);
                it = bc_by_name.find(leaf->result_name);
            }
            out->kind = ValRef::BCAST;
            out->idx = it->second;
            *scalar_valued = true;
            return CN_OK;
        }
        if (leaf->ndims < 1 || leaf->ndims > kMaxDims)
            return fail(CN_ERR_BAD_BLOB, "array leaf without a rank");
        Region reg = op.region.is_global ? Region::full(leaf->ndims, leaf->shape) : op.region;
        if (reg.ndims != leaf->ndims)
            return fail(CN_ERR_SHAPE_MISMATCH, "operand region rank differs from the array rank");
        for (int d = 0; d < reg.ndims; ++d)
            if (reg.stop[d] > leaf->shape[d] || reg.start[d] > reg.stop[d])
                return fail(CN_ERR_SHAPE_MISMATCH, "operand region lies outside its array");
        *nd = leaf->ndims;
        for (int d = 0; d < leaf->ndims; ++d) shape[d] = reg.extent(d);

        // an array written earlier in this group
        auto oit = out_by_name.find(leaf->result_name);
        if (oit != out_by_name.end()) {
            OutIR& o = g.outs[oit->second];
            if (region_equal(reg, o.region)) {  // exactly what was just written
                if (o.value.kind == ValRef::CONST || o.value.kind == ValRef::BCAST)
                    return fail(CN_ERR_HAZARD, "re-reading a region filled in the same group");
                if (o.value.kind == ValRef::LEAF) {  // a plain copy: read its source again
                    Use u = uses[o.value.idx];
                    u.root = ri;
                    u.red = red;
                    u.slot = slot;
                    out->kind = ValRef::LEAF;
                    out->idx = (int)uses.size();
                    uses.push_back(u);
                    return CN_OK;
                }
                *out = o.value;
                return CN_OK;
            }
            if (region_is_full(reg, o.ndims, o.shape)) {
                out->kind = ValRef::OUTVAL;
                out->idx = oit->second;
                return CN_OK;
            }
            return fail(CN_ERR_HAZARD,
                        "a group reads a shifted view of an array it wrote earlier");
        }
        Use u;
        u.name = leaf->result_name;
        u.ndims = leaf->ndims;
        for (int d = 0; d < kMaxDims; ++d) u.shape[d] = d < leaf->ndims ? leaf->shape[d] : 0;
        u.region = reg;
        u.root = ri;
        u.red = red;
        u.slot = slot;
        out->kind = ValRef::LEAF;
        out->idx = (int)uses.size();  // index into `uses`; remapped after de-duplication
        uses.push_back(u);
        return CN_OK;
    }

    int run(const std::vector<const AstNode*>& fused) {
        g = GroupIR();
        std::vector<const AstNode*> roots;
        for (auto& r : node.roots) roots.push_back(r.get());
        size_t n_own = roots.size();
        for (auto* f : fused) roots.push_back(f);

        g.dtype = DT_F32;
        for (size_t i = 0; i < n_own; ++i)
            if (roots[i]->dtype != DT_F32) {
                g.dtype = roots[i]->dtype;
                break;
            }
        if (!dtype_valid(g.dtype)) return fail(CN_ERR_BAD_DTYPE, "bad dtype code in group");

        for (size_t i = 0; i < roots.size(); ++i) {
            const AstNode* r = roots[i];
            int op = r->opcode;
            if (op == OP_NOOP || op == OP_CREATE) continue;
            if (is_elementwise(op)) {
                int need = is_binary_elementwise(op) ? 2 : 1;
                if ((int)r->operands.size() != need)
                    return fail(CN_ERR_BAD_BLOB, "wrong operand count for an elementwise op");
                if ((op == OP_EXP || op == OP_TANH || op == OP_SQRT) &&
                    (g.dtype == DT_I32 || g.dtype == DT_I64))
                    return fail(CN_ERR_BAD_DTYPE, "exp/tanh/sqrt need a floating-point group");
                RootIR ri;
                ri.opcode = op;
                ri.result_name = r->result_name;
                ri.is_temp = r->is_temp;
                int ridx = (int)g.roots.size();
                bool sv[2] = {true, true};
                int nd[2] = {0, 0};
                int64_t sh[2][kMaxDims] = {{0, 0, 0}, {0, 0, 0}};
                ValRef v[2];
                for (int k = 0; k < need; ++k) {
                    int rc = resolve(r->operands[k], ridx, -1, k, &v[k], &sv[k], &nd[k], sh[k]);
                    if (rc) return rc;
                }
                ri.a = v[0];
                ri.b = v[1];
                bool scalar_valued = sv[0] && (need == 1 || sv[1]);
                if (scalar_valued) {
                    ri.domain = DOM_SCALAR;
                } else {
                    int k0 = sv[0] ? 1 : 0;
                    if (!g.ndims) g.ndims = nd[k0];
                    if (nd[k0] != g.ndims)
                        return fail(CN_ERR_SHAPE_MISMATCH, "operands of different rank in one group");
                    if (need == 2 && !sv[0] && !sv[1] &&
                        (nd[0] != nd[1] || !same_shape(nd[0], sh[0], sh[1])))
                        return fail(CN_ERR_SHAPE_MISMATCH,
                                    "elementwise operands have different shapes");
                    for (int d = 0; d < g.ndims; ++d) ri.shape[d] = sh[k0][d];
                }
                g.roots.push_back(ri);
                root_by_name[r->result_name] = ridx;
                if (!r->is_temp) {
                    if (scalar_valued) {
                        if ((int)g.souts.size() >= CN_MAX_SOUT)
                            return fail(CN_ERR_LIMIT, "too many scalar outputs in one group");
                        ScalarOutIR so;
                        so.name = r->result_name;
                        so.value.kind = ValRef::ROOT;
                        so.value.idx = ridx;
                        g.souts.push_back(so);
                    } else {
                        if ((int)g.outs.size() >= CN_MAX_OUT)
                            return fail(CN_ERR_LIMIT, "too many array outputs in one group");
                        OutIR o;
                        o.name = r->result_name;
                        o.is_set = false;
                        o.ndims = g.ndims;
                        for (int d = 0; d < g.ndims; ++d) o.shape[d] = ri.shape[d];
                        o.region = Region::full(g.ndims, ri.shape);
                        o.value.kind = ValRef::ROOT;
                        o.value.idx = ridx;
                        o.root_index = ridx;
                        out_by_name[o.name] = (int)g.outs.size();
                        g.outs.push_back(o);
                    }
                }
            } else if (op == OP_SET_REGION || op == OP_COPY) {
                if (r->operands.size() != 2 || !r->operands[0].leaf)
                    return fail(CN_ERR_BAD_BLOB, "SET_REGION needs (target, rhs)");
                const AstNode* t = r->operands[0].leaf.get();
                if (t->ndims < 1 || t->ndims > kMaxDims)
                    return fail(CN_ERR_BAD_BLOB, "SET_REGION target without a rank");
                int64_t tsize = shape_size(t->ndims, t->shape);
                ValRef v;
                bool sv = false;
                int nd = 0;
                int64_t sh[kMaxDims] = {0, 0, 0};
                int rc = resolve(r->operands[1], -2, -1, 1, &v, &sv, &nd, sh);
                if (rc) return rc;
                if (tsize == 1 && sv) {
                    if ((int)g.souts.size() >= CN_MAX_SOUT)
                        return fail(CN_ERR_LIMIT, "too many scalar outputs in one group");
                    // model as a scalar root so later operands can forward it
                    RootIR ri;
                    ri.opcode = OP_COPY;
                    ri.a = v;
                    ri.result_name = t->result_name;
                    ri.is_temp = true;
                    ri.domain = DOM_SCALAR;
                    int ridx = (int)g.roots.size();
                    g.roots.push_back(ri);
                    root_by_name[t->result_name] = ridx;
                    ScalarOutIR so;
                    so.name = t->result_name;
                    so.value.kind = ValRef::ROOT;
                    so.value.idx = ridx;
                    so.is_set = true;
                    g.souts.push_back(so);
                    continue;
                }
                if (!g.ndims) g.ndims = t->ndims;
                if (t->ndims != g.ndims)
                    return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION target rank differs from the group");
                Region reg = r->region.is_global ? Region::full(t->ndims, t->shape) : r->region;
                if (reg.ndims != t->ndims)
                    return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION region rank differs from target");
                for (int d = 0; d < reg.ndims; ++d)
                    if (reg.stop[d] > t->shape[d] || reg.start[d] > reg.stop[d])
                        return fail(CN_ERR_SHAPE_MISMATCH, "SET_REGION region outside its target");
                if (!sv) {
                    int64_t rs[kMaxDims];
                    for (int d = 0; d < reg.ndims; ++d) rs[d] = reg.extent(d);
                    if (nd != reg.ndims || !same_shape(nd, sh, rs))
                        return fail(CN_ERR_SHAPE_MISMATCH,
                                    "SET_REGION right-hand side does not match the region shape");
                }
                if ((int)g.outs.size() >= CN_MAX_OUT)
                    return fail(CN_ERR_LIMIT, "too many array outputs in one group");
                if (out_by_name.count(t->result_name))
                    return fail(CN_ERR_HAZARD, "an array is assigned twice in one group");
                OutIR o;
                o.name = t->result_name;
                o.is_set = true;
                o.ndims = t->ndims;
                for (int d = 0; d < t->ndims; ++d) o.shape[d] = t->shape[d];
                o.region = reg;
                o.value = v;
                if (v.kind == ValRef::LEAF) uses[v.idx].root = -2 - (int)g.outs.size();
                out_by_name[o.name] = (int)g.outs.size();
                g.outs.push_back(o);
            } else if (op == OP_REDUCE || op == OP_SUM) {
                int need = op == OP_REDUCE ? 2 : 1;
                if ((int)r->operands.size() != need)
                    return fail(CN_ERR_BAD_BLOB, "wrong operand count for a reduction");
                if ((int)g.reds.size() >= CN_MAX_RED)
                    return fail(CN_ERR_LIMIT, "too many fused reductions in one group");
                RedIR rd;
                rd.result_name = r->result_name;
                int redidx = (int)g.reds.size();
                int nd[2] = {0, 0};
                int64_t sh[2][kMaxDims] = {{0, 0, 0}, {0, 0, 0}};
                ValRef v[2];
                int n_scalar = 0;
                for (int k = 0; k < need; ++k) {
                    bool sv = false;
                    int rc = resolve(r->operands[k], -1, redidx, k, &v[k], &sv, &nd[k], sh[k]);
                    if (rc) return rc;
                    if (sv) ++n_scalar;
                }
                if (n_scalar == need) {
                    // sum / dot of size-1 values: a plain scalar root
                    if ((int)g.souts.size() >= CN_MAX_SOUT)
                        return fail(CN_ERR_LIMIT, "too many scalar outputs in one group");
                    RootIR ri;
                    ri.opcode = need == 2 ? OP_MUL : OP_COPY;
                    ri.a = v[0];
                    ri.b = v[1];
                    ri.result_name = r->result_name;
                    ri.domain = DOM_SCALAR;
                    int ridx = (int)g.roots.size();
                    g.roots.push_back(ri);
                    root_by_name[r->result_name] = ridx;
                    ScalarOutIR so;
                    so.name = r->result_name;
                    so.value.kind = ValRef::ROOT;
                    so.value.idx = ridx;
                    g.souts.push_back(so);
                    continue;
                }
                if (n_scalar) return fail(CN_ERR_UNSUPPORTED, "dot of a scalar with an array");
                if (need == 2 && (nd[0] != nd[1] || !same_shape(nd[0], sh[0], sh[1])))
                    return fail(CN_ERR_SHAPE_MISMATCH, "dot operands have different shapes");
                if (!g.ndims) g.ndims = nd[0];
                rd.a = v[0];
                rd.b = v[1];
                g.reds.push_back(rd);
            } else {
                return fail(CN_ERR_BAD_OPCODE, "opcode cannot be part of a fused group");
            }
        }
        if ((int)uses.size() > 64) return fail(CN_ERR_LIMIT, "too many array operands in one group");
        return classify();
    }

    // ---- classification ---------------------------------------------------------------
    void value_shape(const ValRef& v, int64_t* shape, Region* leafreg) const {
        if (v.kind == ValRef::ROOT) {
            for (int d = 0; d < g.ndims; ++d) shape[d] = g.roots[v.idx].shape[d];
        } else if (v.kind == ValRef::LEAF) {
            for (int d = 0; d < g.ndims; ++d) shape[d] = uses[v.idx].region.extent(d);
            if (leafreg) *leafreg = uses[v.idx].region;
        } else if (v.kind == ValRef::OUTVAL) {
            for (int d = 0; d < g.ndims; ++d) shape[d] = g.outs[v.idx].shape[d];
        }
    }

    int classify() {
        bool any_array = !g.outs.empty() || !g.reds.empty();
        for (auto& r : g.roots)
            if (r.domain != DOM_SCALAR) any_array = true;
        if (!any_array) {
            g.cls = GroupIR::SCALAR_ONLY;
            return finish_scalar_only();
        }
        if (!force_strided && try_shifted()) return CN_OK;
        return build_strided();
    }

    int finish_scalar_only() {
        g.leaves.clear();
        return CN_OK;
    }

    bool try_shifted() {
        const int nd = g.ndims;
        // every array touched must have the same shape, every view unit step
        int64_t as[kMaxDims] = {0, 0, 0};
        bool have = false;
        auto take = [&](int n, const int64_t* s) {
            if (n != nd) return false;
            if (!have) {
                for (int d = 0; d < nd; ++d) as[d] = s[d];
                have = true;
                return true;
            }
            return same_shape(nd, as, s);
        };
        for (auto& u : uses)
            if (!take(u.ndims, u.shape) || !u.region.unit_step()) return false;
        for (auto& o : g.outs)
            if (!take(o.ndims, o.shape) || !o.region.unit_step()) return false;
        if (!have) return false;

        // origins: SET_REGION destinations anchor the roots that feed them
        std::vector<RootIR> roots = g.roots;
        auto set_origin = [&](RootIR& r, const int64_t* o) {
            if (r.origin_set) {
                for (int d = 0; d < nd; ++d)
                    if (r.origin[d] != o[d]) return false;
                return true;
            }
            for (int d = 0; d < nd; ++d) r.origin[d] = o[d];
            r.origin_set = true;
            return true;
        };
        for (auto& o : g.outs)
            if (o.value.kind == ValRef::ROOT && roots[o.value.idx].domain != DOM_SCALAR)
                if (!set_origin(roots[o.value.idx], o.region.start)) return false;
        for (int i = (int)roots.size() - 1; i >= 0; --i) {
            RootIR& r = roots[i];
            if (r.domain == DOM_SCALAR || !r.origin_set) continue;
            for (const ValRef* v : {&r.a, &r.b})
                if (v->kind == ValRef::ROOT && roots[v->idx].domain != DOM_SCALAR)
                    if (!set_origin(roots[v->idx], r.origin)) return false;
        }
        for (size_t i = 0; i < roots.size(); ++i) {
            RootIR& r = roots[i];
            if (r.domain == DOM_SCALAR || r.origin_set) continue;
            bool done = false;
            for (const ValRef* v : {&r.a, &r.b}) {
                if (done) break;
                if (v->kind == ValRef::ROOT && roots[v->idx].domain != DOM_SCALAR &&
                    roots[v->idx].origin_set) {
                    set_origin(r, roots[v->idx].origin);
                    done = true;
                } else if (v->kind == ValRef::LEAF) {
                    set_origin(r, uses[v->idx].region.start);
                    done = true;
                } else if (v->kind == ValRef::OUTVAL) {
                    int64_t z[kMaxDims] = {0, 0, 0};
                    set_origin(r, z);
                    done = true;
                }
            }
            if (!done) return false;
            // push the origin down to operand roots that are still free
            for (const ValRef* v : {&r.a, &r.b})
                if (v->kind == ValRef::ROOT && roots[v->idx].domain != DOM_SCALAR)
                    if (!set_origin(roots[v->idx], r.origin)) return false;
        }

        // boxes in frame (= array) coordinates
        struct Box {
            int64_t lo[kMaxDims], hi[kMaxDims];
        };
        std::vector<Box> boxes;
        auto add_box = [&](const int64_t* lo, const int64_t* shape) {
            Box b;
            for (int d = 0; d < nd; ++d) {
                b.lo[d] = lo[d];
                b.hi[d] = lo[d] + shape[d];
                if (b.lo[d] < 0 || b.hi[d] > as[d]) return -1;
            }
            for (size_t i = 0; i < boxes.size(); ++i) {
                bool eq = true;
                for (int d = 0; d < nd; ++d)
                    if (boxes[i].lo[d] != b.lo[d] || boxes[i].hi[d] != b.hi[d]) eq = false;
                if (eq) return (int)i;
            }
            boxes.push_back(b);
            return (int)boxes.size() - 1;
        };
        std::vector<int> root_box(roots.size(), -1);
        for (size_t i = 0; i < roots.size(); ++i)
            if (roots[i].domain != DOM_SCALAR) {
                root_box[i] = add_box(roots[i].origin, roots[i].shape);
                if (root_box[i] < 0) return false;
            }
        std::vector<int> out_box(g.outs.size(), -1);
        for (size_t i = 0; i < g.outs.size(); ++i) {
            int64_t sh[kMaxDims];
            for (int d = 0; d < nd; ++d) sh[d] = g.outs[i].region.extent(d);
            out_box[i] = add_box(g.outs[i].region.start, sh);
            if (out_box[i] < 0) return false;
        }
        std::vector<int> red_box(g.reds.size(), -1);
        const int64_t zero[kMaxDims] = {0, 0, 0};
        for (size_t i = 0; i < g.reds.size(); ++i) {
            const RedIR& rd = g.reds[i];
            int bx = -1;
            for (const ValRef* v : {&rd.a, &rd.b}) {
                int b = -1;
                if (v->kind == ValRef::NONE) continue;
                if (v->kind == ValRef::ROOT) b = root_box[v->idx];
                else if (v->kind == ValRef::LEAF) {
                    // a reduction operand read straight from an array sits where the array does
                    int64_t sh[kMaxDims];
                    for (int d = 0; d < nd; ++d) sh[d] = uses[v->idx].region.extent(d);
                    b = add_box(uses[v->idx].region.start, sh);
                } else if (v->kind == ValRef::OUTVAL) b = add_box(zero, as);
                if (b < 0) return false;
                if (bx >= 0 && bx != b) return false;
                bx = b;
            }
            red_box[i] = bx;
        }

        // hazards: a leaf reads an output array at an index other than the one written
        bool copy_through = false;
        for (size_t i = 0; i < g.outs.size(); ++i) {
            OutIR& o = g.outs[i];
            for (auto& u : uses) {
                if (u.name != o.name) continue;
                const int64_t* org = nullptr;
                if (u.root >= 0) org = roots[u.root].origin;
                else if (u.root <= -2 && (-2 - u.root) < (int)g.outs.size())
                    org = g.outs[-2 - u.root].region.start;
                else org = u.region.start;  // reduction operand: delta 0 by construction
                for (int d = 0; d < nd; ++d)
                    if (u.region.start[d] != org[d]) o.hazard = true;
            }
            if (o.hazard) copy_through = true;
        }
        if (copy_through) {
            if (add_box(zero, as) < 0) return false;
        }
        if (boxes.size() > 2) return false;
        int big = 0, small = 0;
        if (boxes.size() == 2) {
            auto contains = [&](const Box& a, const Box& b) {
                for (int d = 0; d < nd; ++d)
                    if (b.lo[d] < a.lo[d] || b.hi[d] > a.hi[d]) return false;
                return true;
            };
            if (contains(boxes[0], boxes[1])) big = 0, small = 1;
            else if (contains(boxes[1], boxes[0])) big = 1, small = 0;
            else return false;
        }
        if (copy_through) {
            // the sweep must cover the whole array; a hazard output is either a region output
            // (the rest of the array is copied through) or an assignment of the whole array
            // (every element is written anyway: nothing to copy through)
            for (int d = 0; d < nd; ++d)
                if (boxes[big].lo[d] != 0 || boxes[big].hi[d] != as[d]) return false;
            for (size_t i = 0; i < g.outs.size(); ++i)
                if (g.outs[i].hazard && out_box[i] != small && out_box[i] != big) return false;
        }

        // commit
        g.cls = GroupIR::SHIFTED;
        g.roots = roots;
        g.two_domains = boxes.size() == 2;
        g.copy_through = copy_through;
        for (int d = 0; d < nd; ++d) {
            g.array_shape[d] = as[d];
            g.box_lo[d] = boxes[big].lo[d];
            g.box_hi[d] = boxes[big].hi[d];
            g.reg_lo[d] = boxes[small].lo[d];
            g.reg_hi[d] = boxes[small].hi[d];
        }
        auto dom_of = [&](int b) { return (g.two_domains && b == small) ? DOM_REGION : DOM_BOX; };
        for (size_t i = 0; i < g.roots.size(); ++i)
            if (g.roots[i].domain != DOM_SCALAR) g.roots[i].domain = dom_of(root_box[i]);
        for (size_t i = 0; i < g.outs.size(); ++i) g.outs[i].domain = dom_of(out_box[i]);
        for (size_t i = 0; i < g.reds.size(); ++i) g.reds[i].domain = dom_of(red_box[i]);

        // leaf load sites, de-duplicated by (array, delta, domain)
        std::vector<int> remap(uses.size(), -1);
        g.max_halo = 0;
        bool all_zero = true;
        for (size_t ui = 0; ui < uses.size(); ++ui) {
            const Use& u = uses[ui];
            LeafIR l;
            l.name = u.name;
            l.ndims = u.ndims;
            for (int d = 0; d < nd; ++d) l.shape[d] = u.shape[d];
            l.region = u.region;
            const int64_t* org;
            if (u.root >= 0) {
                org = g.roots[u.root].origin;
                l.domain = g.roots[u.root].domain;
            } else if (u.root <= -2 && (-2 - u.root) < (int)g.outs.size()) {
                org = g.outs[-2 - u.root].region.start;
                l.domain = g.outs[-2 - u.root].domain;
            } else {
                org = u.region.start;
                l.domain = g.reds[u.red].domain;
            }
            for (int d = 0; d < nd; ++d) {
                l.delta[d] = u.region.start[d] - org[d];
                if (l.delta[d]) all_zero = false;
            }
            int64_t h = l.delta[0] < 0 ? -l.delta[0] : l.delta[0];
            if (h > g.max_halo) g.max_halo = (int)h;
            int found = -1;
            for (size_t k = 0; k < g.leaves.size(); ++k) {
                const LeafIR& m = g.leaves[k];
                if (m.name == l.name && m.domain == l.domain && m.delta[0] == l.delta[0] &&
                    m.delta[1] == l.delta[1] && m.delta[2] == l.delta[2])
                    found = (int)k;
            }
            if (found < 0) {
                if ((int)g.leaves.size() >= 32) return false;
                found = (int)g.leaves.size();
                g.leaves.push_back(l);
            }
            remap[ui] = found;
        }
        auto fix = [&](ValRef& v) {
            if (v.kind == ValRef::LEAF) v.idx = remap[v.idx];
        };
        for (auto& r : g.roots) {
            fix(r.a);
            fix(r.b);
        }
        for (auto& o : g.outs) fix(o.value);
        for (auto& rd : g.reds) {
            fix(rd.a);
            fix(rd.b);
        }
        // old contents: copy-through of hazard outputs, or forwarding outside the region
        for (size_t i = 0; i < g.outs.size(); ++i) {
            OutIR& o = g.outs[i];
            if (o.hazard && g.two_domains && o.domain == DOM_REGION) o.needs_old = true;
        }
        auto mark_old = [&](const ValRef& v) {
            if (v.kind == ValRef::OUTVAL && g.outs[v.idx].domain == DOM_REGION)
                g.outs[v.idx].needs_old = true;
        };
        for (auto& r : g.roots) {
            mark_old(r.a);
            mark_old(r.b);
        }
        for (auto& rd : g.reds) {
            mark_old(rd.a);
            mark_old(rd.b);
        }
        // whole-array, zero-offset groups walk the slab as one 1-D range
        bool whole = true;
        for (int d = 0; d < nd; ++d)
            if (g.box_lo[d] != 0 || g.box_hi[d] != as[d]) whole = false;
        g.flat = all_zero && whole && !g.two_domains && !copy_through;
        int esz = dtype_size(g.dtype);
        g.vec = 1;
        if (esz == 8 && (g.flat || nd == 1 || as[nd - 1] % 2 == 0)) g.vec = 2;
        // staged variant: exactly one array is read at shifted positions, within a small halo
        g.staged = false;
        const int level = staged_level();
        if (allow_staged && (force_staged || level == 2 || (level == 1 && nd == 3)) && !g.flat && g.vec == 2 &&
            g.dtype == DT_F64 && (nd == 2 || nd == 3)) {
            int name = -1;
            bool ok = true;
            int hx = 0, hy = 0, hz = 0;
            for (auto& l : g.leaves) {
                bool shifted = l.delta[0] || l.delta[1] || l.delta[2];
                if (!shifted) continue;
                if (name >= 0 && name != l.name) ok = false;
                name = l.name;
            }
            if (name >= 0 && ok) {
                for (auto& l : g.leaves) {
                    if (l.name != name) continue;
                    auto mag = [](int64_t v) { return (int)(v < 0 ? -v : v); };
                    hx = std::max(hx, mag(l.delta[nd - 1]));
                    hy = std::max(hy, mag(l.delta[nd - 2]));
                    if (nd == 3) hz = std::max(hz, mag(l.delta[0]));
                }
                // an in-place output on the stencil array would race with other tiles' fetches
                for (auto& o : g.outs)
                    if (o.name == name && !(copy_through && o.hazard)) ok = false;
                if (ok && hx <= 2 && hy <= 2 && hz <= 1) {
                    g.staged = true;
                    g.stage_array = name;
                    g.hy = hy;
                    g.hz = hz;
                }
            }
        }
        return true;
    }

    int build_strided() {
        const int nd = g.ndims;
        g.cls = GroupIR::STRIDED;
        // one iteration shape for every array-valued root, output and reduction
        int64_t S[kMaxDims] = {0, 0, 0};
        bool have = false;
        auto take = [&](const int64_t* s) {
            if (!have) {
                for (int d = 0; d < nd; ++d) S[d] = s[d];
                have = true;
                return true;
            }
            return same_shape(nd, S, s);
        };
        for (auto& r : g.roots)
            if (r.domain != DOM_SCALAR) {
                if (!take(r.shape))
                    return fail(CN_ERR_UNSUPPORTED,
                                "roots of different shapes in one strided group");
                r.domain = DOM_BOX;
            }
        for (auto& o : g.outs) {
            int64_t sh[kMaxDims];
            for (int d = 0; d < nd; ++d) sh[d] = o.region.extent(d);
            if (!take(sh))
                return fail(CN_ERR_UNSUPPORTED, "outputs of different shapes in one strided group");
            o.domain = DOM_BOX;
        }
        for (auto& rd : g.reds) {
            int64_t sh[kMaxDims] = {0, 0, 0};
            value_shape(rd.a, sh, nullptr);
            if (!take(sh))
                return fail(CN_ERR_UNSUPPORTED, "reduction shape differs from the group shape");
            rd.domain = DOM_BOX;
        }
        for (int d = 0; d < nd; ++d) g.extent[d] = S[d];
        // leaves de-duplicated by (array, region)
        std::vector<int> remap(uses.size(), -1);
        for (size_t ui = 0; ui < uses.size(); ++ui) {
            const Use& u = uses[ui];
            int found = -1;
            for (size_t k = 0; k < g.leaves.size(); ++k)
                if (g.leaves[k].name == u.name && region_equal(g.leaves[k].region, u.region))
                    found = (int)k;
            if (found < 0) {
                if ((int)g.leaves.size() >= CN_MAX_IN)
                    return fail(CN_ERR_LIMIT, "too many array operands in one group");
                LeafIR l;
                l.name = u.name;
                l.ndims = u.ndims;
                for (int d = 0; d < u.ndims; ++d) l.shape[d] = u.shape[d];
                l.region = u.region;
                l.domain = DOM_BOX;
                found = (int)g.leaves.size();
                g.leaves.push_back(l);
            }
            remap[ui] = found;
        }
        auto fix = [&](ValRef& v) {
            if (v.kind == ValRef::LEAF) v.idx = remap[v.idx];
        };
        for (auto& r : g.roots) {
            fix(r.a);
            fix(r.b);
        }
        for (auto& o : g.outs) fix(o.value);
        for (auto& rd : g.reds) {
            fix(rd.a);
            fix(rd.b);
        }
        for (auto& o : g.outs) {
            for (auto& l : g.leaves)
                if (l.name == o.name && !region_equal(l.region, o.region)) o.hazard = true;
            for (auto& r : g.roots)
                for (const ValRef* v : {&r.a, &r.b})
                    if (v->kind == ValRef::OUTVAL)
                        return fail(CN_ERR_UNSUPPORTED,
                                    "whole-array re-read of an assigned array in a strided group");
        }
        for (auto& rd : g.reds)
            for (const ValRef* v : {&rd.a, &rd.b})
                if (v->kind == ValRef::OUTVAL)
                    return fail(CN_ERR_UNSUPPORTED,
                                "whole-array re-read of an assigned array in a strided group");
        g.vec = 1;
        return CN_OK;
    }
};

void put(std::ostringstream& s, const ValRef& v) { s << (int)v.kind << ':' << v.idx << ','; }

}  // namespace

namespace {
int g_staged = -1;
}

void set_staged_level(int level) { g_staged = level < 0 ? 0 : (level > 2 ? 2 : level); }

// 0: never, 1: 3-D stencils only (default: measured faster there, slower in 2-D), 2: always
int staged_level() {
    if (g_staged < 0) {
        const char* e = getenv("CN_STAGED");
        g_staged = e ? atoi(e) : 1;
        if (g_staged < 0 || g_staged > 2) g_staged = 1;
    }
    return g_staged;
}

int lower_group(const DagNode& node, const std::vector<const AstNode*>& fused, GroupIR* out,
                std::string* err, bool force_strided) {
    Lowering l{node, *out, err, {}, {}, {}, {}, force_strided, true};
    int rc = l.run(fused);
    if (rc) return rc;
    if ((int)out->leaves.size() > (out->cls == GroupIR::SHIFTED ? 32 : CN_MAX_IN)) {
        if (err) *err = "too many array operands in one group";
        return CN_ERR_LIMIT;
    }
    return CN_OK;
}

int lower_staged_producer(const DagNode& consumer, const DagNode& producer, int pseudo_name, int target_name,
                          const std::vector<const AstNode*>& fused, GroupIR* out, std::string* err) {
    auto unfit = [&](const char* why) {
        if (err) *err = why;
        return (int)CN_ERR_UNSUPPORTED;
    };
    GroupIR gp;
    {
        Lowering lp{producer, gp, err, {}, {}, {}, {}, false, false};
        int rc = lp.run({});
        if (rc) return rc;
    }
    if (gp.cls != GroupIR::SHIFTED || !gp.flat || gp.outs.size() != 1 || !gp.outs[0].is_set ||
        gp.outs[0].name != target_name || !gp.reds.empty() || !gp.souts.empty() || gp.dtype != DT_F64)
        return unfit("producer is not a flat float64 group with one output");
    if (gp.outs[0].value.kind != ValRef::ROOT) return unfit("producer output is not a computed value");
    {
        Lowering lc{consumer, *out, err, {}, {}, {}, {}, false, true};
        lc.force_staged = true;
        int rc = lc.run(fused);
        if (rc) return rc;
    }
    GroupIR& g = *out;
    if (g.cls != GroupIR::SHIFTED || g.flat || !g.staged || g.stage_array != pseudo_name || g.ndims != 2 ||
        g.dtype != DT_F64 || g.vec != 2)
    {
        if (err)
            *err = "consumer does not lower to a staged 2-D float64 stencil over the stand-in (class " +
                   std::to_string((int)g.cls) + ", flat " + std::to_string(g.flat) + ", staged " + std::to_string(g.staged) +
                   ", stage array " + std::to_string(g.stage_array) + ", rank " + std::to_string(g.ndims) + ", vec " +
                   std::to_string(g.vec) + ")";
        return (int)CN_ERR_UNSUPPORTED;
    }
    if (gp.ndims != g.ndims) return unfit("producer and consumer ranks differ");
    for (int d = 0; d < g.ndims; ++d)
        if (gp.array_shape[d] != g.array_shape[d]) return unfit("producer and consumer shapes differ");
    for (int d = 0; d < g.ndims; ++d)
        if (g.box_lo[d] != 0 || g.box_hi[d] != g.array_shape[d]) return unfit("consumer does not sweep the whole array");
    if (g.scalars.size() + gp.scalars.size() > CN_MAX_SC || g.bcast_names.size() + gp.bcast_names.size() > CN_MAX_BC ||
        g.input_arrays().size() + gp.input_arrays().size() > CN_MAX_IN)
        return unfit("too many operands for one launch");
    // Other blocks evaluate the producer on their tiles' halo rings while this block stores:
    // an output that the producer reads must go to the shadow buffer.
    const std::vector<int> pin = gp.input_arrays();
    for (auto& o : g.outs)
        if (std::find(pin.begin(), pin.end(), o.name) != pin.end()) {
            const bool whole = region_is_full(o.region, o.ndims, o.shape);
            if (!whole && o.domain != DOM_REGION) return unfit("an output the producer reads is neither whole nor the region");
            o.hazard = true;
            g.copy_through = true;
            if (g.two_domains && o.domain == DOM_REGION) o.needs_old = true;
        }
    g.producer.clear();
    g.producer.push_back(gp);
    g.producer_target = target_name;
    if ((int)g.leaves.size() > 32) return unfit("too many array operands in one group");
    return CN_OK;
}

std::vector<int> GroupIR::input_arrays() const {
    std::vector<int> names;
    for (auto& l : leaves) {
        if (cls == SHIFTED && std::find(names.begin(), names.end(), l.name) != names.end())
            continue;
        names.push_back(l.name);
    }
    return names;
}

std::string GroupIR::entry_name() const {
    const std::string k = key();
    uint32_t h = 2166136261u;  // FNV-1a
    for (unsigned char c : k) {
        h ^= c;
        h *= 16777619u;
    }
    const char* c = cls == SHIFTED ? (flat ? "flat" : "shifted") : (cls == STRIDED ? "strided" : "scalar");
    char buf[128];
    snprintf(buf, sizeof(buf), "cn_group_%s%dd_i%zuo%zur%zu%s_%08x", c, flat ? 1 : ndims,
             input_arrays().size(), outs.size(), reds.size(), copy_through ? "_ct" : "", h);
    return buf;
}

std::string GroupIR::key() const {
    std::ostringstream s;
    s << "c" << (int)cls << "t" << dtype << "n" << ndims << "v" << vec << "f" << flat << "d"
      << two_domains << "x" << copy_through << "g" << staged << hy << hz << "|L";
    for (auto& l : leaves) {
        s << l.domain << ':';
        if (cls == SHIFTED) {
            s << l.delta[0] << ',' << l.delta[1] << ',' << l.delta[2];
            // which earlier leaf reads the same array (loads of one row are grouped)
            int same = -1;
            for (size_t k = 0; k < leaves.size() && &leaves[k] != &l; ++k)
                if (leaves[k].name == l.name) {
                    same = (int)k;
                    break;
                }
            s << '@' << same;
            int alias = -1;
            for (size_t k = 0; k < outs.size(); ++k)
                if (outs[k].name == l.name) alias = (int)k;
            s << 'a' << alias;
        }
        s << ';';
    }
    s << "|S" << scalars.size() << "|B" << bcast_names.size() << "|R";
    for (auto& r : roots) {
        s << r.opcode << '/' << r.domain << '/';
        put(s, r.a);
        put(s, r.b);
        s << ';';
    }
    s << "|O";
    for (auto& o : outs) {
        s << o.is_set << o.hazard << o.needs_old << '/' << o.domain << '/';
        put(s, o.value);
        s << ';';
    }
    s << "|s";
    for (auto& o : souts) {
        put(s, o.value);
        s << ';';
    }
    s << "|r";
    for (auto& r : reds) {
        s << r.domain << '/';
        put(s, r.a);
        put(s, r.b);
        s << ';';
    }
    if (!producer.empty()) s << "|P{" << producer[0].key() << "}";
    if (!tail.empty()) s << "|T{" << tail[0].key() << "}";
    return s.str();
}

}  // namespace cn
