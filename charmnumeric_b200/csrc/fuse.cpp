// Producer inlining across two consecutive fusible DAG nodes.
//
// Pattern: node A assigns a whole array P from an elementwise expression of whole arrays
// (`p[...] = r + beta * p`), node B right behind it reads P through shifted views (a stencil:
// `Ap[1:-1,1:-1] = 4 p[1:-1,1:-1] - p[:-2,1:-1] - ...`).  Run one after the other, A writes P
// and B reads it back: 16 bytes per point of HBM traffic that carry no information B could
// not recompute from A's inputs.  The merged node evaluates A's expression once per view of
// P that B reads (same operations in the same order, so the values are bit-identical to what
// A would have stored), feeds them to B's roots, and still assigns P itself.  The reference
// has no counterpart: its fusion stops at DAG-node boundaries (src/dag_group_compile.cpp:6-41
// compiles one kernel per node).
#include <climits>
#include <map>
#include <set>

#include "group_ir.hpp"

namespace cn {

namespace {

int64_t elems(const AstNode& n) {
    int64_t v = 1;
    for (int d = 0; d < n.ndims; ++d) v *= n.shape[d];
    return n.ndims >= 1 ? v : 1;
}

bool is_full(const Region& r, const AstNode& leaf) {
    if (r.is_global) return true;
    if (r.ndims != leaf.ndims) return false;
    for (int d = 0; d < r.ndims; ++d)
        if (r.start[d] != 0 || r.stop[d] != leaf.shape[d] || r.step[d] != 1) return false;
    return true;
}

bool same_region(const Region& a, const Region& b) {
    if (a.ndims != b.ndims) return false;
    for (int d = 0; d < a.ndims; ++d)
        if (a.start[d] != b.start[d] || a.stop[d] != b.stop[d] || a.step[d] != b.step[d]) return false;
    return true;
}

std::unique_ptr<AstNode> clone(const AstNode& n);

Operand clone_operand(const Operand& o) {
    Operand c;
    c.is_ref = o.is_ref;
    c.ref_name = o.ref_name;
    c.region = o.region;
    if (o.leaf) c.leaf = clone(*o.leaf);
    return c;
}

std::unique_ptr<AstNode> clone(const AstNode& n) {
    std::unique_ptr<AstNode> c(new AstNode());
    c->result_name = n.result_name;
    c->opcode = n.opcode;
    c->is_temp = n.is_temp;
    c->is_scalar = n.is_scalar;
    c->is_broadcast = n.is_broadcast;
    c->dtype = n.dtype;
    c->ndims = n.ndims;
    c->scalar = n.scalar;
    for (int d = 0; d < kMaxDims; ++d) c->shape[d] = n.shape[d];
    c->region = n.region;
    for (auto& o : n.operands) c->operands.push_back(clone_operand(o));
    return c;
}

bool array_leaf(const Operand& o) {
    return !o.is_ref && o.leaf && !o.leaf->is_scalar && !o.leaf->is_broadcast && elems(*o.leaf) > 1;
}

}  // namespace

namespace {

struct Pattern {
    const AstNode* set = nullptr;       // the whole-array assignment of the producer
    std::set<int> array_temps;          // array-valued temporaries of the producer
    std::set<int> scalar_roots;         // its size-1 values
    std::set<int> a_inputs;             // arrays it reads
    std::set<int> scalar_sets;          // size-1 arrays it assigns
    std::set<const AstNode*> scalar_set_roots;
    std::vector<Region> views;          // distinct views through which the consumer reads the target
    int pname = -1;

    int view_index(const Region& r) const {
        for (size_t i = 0; i < views.size(); ++i)
            if (same_region(views[i], r)) return (int)i;
        return -1;
    }
};

bool analyse(const DagNode& a, const DagNode& b, Pattern* pat) {
    if (!a.fusible || !b.fusible || a.roots.empty() || b.roots.empty()) return false;
    const AstNode*& set = pat->set;
    std::set<int>&array_temps = pat->array_temps, &scalar_roots = pat->scalar_roots, &a_inputs = pat->a_inputs,
    &scalar_sets = pat->scalar_sets;
    std::set<const AstNode*>& scalar_set_roots = pat->scalar_set_roots;
    std::vector<Region>& views = pat->views;

    // ---- the producer: elementwise temporaries over whole arrays, one whole-array assignment
    for (auto& rp : a.roots) {
        const AstNode& r = *rp;
        if (r.opcode == OP_NOOP) continue;
        if (r.opcode == OP_SET_REGION) {
            if (set || r.operands.size() != 2 || !r.operands[0].leaf) return false;
            if (elems(*r.operands[0].leaf) == 1) {
                // a size-1 assignment (`beta[...] = rtr_new / rtr`): stays as it is, up front
                const Operand& v = r.operands[1];
                if (v.is_ref ? !scalar_roots.count(v.ref_name) : (!v.leaf || array_leaf(v))) return false;
                scalar_sets.insert(r.operands[0].leaf->result_name);
                scalar_set_roots.insert(&r);
                continue;
            }
            set = &r;
            continue;
        }
        if (!is_elementwise(r.opcode)) return false;
        if (set) return false;  // the assignment closes the producer
        const bool scalar_valued = elems(r) == 1;
        if (!scalar_valued && !r.is_temp) return false;
        for (auto& o : r.operands) {
            if (o.is_ref) {
                if (!array_temps.count(o.ref_name) && !scalar_roots.count(o.ref_name)) return false;
                if (scalar_valued && array_temps.count(o.ref_name)) return false;
            } else if (!o.leaf) {
                return false;
            } else if (array_leaf(o)) {
                if (scalar_valued || !is_full(o.region, *o.leaf)) return false;
                a_inputs.insert(o.leaf->result_name);
            }
        }
        (scalar_valued ? scalar_roots : array_temps).insert(r.result_name);
    }
    if (!set) return false;
    const AstNode& target = *set->operands[0].leaf;
    if (elems(target) <= 1 || !is_full(set->region, target)) return false;
    const Operand& rhs = set->operands[1];
    if (!rhs.is_ref || !array_temps.count(rhs.ref_name)) return false;
    const int pname = target.result_name;
    pat->pname = pname;
    // every array the producer reads has the target's shape (the views of B apply to all of them)
    for (auto& rp : a.roots)
        for (auto& o : rp->operands)
            if (array_leaf(o)) {
                if (o.leaf->ndims != target.ndims) return false;
                for (int d = 0; d < target.ndims; ++d)
                    if (o.leaf->shape[d] != target.shape[d]) return false;
            }

    // ---- the consumer: reads the target through unit-step views, writes neither the target
    // nor anything the producer reads
    auto view_index = [&](const Region& r) { return pat->view_index(r); };
    for (auto& rp : b.roots) {
        const AstNode& r = *rp;
        if (r.opcode == OP_NOOP) continue;
        if (r.opcode == OP_SET_REGION) {
            if (r.operands.size() != 2 || !r.operands[0].leaf) return false;
            const int t = r.operands[0].leaf->result_name;
            if (t == pname || a_inputs.count(t)) return false;
        } else if (!is_elementwise(r.opcode)) {
            return false;
        }
        if (array_temps.count(r.result_name) || scalar_roots.count(r.result_name)) return false;
        for (size_t k = 0; k < r.operands.size(); ++k) {
            const Operand& o = r.operands[k];
            if (r.opcode == OP_SET_REGION && k == 0) continue;
            if (o.is_ref || !o.leaf) continue;
            if (scalar_roots.count(o.leaf->result_name) || scalar_sets.count(o.leaf->result_name))
                return false;  // a size-1 result of A read back
            if (!array_leaf(o) || o.leaf->result_name != pname) continue;
            Region reg = o.region.is_global ? Region::full(o.leaf->ndims, o.leaf->shape) : o.region;
            if (!reg.unit_step() || reg.ndims != target.ndims) return false;
            if (view_index(reg) < 0) views.push_back(reg);
        }
    }
    if (views.empty() || views.size() > 8) return false;
    // recomputing pays while the producer is cheap next to the pass over the target it saves
    if (array_temps.size() * views.size() > 48 || a_inputs.size() > 4) return false;
    return true;
}

}  // namespace

// Build in `out` the node that does the work of `a` followed by `b`, or return false when the
// pair does not fit the pattern (the caller then runs the two nodes as they are).
bool inline_producer(const DagNode& a, const DagNode& b, DagNode* out) {
    Pattern pat;
    if (!analyse(a, b, &pat)) return false;
    const AstNode* set = pat.set;
    const std::set<int>&array_temps = pat.array_temps, &scalar_roots = pat.scalar_roots;
    const std::set<const AstNode*>& scalar_set_roots = pat.scalar_set_roots;
    const std::vector<Region>& views = pat.views;
    const AstNode& target = *set->operands[0].leaf;
    const Operand& rhs = set->operands[1];
    const int pname = pat.pname;
    auto view_index = [&](const Region& r) { return pat.view_index(r); };

    // ---- the merged node
    out->id = b.id;
    out->identifier = b.identifier;
    out->fusible = true;
    out->deps = a.deps;
    out->roots.clear();
    // size-1 work of the producer, once
    for (auto& rp : a.roots)
        if ((scalar_roots.count(rp->result_name) && rp->opcode != OP_SET_REGION) || scalar_set_roots.count(rp.get()))
            out->roots.push_back(clone(*rp));
    // the producer's expression at every view the consumer reads
    auto temp_name = [&](int name, size_t view) {
        int k = 0;
        for (int t : array_temps) {
            if (t == name) break;
            ++k;
        }
        return INT_MIN / 2 + (int)(view * array_temps.size()) + k;
    };
    for (size_t v = 0; v < views.size(); ++v) {
        for (auto& rp : a.roots) {
            if (!array_temps.count(rp->result_name) || rp->opcode == OP_SET_REGION) continue;
            std::unique_ptr<AstNode> c = clone(*rp);
            c->result_name = temp_name(rp->result_name, v);
            c->is_temp = true;
            for (int d = 0; d < target.ndims; ++d) c->shape[d] = views[v].extent(d);
            for (auto& o : c->operands) {
                if (o.is_ref) {
                    if (array_temps.count(o.ref_name)) o.ref_name = temp_name(o.ref_name, v);
                } else if (array_leaf(o)) {
                    o.region = views[v];
                }
            }
            out->roots.push_back(std::move(c));
        }
    }
    // the consumer, fed from those values
    for (auto& rp : b.roots) {
        std::unique_ptr<AstNode> c = clone(*rp);
        for (size_t k = 0; k < c->operands.size(); ++k) {
            Operand& o = c->operands[k];
            if (c->opcode == OP_SET_REGION && k == 0) continue;
            if (!array_leaf(o) || o.leaf->result_name != pname) continue;
            Region reg = o.region.is_global ? Region::full(o.leaf->ndims, o.leaf->shape) : o.region;
            const int v = view_index(reg);
            o.is_ref = true;
            o.ref_name = temp_name(rhs.ref_name, (size_t)v);
            o.leaf.reset();
            o.region = Region();
        }
        out->roots.push_back(std::move(c));
    }
    // the producer itself, last: every read of the target above sees its old contents, every
    // whole-array read of it after this point (a fused dot product) sees the new ones
    for (auto& rp : a.roots)
        if (array_temps.count(rp->result_name) || rp.get() == set) out->roots.push_back(clone(*rp));
    return true;
}

// The same pair as two nodes for the staged form: `consumer` is `b` with its reads of the
// target turned into reads of a stand-in array `pseudo_name` (which never exists: the kernel
// computes its tiles in shared memory), followed by the assignment of the target from that
// stand-in; `producer` is `a` as it is.  Only producers without size-1 results qualify.
bool stage_producer(const DagNode& a, const DagNode& b, DagNode* consumer, DagNode* producer, int* pseudo_name,
                    int* target_name) {
    Pattern pat;
    if (!analyse(a, b, &pat)) return false;
    if (!pat.scalar_sets.empty()) return false;
    for (auto& rp : a.roots)
        if (pat.scalar_roots.count(rp->result_name) && !rp->is_temp) return false;
    const AstNode& target = *pat.set->operands[0].leaf;
    const int pseudo = INT_MAX - 7;  // no real array carries this name
    producer->id = a.id;
    producer->identifier = a.identifier;
    producer->fusible = true;
    producer->roots.clear();
    for (auto& rp : a.roots) producer->roots.push_back(clone(*rp));
    consumer->id = b.id;
    consumer->identifier = b.identifier;
    consumer->fusible = true;
    consumer->deps = a.deps;
    consumer->roots.clear();
    for (auto& rp : b.roots) {
        std::unique_ptr<AstNode> c = clone(*rp);
        for (size_t k = 0; k < c->operands.size(); ++k) {
            Operand& o = c->operands[k];
            if (c->opcode == OP_SET_REGION && k == 0) continue;
            if (array_leaf(o) && o.leaf->result_name == pat.pname) o.leaf->result_name = pseudo;
        }
        consumer->roots.push_back(std::move(c));
    }
    // target[...] = stand-in[...]
    std::unique_ptr<AstNode> s = clone(*pat.set);
    Operand& v = s->operands[1];
    v.is_ref = false;
    v.ref_name = -1;
    v.leaf = clone(target);
    v.leaf->result_name = pseudo;
    v.leaf->opcode = OP_NOOP;
    v.region = Region();
    consumer->roots.push_back(std::move(s));
    *pseudo_name = pseudo;
    *target_name = pat.pname;
    return true;
}

}  // namespace cn
