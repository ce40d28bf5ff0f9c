// Tile sizes and alignment offsets of newly created arrays, chosen so that their tiles line
// up with the tiles of the arrays they are computed from or stored into.
//
// Restates the observable rules of the reference's decomposition solver
// (src/decomposition_solver.hpp:95-1716; pinned by tests/test_compute_decompositions.cpp:128-396)
// in a compact form:
//   * tiles (:100-122): an unset tile is the minimum tile of its rank; a tile that is not
//     final is rounded up to a power of two, kept at or above the minimum, and doubled while
//     the array would have more than odf x PEs tiles;
//   * tile propagation (:145-287): an array computed from a view of S proposes S's tile
//     divided by the view's stride factor (the gcd of its steps > 1); a proposal is taken
//     when it is smaller than the current tile;
//   * offsets (:907-1420): every view the array is computed from proposes the absolute
//     offset (S.offset + view start) / step, every SET_REGION that stores the array proposes
//     target.offset + region start, every array computed from it proposes the offset that
//     would line the two up; per dimension the candidate with the least total distance to
//     all proposals wins (the smaller one on a tie).
// The slab executor of this backend does not need per-array offsets (one slab per rank, rows
// that do not line up are fetched); the solver is provided for hosts that keep the
// reference's tile grids.
#include <algorithm>
#include <cstring>
#include <map>
#include <set>
#include <vector>

#include "../../include/cnb200.h"
#include "cn_types.hpp"

namespace cn {

namespace {

int64_t next_pow2(int64_t v) {
    int64_t p = 1;
    while (p < v) p <<= 1;
    return p;
}

int64_t gcd64(int64_t a, int64_t b) {
    while (b) {
        int64_t t = a % b;
        a = b;
        b = t;
    }
    return a < 0 ? -a : a;
}

// One alignment relation: index i of `out` sits on index start + i * step of `src`.
struct Edge {
    int out, src;
    int ndims;
    int64_t start[3], step[3];
};

struct Solver {
    std::map<int, cn_array_meta*> meta;
    std::vector<Edge> edges;
    int64_t min_tile[4] = {1, 262144, 512, 64};

    cn_array_meta* find(int name) {
        auto it = meta.find(name);
        return it == meta.end() ? nullptr : it->second;
    }

    // leaves of the expression behind `op`, looked up through roots that are no arrays of their own
    void collect(const Operand& op, const std::map<int, const AstNode*>& defs, int out, int depth) {
        if (depth > 16) return;
        if (op.is_ref) {
            if (find(op.ref_name)) {
                add_edge(out, op.ref_name, Region());
                return;
            }
            auto it = defs.find(op.ref_name);
            if (it != defs.end())
                for (auto& o : it->second->operands) collect(o, defs, out, depth + 1);
            return;
        }
        if (!op.leaf || op.leaf->is_scalar || op.leaf->is_broadcast) return;
        if (find(op.leaf->result_name)) {
            add_edge(out, op.leaf->result_name, op.region);
            return;
        }
        auto it = defs.find(op.leaf->result_name);  // a temporary named like a leaf
        if (it != defs.end())
            for (auto& o : it->second->operands) collect(o, defs, out, depth + 1);
    }

    void add_edge(int out, int src, const Region& r) {
        cn_array_meta *mo = find(out), *ms = find(src);
        if (!mo || !ms || mo->ndims != ms->ndims || out == src) return;
        Edge e;
        e.out = out;
        e.src = src;
        e.ndims = mo->ndims;
        for (int d = 0; d < 3; ++d) {
            e.start[d] = (!r.is_global && d < r.ndims) ? r.start[d] : 0;
            e.step[d] = (!r.is_global && d < r.ndims && r.step[d] > 1) ? r.step[d] : 1;
        }
        edges.push_back(e);
    }
};

}  // namespace

int compute_decompositions(cn_array_meta* arrays, int n_arrays, const Dag* dag, int odf, int num_pes,
                           const int64_t* min_tile) {
    Solver s;
    if (min_tile)
        for (int d = 1; d <= 3; ++d)
            if (min_tile[d - 1] > 0) s.min_tile[d] = min_tile[d - 1];
    for (int i = 0; i < n_arrays; ++i) {
        if (arrays[i].ndims < 1 || arrays[i].ndims > 3) return CN_ERR_INVALID_ARGUMENT;
        s.meta[arrays[i].name] = &arrays[i];
    }
    const int64_t max_tiles = (int64_t)std::max(1, odf) * std::max(1, num_pes);
    for (auto& kv : s.meta) {
        cn_array_meta& m = *kv.second;
        if (m.tile <= 0) m.tile = s.min_tile[m.ndims];
        if (!m.decomp_final) {
            m.tile = std::max(next_pow2(m.tile), s.min_tile[m.ndims]);
            auto count = [&]() {
                int64_t c = 1;
                for (int d = 0; d < m.ndims; ++d) c *= (m.shape[d] + m.tile - 1) / m.tile;
                return c;
            };
            while (count() > max_tiles) m.tile *= 2;
            m.offset[0] = m.offset[1] = m.offset[2] = 0;
        }
    }
    if (!dag) return CN_OK;

    // alignment relations of every root that defines or stores an array
    for (auto& node : dag->nodes) {
        std::map<int, const AstNode*> defs;
        for (auto& rp : node.roots) {
            const AstNode& r = *rp;
            if (r.opcode == OP_SET_REGION) {
                if (r.operands.size() != 2 || !r.operands[0].leaf) continue;
                const int target = r.operands[0].leaf->result_name;
                const Operand& rhs = r.operands[1];
                const int value = rhs.is_ref ? rhs.ref_name : (rhs.leaf && !rhs.leaf->is_scalar ? rhs.leaf->result_name : -1);
                // the stored array lines up with the target's region: stored[i] sits on target[start + i * step]
                if (value >= 0 && s.find(value)) s.add_edge(value, target, r.region);
                continue;
            }
            if (!(is_elementwise(r.opcode) || r.opcode == OP_COPY)) continue;
            defs[r.result_name] = &r;
            if (!s.find(r.result_name)) continue;
            for (auto& o : r.operands) s.collect(o, defs, r.result_name, 0);
        }
    }

    // tiles: proposals from the arrays an array is aligned with, to a fixed point
    for (int pass = 0; pass < 64; ++pass) {
        bool changed = false;
        for (const Edge& e : s.edges) {
            cn_array_meta *out = s.find(e.out), *src = s.find(e.src);
            if (out->decomp_final) continue;
            int64_t factor = 0;
            for (int d = 0; d < e.ndims; ++d)
                if (e.step[d] > 1) factor = factor ? gcd64(factor, e.step[d]) : e.step[d];
            int64_t cand = src->tile;
            if (factor > 1) cand = std::max<int64_t>(1, cand / factor);
            cand = std::max(next_pow2(cand), s.min_tile[out->ndims]);
            if (cand < out->tile) {
                out->tile = cand;
                changed = true;
            }
        }
        if (!changed) break;
    }

    // offsets: relax until nothing moves; arrays whose offset is fixed never move
    std::set<int> known;
    for (auto& kv : s.meta)
        if (kv.second->decomp_final) known.insert(kv.first);
    std::vector<int> order;  // arrays in the order the DAG defines them
    for (const Edge& e : s.edges)
        if (!s.find(e.out)->decomp_final && std::find(order.begin(), order.end(), e.out) == order.end())
            order.push_back(e.out);
    for (int sweep = 0; sweep < 8; ++sweep) {
        bool moved = false;
        for (int name : order) {
            cn_array_meta& m = *s.find(name);
            for (int d = 0; d < m.ndims; ++d) {
                std::vector<int64_t> props;
                for (const Edge& e : s.edges) {
                    if (e.out == name && known.count(e.src))  // computed from / stored into src
                        props.push_back((s.find(e.src)->offset[d] + e.start[d]) / e.step[d]);
                    else if (e.src == name && known.count(e.out) && e.out != name)  // out is computed from this array
                        props.push_back(s.find(e.out)->offset[d] * e.step[d] - e.start[d]);
                }
                if (props.empty()) continue;
                std::vector<int64_t> cands = props;
                std::sort(cands.begin(), cands.end());
                cands.erase(std::unique(cands.begin(), cands.end()), cands.end());
                int64_t best = cands[0], best_cost = -1;
                for (int64_t c : cands) {
                    int64_t cost = 0;
                    for (int64_t p : props) cost += c > p ? c - p : p - c;
                    if (best_cost < 0 || cost < best_cost) {
                        best_cost = cost;
                        best = c;
                    }
                }
                if (m.offset[d] != best) {
                    m.offset[d] = best;
                    moved = true;
                }
            }
            known.insert(name);
        }
        if (!moved) break;
    }
    for (int name : order) s.find(name)->decomp_final = 1;
    return CN_OK;
}

}  // namespace cn

extern "C" int cn_compute_decompositions(cn_array_meta* arrays, int n_arrays, const char* dag_blob, int64_t size,
                                         int odf, int num_pes, const int64_t min_tile[3]) {
    if ((!arrays && n_arrays > 0) || n_arrays < 0) return cn::CN_ERR_INVALID_ARGUMENT;
    cn::Dag dag;
    if (dag_blob) {
        std::string err;
        int rc = cn::parse_dag(dag_blob, size, &dag, &err);
        if (rc) return rc;
    }
    return cn::compute_decompositions(arrays, n_arrays, dag_blob ? &dag : nullptr, odf, num_pes, min_tile);
}
