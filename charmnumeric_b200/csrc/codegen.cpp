// GroupIR -> CUDA source for one fused group kernel (entry point `cn_group`).
//
// The reference builds one linalg.generic per root and relies on MLIR loop fusion
// (src/jit.cpp:28-185), then launches one 256-thread-per-block kernel per aligned fragment
// (src/dispatch.hpp:187-194).  Here each group becomes ONE persistent kernel over the whole
// local slab: blocks walk a list of tiles, every thread owns `vec` adjacent elements of
// `CN_R` consecutive rows, loads are 128-bit where the column offset is even, every root is
// one separately rounded statement (the program is compiled with --fmad=false so that
// a*b+c is never contracted), and fused reductions end in the deterministic last-block
// finish of cn_device.cuh.
#include <map>
#include <algorithm>
#include <set>
#include <sstream>

#include "cn_device.cuh"
#include "group_ir.hpp"

namespace cn {

namespace {

const char* type_name(int dt) {
    switch (dt) {
        case DT_F32: return "float";
        case DT_F64: return "double";
        case DT_I32: return "int";
        default: return "long long";
    }
}

struct Gen {
    const GroupIR& g;
    std::ostringstream o;
    bool is_float() const { return g.dtype == DT_F32 || g.dtype == DT_F64; }
    int nd() const { return g.flat ? 1 : g.ndims; }

    std::string val(const ValRef& v, int e) const {
        std::ostringstream s;
        switch (v.kind) {
            case ValRef::LEAF: s << pfx << "l" << v.idx << "_" << e; break;
            case ValRef::CONST: s << pfx << "c" << v.idx; break;
            case ValRef::BCAST: s << pfx << "b" << v.idx; break;
            case ValRef::ROOT:
                if (g.roots[v.idx].domain == DOM_SCALAR) s << pfx << "r" << v.idx;
                else s << pfx << "r" << v.idx << "_" << e;
                break;
            case ValRef::OUTVAL: s << "w" << v.idx << "_" << e; break;
            default: s << "(T)0";
        }
        return s.str();
    }

    std::string expr(int opcode, const std::string& a, const std::string& b) const {
        switch (opcode) {
            case OP_ADD: return a + " + " + b;
            case OP_SUB: return a + " - " + b;
            case OP_MUL: return a + " * " + b;
            case OP_DIV: return a + " / " + b;
            case OP_COPY: return a;
            case OP_EXP:
                return g.dtype == DT_F64 ? "cn_exp(" + a + ")" : "(T)cn_exp((double)" + a + ")";
            case OP_TANH:
                return g.dtype == DT_F64 ? "cn_tanh(" + a + ")" : "(T)cn_tanh((double)" + a + ")";
            case OP_SQRT: return g.dtype == DT_F64 ? "sqrt(" + a + ")" : "sqrtf(" + a + ")";
            case OP_ABS:
                if (g.dtype == DT_F64) return "fabs(" + a + ")";
                if (g.dtype == DT_F32) return "fabsf(" + a + ")";
                return "(" + a + " < 0 ? -" + a + " : " + a + ")";
        }
        return "(T)0";
    }

    std::string pfx;           // name prefix of this group's values (a staged producer's are "P...")
    bool staged_mode = false;  // stencil array comes from the shared-memory ring
    bool fast_loads = false;   // inside a row-interior tile: every load is unconditional
    bool carry_mode = false;   // staged 3-D march: the thread's own column is carried in registers
    bool pref_mode = false;    // flat interior tile: inputs were loaded ahead into cu<row>[r]
    // slot of each distinct input array, in order of first use (SHIFTED class)
    std::vector<int> in_names;
    int in_slot(int name) {
        for (size_t i = 0; i < in_names.size(); ++i)
            if (in_names[i] == name) return (int)i;
        in_names.push_back(name);
        return (int)in_names.size() - 1;
    }
    // an input buffer may be the very buffer an output is written to (in-place update)
    bool aliases_written_buffer(int name) const {
        for (auto& out : g.outs)
            if (out.name == name && out.is_set && !(g.copy_through && out.hazard)) return true;
        return false;
    }
    bool any_inplace() const {
        for (auto& out : g.outs)
            if (out.is_set && !(g.copy_through && out.hazard)) return true;
        return false;
    }

    void prologue() {
        o << "#include \"cn_device.cuh\"\n";
        o << "typedef " << type_name(g.dtype) << " T;\n";
        o << "typedef " << (is_float() ? "double" : "long long") << " ACC;\n";
        if (g.vec == 2) o << "typedef " << (g.dtype == DT_I64 ? "longlong2" : "double2") << " T2;\n";
        o << "extern \"C\" __global__ void __launch_bounds__(CN_BLOCK, CN_MINB) " << g.entry_name() << "("
             "const __grid_constant__ CnGroupArgs a) {\n";
        o << "  cn_stream_dependency();\n";
        for (size_t i = 0; i < g.scalars.size(); ++i)
            o << "  const T c" << i << " = (T)a.sc[" << i << "];\n";
        for (size_t i = 0; i < g.bcast_names.size(); ++i)
            o << "  const T b" << i << " = *(const T*)a.bc[" << i << "];\n";
        for (size_t i = 0; i < g.roots.size(); ++i) {
            const RootIR& r = g.roots[i];
            if (r.domain != DOM_SCALAR) continue;
            o << "  const T r" << i << " = " << expr(r.opcode, val(r.a, 0), val(r.b, 0)) << ";\n";
        }
    }

    void scalar_outs() {
        if (g.souts.empty()) return;
        o << "  if (blockIdx.x == 0 && threadIdx.x == 0) {\n";
        for (size_t i = 0; i < g.souts.size(); ++i)
            o << "    *(T*)a.sout[" << i << "] = " << val(g.souts[i].value, 0) << ";\n";
        o << "  }\n";
    }

    // stores into other GPUs' mailboxes are made visible there before the kernel ends
    void push_fence() {
        o << "#if CN_PUSH\n  if (a.push_mask) __threadfence_system();\n#endif\n";
    }

    void red_decl() {
        for (size_t i = 0; i < g.reds.size(); ++i) o << "  ACC acc" << i << " = (ACC)0;\n";
    }

    void red_epilogue() {
        if (g.reds.empty()) return;
        o << "  __shared__ ACC cn_sm[32];\n  __shared__ int cn_flag;\n";
        for (size_t i = 0; i < g.reds.size(); ++i)
            o << "  ACC bt" << i << " = cn_block_sum(acc" << i << ", cn_sm);\n";
        o << "  if (threadIdx.x == 0) {\n";
        for (size_t i = 0; i < g.reds.size(); ++i)
            o << "    ((ACC*)a.partials)[" << i << " * gridDim.x + blockIdx.x] = bt" << i << ";\n";
        o << "  }\n";
        o << "  if (cn_grid_ticket(a.counter, &cn_flag)) {\n";
        o << "    ACC tv[" << g.reds.size() << "];\n";
        for (size_t i = 0; i < g.reds.size(); ++i)
            o << "    tv[" << i << "] = cn_sum_partials(((const ACC*)a.partials) + " << i
              << " * gridDim.x, cn_sm);\n";
        // more than one rank: the block that holds the local totals also exchanges them with
        // the other GPUs' mailboxes and adds them up, so no separate collective follows
        o << "    if (a.peer_n > 1) cn_peer_allreduce(a, tv, " << g.reds.size() << ", cn_sm);\n";
        for (size_t i = 0; i < g.reds.size(); ++i)
            o << "    if (threadIdx.x == 0) *(T*)a.red[" << i << "] = (T)tv[" << i << "];\n";
        scalar_tail();
        o << "    if (threadIdx.x == 0) *a.counter = 0u;\n";
        o << "  }\n";
    }

    // The scalar group behind the reductions, evaluated by the thread that has just stored
    // their results (it reads them back through the size-1 operand pointers).  Every block of
    // the launch has finished its own work by now -- this block drew the last ticket -- so a
    // size-1 array the group's blocks read in their prologue may be overwritten here.
    void scalar_tail() {
        if (g.tail.empty()) return;
        const GroupIR& S = g.tail[0];
        Gen sg{S, {}, {}};
        sg.pfx = "S";
        size_t sc_base = g.scalars.size(), bc_base = g.bcast_names.size();
        if (!g.producer.empty()) {
            sc_base += g.producer[0].scalars.size();
            bc_base += g.producer[0].bcast_names.size();
        }
        const size_t so_base = g.souts.size();
        o << "    if (threadIdx.x == 0) {\n";
        for (size_t i = 0; i < S.scalars.size(); ++i)
            o << "      const T Sc" << i << " = (T)a.sc[" << (sc_base + i) << "];\n";
        for (size_t i = 0; i < S.bcast_names.size(); ++i)
            o << "      const T Sb" << i << " = *(const volatile T*)a.bc[" << (bc_base + i) << "];\n";
        for (size_t i = 0; i < S.roots.size(); ++i) {
            const RootIR& r = S.roots[i];
            if (r.domain != DOM_SCALAR) continue;
            o << "      const T Sr" << i << " = " << sg.expr(r.opcode, sg.val(r.a, 0), sg.val(r.b, 0)) << ";\n";
        }
        for (size_t i = 0; i < S.souts.size(); ++i)
            o << "      *(T*)a.sout[" << (so_base + i) << "] = " << sg.val(S.souts[i].value, 0) << ";\n";
        o << "    }\n";
    }

    std::string guard(int domain, int e) const {
        std::ostringstream s;
        s << ((domain == DOM_REGION && g.two_domains) ? "act" : "bx") << e;
        return s.str();
    }
    std::string guard_any(int domain) const {
        if (fast_loads) return "(true)";
        std::string base = (domain == DOM_REGION && g.two_domains) ? "act" : "bx";
        if (g.vec == 1) return "(" + base + "0)";
        return "(" + base + "0 | " + base + "1)";
    }

    // ---- SHIFTED class ----------------------------------------------------------------
    void shifted_body(const std::string& ind) {
        const int N = nd();
        const int V = g.vec;
        // row offset expression of a leaf: deltas of all but the last dimension
        auto rowoff = [&](const LeafIR& l) {
            std::ostringstream s;
            if (g.flat) return std::string("");
            if (N == 2 && l.delta[0]) s << " + (" << l.delta[0] << "LL) * s0";
            if (N == 3) {
                if (l.delta[0]) s << " + (" << l.delta[0] << "LL) * s0";
                if (l.delta[1]) s << " + (" << l.delta[1] << "LL) * s1";
            }
            return s.str();
        };
        // group leaves into rows: (array, domain, outer deltas)
        struct Row {
            int name, domain;
            int64_t d0, d1;
            std::string off;
            std::set<int64_t> cols;
        };
        std::vector<Row> rows;
        std::vector<int> leaf_row(g.leaves.size());
        for (size_t k = 0; k < g.leaves.size(); ++k) {
            const LeafIR& l = g.leaves[k];
            int64_t d0 = 0, d1 = 0, dl = 0;
            if (!g.flat) {
                if (N == 1) dl = l.delta[0];
                if (N == 2) d0 = l.delta[0], dl = l.delta[1];
                if (N == 3) d0 = l.delta[0], d1 = l.delta[1], dl = l.delta[2];
            }
            int found = -1;
            for (size_t r = 0; r < rows.size(); ++r)
                if (rows[r].name == l.name && rows[r].domain == l.domain && rows[r].d0 == d0 &&
                    rows[r].d1 == d1)
                    found = (int)r;
            if (found < 0) {
                Row r{l.name, l.domain, d0, d1, rowoff(l), {}};
                rows.push_back(r);
                found = (int)rows.size() - 1;
            }
            leaf_row[k] = found;
            for (int e = 0; e < V; ++e) rows[found].cols.insert(dl + e);
        }
        auto colname = [](int row, int64_t c) {
            std::ostringstream s;
            s << "m" << row << (c < 0 ? "n" : "p") << (c < 0 ? -c : c);
            return s.str();
        };
        // loads
        for (size_t r = 0; r < rows.size(); ++r) {
            Row& row = rows[r];
            int slot = in_slot(row.name);
            std::ostringstream decl;
            for (int64_t c : row.cols) decl << ind << "T " << colname((int)r, c) << " = (T)0;\n";
            o << decl.str();
            // where the row lives: global memory (guarded) or the shared-memory ring (always
            // there: the TMA unit zero-fills whatever lies outside the array)
            const bool smem = staged_mode && row.name == g.stage_array;
            std::ostringstream base;
            if (smem) {
                const int64_t dz = N == 3 ? row.d0 : 0, dy = N == 3 ? row.d1 : row.d0;
                base << "sp" << (dz + g.hz) << " + sq + (" << dy << ") * CN_SW + 2";
                o << ind << "{\n";
            } else {
                base << "in" << slot << " + p" << row.off;
                o << ind << "if " << guard_any(row.domain) << " {\n";
            }
            std::set<int64_t> done;
            if (pref_mode && !smem) {
                o << ind << "  " << colname((int)r, 0) << " = cu" << r << "[r].x; " << colname((int)r, 1)
                  << " = cu" << r << "[r].y;\n";
                done.insert(0);
                done.insert(1);
            }
            if (smem && carry_mode && N == 3 && row.d1 == 0) {
                // the thread's own two columns of planes z-1, z, z+1 sit in registers
                for (int64_t c = 0; c < 2; ++c)
                    if (row.cols.count(c)) {
                        o << ind << "  " << colname((int)r, c) << " = cz" << (row.d0 + g.hz) << "[r][" << c
                          << "];\n";
                        done.insert(c);
                    }
            }
            // 128-bit pair loads first, so that single neighbours can be taken from them
            for (int64_t c : row.cols) {
                if (done.count(c)) continue;
                bool even = ((c % 2) + 2) % 2 == 0;
                if (V == 2 && even && row.cols.count(c + 1) && !done.count(c + 1)) {
                    o << ind << "  { const T2 q = *(const T2*)(" << base.str() << " + (" << c
                      << "LL)); " << colname((int)r, c) << " = q.x; " << colname((int)r, c + 1)
                      << " = q.y; }\n";
                    done.insert(c);
                    done.insert(c + 1);
                }
            }
            // In a row-interior tile the lanes of a warp hold consecutive pairs of one row: the
            // elements just left and right of a thread's own pair sit in its neighbour lanes'
            // registers.  A shuffle fetches them; only the warp's edge lanes still load.
            const bool can_shfl = fast_loads && !smem && V == 2 && N >= 2 && row.cols.count(0) &&
                                  row.cols.count(1) && done.count(0) && done.count(1);
            bool shfl_open = false;
            if (can_shfl) {
                for (int64_t c : row.cols) {
                    if (done.count(c) || c < -2 || c > 3) continue;
                    if (!shfl_open) o << "#if CN_SHFL && (CN_TX % 32) == 0\n";
                    shfl_open = true;
                    const bool up = c < 0;
                    o << ind << "  " << colname((int)r, c) << " = __shfl_" << (up ? "up" : "down") << "_sync(wm, "
                      << colname((int)r, up ? c + 2 : c - 2) << ", 1);\n";
                    o << ind << "  if (" << (up ? "lane == 0" : "(lane == 31) | (x + 2 >= xhi)") << ") "
                      << colname((int)r, c) << " = *(" << base.str() << " + (" << c << "LL));\n";
                }
                if (shfl_open) {
                    o << "#else\n";
                    for (int64_t c : row.cols) {
                        if (done.count(c) || c < -2 || c > 3) continue;
                        o << ind << "  " << colname((int)r, c) << " = *(" << base.str() << " + (" << c << "LL));\n";
                    }
                    o << "#endif\n";
                    for (int64_t c : row.cols)
                        if (c >= -2 && c <= 3) done.insert(c);
                }
            }
            for (int64_t c : row.cols) {
                if (done.count(c)) continue;
                o << ind << "  " << colname((int)r, c) << " = *(" << base.str() << " + (" << c << "LL));\n";
                done.insert(c);
            }
            o << ind << "}\n";
        }
        for (size_t k = 0; k < g.leaves.size(); ++k) {
            const LeafIR& l = g.leaves[k];
            int64_t dl = g.flat ? 0 : l.delta[N - 1];
            for (int e = 0; e < V; ++e)
                o << ind << "const T l" << k << "_" << e << " = " << colname(leaf_row[k], dl + e)
                  << ";\n";
        }
        // old contents of outputs
        for (size_t m = 0; m < g.outs.size(); ++m) {
            if (!g.outs[m].needs_old) continue;
            for (int e = 0; e < V; ++e) o << ind << "T old" << m << "_" << e << " = (T)0;\n";
            // only elements of the sweep that lie outside the assigned region keep their
            // old value; inside it nothing of the old contents is needed
            if (g.two_domains && g.outs[m].domain == DOM_REGION) {
                if (V == 2) o << ind << "if ((bx0 & !act0) | (bx1 & !act1)) {\n";
                else o << ind << "if (bx0 & !act0) {\n";
            } else {
                o << ind << "if " << guard_any(DOM_BOX) << " {\n";
            }
            // the old contents live in the buffer the group also reads as an input: go through
            // that pointer so that the load coincides with the stencil's centre-row load
            std::ostringstream ptr;
            ptr << "old" << m << " + p";
            for (size_t s = 0; s < in_names.size(); ++s)
                if (in_names[s] == g.outs[m].name) {
                    ptr.str("");
                    ptr << "in" << s << " + p";
                }
            if (staged_mode && g.outs[m].name == g.stage_array) {
                ptr.str("");
                ptr << "sp" << g.hz << " + sq + (0) * CN_SW + 2";
            }
            if (carry_mode && staged_mode && g.outs[m].name == g.stage_array) {
                o << ind << "  old" << m << "_0 = cz" << g.hz << "[r][0]; old" << m << "_1 = cz" << g.hz
                  << "[r][1];\n";
            } else if (V == 2) {
                o << ind << "  const T2 q = *(const T2*)(" << ptr.str() << " + (0LL));\n";
                o << ind << "  old" << m << "_0 = q.x; old" << m << "_1 = q.y;\n";
            } else {
                o << ind << "  old" << m << "_0 = *(" << ptr.str() << " + (0LL));\n";
            }
            o << ind << "}\n";
        }
        auto emit_merged = [&](size_t m) {
            const OutIR& out = g.outs[m];
            for (int e = 0; e < V; ++e) {
                o << ind << "const T w" << m << "_" << e << " = ";
                if (out.needs_old)
                    o << guard(out.domain, e) << " ? " << val(out.value, e) << " : old" << m << "_"
                      << e << ";\n";
                else
                    o << val(out.value, e) << ";\n";
            }
        };
        for (size_t m = 0; m < g.outs.size(); ++m)
            if (g.outs[m].value.kind != ValRef::ROOT ||
                g.roots[g.outs[m].value.idx].domain == DOM_SCALAR)
                emit_merged(m);
        for (size_t i = 0; i < g.roots.size(); ++i) {
            const RootIR& r = g.roots[i];
            if (r.domain == DOM_SCALAR) continue;
            for (int e = 0; e < V; ++e)
                o << ind << "const T r" << i << "_" << e << " = "
                  << expr(r.opcode, val(r.a, e), val(r.b, e)) << ";\n";
            for (size_t m = 0; m < g.outs.size(); ++m)
                if (g.outs[m].value.kind == ValRef::ROOT && g.outs[m].value.idx == (int)i)
                    emit_merged(m);
        }
        // stores
        for (size_t m = 0; m < g.outs.size(); ++m) {
            const OutIR& out = g.outs[m];
            int dom = (g.copy_through && out.hazard) ? DOM_BOX : out.domain;
            if (V == 2) {
                o << ind << "if (" << guard(dom, 0) << " & " << guard(dom, 1) << ") {\n";
                o << ind << "  T2 q; q.x = w" << m << "_0; q.y = w" << m << "_1;\n";
                o << ind << "  *(T2*)(out" << m << " + p) = q;\n";
                o << ind << "} else if (" << guard(dom, 0) << ") {\n";
                o << ind << "  out" << m << "[p] = w" << m << "_0;\n";
                o << ind << "} else if (" << guard(dom, 1) << ") {\n";
                o << ind << "  out" << m << "[p + 1] = w" << m << "_1;\n";
                o << ind << "}\n";
            } else {
                o << ind << "if (" << guard(dom, 0) << ") out" << m << "[p] = w" << m << "_0;\n";
            }
            // the slab's edge rows also go straight into the neighbours' mailboxes
            o << "#if CN_PUSH\n";
            o << ind << "if (a.push_mask & " << (1u << m) << "u) {\n";
            for (int e = 0; e < V; ++e) {
                o << ind << "  if (" << guard(dom, e) << ") {\n";
                o << ind << "    const unsigned long long q = (unsigned long long)(p + " << e << ");\n";
                o << ind << "    if (a.push_prev[" << m << "] && q < (unsigned long long)a.push_elems) ((T*)a.push_prev[" << m
                  << "])[q] = w" << m << "_" << e << ";\n";
                o << ind << "    const unsigned long long t = q - (unsigned long long)a.push_last;\n";
                o << ind << "    if (a.push_next[" << m << "] && t < (unsigned long long)a.push_elems) ((T*)a.push_next[" << m
                  << "])[t] = w" << m << "_" << e << ";\n";
                o << ind << "  }\n";
            }
            o << ind << "}\n";
            o << "#endif\n";
        }
        // reductions
        for (size_t q = 0; q < g.reds.size(); ++q) {
            const RedIR& rd = g.reds[q];
            for (int e = 0; e < V; ++e) {
                std::string prod = rd.b.kind == ValRef::NONE
                                       ? "(ACC)" + val(rd.a, e)
                                       : "(ACC)(" + val(rd.a, e) + " * " + val(rd.b, e) + ")";
                o << ind << "if (" << guard(rd.domain, e) << (nd() >= 2 ? " & ownr" : "") << ") acc" << q << " += " << prod
                  << ";\n";
            }
        }
    }

    void shifted() {
        const int N = nd();
        const int V = g.vec;
        prologue();
        scalar_outs();
        // resolve input slots first so the pointer declarations are complete
        for (auto& l : g.leaves) in_slot(l.name);
        const bool inplace = any_inplace();
        for (size_t i = 0; i < in_names.size(); ++i) {
            bool alias = inplace && aliases_written_buffer(in_names[i]);
            o << "  const T* " << (alias ? "" : "__restrict__ ") << "in" << i << " = (const T*)a.in["
              << i << "];\n";
        }
        for (size_t m = 0; m < g.outs.size(); ++m) {
            bool shadow = g.copy_through && g.outs[m].hazard;
            o << "  T* " << (shadow ? "__restrict__ " : "") << "out" << m << " = (T*)a.out[" << m
              << "];\n";
            if (g.outs[m].needs_old)
                o << "  const T* old" << m << " = (const T*)a.old[" << m << "];\n";
        }
        red_decl();
        const int L = N - 1;
        if (N >= 2) o << "  const long long s0 = CN_S0 ? CN_S0 : a.stride[0];\n";
        if (N == 3) o << "  const long long s1 = CN_S1 ? CN_S1 : a.stride[1];\n";
        o << "  const long long xlo = a.lo[" << L << "], xhi = a.hi[" << L << "];\n";
        if (g.two_domains)
            o << "  const long long rxlo = a.rlo[" << L << "], rxhi = a.rhi[" << L << "];\n";
        o << "  const long long xbase = " << (V == 2 ? "xlo & ~1LL" : "xlo") << ";\n";
        o << "  const unsigned int ntiles = (unsigned int)a.ntiles;\n";
        // Tiles that lie completely inside the region take a path without any per-element
        // guard: every load is unconditional, so the compiler can issue the loads of all
        // CN_R rows up front and reuse rows shared by consecutive stencil rows.
        auto emit_guards = [&](bool fast) {
            if (fast && N == 1) {
                // a flat interior tile lies inside the region from end to end
                for (int e = 0; e < V; ++e) o << "      const bool bx" << e << " = true;\n";
                if (g.two_domains)
                    for (int e = 0; e < V; ++e) o << "      const bool act" << e << " = true;\n";
                return;
            }
            if (fast) {
                // rows (and planes) of the tile are all inside the region: only the position
                // along the last dimension still decides what an element does
                for (int e = 0; e < V; ++e)
                    o << "      const bool bx" << e << " = (x + " << e << " >= xlo) & (x + " << e
                      << " < xhi);\n";
                if (g.two_domains)
                    for (int e = 0; e < V; ++e)
                        o << "      const bool act" << e << " = (x + " << e << " >= rxlo) & (x + "
                          << e << " < rxhi);\n";
                return;
            }
            for (int e = 0; e < V; ++e)
                o << "      const bool bx" << e << " = (x + " << e << " >= xlo) & (x + " << e
                  << " < xhi);\n";
            if (g.two_domains) {
                std::ostringstream rowin;
                rowin << "true";
                if (N == 2) rowin << " & (y >= a.rlo[0]) & (y < a.rhi[0])";
                if (N == 3)
                    rowin << " & (z >= a.rlo[0]) & (z < a.rhi[0]) & (y >= a.rlo[1]) & (y < a.rhi[1])";
                o << "      const bool rowin = " << rowin.str() << ";\n";
                for (int e = 0; e < V; ++e)
                    o << "      const bool act" << e << " = rowin & (x + " << e << " >= rxlo) & (x + "
                      << e << " < rxhi);\n";
            }
        };
        auto emit_rows = [&](bool fast) {
            o << "#pragma unroll\n";
            o << "    for (int r = 0; r < CN_R; ++r) {\n";
            if (N == 1) {
                o << "      const long long x = t0 + (long long)r * (CN_BLOCK * " << V
                  << ") + threadIdx.x * " << V << ";\n";
                o << "      const long long p = x;\n";
            } else {
                o << "      const long long y = ybase + r;\n";
                if (!fast) o << "      if (y >= a.hi[" << (N - 2) << "]) break;\n";
                if (N == 2) o << "      const long long p = y * s0 + x;\n";
                else o << "      const long long p = z * s0 + y * s1 + x;\n";
                if (!g.reds.empty())
                    o << "      const bool ownr = (" << (N == 2 ? "y" : "z") << " >= a.own_lo) & (" << (N == 2 ? "y" : "z")
                      << " < a.own_hi);\n";
            }
            emit_guards(fast);
            if (fast && N == 1) o << "      {\n";
            else if (fast) {
                // all lanes of the warp are here (the tile is interior for the whole block):
                // the lanes that go on form a prefix of the warp
                o << "#if CN_SHFL && (CN_TX % 32) == 0\n";
                o << "      const unsigned int wm = __ballot_sync(0xffffffffu, x < xhi);\n";
                o << "      const int lane = threadIdx.x & 31;\n";
                o << "#endif\n";
                o << "      if (x < xhi) {\n";
            }
            else o << "      if " << guard_any(DOM_BOX) << " {\n";
            fast_loads = fast;
            shifted_body("        ");
            fast_loads = false;
            o << "      }\n";
            o << "    }\n";
        };
        const char* ilo = g.two_domains ? "rxlo" : "xlo";
        const char* ihi = g.two_domains ? "rxhi" : "xhi";
        // distinct (array, domain) pairs of a flat group, in the order shifted_body numbers them
        std::vector<std::pair<int, int>> flat_rows;
        if (N == 1)
            for (auto& l : g.leaves) {
                std::pair<int, int> key(l.name, l.domain);
                if (std::find(flat_rows.begin(), flat_rows.end(), key) == flat_rows.end())
                    flat_rows.push_back(key);
            }
        const bool prefetch = g.flat && V == 2 && !flat_rows.empty();
        if (prefetch) {
            o << "#if CN_PREFETCH == 1\n  bool have = false;\n";
            for (size_t k = 0; k < flat_rows.size(); ++k) o << "  T2 nx" << k << "[CN_R] = {};\n";
            o << "#endif\n";
        }
        if (N == 1) {
            o << "  for (unsigned int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {\n";
            o << "    const long long t0 = xbase + (long long)tile * (CN_R * CN_BLOCK * " << V << ");\n";
            o << "    const bool interior = (t0 >= " << ilo << ") & (t0 + CN_R * CN_BLOCK * " << V
              << " <= " << ihi << ");\n";
        } else {
            o << "  const unsigned int ntx = (unsigned int)a.ntx;\n";
            if (N == 3) o << "  const unsigned int nty = (unsigned int)a.nty;\n";
            o << "  const int lx = threadIdx.x % CN_TX, ly = threadIdx.x / CN_TX;\n";
            o << "  for (unsigned int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {\n";
            o << "    const unsigned int tx = tile % ntx; const unsigned int t2 = tile / ntx;\n";
            if (N == 3) {
                o << "    const unsigned int ty = t2 % nty;\n";
                o << "    const long long z = a.lo[0] + (long long)(t2 / nty);\n";
            } else {
                o << "    const unsigned int ty = t2;\n";
            }
            o << "    const long long tx0 = xbase + (long long)tx * (CN_TX * " << V << ");\n";
            o << "    const long long ty0 = a.lo[" << (N - 2) << "] + (long long)ty * ((CN_BLOCK / CN_TX) * CN_R);\n";
            o << "    const long long x = tx0 + lx * " << V << ";\n";
            o << "    const long long ybase = ty0 + ly * CN_R;\n";
            const std::string dom = g.two_domains ? "a.rlo" : "a.lo";
            const std::string domh = g.two_domains ? "a.rhi" : "a.hi";
            o << "    const bool interior = (ty0 >= " << dom << "[" << (N - 2)
              << "]) & (ty0 + (CN_BLOCK / CN_TX) * CN_R <= " << domh << "[" << (N - 2) << "])";
            if (N == 3 && g.two_domains) o << " & (z >= a.rlo[0]) & (z < a.rhi[0])";
            o << ";\n";
        }
        o << "    if (interior) {\n";
        if (prefetch) {
            // Software pipeline over the block's list of tiles: the inputs of the next
            // interior tile are requested before this tile's arithmetic starts, so that long
            // dependent chains (exp, sqrt, division) do not leave the memory system idle.
            const std::string tstep = "(CN_R * CN_BLOCK * 2)";
            auto load_all = [&](const char* dst, const char* base) {
                o << "#pragma unroll\n      for (int r = 0; r < CN_R; ++r) {\n";
                for (size_t k = 0; k < flat_rows.size(); ++k)
                    o << "        " << dst << k << "[r] = *(const T2*)(in" << in_slot(flat_rows[k].first)
                      << " + " << base << " + (long long)r * (CN_BLOCK * 2) + threadIdx.x * 2);\n";
                o << "      }\n";
            };
            o << "#if CN_PREFETCH\n";
            for (size_t k = 0; k < flat_rows.size(); ++k) o << "      T2 cu" << k << "[CN_R];\n";
            o << "#if CN_PREFETCH == 1\n";
            o << "      if (have) {\n#pragma unroll\n        for (int r = 0; r < CN_R; ++r) {";
            for (size_t k = 0; k < flat_rows.size(); ++k) o << " cu" << k << "[r] = nx" << k << "[r];";
            o << " }\n      } else {\n";
            load_all("cu", "t0");
            o << "      }\n";
            o << "      const unsigned int ntile = tile + gridDim.x;\n";
            o << "      const long long n0 = xbase + (long long)ntile * " << tstep << ";\n";
            o << "      have = (ntile < ntiles) & (n0 + " << tstep << " <= " << ihi << ");\n";
            o << "      if (have) {\n";
            load_all("nx", "n0");
            o << "      }\n";
            o << "#else\n";
            // every load of the tile ahead of its arithmetic
            load_all("cu", "t0");
            o << "#endif\n";
            pref_mode = true;
            emit_rows(true);
            pref_mode = false;
            o << "#else\n";
            emit_rows(true);
            o << "#endif\n";
        } else {
            emit_rows(true);
        }
        o << "    } else {\n";
        if (prefetch) o << "#if CN_PREFETCH == 1\n      have = false;\n#endif\n";
        emit_rows(false);
        o << "    }\n";
        o << "  }\n";
        push_fence();
        red_epilogue();
        o << "}\n";
    }

    // ---- staged producer: constants and inputs of the flat group that fills the tiles ------
    void producer_prologue() {
        const GroupIR& P = g.producer[0];
        Gen pg{P, {}, {}};
        pg.pfx = "P";
        const size_t sc_base = g.scalars.size(), bc_base = g.bcast_names.size();
        for (auto& l : g.leaves) in_slot(l.name);
        const size_t in_base = in_names.size();
        for (size_t i = 0; i < P.scalars.size(); ++i)
            o << "  const T Pc" << i << " = (T)a.sc[" << (sc_base + i) << "];\n";
        for (size_t i = 0; i < P.bcast_names.size(); ++i)
            o << "  const T Pb" << i << " = *(const T*)a.bc[" << (bc_base + i) << "];\n";
        for (size_t i = 0; i < P.roots.size(); ++i) {
            const RootIR& r = P.roots[i];
            if (r.domain != DOM_SCALAR) continue;
            o << "  const T Pr" << i << " = " << pg.expr(r.opcode, pg.val(r.a, 0), pg.val(r.b, 0)) << ";\n";
        }
        const std::vector<int> pin = P.input_arrays();
        for (size_t k = 0; k < pin.size(); ++k)
            o << "  const T* __restrict__ Pin" << k << " = (const T*)a.in[" << (in_base + k) << "];\n";
    }

    // One pass of the block over the tile's (rows + 2 hy) x (cols + 4) points, two adjacent
    // points per thread and step: load the producer's inputs there, evaluate its roots in
    // their own order (each a separately rounded statement, as everywhere), store the pair.
    // Points outside the arrays get zeros; no valid stencil point reads them.
    void producer_fill() {
        const GroupIR& P = g.producer[0];
        Gen pg{P, {}, {}};
        pg.pfx = "P";
        const std::vector<int> pin = P.input_arrays();
        // CN_FILL_U points' loads are issued together before any of them is used
        o << "    enum { CN_FILL_N = CN_SH * (CN_SW / 2), CN_FILL_IT = (CN_FILL_N + CN_BLOCK - 1) / CN_BLOCK };\n";
        o << "    for (int it0 = 0; it0 < CN_FILL_IT; it0 += CN_FILL_U) {\n";
        o << "      bool fin[CN_FILL_U];\n";
        for (size_t k = 0; k < pin.size(); ++k) o << "      T2 Pq" << k << "[CN_FILL_U];\n";
        o << "#pragma unroll\n";
        o << "      for (int u = 0; u < CN_FILL_U; ++u) {\n";
        o << "        const int i = threadIdx.x + (it0 + u) * CN_BLOCK;\n";
        o << "        const int sy = i / (CN_SW / 2), sx = i - sy * (CN_SW / 2);\n";
        o << "        const long long gy = ty0 - CN_HY + sy, gx = tx0 - 2 + 2 * sx;\n";
        o << "        fin[u] = (i < CN_FILL_N) & (gy >= fy0) & (gy < fy1) & (gx >= 0) & (gx < fx1);\n";
        o << "        const long long pp = gy * s0 + gx;\n";
        for (size_t k = 0; k < pin.size(); ++k) {
            o << "        Pq" << k << "[u].x = (T)0; Pq" << k << "[u].y = (T)0;\n";
            o << "        if (fin[u]) Pq" << k << "[u] = *(const T2*)(Pin" << k << " + pp);\n";
        }
        o << "      }\n";
        o << "#pragma unroll\n";
        o << "      for (int u = 0; u < CN_FILL_U; ++u) {\n";
        o << "        const int i = threadIdx.x + (it0 + u) * CN_BLOCK;\n";
        o << "        const int sy = i / (CN_SW / 2), sx = i - sy * (CN_SW / 2);\n";
        for (size_t k = 0; k < P.leaves.size(); ++k) {
            size_t slot = 0;
            for (size_t q = 0; q < pin.size(); ++q)
                if (pin[q] == P.leaves[k].name) slot = q;
            o << "        const T Pl" << k << "_0 = Pq" << slot << "[u].x, Pl" << k << "_1 = Pq" << slot << "[u].y;\n";
        }
        for (size_t i = 0; i < P.roots.size(); ++i) {
            const RootIR& r = P.roots[i];
            if (r.domain == DOM_SCALAR) continue;
            for (int e = 0; e < 2; ++e)
                o << "        const T Pr" << i << "_" << e << " = " << pg.expr(r.opcode, pg.val(r.a, e), pg.val(r.b, e))
                  << ";\n";
        }
        o << "        T2 v; v.x = fin[u] ? " << pg.val(P.outs[0].value, 0) << " : (T)0; v.y = fin[u] ? "
          << pg.val(P.outs[0].value, 1) << " : (T)0;\n";
        o << "        if (i < CN_FILL_N) *(T2*)(ring + sy * CN_SW + 2 * sx) = v;\n";
        o << "      }\n";
        o << "    }\n";
    }

    // ---- SHIFTED class, staged variant -----------------------------------------------------
    // The array that is read at shifted positions is brought into shared memory by the TMA
    // unit: 2-D groups fetch one (rows + 2 hy) x (cols + 4) tile per stage and keep three
    // stages in flight along the block's list of tiles; 3-D groups march along dimension 0
    // through a ring of plane tiles, so every plane is fetched once per column of tiles
    // instead of once per stencil arm.  One elected thread issues the copies; an mbarrier per
    // slot counts the bytes; all waits are bounded.  Everything else (other inputs, outputs,
    // reductions) goes through the same code as the cache-served variant.
    void staged() {
        const int N = g.ndims;
        const int V = 2;
        staged_mode = true;
        prologue();
        scalar_outs();
        for (auto& l : g.leaves) in_slot(l.name);
        const bool inplace = any_inplace();
        for (size_t i = 0; i < in_names.size(); ++i) {
            bool alias = inplace && aliases_written_buffer(in_names[i]);
            o << "  const T* " << (alias ? "" : "__restrict__ ") << "in" << i << " = (const T*)a.in["
              << i << "];\n";
        }
        for (size_t m = 0; m < g.outs.size(); ++m) {
            bool shadow = g.copy_through && g.outs[m].hazard;
            o << "  T* " << (shadow ? "__restrict__ " : "") << "out" << m << " = (T*)a.out[" << m
              << "];\n";
            if (g.outs[m].needs_old)
                o << "  const T* old" << m << " = (const T*)a.old[" << m << "];\n";
        }
        red_decl();
        const int L = N - 1;
        const bool prod = !g.producer.empty();  // tiles are computed, not copied (2-D only)
        const int NS = prod ? 1 : (N == 3 ? 2 * g.hz + 3 : 3);
        carry_mode = N == 3 && g.hz == 1;
        if (prod) producer_prologue();
        o << "  enum { CN_HY = " << g.hy << ", CN_HZ = " << g.hz << ", CN_NS = CN_NS_OVERRIDE ? CN_NS_OVERRIDE : " << NS
          << ", CN_TXE = CN_TX * 2, CN_SW = CN_TXE + 4, CN_TYT = (CN_BLOCK / CN_TX) * CN_R, "
             "CN_SH = CN_TYT + 2 * CN_HY, CN_BOX = CN_SH * CN_SW, CN_SLOT = (CN_BOX + 15) / 16 * 16 };\n";
        o << "  extern __shared__ __align__(128) unsigned char cn_dyn[];\n";
        o << "  T* const ring = (T*)cn_dyn;\n";
        o << "  unsigned long long* const full = (unsigned long long*)(cn_dyn + (size_t)CN_NS * CN_SLOT * sizeof(T));\n";
        if (!prod) {
            o << "  if (threadIdx.x == 0) {\n";
            o << "    for (int s = 0; s < CN_NS; ++s) cn_mbar_init(&full[s], 1u);\n";
            o << "    cn_mbar_init_fence();\n";
            o << "  }\n";
            o << "  __syncthreads();\n";
        } else {
            o << "  (void)full;\n";
        }
        o << "  const long long s0 = CN_S0 ? CN_S0 : a.stride[0];\n";
        if (N == 3) o << "  const long long s1 = CN_S1 ? CN_S1 : a.stride[1];\n";
        o << "  const long long xlo = a.lo[" << L << "], xhi = a.hi[" << L << "];\n";
        if (g.two_domains)
            o << "  const long long rxlo = a.rlo[" << L << "], rxhi = a.rhi[" << L << "];\n";
        o << "  const long long xbase = xlo & ~1LL;\n";
        o << "  const unsigned int ntiles = (unsigned int)a.ntiles;\n";
        o << "  const unsigned int ntx = (unsigned int)a.ntx;\n";
        if (N == 3) o << "  const unsigned int nty = (unsigned int)a.nty;\n";
        o << "  const int lx = threadIdx.x % CN_TX, ly = threadIdx.x / CN_TX;\n";
        o << "  bool timed_out = false;\n";
        if (N == 3 && g.two_domains) o << "  const long long rz0 = a.rlo[0], rz1 = a.rhi[0];\n";
        const std::string dom = g.two_domains ? "a.rlo" : "a.lo";
        const std::string domh = g.two_domains ? "a.rhi" : "a.hi";

        // In the 3-D march a thread keeps its (x, y) for a whole chunk of planes: what depends
        // on x alone is worked out once per chunk (pbx*, pact*), not once per plane.
        const bool hoist = N == 3;
        auto emit_guards = [&](bool fast) {
            for (int e = 0; e < V; ++e) {
                if (hoist) o << "        const bool bx" << e << " = pbx" << e << ";\n";
                else o << "        const bool bx" << e << " = (x + " << e << " >= xlo) & (x + " << e
                       << " < xhi);\n";
            }
            if (!g.two_domains) return;
            if (!fast) {
                std::ostringstream rowin;
                rowin << "true";
                if (N == 2) rowin << " & (y >= a.rlo[0]) & (y < a.rhi[0])";
                if (N == 3) rowin << " & zin & (y >= a.rlo[1]) & (y < a.rhi[1])";
                o << "        const bool rowin = " << rowin.str() << ";\n";
            }
            for (int e = 0; e < V; ++e) {
                o << "        const bool act" << e << " = " << (fast ? "" : "rowin & ");
                if (hoist) o << "pact" << e << ";\n";
                else o << "(x + " << e << " >= rxlo) & (x + " << e << " < rxhi);\n";
            }
        };
        auto emit_rows = [&](bool fast) {
            o << "#pragma unroll\n";
            o << "      for (int r = 0; r < CN_R; ++r) {\n";
            o << "        const long long y = ybase + r;\n";
            if (!fast) o << "        if (y >= a.hi[" << (N - 2) << "]) break;\n";
            if (N == 2) o << "        const long long p = y * s0 + x;\n";
            else o << "        const long long p = z * s0 + y * s1 + x;\n";
            o << "        const int sq = (ly * CN_R + r + CN_HY) * CN_SW + lx * 2;\n";
            if (!g.reds.empty())
                o << "        const bool ownr = (" << (N == 2 ? "y" : "z") << " >= a.own_lo) & (" << (N == 2 ? "y" : "z")
                  << " < a.own_hi);\n";
            emit_guards(fast);
            if (fast) o << "        if (x < xhi) {\n";
            else o << "        if " << guard_any(DOM_BOX) << " {\n";
            fast_loads = fast;
            shifted_body("          ");
            fast_loads = false;
            o << "        }\n";
            o << "      }\n";
        };
        auto emit_interior = [&]() {
            if (hoist) {
                if (g.two_domains) o << "      const bool zin = (z >= rz0) & (z < rz1);\n";
                o << "      const bool interior = yin" << (g.two_domains ? " & zin" : "") << ";\n";
            } else {
                o << "      const bool interior = (ty0 >= " << dom << "[" << (N - 2) << "]) & (ty0 + CN_TYT <= "
                  << domh << "[" << (N - 2) << "]);\n";
            }
            o << "      if (interior) {\n";
            emit_rows(true);
            o << "      } else {\n";
            emit_rows(false);
            o << "      }\n";
        };

        if (N == 2 && prod) {
            // every tile: all threads compute the stand-in's values for the tile and its halo
            // ring into shared memory, then the stencil reads them from there
            o << "  const long long fy0 = a.fill_lo[0], fy1 = a.fill_hi[0], fx1 = a.fill_hi[1];\n";
            o << "  for (unsigned int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {\n";
            o << "    const unsigned int tx = tile % ntx, ty = tile / ntx;\n";
            o << "    const long long tx0 = xbase + (long long)tx * CN_TXE;\n";
            o << "    const long long ty0 = a.lo[0] + (long long)ty * CN_TYT;\n";
            o << "    __syncthreads();  // the previous tile's readers are done with the ring\n";
            producer_fill();
            o << "    __syncthreads();\n";
            o << "    {\n";
            o << "      const T* const sp0 = ring;\n";
            o << "      const long long x = tx0 + lx * 2;\n";
            o << "      const long long ybase = ty0 + ly * CN_R;\n";
            emit_interior();
            o << "    }\n";
            o << "  }\n";
        } else if (N == 2) {
            // tile k of this block: index blockIdx.x + k * gridDim.x, slot k % CN_NS
            o << "  const unsigned int nmine = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;\n";
            o << "  auto issue = [&](unsigned int k) {\n";
            o << "    const unsigned int tile = blockIdx.x + k * gridDim.x;\n";
            o << "    const long long fx = xbase + (long long)(tile % ntx) * CN_TXE - 2 + a.tm_off[1];\n";
            o << "    const long long fy = a.lo[0] + (long long)(tile / ntx) * CN_TYT - CN_HY + a.tm_off[0];\n";
            o << "    const unsigned int s = k % CN_NS;\n";
            o << "    if (CN_DEBUG_DROP_COPIES) return;\n";
            o << "    cn_mbar_expect_tx(&full[s], (unsigned int)(CN_BOX * sizeof(T)));\n";
            o << "    cn_tma_load_2d(ring + (size_t)s * CN_SLOT, a.tmap, (int)fx, (int)fy, &full[s]);\n";
            o << "  };\n";
            o << "  if (threadIdx.x == 0)\n";
            o << "    for (unsigned int k = 0; k < nmine && k < CN_NS; ++k) issue(k);\n";
            o << "  for (unsigned int k = 0; k < nmine; ++k) {\n";
            o << "    const unsigned int tile = blockIdx.x + k * gridDim.x;\n";
            o << "    const unsigned int slot = k % CN_NS;\n";
            // the verdict of the bounded wait is made block-uniform, so that no thread can
            // leave the loop while others go on to the barrier below
            o << "    const bool ok = cn_mbar_wait(&full[slot], (k / CN_NS) & 1u);\n";
            o << "    if (__syncthreads_or(ok ? 0 : 1)) { timed_out = true; break; }\n";
            o << "    {\n";
            o << "      const T* const sp0 = ring + (size_t)slot * CN_SLOT;\n";
            o << "      const unsigned int tx = tile % ntx, ty = tile / ntx;\n";
            o << "      const long long tx0 = xbase + (long long)tx * CN_TXE;\n";
            o << "      const long long ty0 = a.lo[0] + (long long)ty * CN_TYT;\n";
            o << "      const long long x = tx0 + lx * 2;\n";
            o << "      const long long ybase = ty0 + ly * CN_R;\n";
            emit_interior();
            o << "    }\n";
            o << "    __syncthreads();\n";
            o << "    if (threadIdx.x == 0 && k + CN_NS < nmine) issue(k + CN_NS);\n";
            o << "  }\n";
        } else {
            // march along dimension 0 in chunks; plane i of a chunk is (zs - hz + i), and the
            // running load counter `gs` picks its slot and the parity of its barrier phase
            o << "  unsigned int gs = 0;\n";
            o << "  for (unsigned int tile = blockIdx.x; tile < ntiles && !timed_out; tile += gridDim.x) {\n";
            o << "    const unsigned int tx = tile % ntx; const unsigned int t2 = tile / ntx;\n";
            o << "    const unsigned int ty = t2 % nty; const unsigned int zc = t2 / nty;\n";
            o << "    const long long tx0 = xbase + (long long)tx * CN_TXE;\n";
            o << "    const long long ty0 = a.lo[1] + (long long)ty * CN_TYT;\n";
            o << "    const long long zs = a.lo[0] + (long long)zc * a.zchunk;\n";
            o << "    const long long ze = zs + a.zchunk < a.hi[0] ? zs + a.zchunk : a.hi[0];\n";
            o << "    const unsigned int total = (unsigned int)(ze - zs) + 2 * CN_HZ;\n";
            o << "    const long long x = tx0 + lx * 2;\n";
            o << "    const long long ybase = ty0 + ly * CN_R;\n";
            o << "    auto issue = [&](unsigned int i) {\n";
            o << "      const unsigned int s = (gs + i) % CN_NS;\n";
            o << "      if (CN_DEBUG_DROP_COPIES) return;\n";
            o << "      cn_mbar_expect_tx(&full[s], (unsigned int)(CN_BOX * sizeof(T)));\n";
            o << "      cn_tma_load_3d(ring + (size_t)s * CN_SLOT, a.tmap, (int)(tx0 - 2 + a.tm_off[2]), "
                 "(int)(ty0 - CN_HY + a.tm_off[1]), (int)(zs - CN_HZ + (long long)i + a.tm_off[0]), &full[s]);\n";
            o << "    };\n";
            o << "    if (threadIdx.x == 0)\n";
            o << "      for (unsigned int i = 0; i < total && i < CN_NS; ++i) issue(i);\n";
            o << "    unsigned int waited = 0;\n";
            for (int e = 0; e < V; ++e)
                o << "    const bool pbx" << e << " = (x + " << e << " >= xlo) & (x + " << e << " < xhi);\n";
            if (g.two_domains)
                for (int e = 0; e < V; ++e)
                    o << "    const bool pact" << e << " = (x + " << e << " >= rxlo) & (x + " << e << " < rxhi);\n";
            o << "    const bool yin = (ty0 >= " << dom << "[1]) & (ty0 + CN_TYT <= " << domh << "[1]);\n";
            if (carry_mode)
                o << "    T cz0[CN_R][2], cz1[CN_R][2], cz2[CN_R][2];  // own columns at z-1, z, z+1\n";
            o << "    for (long long z = zs; z < ze; ++z) {\n";
            o << "      const unsigned int i0 = (unsigned int)(z - zs);\n";
            // the verdict of the bounded wait is made block-uniform (see the 2-D loop above);
            // the barrier also keeps the block's warps on the same plane, which measured faster
            // than letting them drift
            o << "      while (waited <= i0 + 2 * CN_HZ) {\n";
            o << "        const bool ok = cn_mbar_wait(&full[(gs + waited) % CN_NS], ((gs + waited) / CN_NS) & 1u);\n";
            o << "        if (__syncthreads_or(ok ? 0 : 1)) { timed_out = true; break; }\n";
            o << "        ++waited;\n";
            o << "      }\n";
            o << "      if (timed_out) break;\n";
            for (int d = 0; d <= 2 * g.hz; ++d)
                o << "      const T* const sp" << d << " = ring + (size_t)((gs + i0 + " << d
                  << ") % CN_NS) * CN_SLOT;\n";
            if (carry_mode) {
                // one 128-bit shared-memory read per row brings in plane z+1; planes z-1 and z
                // were read on the two previous steps (on the first step of a chunk, now)
                o << "#pragma unroll\n";
                o << "      for (int r = 0; r < CN_R; ++r) {\n";
                o << "        const int sq = (ly * CN_R + r + CN_HY) * CN_SW + lx * 2;\n";
                o << "        if (i0 == 0) {\n";
                o << "          const T2 q0 = *(const T2*)(sp0 + sq + 2); cz0[r][0] = q0.x; cz0[r][1] = q0.y;\n";
                o << "          const T2 q1 = *(const T2*)(sp1 + sq + 2); cz1[r][0] = q1.x; cz1[r][1] = q1.y;\n";
                o << "        }\n";
                o << "        const T2 q2 = *(const T2*)(sp2 + sq + 2); cz2[r][0] = q2.x; cz2[r][1] = q2.y;\n";
                o << "      }\n";
            }
            emit_interior();
            if (carry_mode) {
                o << "#pragma unroll\n";
                o << "      for (int r = 0; r < CN_R; ++r) {\n";
                o << "        cz0[r][0] = cz1[r][0]; cz0[r][1] = cz1[r][1];\n";
                o << "        cz1[r][0] = cz2[r][0]; cz1[r][1] = cz2[r][1];\n";
                o << "      }\n";
            }
            o << "      __syncthreads();\n";
            o << "      if (threadIdx.x == 0 && i0 + CN_NS < total) issue(i0 + CN_NS);\n";
            o << "    }\n";
            o << "    gs += total;\n";
            o << "  }\n";
        }
        o << "  if (timed_out && a.error) atomicExch(a.error, 1u);\n";
        push_fence();
        red_epilogue();
        o << "}\n";
    }

    // ---- STRIDED class ----------------------------------------------------------------
    void strided() {
        const int N = g.ndims;
        prologue();
        scalar_outs();
        for (size_t k = 0; k < g.leaves.size(); ++k)
            o << "  const T* in" << k << " = (const T*)a.in[" << k << "];\n";
        for (size_t m = 0; m < g.outs.size(); ++m)
            o << "  T* out" << m << " = (T*)a.out[" << m << "];\n";
        red_decl();
        o << "  const long long e0 = a.ext[0]";
        if (N >= 2) o << ", e1 = a.ext[1]";
        if (N == 3) o << ", e2 = a.ext[2]";
        o << ";\n";
        o << "  const long long total = e0" << (N >= 2 ? " * e1" : "") << (N == 3 ? " * e2" : "")
          << ";\n";
        o << "  for (long long i = (long long)blockIdx.x * CN_BLOCK + threadIdx.x; i < total; "
             "i += (long long)gridDim.x * CN_BLOCK) {\n";
        if (N == 1) o << "    const long long i0 = i;\n";
        if (N == 2) o << "    const long long i0 = i / e1, i1 = i - i0 * e1;\n";
        if (N == 3)
            o << "    const long long i0 = i / (e1 * e2); const long long rem = i - i0 * e1 * e2;\n"
                 "    const long long i1 = rem / e2, i2 = rem - i1 * e2;\n";
        auto addr = [&](const char* what, size_t k) {
            std::ostringstream s;
            s << "a." << what << "_off[" << k << "] + i0 * a." << what << "_str[" << k << "][0]";
            if (N >= 2) s << " + i1 * a." << what << "_str[" << k << "][1]";
            if (N == 3) s << " + i2 * a." << what << "_str[" << k << "][2]";
            return s.str();
        };
        for (size_t k = 0; k < g.leaves.size(); ++k)
            o << "    const T l" << k << "_0 = in" << k << "[" << addr("in", k) << "];\n";
        for (size_t i = 0; i < g.roots.size(); ++i) {
            const RootIR& r = g.roots[i];
            if (r.domain == DOM_SCALAR) continue;
            o << "    const T r" << i << "_0 = " << expr(r.opcode, val(r.a, 0), val(r.b, 0)) << ";\n";
        }
        for (size_t m = 0; m < g.outs.size(); ++m)
            o << "    out" << m << "[" << addr("out", m) << "] = " << val(g.outs[m].value, 0)
              << ";\n";
        for (size_t q = 0; q < g.reds.size(); ++q) {
            const RedIR& rd = g.reds[q];
            std::string prod = rd.b.kind == ValRef::NONE
                                   ? "(ACC)" + val(rd.a, 0)
                                   : "(ACC)(" + val(rd.a, 0) + " * " + val(rd.b, 0) + ")";
            o << "    acc" << q << " += " << prod << ";\n";
        }
        o << "  }\n";
        red_epilogue();
        o << "}\n";
    }

    void scalar_only() {
        prologue();
        scalar_outs();
        o << "}\n";
    }
};

}  // namespace

int generate_source(const GroupIR& g, std::string* src, std::string* err) {
    Gen gen{g, {}, {}};
    switch (g.cls) {
        case GroupIR::SCALAR_ONLY: gen.scalar_only(); break;
        case GroupIR::SHIFTED:
            if (g.staged) gen.staged();
            else gen.shifted();
            break;
        case GroupIR::STRIDED: gen.strided(); break;
        default:
            if (err) *err = "unknown group class";
            return CN_ERR_UNSUPPORTED;
    }
    *src = gen.o.str();
    return CN_OK;
}

}  // namespace cn
