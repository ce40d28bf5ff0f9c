// Region algebra of the slab planner: which rows of which operand a rank reads when a group
// iterates over views that are stepped or offset against each other, and which rows therefore
// have to move between ranks.
//
// Reference counterparts: ArrayRegion intersect / map (src/array_region.hpp:136-222, 461-536),
// local_inputs and send_remote_inputs (src/array_region.hpp:553-663), which do the same job
// per chare tile and per fragment.  Here every array is one slab per rank along dimension 0,
// so the algebra is one-dimensional: (start, stop, step) lattices of row indices.
#include <algorithm>

#include "regions.hpp"

namespace cn {

namespace {

int64_t ceil_div(int64_t a, int64_t b) {  // b > 0
    return a >= 0 ? (a + b - 1) / b : -((-a) / b);
}

}  // namespace

int64_t lattice_size(const Lattice& r) {
    if (r.stop <= r.start || r.step <= 0) return 0;
    return (r.stop - r.start + r.step - 1) / r.step;
}

// Points of `r` that lie in [lo, hi): again a lattice with r's step.
Lattice lattice_clip(const Lattice& r, int64_t lo, int64_t hi) {
    Lattice out = r;
    if (r.step <= 0) {
        out.stop = out.start;
        return out;
    }
    if (lo > out.start) out.start = r.start + ceil_div(lo - r.start, r.step) * r.step;
    out.stop = std::min(r.stop, hi);
    if (out.stop < out.start) out.stop = out.start;
    return out;
}

// Common points of two lattices (src/array_region.hpp:136-222 solves the same congruence per
// dimension): empty, or a lattice whose step is lcm(a.step, b.step).
Lattice lattice_intersect(const Lattice& a, const Lattice& b) {
    Lattice none{0, 0, 1};
    if (a.step <= 0 || b.step <= 0) return none;
    const int64_t lo = std::max(a.start, b.start), hi = std::min(a.stop, b.stop);
    if (hi <= lo) return none;
    int64_t g = a.step, h = b.step;
    while (h) {
        int64_t t = g % h;
        g = h;
        h = t;
    }
    if ((b.start - a.start) % g != 0) return none;
    const int64_t lcm = a.step / g * b.step;
    // first x >= lo with x = a.start (mod a.step) and x = b.start (mod b.step); the steps of
    // real programs are tiny, so walking a's lattice is as good as the extended Euclid
    int64_t x = a.start + ceil_div(lo - a.start, a.step) * a.step;
    for (int64_t k = 0; k < b.step / g && x < hi; ++k, x += a.step)
        if ((x - b.start) % b.step == 0) break;
    if (x >= hi || (x - b.start) % b.step != 0) return none;
    return Lattice{x, hi, lcm};
}

// `part` is a sub-lattice of `from`; the result is the lattice of the same positions in `to`
// (position k of `from` corresponds to position k of `to`; src/array_region.hpp:461-536).
Lattice lattice_map(const Lattice& part, const Lattice& from, const Lattice& to) {
    const int64_t first = (part.start - from.start) / from.step;
    const int64_t count = lattice_size(part);
    const int64_t stride = part.step / from.step;  // positions of `from` per step of `part`
    Lattice out;
    out.start = to.start + first * to.step;
    out.step = to.step * (stride > 0 ? stride : 1);
    out.stop = out.start + count * out.step;
    return out;
}

// Iteration rows [lo, hi) of a group that rank `rank` executes: those whose anchor row
// anchor.start + i * anchor.step lies in the rank's slab of the anchor array (n0 rows).
void iteration_rows(const Lattice& anchor, int64_t n0, int nranks, int rank, int64_t* lo, int64_t* hi) {
    int64_t b, e;
    slab_rows(n0, nranks, rank, &b, &e);
    const int64_t extent = lattice_size(anchor);
    int64_t i0 = b > anchor.start ? ceil_div(b - anchor.start, anchor.step) : 0;
    int64_t i1 = e > anchor.start ? ceil_div(e - anchor.start, anchor.step) : 0;
    i0 = std::min(i0, extent);
    i1 = std::min(i1, extent);
    if (i1 < i0) i1 = i0;
    *lo = i0;
    *hi = i1;
}

void slab_rows(int64_t n0, int nranks, int rank, int64_t* begin, int64_t* end) {
    const int64_t per = (n0 + nranks - 1) / nranks;
    *begin = std::min<int64_t>((int64_t)rank * per, n0);
    *end = std::min<int64_t>((int64_t)(rank + 1) * per, n0);
}

// Rows [lo, hi) of an operand (view `leaf` of an array with `leaf_n0` rows) that rank `rank`
// reads while it executes its iteration rows of the anchor: the bounding range of the rows
// leaf.start + i * leaf.step.  Empty (lo == hi) when the rank has no iteration rows.
void rows_read(const Lattice& anchor, int64_t anchor_n0, const Lattice& leaf, int nranks, int rank, int64_t* lo,
               int64_t* hi) {
    int64_t i0, i1;
    iteration_rows(anchor, anchor_n0, nranks, rank, &i0, &i1);
    if (i1 <= i0) {
        *lo = *hi = 0;
        return;
    }
    *lo = leaf.start + i0 * leaf.step;
    *hi = leaf.start + (i1 - 1) * leaf.step + 1;
}

// Every transfer of one operand: rows [lo, hi) go from rank `src` to rank `dst` (src != dst)
// wherever what `dst` reads overlaps what `src` owns.  All ranks compute the same list.
std::vector<RowTransfer> plan_transfers(const Lattice& anchor, int64_t anchor_n0, const Lattice& leaf, int64_t leaf_n0,
                                        int nranks) {
    std::vector<RowTransfer> out;
    for (int dst = 0; dst < nranks; ++dst) {
        int64_t lo, hi;
        rows_read(anchor, anchor_n0, leaf, nranks, dst, &lo, &hi);
        if (hi <= lo) continue;
        for (int src = 0; src < nranks; ++src) {
            if (src == dst) continue;
            int64_t b, e;
            slab_rows(leaf_n0, nranks, src, &b, &e);
            const int64_t t0 = std::max(lo, b), t1 = std::min(hi, e);
            if (t1 > t0) out.push_back(RowTransfer{src, dst, t0, t1});
        }
    }
    return out;
}

}  // namespace cn
