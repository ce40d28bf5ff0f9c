// One-dimensional region algebra of the slab planner (see regions.cpp).
#pragma once
#include <cstdint>
#include <vector>

namespace cn {

struct Lattice {  // rows start, start + step, ... below stop
    int64_t start = 0, stop = 0, step = 1;
};

struct RowTransfer {
    int src = 0, dst = 0;
    int64_t lo = 0, hi = 0;  // global rows [lo, hi) of the operand array
};

int64_t lattice_size(const Lattice& r);
Lattice lattice_clip(const Lattice& r, int64_t lo, int64_t hi);
Lattice lattice_intersect(const Lattice& a, const Lattice& b);
Lattice lattice_map(const Lattice& part, const Lattice& from, const Lattice& to);
void slab_rows(int64_t n0, int nranks, int rank, int64_t* begin, int64_t* end);
void iteration_rows(const Lattice& anchor, int64_t n0, int nranks, int rank, int64_t* lo, int64_t* hi);
void rows_read(const Lattice& anchor, int64_t anchor_n0, const Lattice& leaf, int nranks, int rank, int64_t* lo,
               int64_t* hi);
std::vector<RowTransfer> plan_transfers(const Lattice& anchor, int64_t anchor_n0, const Lattice& leaf, int64_t leaf_n0,
                                        int nranks);

}  // namespace cn
