// Intermediate form of one fused DAG group, between the AST that arrives over the wire
// and the CUDA source handed to NVRTC.
//
// The reference lowers each fusible DAG node to one `fused_kernel` whose arguments are a
// strided memref per (array, operand region) use, one by-value scalar per size-1 array and
// one memref per non-temp root (src/jit.cpp:28-158, 223-263).  Here the same information is
// kept, plus what the slab executor needs: per-leaf offsets relative to the output, which
// outputs alias inputs, and which reductions were fused behind the group.
#pragma once
#include <string>
#include <vector>

#include "cn_types.hpp"

namespace cn {

struct ValRef {
    enum Kind { NONE, LEAF, CONST, BCAST, ROOT, OUTVAL } kind = NONE;
    int idx = -1;
};

enum Domain { DOM_SCALAR = 0, DOM_REGION = 1, DOM_BOX = 2 };

struct LeafIR {
    int name = -1;
    int ndims = 0;
    int64_t shape[kMaxDims] = {0, 0, 0};  // global shape of the array read
    Region region;                        // explicit (never global)
    int64_t delta[kMaxDims] = {0, 0, 0};  // shifted class: region.start - origin of its user
    int domain = DOM_REGION;              // guard under which the load is issued
};

struct RootIR {
    int opcode = OP_NOOP;
    ValRef a, b;
    int result_name = -1;
    bool is_temp = true;
    int domain = DOM_REGION;
    int64_t shape[kMaxDims] = {0, 0, 0};
    int64_t origin[kMaxDims] = {0, 0, 0};
    bool origin_set = false;
};

struct OutIR {
    int name = -1;
    bool is_set = false;                  // SET_REGION into an existing array vs new array
    int ndims = 0;
    int64_t shape[kMaxDims] = {0, 0, 0};  // global shape of the array written
    Region region;                        // explicit destination region
    ValRef value;
    int domain = DOM_REGION;
    bool hazard = false;                  // some leaf reads this array at a different index
    bool needs_old = false;               // old contents are read (copy-through / forwarding)
    int root_index = -1;                  // root that defines the output
};

struct ScalarOutIR {
    int name = -1;
    ValRef value;
    bool is_set = false;
};

struct RedIR {
    ValRef a, b;  // b.kind == NONE for SUM
    int result_name = -1;
    int domain = DOM_BOX;
};

struct GroupIR {
    enum Class { SCALAR_ONLY, SHIFTED, STRIDED } cls = SCALAR_ONLY;
    int dtype = DT_F64;
    int ndims = 0;
    int64_t array_shape[kMaxDims] = {0, 0, 0};  // SHIFTED: common shape of every array touched
    int64_t box_lo[kMaxDims] = {0, 0, 0}, box_hi[kMaxDims] = {0, 0, 0};  // global frame coords
    int64_t reg_lo[kMaxDims] = {0, 0, 0}, reg_hi[kMaxDims] = {0, 0, 0};
    int64_t extent[kMaxDims] = {0, 0, 0};       // STRIDED: iteration extents
    bool two_domains = false;   // region box is a strict subset of the iteration box
    bool copy_through = false;  // hazard outputs are written out of place over the whole array
    bool flat = false;          // SHIFTED with zero deltas over whole arrays: 1-D walk
    int vec = 1;                // elements per thread along the last dimension
    int max_halo = 0;           // SHIFTED: largest |delta| along dimension 0
    // Staged variant (2-D / 3-D float64 stencils): the one array that is read at shifted
    // positions is fetched tile by tile into shared memory by the TMA unit.
    bool staged = false;
    int stage_array = -1;       // name of that array
    int hy = 0, hz = 0;         // halo rows / planes a tile carries on each side

    // Staged producer: the stage array is a stand-in that exists nowhere; the kernel computes
    // its tiles (halo included) in shared memory by evaluating this flat group, whose single
    // output is the array the stand-in takes the place of (`producer_target`), at every point
    // of the tile.  Empty, or exactly one element.
    std::vector<GroupIR> producer;
    int producer_target = -1;

    // Scalar tail: a SCALAR_ONLY group (size-1 arrays in, size-1 arrays out) that directly
    // follows a group with fused reductions and is evaluated by the thread that has just
    // written the reduction results, instead of by a kernel of its own (CG's
    // beta = r.r / rtr, rtr = r.r; a Jacobi sweep's res = sum).  Its literal scalars,
    // size-1 operands and results take the slots behind the group's (and its producer's)
    // own.  Empty, or exactly one element.
    std::vector<GroupIR> tail;

    std::vector<LeafIR> leaves;
    std::vector<double> scalars;
    std::vector<int> bcast_names;
    std::vector<RootIR> roots;
    std::vector<OutIR> outs;
    std::vector<ScalarOutIR> souts;
    std::vector<RedIR> reds;

    // Structural key: equal keys <=> identical generated source.
    std::string key() const;
    // Name of the kernel entry point: class, rank and operand counts in clear plus a hash of
    // the key, so that a profiler's kernel filter can pick one group kernel.
    std::string entry_name() const;
    // SHIFTED class: distinct input arrays in order of first use; slot i of the launch
    // arguments' `in[]` is array input_arrays()[i].  STRIDED class: one slot per leaf.
    std::vector<int> input_arrays() const;
};

// Lower one fusible DAG node (plus REDUCE / SUM roots fused behind it) to GroupIR.
// `fused` lists extra REDUCE/SUM roots taken from following DAG nodes.
// `force_strided` skips the shifted-class analysis (used by the raw kernel-ABI entry point,
// whose caller supplies explicit strided views).
int lower_group(const DagNode& node, const std::vector<const AstNode*>& fused, GroupIR* out,
                std::string* err, bool force_strided = false);

// Producer inlining (fuse.cpp): when node `a` assigns a whole array from an elementwise
// expression of whole arrays and node `b`, right behind it, reads that array through shifted
// views, build in `out` one node that does the work of both without the round trip of the
// array through memory.  False when the pair does not fit.
bool inline_producer(const DagNode& a, const DagNode& b, DagNode* out);

// The staged form of the same pair: `consumer` / `producer` / the stand-in's name as built by
// stage_producer; lower_staged_producer lowers both and joins them into one GroupIR (2-D
// float64 groups only; CN_ERR_UNSUPPORTED when the pair does not fit the staged kernel).
bool stage_producer(const DagNode& a, const DagNode& b, DagNode* consumer, DagNode* producer, int* pseudo_name,
                    int* target_name);
int lower_staged_producer(const DagNode& consumer, const DagNode& producer, int pseudo_name, int target_name,
                          const std::vector<const AstNode*>& fused, GroupIR* out, std::string* err);

// Shared-memory / TMA staging of stencil groups.  Level 0: never; 1 (default): 3-D groups
// only; 2: 2-D groups too.  Set with CN_STAGED or cn_set_option(ctx, "staged", level).
void set_staged_level(int level);
int staged_level();

// Emit the CUDA source of the group kernel (entry point g.entry_name()).
int generate_source(const GroupIR& g, std::string* src, std::string* err);

}  // namespace cn
