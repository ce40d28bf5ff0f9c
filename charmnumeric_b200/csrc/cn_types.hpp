// Host-side data model of the backend: opcodes, dtypes, regions, AST / DAG nodes and the
// wire format they arrive in.
//
// Opcode and dtype numbering is the reference protocol's (src/opcodes.hpp:3-20,
// charmnumeric/charmnumeric.py:37-40, 139-150); opcodes >= 11 are additions.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace cn {

enum Opcode : int {
    OP_COPY = -5,
    OP_SET_REGION = -4,
    OP_GET_REGION = -3,
    OP_CREATE = -2,
    OP_NOOP = -1,
    OP_ADD = 0,
    OP_SUB = 1,
    OP_MUL = 2,
    OP_DIV = 3,
    OP_MATMUL = 4,
    OP_TANH = 5,
    OP_EXP = 6,
    OP_TILE = 7,
    OP_REDUCE = 8,
    OP_MATMATMUL = 9,
    OP_DIAG = 10,
    // additions (absent from the reference protocol)
    OP_SQRT = 11,
    OP_ABS = 12,
    OP_SUM = 13,    // sum of all elements of one array -> size-1 array
    OP_RANDU = 14,  // seeded uniform fill: operands (seed, lo, hi) as literal scalars
};

inline bool is_binary_elementwise(int op) { return op >= OP_ADD && op <= OP_DIV; }
inline bool is_unary_elementwise(int op) {
    return op == OP_TANH || op == OP_EXP || op == OP_SQRT || op == OP_ABS;
}
inline bool is_elementwise(int op) { return is_binary_elementwise(op) || is_unary_elementwise(op); }

enum DType : int { DT_F32 = 0, DT_F64 = 1, DT_I32 = 2, DT_I64 = 3 };
inline int dtype_size(int dt) { return (dt == DT_F64 || dt == DT_I64) ? 8 : 4; }
inline bool dtype_valid(int dt) { return dt >= 0 && dt <= 3; }

// Status codes returned through the C ABI (the reference aborts the process instead).
enum Status : int {
    CN_OK = 0,
    CN_ERR_INVALID_ARGUMENT = 1,
    CN_ERR_BAD_BLOB = 2,
    CN_ERR_UNKNOWN_ARRAY = 3,
    CN_ERR_SHAPE_MISMATCH = 4,
    CN_ERR_UNSUPPORTED = 5,
    CN_ERR_BAD_OPCODE = 6,
    CN_ERR_BAD_DTYPE = 7,
    CN_ERR_CUDA = 8,
    CN_ERR_COMPILE = 9,
    CN_ERR_COMM = 10,
    CN_ERR_HAZARD = 11,
    CN_ERR_OUT_OF_MEMORY = 12,
    CN_ERR_LIMIT = 13,
    CN_ERR_RANK_FAILED = 14,
    CN_ERR_NO_DEVICE = 15,
};

constexpr int kMaxDims = 3;

// (start, stop, step) per dimension; `is_global` means "the whole array".
// Same meaning as ArrayRegion in the reference (charmnumeric/charmnumeric.py:153-207,
// src/array_region.hpp:22-134).
struct Region {
    bool is_global = true;
    int ndims = 0;
    int64_t start[kMaxDims] = {0, 0, 0};
    int64_t stop[kMaxDims] = {0, 0, 0};
    int64_t step[kMaxDims] = {1, 1, 1};

    int64_t extent(int d) const {
        if (stop[d] <= start[d]) return 0;
        return (stop[d] - start[d] + step[d] - 1) / step[d];
    }
    int64_t size() const {
        int64_t n = 1;
        for (int d = 0; d < ndims; ++d) n *= extent(d);
        return n;
    }
    static Region full(int nd, const int64_t* shape) {
        Region r;
        r.is_global = false;
        r.ndims = nd;
        for (int d = 0; d < nd; ++d) {
            r.start[d] = 0;
            r.stop[d] = shape[d];
            r.step[d] = 1;
        }
        return r;
    }
    bool unit_step() const {
        for (int d = 0; d < ndims; ++d)
            if (step[d] != 1) return false;
        return true;
    }
};

struct AstNode;

struct Operand {
    bool is_ref = false;             // true: refers to an earlier root of the same group
    int ref_name = -1;               // result_name of that root
    std::unique_ptr<AstNode> leaf;   // otherwise: an inline NOOP/CREATE leaf
    Region region;                   // operand region (global = whole array)
};

struct AstNode {
    int result_name = -1;
    int opcode = OP_NOOP;
    bool is_temp = false;
    bool is_scalar = false;
    bool is_broadcast = false;
    int dtype = DT_F64;
    int ndims = 0;
    double scalar = 0.0;
    int64_t shape[kMaxDims] = {0, 0, 0};
    Region region;                   // SET_REGION destination / CREATE shape
    std::vector<Operand> operands;
};

struct DagNode {
    int id = 0;
    int64_t identifier = 0;
    bool fusible = false;
    std::vector<int> deps;
    std::vector<std::unique_ptr<AstNode>> roots;
};

struct Dag {
    int epoch = 0;
    std::vector<DagNode> nodes;
    std::vector<int> deletes;        // arrays released after the DAG has run
};

// Parse a DAG blob ("CNB1" format; the grammar is written out at the top of wire.cpp).
// Returns CN_OK or CN_ERR_BAD_BLOB with a message.
int parse_dag(const char* msg, int64_t size, Dag* out, std::string* err);
// Parse a single serialized group (the `node` production) for cn_compile_group.
int parse_node(const char* msg, int64_t size, DagNode* out, std::string* err);

const char* status_string(int status);

}  // namespace cn
