// "CNB1" DAG blob reader.
//
// The reference receives its DAGs through charmtyles' DAG::deserialize
// (src/dag_group_receive.cpp:192), whose byte format is not part of the reference tree.
// This backend therefore defines its own container for the same fields
// (DAGNode: id, identifier, fusible, parents; ASTNode: result_name, opcode, is_temp,
// is_scalar, is_broadcast, dtype, ndims, scalar, operands, operand_regions, region).
// Regions use the reference's own encoding (ArrayRegion.serialize,
// charmnumeric/charmnumeric.py:194-207).  All integers little-endian.
//
//   blob     := "CNB1" i32 epoch  i32 n_nodes  node*  i32 n_deletes  i32 name*
//   node     := i32 id  i64 identifier  i32 fusible  i32 n_deps  i32 dep*  i32 n_roots  ast*
//   ast      := i32 result_name  i32 opcode  i32 flags  i32 dtype  i32 ndims  f64 scalar
//               i32 shape[ndims]  region  i32 n_operands  operand*
//               flags: bit0 is_temp, bit1 is_scalar, bit2 is_broadcast
//   operand  := i32 kind  (kind 0: ast (inline leaf) | kind 1: i32 result_name)  region
//   region   := i32 is_global  [ i32 ndims  (i32 start  i32 stop  i32 step) * ndims ]
#include <cstring>

#include "cn_types.hpp"

namespace cn {

namespace {

struct Reader {
    const char* p;
    const char* end;
    std::string* err;
    bool ok = true;

    bool need(size_t n) {
        if (!ok) return false;
        if ((size_t)(end - p) < n) {
            ok = false;
            if (err) *err = "DAG blob truncated";
            return false;
        }
        return true;
    }
    int32_t i32() {
        int32_t v = 0;
        if (need(4)) {
            memcpy(&v, p, 4);
            p += 4;
        }
        return v;
    }
    int64_t i64() {
        int64_t v = 0;
        if (need(8)) {
            memcpy(&v, p, 8);
            p += 8;
        }
        return v;
    }
    double f64() {
        double v = 0;
        if (need(8)) {
            memcpy(&v, p, 8);
            p += 8;
        }
        return v;
    }
    void fail(const std::string& m) {
        if (ok && err) *err = m;
        ok = false;
    }
    // A count read from the blob can never exceed what the bytes that are left could hold:
    // checked before anything is sized by it, so a few bytes cannot ask for gigabytes.
    bool fits(int64_t count, size_t min_bytes_each) const {
        return count >= 0 && (uint64_t)count <= (uint64_t)(end - p) / min_bytes_each;
    }
};

void read_region(Reader& r, Region* out) {
    int g = r.i32();
    out->is_global = (g != 0);
    out->ndims = 0;
    if (out->is_global) return;
    int nd = r.i32();
    if (nd < 1 || nd > kMaxDims) {
        r.fail("region rank out of range");
        return;
    }
    out->ndims = nd;
    for (int d = 0; d < nd; ++d) {
        out->start[d] = r.i32();
        out->stop[d] = r.i32();
        out->step[d] = r.i32();
        if (r.ok && out->step[d] <= 0) r.fail("region step must be positive");
        if (r.ok && out->start[d] < 0) r.fail("region start must be non-negative");
    }
}

std::unique_ptr<AstNode> read_ast(Reader& r, int depth) {
    auto n = std::make_unique<AstNode>();
    if (depth > 4) {
        r.fail("AST nesting too deep");
        return n;
    }
    n->result_name = r.i32();
    n->opcode = r.i32();
    int flags = r.i32();
    n->is_temp = flags & 1;
    n->is_scalar = flags & 2;
    n->is_broadcast = flags & 4;
    n->dtype = r.i32();
    n->ndims = r.i32();
    n->scalar = r.f64();
    if (!r.ok) return n;
    if (n->ndims < 0 || n->ndims > kMaxDims) {
        r.fail("array rank out of range (1..3 supported)");
        return n;
    }
    for (int d = 0; d < n->ndims; ++d) {
        n->shape[d] = r.i32();
        if (r.ok && n->shape[d] < 0) r.fail("negative extent");
    }
    read_region(r, &n->region);
    int nops = r.i32();
    if (!r.ok) return n;
    if (nops < 0 || nops > 8) {
        r.fail("operand count out of range");
        return n;
    }
    n->operands.resize(nops);
    for (int i = 0; i < nops && r.ok; ++i) {
        Operand& o = n->operands[i];
        int kind = r.i32();
        if (kind == 0) {
            o.is_ref = false;
            o.leaf = read_ast(r, depth + 1);
        } else if (kind == 1) {
            o.is_ref = true;
            o.ref_name = r.i32();
        } else {
            r.fail("bad operand kind");
        }
        read_region(r, &o.region);
    }
    return n;
}

void read_node(Reader& r, DagNode* node) {
    node->id = r.i32();
    node->identifier = r.i64();
    node->fusible = r.i32() != 0;
    int ndeps = r.i32();
    if (!r.ok) return;
    if (ndeps < 0 || ndeps > 1 << 20 || !r.fits(ndeps, 4)) {
        r.fail("dependency count out of range");
        return;
    }
    node->deps.resize(ndeps);
    for (int i = 0; i < ndeps; ++i) node->deps[i] = r.i32();
    int nroots = r.i32();
    if (!r.ok) return;
    if (nroots < 0 || nroots > 4096 || !r.fits(nroots, 36)) {  // an ast is at least 36 bytes
        r.fail("root count out of range");
        return;
    }
    for (int i = 0; i < nroots && r.ok; ++i) node->roots.push_back(read_ast(r, 0));
}

}  // namespace

int parse_dag(const char* msg, int64_t size, Dag* out, std::string* err) {
    if (!msg || size < 16) {
        if (err) *err = "DAG blob too short";
        return CN_ERR_BAD_BLOB;
    }
    if (memcmp(msg, "CNB1", 4) != 0) {
        if (err) *err = "DAG blob has no CNB1 magic";
        return CN_ERR_BAD_BLOB;
    }
    Reader r{msg + 4, msg + size, err};
    out->epoch = r.i32();
    int n = r.i32();
    if (r.ok && (n < 0 || n > 1 << 22 || !r.fits(n, 24))) r.fail("node count out of range");  // a node is at least 24 bytes
    if (r.ok) out->nodes.resize(n);
    for (int i = 0; i < n && r.ok; ++i) read_node(r, &out->nodes[i]);
    int nd = r.i32();
    if (r.ok && (nd < 0 || nd > 1 << 24 || !r.fits(nd, 4))) r.fail("delete count out of range");
    for (int i = 0; i < nd && r.ok; ++i) out->deletes.push_back(r.i32());
    if (r.ok && r.p != r.end) r.fail("trailing bytes after DAG blob");
    return r.ok ? CN_OK : CN_ERR_BAD_BLOB;
}

int parse_node(const char* msg, int64_t size, DagNode* out, std::string* err) {
    if (!msg || size < 24) {
        if (err) *err = "group blob too short";
        return CN_ERR_BAD_BLOB;
    }
    Reader r{msg, msg + size, err};
    read_node(r, out);
    if (r.ok && r.p != r.end) r.fail("trailing bytes after group blob");
    return r.ok ? CN_OK : CN_ERR_BAD_BLOB;
}

const char* status_string(int s) {
    switch (s) {
        case CN_OK: return "ok";
        case CN_ERR_INVALID_ARGUMENT: return "invalid argument";
        case CN_ERR_BAD_BLOB: return "malformed DAG blob";
        case CN_ERR_UNKNOWN_ARRAY: return "unknown array name";
        case CN_ERR_SHAPE_MISMATCH: return "shape mismatch";
        case CN_ERR_UNSUPPORTED: return "unsupported operation";
        case CN_ERR_BAD_OPCODE: return "bad opcode";
        case CN_ERR_BAD_DTYPE: return "bad dtype";
        case CN_ERR_CUDA: return "CUDA error";
        case CN_ERR_COMPILE: return "kernel compilation failed";
        case CN_ERR_COMM: return "communication error";
        case CN_ERR_HAZARD: return "read/write hazard inside a fused group";
        case CN_ERR_OUT_OF_MEMORY: return "out of device memory";
        case CN_ERR_LIMIT: return "group exceeds a compiled-in limit";
        case CN_ERR_RANK_FAILED: return "a rank was marked failed";
        case CN_ERR_NO_DEVICE: return "no CUDA device";
        default: return "unknown status";
    }
}

}  // namespace cn
