"""Serialiser for the CNB1 DAG blob consumed by ``cn_receive_dag``.

The reference ships its DAGs in charmtyles' own byte format, which is not part of the
reference tree; this container carries the same fields (DAGNode: id, identifier, fusible,
parents; ASTNode: result_name, opcode, is_temp, is_scalar, is_broadcast, dtype, ndims,
scalar, operands, operand_regions, region).  Regions are encoded exactly as
``ArrayRegion.serialize`` does (charmnumeric/charmnumeric.py:194-207).  Grammar (all
little-endian)::

    blob     := "CNB1" i32 epoch  i32 n_nodes  node*  i32 n_deletes  i32 name*
    node     := i32 id  i64 identifier  i32 fusible  i32 n_deps  i32 dep*  i32 n_roots  ast*
    ast      := i32 result_name  i32 opcode  i32 flags  i32 dtype  i32 ndims  f64 scalar
                i32 shape[ndims]  region  i32 n_operands  operand*
                flags: bit0 is_temp, bit1 is_scalar, bit2 is_broadcast
    operand  := i32 kind  (kind 0: ast | kind 1: i32 result_name)  region
    region   := i32 is_global  [ i32 ndims  (i32 start  i32 stop  i32 step) * ndims ]
"""
import struct

# opcode numbering: src/opcodes.hpp:3-20 == charmnumeric/charmnumeric.py:139-150
OP_COPY, OP_SET_REGION, OP_GET_REGION, OP_CREATE, OP_NOOP = -5, -4, -3, -2, -1
OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_MATMUL, OP_TANH, OP_EXP = 0, 1, 2, 3, 4, 5, 6
OP_TILE, OP_REDUCE, OP_MATMATMUL, OP_DIAG = 7, 8, 9, 10
# additions of this backend
OP_SQRT, OP_ABS, OP_SUM, OP_RANDU = 11, 12, 13, 14

# dtype codes: charmnumeric/charmnumeric.py:37-40
F32, F64, I32, I64 = 0, 1, 2, 3


class Region:
    """(start, stop, step) per dimension; ``None`` fields mean the whole array."""

    __slots__ = ("start", "stop", "step")

    def __init__(self, start, stop, step=None):
        self.start = tuple(int(v) for v in start)
        self.stop = tuple(int(v) for v in stop)
        self.step = tuple(int(v) for v in step) if step is not None else (1,) * len(self.start)

    def shape(self):
        return tuple((b - a + s - 1) // s if b > a else 0
                     for a, b, s in zip(self.start, self.stop, self.step))

    def __eq__(self, other):
        return (isinstance(other, Region) and self.start == other.start
                and self.stop == other.stop and self.step == other.step)

    def __hash__(self):
        return hash((self.start, self.stop, self.step))

    def __repr__(self):
        return f"Region({self.start}, {self.stop}, {self.step})"


def pack_region(region):
    if region is None:
        return struct.pack("<i", 1)
    out = [struct.pack("<ii", 0, len(region.start))]
    for a, b, s in zip(region.start, region.stop, region.step):
        out.append(struct.pack("<iii", a, b, s))
    return b"".join(out)


class Ast:
    """One AST node: a root of a group, or an inline NOOP leaf."""

    def __init__(self, result_name, opcode=OP_NOOP, *, is_temp=False, is_scalar=False,
                 is_broadcast=False, dtype=F64, shape=(), scalar=0.0, region=None, operands=()):
        self.result_name = int(result_name)
        self.opcode = int(opcode)
        self.is_temp = bool(is_temp)
        self.is_scalar = bool(is_scalar)
        self.is_broadcast = bool(is_broadcast)
        self.dtype = int(dtype)
        self.shape = tuple(int(v) for v in shape)
        self.scalar = float(scalar)
        self.region = region
        self.operands = list(operands)  # (Ast | Ref, Region | None)

    def pack(self):
        flags = (1 if self.is_temp else 0) | (2 if self.is_scalar else 0) | \
                (4 if self.is_broadcast else 0)
        out = [struct.pack("<iiiiid", self.result_name, self.opcode, flags, self.dtype,
                           len(self.shape), self.scalar)]
        out.append(struct.pack(f"<{len(self.shape)}i", *self.shape))
        out.append(pack_region(self.region))
        out.append(struct.pack("<i", len(self.operands)))
        for node, region in self.operands:
            if isinstance(node, Ref):
                out.append(struct.pack("<ii", 1, node.name))
            else:
                out.append(struct.pack("<i", 0))
                out.append(node.pack())
            out.append(pack_region(region))
        return b"".join(out)


class Ref:
    """Operand that names an earlier root of the same group."""

    __slots__ = ("name",)

    def __init__(self, name):
        self.name = int(name)


def leaf(name, shape, dtype=F64):
    """Array leaf (NOOP)."""
    size = 1
    for v in shape:
        size *= v
    return Ast(name, OP_NOOP, shape=shape, dtype=dtype, is_broadcast=(size == 1))


def scalar(value, dtype=F64):
    """Literal scalar leaf."""
    return Ast(-1, OP_NOOP, is_scalar=True, scalar=value, dtype=dtype)


class Node:
    """One DAG node: a fusible group (flat list of roots) or a single non-fusible root."""

    def __init__(self, node_id, roots, *, fusible=True, deps=(), identifier=0):
        self.id = int(node_id)
        self.roots = list(roots)
        self.fusible = bool(fusible)
        self.deps = [int(d) for d in deps]
        self.identifier = int(identifier)

    def pack(self):
        out = [struct.pack("<iqii", self.id, self.identifier, 1 if self.fusible else 0,
                           len(self.deps))]
        out.append(struct.pack(f"<{len(self.deps)}i", *self.deps))
        out.append(struct.pack("<i", len(self.roots)))
        out.extend(r.pack() for r in self.roots)
        return b"".join(out)


def dag_blob(nodes, deletes=(), epoch=0):
    out = [b"CNB1", struct.pack("<ii", int(epoch), len(nodes))]
    out.extend(n.pack() for n in nodes)
    out.append(struct.pack("<i", len(deletes)))
    out.append(struct.pack(f"<{len(deletes)}i", *[int(d) for d in deletes]))
    return b"".join(out)
