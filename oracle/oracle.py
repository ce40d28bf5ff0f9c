"""CPU oracle, Python side.  TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check
and by the CPU-baseline leg of the benchmark, never by the product package.

Two parts:

* ``Oracle`` interprets the very DAG node objects that get serialised for the GPU
  (``charmnumeric_b200.wire.Node`` / ``Ast``) with the reference's semantics, one numpy
  operation per root so that every op is one separately rounded IEEE operation in
  (lhs, rhs) order (src/jit.cpp:296-385, 411-459); roots run in flat list order
  (src/jit.cpp:119-120); SET_REGION evaluates its right-hand side completely before the
  copy into the target (src/execute_node.cpp:1581-1584), so in-place stencils are true
  Jacobi steps; arrays start as zeros (src/backend.hpp:141-143); dot is a plain sum of
  products per tile, tiles added in order (src/backend_internal.hpp:88-93,
  src/executor_reducer.cpp:18-55); matvec is a per-tile gemv with partials accumulated
  tile by tile (src/backend_internal.hpp:15-41, src/execute_node.cpp:572-576).
* ``clib`` is the C restatement (cn_oracle.c): exp / tanh, the seeded generator, and the
  threaded workload loops used as the CPU baseline.

Pinning status is stated in the header of cn_oracle.c.
"""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = _HERE / "libcn_oracle.so"

OP_COPY, OP_SET_REGION, OP_CREATE, OP_NOOP = -5, -4, -2, -1
OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_MATMUL, OP_TANH, OP_EXP, OP_REDUCE = 0, 1, 2, 3, 4, 5, 6, 8
OP_TILE, OP_DIAG = 7, 10
OP_SQRT, OP_ABS, OP_SUM, OP_RANDU = 11, 12, 13, 14
NP_DTYPES = {0: np.dtype("float32"), 1: np.dtype("float64"), 2: np.dtype("int32"),
             3: np.dtype("int64")}


def build(force=False):
    """Compile cn_oracle.c with the committed Makefile (idempotent)."""
    src = _HERE / "cn_oracle.c"
    if force or not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)] + (["-B"] if force else []), check=True,
                       capture_output=True)
    return _LIB


_clib = None


def clib():
    global _clib
    if _clib is None:
        if not _LIB.exists():
            build()
        lib = C.CDLL(str(_LIB))
        d, i64, p = C.c_double, C.c_int64, C.c_void_p
        lib.cno_exp.restype = d
        lib.cno_exp.argtypes = [d]
        lib.cno_tanh.restype = d
        lib.cno_tanh.argtypes = [d]
        lib.cno_exp_v.argtypes = [p, p, i64]
        lib.cno_tanh_v.argtypes = [p, p, i64]
        lib.cno_randu.argtypes = [p, i64, C.c_uint64, C.c_uint64, d, d]
        lib.cno_tile.restype = i64
        lib.cno_tile.argtypes = [i64, C.c_int, C.c_int]
        lib.cno_dot.restype = d
        lib.cno_dot.argtypes = [p, p, i64, i64]
        lib.cno_gemv.argtypes = [p, i64, p, p, i64, i64, i64]
        lib.cno_set_threads.argtypes = [C.c_int]
        lib.cno_jacobi2d.argtypes = [p, p, i64, i64, d, C.c_int, C.c_int, p, i64]
        lib.cno_jacobi3d.argtypes = [p, p, i64, i64, i64, d, C.c_int, C.c_int, p, i64]
        lib.cno_chain_value.restype = d
        lib.cno_chain_value.argtypes = [d, d]
        lib.cno_chain_v.argtypes = [p, p, p, i64]
        lib.cno_chain_sum.restype = d
        lib.cno_chain_sum.argtypes = [p, p, i64, i64]
        lib.cno_cg_poisson.argtypes = [p, p, p, p, p, i64, C.c_int, p, i64]
        lib.cno_power_iteration.argtypes = [p, p, p, i64, C.c_int, p, i64]
        lib.cno_cg_poisson_tiled.argtypes = [p, p, i64, C.c_int, p, i64, C.c_int, p]
        lib.cno_jacobi2d_tiled.argtypes = [p, i64, d, C.c_int, C.c_int, p, i64, C.c_int, p]
        _clib = lib
    return _clib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def exp(x):
    x = np.ascontiguousarray(x, dtype=np.float64)
    y = np.empty_like(x)
    clib().cno_exp_v(_ptr(x), _ptr(y), x.size)
    return y


def tanh(x):
    x = np.ascontiguousarray(x, dtype=np.float64)
    y = np.empty_like(x)
    clib().cno_tanh_v(_ptr(x), _ptr(y), x.size)
    return y


def randu(shape, seed, lo=0.0, hi=1.0, dtype=np.float64, offset=0):
    n = int(np.prod(shape))
    out = np.empty(n, dtype=np.float64)
    clib().cno_randu(_ptr(out), n, int(offset), int(seed), float(lo), float(hi))
    return out.reshape(shape).astype(dtype, copy=False)


def ref_tile(extent, ndims, max_tiles=16):
    """Tile edge the reference's CPU build would choose (odf 4 x 4 PEs -> 16 tiles)."""
    return int(clib().cno_tile(int(extent), int(ndims), int(max_tiles)))


def dot(a, b, tile=None):
    a = np.ascontiguousarray(a, dtype=np.float64).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float64).reshape(-1)
    if tile is None:
        tile = 262144
    return float(clib().cno_dot(_ptr(a), _ptr(b), a.size, int(tile)))


def gemv(A, x, tile=None):
    A = np.ascontiguousarray(A, dtype=np.float64)
    x = np.ascontiguousarray(x, dtype=np.float64)
    y = np.empty(A.shape[0], dtype=np.float64)
    if tile is None:
        tile = 512
    clib().cno_gemv(_ptr(A), A.shape[1], _ptr(x), _ptr(y), A.shape[0], A.shape[1], int(tile))
    return y


def _slices(region, shape):
    if region is None:
        return tuple(slice(0, n, 1) for n in shape)
    return tuple(slice(a, b, s) for a, b, s in zip(region.start, region.stop, region.step))


def _store_scalar(s, dtype):
    """A reduction result as a size-1 array of the group's element type.  Integer sums are
    accumulated in 64 bits and then converted like a C cast (two's-complement wrap), which is what
    the kernels' `(T)total` does."""
    if np.dtype(dtype).kind == "i":
        return np.array([int(s)], dtype=np.int64).astype(dtype)
    return np.array([s], dtype=dtype)


class Oracle:
    """Interpreter of DAG nodes over numpy arrays (name -> ndarray)."""

    def __init__(self):
        self.arrays = {}

    # -- helpers --
    def _leaf_value(self, ast, region, dtype):
        if ast.is_scalar:
            return dtype.type(ast.scalar)
        arr = self.arrays[ast.result_name]
        if tuple(arr.shape) != tuple(ast.shape):
            raise ValueError(f"leaf {ast.result_name}: shape {ast.shape} != stored {arr.shape}")
        if arr.size == 1 and region is None:
            return arr.reshape(-1)[0]
        return arr[_slices(region, arr.shape)]

    def _operand(self, operand, values, dtype):
        node, region = operand
        if hasattr(node, "name") and not hasattr(node, "opcode"):  # wire.Ref
            return values[node.name]
        if node.result_name in values and not node.is_scalar:
            # an array assigned earlier in this group is read back from the table
            pass
        return self._leaf_value(node, region, dtype)

    @staticmethod
    def _group_dtype(roots):
        for r in roots:
            if r.dtype != 0:
                return NP_DTYPES[r.dtype]
        return NP_DTYPES[0]

    def _apply(self, opcode, a, b, dtype):
        is_int = dtype.kind == "i"
        with np.errstate(all="ignore"):
            if opcode == OP_ADD:
                return np.add(a, b, dtype=dtype)
            if opcode == OP_SUB:
                return np.subtract(a, b, dtype=dtype)
            if opcode == OP_MUL:
                return np.multiply(a, b, dtype=dtype)
            if opcode == OP_DIV:
                if is_int:  # arith.divsi: truncation toward zero (src/jit.cpp:438-440)
                    q = np.trunc(np.asarray(a, dtype=np.float64) / np.asarray(b, dtype=np.float64))
                    return q.astype(dtype)
                return np.divide(a, b, dtype=dtype)
            if opcode == OP_EXP:
                return exp(np.asarray(a, dtype=np.float64)).astype(dtype).reshape(np.shape(a))
            if opcode == OP_TANH:
                return tanh(np.asarray(a, dtype=np.float64)).astype(dtype).reshape(np.shape(a))
            if opcode == OP_SQRT:
                return np.sqrt(a, dtype=dtype)
            if opcode == OP_ABS:
                return np.abs(a).astype(dtype)
        raise ValueError(f"opcode {opcode} is not elementwise")

    # -- nodes --
    def run(self, nodes, deletes=()):
        for node in nodes:
            self.run_node(node)
        for name in deletes:
            self.arrays.pop(name, None)

    def run_node(self, node):
        roots = node.roots
        dtype = self._group_dtype(roots)
        values = {}
        for r in roots:
            op = r.opcode
            if op == OP_NOOP:
                continue
            if op == OP_CREATE:
                self.arrays[r.result_name] = np.zeros(r.shape, dtype=NP_DTYPES[r.dtype])
            elif op in (OP_ADD, OP_SUB, OP_MUL, OP_DIV):
                a = self._operand(r.operands[0], values, dtype)
                b = self._operand(r.operands[1], values, dtype)
                v = self._apply(op, a, b, dtype)
                values[r.result_name] = v
                if not r.is_temp:
                    self.arrays[r.result_name] = np.array(v, dtype=dtype).reshape(r.shape)
            elif op in (OP_EXP, OP_TANH, OP_SQRT, OP_ABS):
                a = self._operand(r.operands[0], values, dtype)
                v = self._apply(op, a, None, dtype)
                values[r.result_name] = v
                if not r.is_temp:
                    self.arrays[r.result_name] = np.array(v, dtype=dtype).reshape(r.shape)
            elif op in (OP_SET_REGION, OP_COPY):
                target = self.arrays[r.operands[0][0].result_name]
                rhs = self._operand(r.operands[1], values, dtype)
                rhs = np.array(rhs, dtype=target.dtype, copy=True)  # result buffer first
                if target.size == 1 and r.region is None:
                    target.reshape(-1)[0] = rhs.reshape(-1)[0]
                else:
                    dest = target[_slices(r.region, target.shape)]
                    if rhs.shape != dest.shape and rhs.size == dest.size and rhs.size > 1:
                        # cross-dimension assignment (src/executor_transfer.cpp:66-177): the same
                        # elements in the same order, singleton dimensions placed differently
                        rhs = rhs.reshape(dest.shape)
                    target[_slices(r.region, target.shape)] = rhs
            elif op == OP_REDUCE:
                a = self._operand(r.operands[0], values, dtype)
                b = self._operand(r.operands[1], values, dtype)
                if dtype.kind == "f":
                    s = dot(a, b, ref_tile(np.size(a), 1)) if dtype == np.float64 else \
                        np.dot(np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel())
                else:
                    s = np.sum(np.asarray(a, np.int64) * np.asarray(b, np.int64))
                self.arrays[r.result_name] = _store_scalar(s, dtype)
            elif op == OP_SUM:
                a = self._operand(r.operands[0], values, dtype)
                if dtype.kind == "f":
                    s = dot(a, np.ones(np.size(a)), ref_tile(np.size(a), 1))
                else:
                    s = np.sum(np.asarray(a, np.int64))
                self.arrays[r.result_name] = _store_scalar(s, dtype)
            elif op == OP_MATMUL:
                A = self.arrays[r.operands[0][0].result_name]
                A = A[_slices(r.operands[0][1], A.shape)]
                x = self.arrays[r.operands[1][0].result_name]
                x = x[_slices(r.operands[1][1], x.shape)]
                column = x.ndim == 2  # (n, 1) column vector: same values, result (m, 1)
                x = np.ascontiguousarray(x).reshape(-1)
                if dtype == np.float64:
                    y = gemv(A, x, ref_tile(A.shape[1], 2))
                else:
                    y = (np.asarray(A) @ np.asarray(x)).astype(dtype)
                y = y.astype(dtype)
                self.arrays[r.result_name] = y.reshape(-1, 1) if column else y
            elif op == OP_TILE:
                # charmnumeric/operations.py:52-72: numpy.tile with the padded repeat counts
                v = self.arrays[r.operands[0][0].result_name]
                reps = tuple(int(o[0].scalar) for o in r.operands[1:])
                self.arrays[r.result_name] = np.ascontiguousarray(np.tile(v, reps)).astype(dtype)
            elif op == OP_DIAG:
                # src/execute_node.cpp:600-750: vector -> diagonal matrix, matrix -> k-th diagonal
                v = self.arrays[r.operands[0][0].result_name]
                k = int(r.operands[1][0].scalar)
                self.arrays[r.result_name] = np.ascontiguousarray(np.diag(v, k)).astype(dtype)
            elif op == OP_RANDU:
                seed, lo, hi = (o[0].scalar for o in r.operands)
                self.arrays[r.result_name] = randu(r.shape, int(seed), lo, hi, NP_DTYPES[r.dtype])
            else:
                raise ValueError(f"oracle: opcode {op} not covered")

    def put(self, name, host):
        self.arrays[name] = np.array(host, copy=True)

    def get(self, name):
        return self.arrays[name]
