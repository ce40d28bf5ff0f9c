"""Lazy ndarray frontend: the same user-facing API as the reference's Python package
(``charmnumeric/charmnumeric.py``, ``charmnumeric/operations.py``), producing the same opcode
stream, executed by the B200 backend through the C ABI.

The reference frontend sits on charmtyles' ``FrontendObject`` / ``fusible_op`` /
``nonfusible_op`` / ``execute`` machinery, which is not part of the reference tree; the
small amount of it that the array API needs is restated here:

* every operator records one op and returns a new lazy ``Array`` (charmnumeric.py:394-489);
* ``a @ b`` on two vectors is a non-fusible REDUCE, matrix @ vector a non-fusible MATMUL
  (charmnumeric.py:492-576);
* ``x[key] = rhs`` records SET_REGION (charmnumeric.py:708-711);
* nothing runs until ``execute(interface)`` / ``Array.get(interface)`` / the auto-flush
  threshold (charmnumeric.py:683-688, examples/jacobi2d.py:6);
* consecutive fusible ops are grouped into one DAG node with a flat root list; results
  whose Python object is already gone and that are only used inside their group become
  temporaries of the fused kernel.
"""
import numbers
import weakref

import numpy as np

from . import wire
from .context import NP_DTYPES, WIRE_DTYPES, Context
from .wire import Region

_DEFAULT_DTYPE = np.dtype("float64")


class ArrayOperation:
    """Opcode values of the wire protocol (charmnumeric.py:139-150) plus additions."""
    add, sub, mul, div, matmul, tanh, exp, tile, reduce, matmatmul, diag = range(11)
    sqrt, abs, sum, randu = 11, 12, 13, 14


class DType:
    """Element type encoding shared with the wire protocol (charmnumeric.py:34-75)."""
    FLOAT32, FLOAT64, INT32, INT64 = 0, 1, 2, 3

    @staticmethod
    def from_numpy(dt):
        return WIRE_DTYPES[_normalize_dtype(dt)]

    @staticmethod
    def to_numpy(code):
        if code not in NP_DTYPES:
            raise TypeError(f"Unsupported wire dtype {code!r}")
        return NP_DTYPES[code]

    @staticmethod
    def promote(a, b):
        """Promoted wire dtype of two wire dtypes (charmnumeric.py:71-75)."""
        return DType.from_numpy(np.result_type(DType.to_numpy(a), DType.to_numpy(b)))


class _CallableInt(int):
    """An int that can also be called: the reference keeps ``obj.size()`` working next to
    ``obj.size`` (charmnumeric.py:24-31)."""

    def __new__(cls, value):
        return int.__new__(cls, int(value))

    def __call__(self):
        return int(self)


def _normalize_dtype(dtype):
    if dtype is None:
        return _DEFAULT_DTYPE
    dt = np.dtype(dtype)
    if dt not in WIRE_DTYPES:
        raise TypeError("charmnumeric only supports float32, float64, int32, and int64; "
                        f"got {dt}")
    return dt


def _normalize_shape(shape):
    if isinstance(shape, numbers.Integral):
        shape = (int(shape),)
    shape = tuple(int(d) for d in shape)
    for d in shape:
        if d < 0:
            raise ValueError(f"negative dimensions are not allowed: {shape}")
    if not 1 <= len(shape) <= 3:
        raise NotImplementedError("charmnumeric arrays have 1 to 3 dimensions")
    return shape


def _is_scalar_like(v):
    if isinstance(v, np.ndarray):
        return v.ndim == 0
    return isinstance(v, (bool, numbers.Real, np.generic))


def _coerce_scalar(v):
    if isinstance(v, (np.ndarray, np.generic)):
        v = v.item()
    if isinstance(v, bool):
        return int(v)
    if isinstance(v, numbers.Integral):
        return int(v)
    return float(v)


def _size(shape):
    n = 1
    for d in shape:
        n *= d
    return n


# ---- recording state ----------------------------------------------------------------------

class _Info:
    """Identity of one backend array; op records keep these, never the user objects."""
    __slots__ = ("name", "shape", "dtype", "alive", "materialised", "__weakref__")

    def __init__(self, name, shape, dtype):
        self.name = name
        self.shape = shape
        self.dtype = dtype
        self.alive = True          # a user-facing Array / ArrayView still refers to it
        self.materialised = False  # exists in the backend's array table


class _Op:
    __slots__ = ("kind", "opcode", "result", "operands", "region", "payload")

    def __init__(self, kind, opcode=None, result=None, operands=(), region=None, payload=None):
        self.kind = kind          # "ew", "set", "xset" (cross-dimension assignment), "create", "reduce", "sum", "matmul", "diag", "tile", "randu", "put"
        self.opcode = opcode
        self.result = result      # _Info
        self.operands = list(operands)  # (_Info, Region | None) or python scalar
        self.region = region      # destination region of "set"
        self.payload = payload


class _State:
    def __init__(self):
        self.reset()

    def reset(self):
        self.pending = []
        self.next_node = 0
        self.auto_flush = None    # (interface, threshold)
        # Names keep counting up across resets and the list of dead arrays is kept: arrays of
        # an earlier program may still live in a backend context and be released later, and a
        # late release must never hit a new array that happens to reuse the name.
        if not hasattr(self, "next_name"):
            self.next_name = 1
            self.dead = []        # names of materialised arrays whose user object is gone

    def new_name(self):
        n = self.next_name
        self.next_name += 1
        return n


_state = _State()


def reset_frontend_state():
    """Forget every pending op (the test fixtures call this); array names stay unique."""
    _state.reset()


def set_auto_flush(interface, threshold):
    """Execute automatically once ``threshold`` ops are pending (examples/jacobi2d.py:6)."""
    _state.auto_flush = (interface, int(threshold))


def _record(op):
    _state.pending.append(op)
    if _state.auto_flush is not None and len(_state.pending) >= _state.auto_flush[1]:
        execute(_state.auto_flush[0])


def _retire(info):
    info.alive = False
    if info.materialised:
        _state.dead.append(info.name)


# ---- regions ------------------------------------------------------------------------------

def _full_region(shape):
    return Region((0,) * len(shape), shape, (1,) * len(shape))


def _parse_key(key, shape):
    """Index expression -> Region (charmnumeric.py:272-343: ints, slices, one ellipsis)."""
    ndims = len(shape)
    if key is Ellipsis:
        key = (Ellipsis,)
    elif not isinstance(key, tuple):
        key = (key,)
    if any(k is None for k in key):
        raise NotImplementedError("np.newaxis is not supported yet")
    if sum(1 for k in key if k is Ellipsis) > 1:
        raise IndexError("an index can only have a single ellipsis")
    explicit = sum(1 for k in key if k is not Ellipsis)
    if explicit > ndims:
        raise IndexError(f"too many indices for array: array is {ndims}-dimensional, "
                         f"but {explicit} were indexed")
    items = []
    for k in key:
        if k is Ellipsis:
            items.extend([slice(None)] * (ndims - explicit))
        else:
            items.append(k)
    items.extend([slice(None)] * (ndims - len(items)))
    start, stop, step = [], [], []
    for i, it in enumerate(items):
        if isinstance(it, slice):
            st = 1 if it.step is None else int(it.step)
            if st == 0:
                raise ValueError("slice step cannot be zero")
            if st < 0:
                raise NotImplementedError("negative slicing is not supported yet")
            a, b, st = it.indices(shape[i])
            b = max(a, b)
        elif isinstance(it, numbers.Integral):
            a = int(it)
            if a < 0:
                a += shape[i]
            if a < 0 or a >= shape[i]:
                raise IndexError(f"index {it} is out of bounds for axis {i} with size {shape[i]}")
            b, st = a + 1, 1
        else:
            raise TypeError("only integers, slices, and ellipsis are valid charmnumeric indices")
        start.append(a)
        stop.append(b)
        step.append(st)
    return Region(start, stop, step)


def _compose(outer, inner):
    """Region of a view of a view (charmnumeric.py:212-230)."""
    start = [o + i * s for o, i, s in zip(outer.start, inner.start, outer.step)]
    stop = [o + i * s for o, i, s in zip(outer.start, inner.stop, outer.step)]
    step = [s * t for s, t in zip(outer.step, inner.step)]
    # a stop computed through a step may overshoot by less than one step: clip to the outer stop
    stop = [min(b, ob) if b > a else a for a, b, ob in zip(start, stop, outer.stop)]
    return Region(start, stop, step)


# ---- user-facing objects --------------------------------------------------------------------

class _ArrayOps:
    __array_priority__ = 1000

    # subclasses provide: _info, _region (None = whole array), shape, dtype
    @property
    def ndims(self):
        return len(self.shape)

    ndim = ndims

    @property
    def size(self):
        return _CallableInt(_size(self.shape))

    @property
    def itemsize(self):
        return self.dtype.itemsize

    @property
    def nbytes(self):
        return self.size * self.itemsize

    @property
    def name(self):
        return self._info.name

    def __len__(self):
        return self.shape[0]

    def __bool__(self):
        raise ValueError("The truth value of a charmnumeric array is ambiguous. "
                         "Use .get(interface) to materialize it first.")

    def __array__(self, dtype=None, copy=None):
        raise TypeError("charmnumeric arrays are lazy frontend objects. "
                        "Call .get(interface) before converting to numpy.")

    def _operand(self):
        return (self._info, self._region)

    def __add__(self, other):
        return _binary(ArrayOperation.add, self, other)

    def __radd__(self, other):
        return _binary(ArrayOperation.add, other, self)

    def __sub__(self, other):
        return _binary(ArrayOperation.sub, self, other)

    def __rsub__(self, other):
        return _binary(ArrayOperation.sub, other, self)

    def __mul__(self, other):
        return _binary(ArrayOperation.mul, self, other)

    def __rmul__(self, other):
        return _binary(ArrayOperation.mul, other, self)

    def __truediv__(self, other):
        return _binary(ArrayOperation.div, self, other)

    def __rtruediv__(self, other):
        return _binary(ArrayOperation.div, other, self)

    def __neg__(self):
        # the reference spells -x as x * -1 (charmnumeric.py:427-434)
        return _binary(ArrayOperation.mul, self, -1)

    def __matmul__(self, other):
        return _matmul(self, other)

    def dot(self, other):
        return _matmul(self, other)

    def matvec(self, vec):
        return _matvec(self, vec)

    def copy(self):
        out = empty(self.shape, dtype=self.dtype)
        out[...] = self
        return out

    def fill(self, value):
        self[...] = value

    def astype(self, dtype, copy=True):
        if _normalize_dtype(dtype) != self.dtype:
            raise NotImplementedError(
                "dtype conversion for existing charmnumeric arrays is not implemented yet")
        return self.copy() if copy else self

    def __getitem__(self, key):
        region = _parse_key(key, self.shape)
        if self._region is not None:
            region = _compose(self._region, region)
        return ArrayView(self._root(), region)

    def __setitem__(self, key, rhs):
        region = _parse_key(key, self.shape)
        if self._region is not None:
            region = _compose(self._region, region)
        rhs = _coerce_assignment(rhs, region.shape(), self.dtype)
        if isinstance(rhs, _ArrayOps):
            if tuple(rhs.shape) != tuple(region.shape()) and rhs.size != 1:
                # the same elements with the singleton dimensions elsewhere (`A[i, :] = v`,
                # `v[:] = A[:, j]`): a cross-dimension assignment, its own node
                # (src/executor_transfer.cpp:66-177)
                if [d for d in rhs.shape if d != 1] != [d for d in region.shape() if d != 1]:
                    raise ValueError(f"could not broadcast input from shape {rhs.shape} "
                                     f"into shape {region.shape()}")
                if rhs.dtype != self.dtype:
                    raise TypeError("cross-dimension assignment needs matching dtypes")
                _record(_Op("xset", wire.OP_SET_REGION, self._info, [rhs._operand()], region=region))
                return
            operand = rhs._operand()
        else:
            operand = rhs
        _record(_Op("set", wire.OP_SET_REGION, self._info, [operand], region=region))


class Array(_ArrayOps):
    """A whole lazy array."""

    def __init__(self, info):
        self._info = info
        self._region = None
        self.shape = info.shape
        self.dtype = info.dtype
        weakref.finalize(self, _retire, info)

    def _root(self):
        return self

    def __repr__(self):
        return f"Array(shape={self.shape}, dtype={self.dtype.name}, name={self.name})"

    def wire_dtype(self):
        return WIRE_DTYPES[self.dtype]

    def get(self, interface):
        execute(interface)
        data = interface.get(self.ndims, self.name, self.size, dtype=self.dtype)
        return data.reshape(self.shape)


class ArrayView(_ArrayOps):
    """A (start, stop, step) window of an Array; keeps its Array alive."""

    def __init__(self, base, region):
        self._base = base
        self._info = base._info
        self._region = region
        self.shape = tuple(region.shape())
        self.dtype = base.dtype

    def _root(self):
        return self._base

    def __repr__(self):
        return f"ArrayView(shape={self.shape}, dtype={self.dtype.name}, name={self.name})"

    def get(self, interface):
        return self.copy().get(interface)


def _new_array(shape, dtype):
    return Array(_Info(_state.new_name(), tuple(shape), np.dtype(dtype)))


def _coerce_operand(v):
    if isinstance(v, _ArrayOps):
        return v
    if _is_scalar_like(v):
        return _coerce_scalar(v)
    host = np.asarray(v)
    if host.ndim == 0:
        return _coerce_scalar(host.item())
    return asarray(host)


def _coerce_assignment(rhs, shape, dtype):
    if isinstance(rhs, _ArrayOps):
        return rhs
    if _is_scalar_like(rhs):
        return _coerce_scalar(rhs)
    host = np.asarray(rhs, dtype=dtype)
    if host.ndim == 0:
        return _coerce_scalar(host.item())
    host = np.broadcast_to(host, shape)
    return asarray(host)


def _result_shape(a, b):
    sa = a.shape if isinstance(a, _ArrayOps) else ()
    sb = b.shape if isinstance(b, _ArrayOps) else ()
    if isinstance(a, _ArrayOps) and isinstance(b, _ArrayOps):
        if a.size == 1 and b.size != 1:
            return tuple(sb)
        if b.size == 1:
            return tuple(sa)
        if tuple(sa) != tuple(sb):
            raise ValueError("operands could not be broadcast together with shapes "
                             f"{tuple(sa)} and {tuple(sb)} (only scalars and size-1 arrays "
                             "broadcast)")
        return tuple(sa)
    return tuple(sa) if isinstance(a, _ArrayOps) else tuple(sb)


def _result_dtype(a, b):
    da = a.dtype if isinstance(a, _ArrayOps) else None
    db = b.dtype if isinstance(b, _ArrayOps) else None
    if da is None:
        return db
    if db is None:
        return da
    return _normalize_dtype(np.result_type(da, db))


def _binary(opcode, a, b):
    a, b = _coerce_operand(a), _coerce_operand(b)
    out = _new_array(_result_shape(a, b), _result_dtype(a, b))
    operands = [x._operand() if isinstance(x, _ArrayOps) else x for x in (a, b)]
    _record(_Op("ew", opcode, out._info, operands))
    return out


def _unary(opcode, x):
    x = asarray(x)
    out = _new_array(x.shape, x.dtype)
    _record(_Op("ew", opcode, out._info, [x._operand()]))
    return out


def _whole(x):
    """Non-fusible ops take whole arrays: materialise a view first."""
    return x.copy() if isinstance(x, ArrayView) else x


def _matmul(a, b):
    b = _coerce_operand(b)
    if not isinstance(b, _ArrayOps):
        raise ValueError("matmul does not support scalar operands")
    if a.ndims == b.ndims and (a.ndims == 1 or tuple(a.shape) == tuple(b.shape)) and \
            not (a.ndims == 2 and b.ndims == 2):
        if tuple(a.shape) != tuple(b.shape):
            raise ValueError(f"Shape mismatch for dot product: {a.shape} @ {b.shape}")
        a, b = _whole(a), _whole(b)
        out = _new_array((1,), _result_dtype(a, b))
        _record(_Op("reduce", wire.OP_REDUCE, out._info, [a._operand(), b._operand()]))
        return out
    if a.ndims != 2:
        raise ValueError(f"matmul requires a 2D matrix, got {a.ndims}D")
    if b.ndims == 1:
        return _matvec(a, b)
    raise NotImplementedError("matrix-matrix products are outside this backend's scope")


def _matvec(mat, vec):
    if not isinstance(vec, _ArrayOps):
        raise ValueError("matvec requires an Array vector")
    # a column vector (n, 1) has the memory layout and the partition of a 1-D vector of n
    column = vec.ndims == 2 and vec.shape[1] == 1
    if mat.ndims != 2 or not (vec.ndims == 1 or column):
        raise ValueError("matvec requires a 2D matrix and a 1D vector (or an (n, 1) column)")
    if mat.shape[1] != vec.shape[0]:
        raise ValueError(f"Shape mismatch: matrix cols {mat.shape[1]} != vector size {vec.shape[0]}")
    out = _new_array((mat.shape[0], 1) if column else (mat.shape[0],), _result_dtype(mat, vec))
    _record(_Op("matmul", wire.OP_MATMUL, out._info, [mat._operand(), vec._operand()]))
    return out


def tile(x, reps):
    """numpy.tile for backend arrays (charmnumeric/operations.py:52-72)."""
    if _is_scalar_like(x):
        return asarray(np.tile(np.asarray(x), reps))
    x = _whole(asarray(x))
    reps = (int(reps),) if isinstance(reps, (int, np.integer)) else tuple(int(r) for r in reps)
    if any(r < 1 for r in reps):
        raise ValueError("tile: repeat counts must be positive")
    nd = max(x.ndims, len(reps))
    if nd > 3:
        raise NotImplementedError("tile: results with more than three dimensions are outside this backend's scope")
    shape = (1,) * (nd - x.ndims) + tuple(x.shape)
    full = (1,) * (nd - len(reps)) + reps
    out = _new_array(tuple(s * r for s, r in zip(shape, full)), x.dtype)
    _record(_Op("tile", wire.OP_TILE, out._info, [x._operand()], payload=full))
    return out


def diag(v, k=0):
    """Diagonal matrix from a vector, or the k-th diagonal of a matrix
    (charmnumeric/operations.py:125-148)."""
    v = _whole(asarray(v))
    k = int(k)
    if v.ndims == 1:
        n = v.shape[0] + (k if k >= 0 else -k)
        shape = (n, n)
    elif v.ndims == 2:
        rows, cols = v.shape
        length = max(0, min(rows, cols - k)) if k >= 0 else max(0, min(rows + k, cols))
        if length == 0:
            raise ValueError(f"k={k} is out of range for shape ({rows}, {cols})")
        shape = (length,)
    else:
        raise ValueError(f"diag requires a 1D or 2D array, got {v.ndims}D")
    out = _new_array(shape, v.dtype)
    _record(_Op("diag", wire.OP_DIAG, out._info, [v._operand()], payload=k))
    return out


def dot2d(a, b):
    """dot of two same-shaped arrays of any rank (the reference accepts 1-D only)."""
    a, b = _whole(asarray(a)), _whole(asarray(b))
    if tuple(a.shape) != tuple(b.shape):
        raise ValueError(f"Shape mismatch for dot product: {a.shape} vs {b.shape}")
    out = _new_array((1,), _result_dtype(a, b))
    _record(_Op("reduce", wire.OP_REDUCE, out._info, [a._operand(), b._operand()]))
    return out


def sum_all(x):
    """Sum of all elements -> size-1 array (an addition; fuses behind the expression)."""
    x = asarray(x)
    out = _new_array((1,), x.dtype)
    _record(_Op("sum", wire.OP_SUM, out._info, [x._operand()]))
    return out


# ---- constructors ---------------------------------------------------------------------------

def create_array(shape, dtype=_DEFAULT_DTYPE):
    shape = _normalize_shape(shape)
    out = _new_array(shape, _normalize_dtype(dtype))
    _record(_Op("create", wire.OP_CREATE, out._info))
    return out


def empty(shape, dtype=_DEFAULT_DTYPE):
    return create_array(shape, dtype=dtype)


def zeros(shape, dtype=_DEFAULT_DTYPE):
    return create_array(shape, dtype=dtype)


def full(shape, fill_value, dtype=None):
    if not _is_scalar_like(fill_value):
        host = np.broadcast_to(np.asarray(fill_value, dtype=dtype), _normalize_shape(shape))
        return asarray(host)
    if dtype is None:
        dtype = _normalize_dtype(np.asarray(fill_value).dtype)
    out = create_array(shape, dtype=dtype)
    out[...] = _coerce_scalar(fill_value)
    return out


def ones(shape, dtype=_DEFAULT_DTYPE):
    return full(shape, 1, dtype=dtype)


def _like(a, dtype, shape):
    if isinstance(a, _ArrayOps):
        bs, bd = a.shape, a.dtype
    else:
        host = np.asarray(a)
        bs, bd = host.shape, _normalize_dtype(host.dtype)
    return (bs if shape is None else _normalize_shape(shape),
            bd if dtype is None else _normalize_dtype(dtype))


def empty_like(a, dtype=None, shape=None):
    s, d = _like(a, dtype, shape)
    return empty(s, dtype=d)


def zeros_like(a, dtype=None, shape=None):
    s, d = _like(a, dtype, shape)
    return zeros(s, dtype=d)


def ones_like(a, dtype=None, shape=None):
    s, d = _like(a, dtype, shape)
    return ones(s, dtype=d)


def full_like(a, fill_value, dtype=None, shape=None):
    s, d = _like(a, dtype, shape)
    return full(s, fill_value, dtype=d)


def asarray(a, dtype=None):
    """Arrays pass through; host data is uploaded in bulk (the reference assigns it one
    SET_REGION per element, charmnumeric.py:863-878)."""
    if isinstance(a, _ArrayOps):
        if dtype is not None and _normalize_dtype(dtype) != a.dtype:
            raise NotImplementedError(
                "dtype conversion for existing charmnumeric arrays is not implemented yet")
        return a
    host = np.array(a, dtype=None if dtype is None else _normalize_dtype(dtype), copy=True)
    if host.ndim == 0:
        raise NotImplementedError("0D charmnumeric arrays are not supported yet")
    host = np.ascontiguousarray(host, dtype=_normalize_dtype(host.dtype))
    out = _new_array(_normalize_shape(host.shape), host.dtype)
    _record(_Op("put", None, out._info, payload=host))
    return out


def array(a, dtype=None, copy=True, ndmin=0):
    if isinstance(a, _ArrayOps):
        a = asarray(a, dtype)
        return a.copy() if copy else a
    host = np.array(a, dtype=dtype, copy=True, ndmin=ndmin)
    return asarray(host)


def copy(a, order="K"):
    return array(a, copy=True)


def copyto(dst, src):
    if not isinstance(dst, _ArrayOps):
        raise TypeError("copyto destination must be a charmnumeric Array or ArrayView")
    dst[...] = src
    return dst


def arange(start, stop=None, step=1, dtype=None):
    return asarray(np.arange(start, stop, step, dtype=dtype))


def eye(N, M=None, k=0, dtype=_DEFAULT_DTYPE):
    return asarray(np.eye(int(N), None if M is None else int(M), int(k), dtype=dtype))


def identity(n, dtype=_DEFAULT_DTYPE):
    return eye(n, dtype=dtype)


def uniform(shape, seed=0, low=0.0, high=1.0, dtype=_DEFAULT_DTYPE):
    """Seeded uniform array in [low, high): element with row-major index g depends only on
    (seed, g), whatever the number of GPUs.  (The reference's random.randn returns zeros,
    charmnumeric/random.py:4-5.)"""
    out = _new_array(_normalize_shape(shape), _normalize_dtype(dtype))
    _record(_Op("randu", wire.OP_RANDU, out._info, [int(seed), float(low), float(high)]))
    return out


# ---- functional API (charmnumeric/operations.py:38-148) ------------------------------------------

def tanh(x):
    if _is_scalar_like(x):
        return np.tanh(_coerce_scalar(x))
    return _unary(ArrayOperation.tanh, x)


def exp(x):
    if _is_scalar_like(x):
        return np.exp(_coerce_scalar(x))
    return _unary(ArrayOperation.exp, x)


def sqrt(x):
    if _is_scalar_like(x):
        return np.sqrt(_coerce_scalar(x))
    return _unary(ArrayOperation.sqrt, x)


def absolute(x):
    if _is_scalar_like(x):
        return np.abs(_coerce_scalar(x))
    return _unary(ArrayOperation.abs, x)


def add(x1, x2):
    return asarray(x1) + x2 if not _is_scalar_like(x1) else x1 + asarray(x2)


def subtract(x1, x2):
    return asarray(x1) - x2 if not _is_scalar_like(x1) else x1 - asarray(x2)


def multiply(x1, x2):
    return asarray(x1) * x2 if not _is_scalar_like(x1) else x1 * asarray(x2)


def divide(x1, x2):
    return asarray(x1) / x2 if not _is_scalar_like(x1) else x1 / asarray(x2)


def matmul(x1, x2):
    return asarray(x1) @ x2


def dot(x1, x2):
    return asarray(x1).dot(x2)


def norm2(x):
    x = asarray(x)
    return x.dot(x)


# ---- interface ------------------------------------------------------------------------------------

class CharmNumericInterface:
    """Connection to the backend.  The reference's interface is a CCS socket to a
    ``charmrun`` server (charmnumeric/interface.py:12-23); here it owns the context of this
    process's GPU.  With several GPUs every rank runs the same program and passes its rank,
    the world size and the shared 128-byte id."""

    def __init__(self, device=0, rank=0, nranks=1, unique_id=None):
        self.context = Context(device=device, rank=rank, nranks=nranks)
        if nranks > 1:
            if unique_id is None:
                raise ValueError("nranks > 1 needs the unique_id shared by all ranks")
            self.context.comm_init(unique_id)

    def connect(self, *args, **kwargs):
        """Accepted for source compatibility; the context is already live."""
        return self

    def get(self, ndims, name, size, dtype=None):
        return self.context.get(name).reshape(-1)

    def close(self):
        self.context.close()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.close()


class LocalCluster(CharmNumericInterface):
    """Source-compatible stand-in for the reference's LocalCluster
    (charmnumeric/interface.py:26-129), which starts a ``charmrun`` server and connects to it.
    There is no server process here: the backend lives in this process, so the launcher's
    arguments (server binary, port, odf, PE count ...) are accepted and ignored, and the object
    is simply the interface of GPU ``device``, usable as a context manager."""

    def __init__(self, server_binary=None, *, device=0, **_launcher_options):
        super().__init__(device=device)


# ---- DAG building -------------------------------------------------------------------------------------

def _is_size1(info):
    return _size(info.shape) == 1


class _Group:
    def __init__(self):
        self.ops = []
        self.shape = None          # iteration shape of the array-valued ops
        self.array_shape = None    # shape of the arrays touched (for the two-domain rule)
        self.uniform = True        # every array touched has array_shape and unit-step views
        self.written = {}          # info.name -> destination Region
        self.produced = set()      # names of elementwise results inside the group
        self.filled = set()        # arrays assigned from a literal inside the group


def _op_views(op):
    for o in op.operands:
        if isinstance(o, tuple):
            yield o


def _op_shape(op):
    if op.kind == "set":
        return tuple(op.region.shape())
    return tuple(op.result.shape)


def _scalar_valued(op):
    if op.kind == "set":
        return _is_size1(op.result)
    return _is_size1(op.result) and all(
        (not isinstance(o, tuple)) or _is_size1(o[0]) for o in op.operands)


def _can_join(g, op):
    if not g.ops:
        return True
    # hazards first
    for info, region in _op_views(op):
        if info.name in g.filled:
            return False
        # a value computed inside the group is handed on element by element (a register of
        # the fused kernel): a part of it, or a shifted view of it, has to come from memory
        if info.name in g.produced and region is not None and region != _full_region(info.shape):
            return False
        if info.name in g.written and not _is_size1(info):
            dest = g.written[info.name]
            reg = region if region is not None else _full_region(info.shape)
            if reg != dest and reg != _full_region(info.shape):
                return False
            if reg != dest and not g.uniform:
                return False
    if op.kind == "set" and op.result.name in g.written:
        return False
    if op.kind == "set" and op.result.name in g.produced:
        return False
    if _scalar_valued(op):
        return True
    shape = _op_shape(op)
    if g.shape is None or shape == g.shape:
        return True
    # ops of another shape start a new group: the backend's kernels iterate over one shape
    # (reductions over whole arrays are folded into a region group by the backend itself)
    return False


def _join(g, op):
    g.ops.append(op)
    if not _scalar_valued(op):
        if g.shape is None:
            g.shape = _op_shape(op)
        touched = [(i, r) for i, r in _op_views(op) if not _is_size1(i) and i.name not in g.produced]
        if op.kind == "set":
            touched.append((op.result, op.region))
        for info, region in touched:
            if g.array_shape is None:
                g.array_shape = info.shape
            if info.shape != g.array_shape:
                g.uniform = False
            if region is not None and any(s != 1 for s in region.step):
                g.uniform = False
    if op.kind == "set":
        g.written[op.result.name] = op.region
        if not isinstance(op.operands[0], tuple):
            g.filled.add(op.result.name)
    elif op.kind == "ew":
        g.produced.add(op.result.name)


def _leaf(info, dtype_code=None):
    return wire.Ast(info.name, wire.OP_NOOP, shape=info.shape, dtype=WIRE_DTYPES[info.dtype],
                    is_broadcast=_is_size1(info))


def _operand_ast(o, produced, dtype):
    if isinstance(o, tuple):
        info, region = o
        if info.name in produced:
            return (wire.Ref(info.name), None)
        return (_leaf(info), region)
    return (wire.scalar(o, WIRE_DTYPES[dtype]), None)


def _group_node(g, consumers_outside):
    roots = []
    produced = set()
    for op in g.ops:
        if op.kind == "ew":
            res = op.result
            temp = (not res.alive) and res.name not in consumers_outside
            roots.append(wire.Ast(res.name, op.opcode, is_temp=temp, shape=res.shape,
                                  dtype=WIRE_DTYPES[res.dtype],
                                  operands=[_operand_ast(o, produced, res.dtype) for o in op.operands]))
            produced.add(res.name)
            if not temp:
                res.materialised = True
        elif op.kind == "set":
            tgt = op.result
            roots.append(wire.Ast(_state.new_name(), wire.OP_SET_REGION, shape=tuple(op.region.shape()),
                                  dtype=WIRE_DTYPES[tgt.dtype], region=op.region,
                                  operands=[(_leaf(tgt), None),
                                            _operand_ast(op.operands[0], produced, tgt.dtype)]))
        elif op.kind == "sum":
            res = op.result
            roots.append(wire.Ast(res.name, wire.OP_SUM, shape=(1,), dtype=WIRE_DTYPES[res.dtype],
                                  operands=[_operand_ast(op.operands[0], produced, res.dtype)]))
            res.materialised = True
    node = wire.Node(_state.next_node, roots, fusible=True)
    _state.next_node += 1
    return node


def _single_node(op):
    res = op.result
    dt = WIRE_DTYPES[res.dtype]
    if op.kind == "create":
        root = wire.Ast(res.name, wire.OP_CREATE, shape=res.shape, dtype=dt)
    elif op.kind in ("reduce", "matmul", "sum"):
        root = wire.Ast(res.name, op.opcode, shape=res.shape, dtype=dt,
                        operands=[(_leaf(i), r) for i, r in op.operands])
    elif op.kind == "tile":
        root = wire.Ast(res.name, wire.OP_TILE, shape=res.shape, dtype=dt,
                        operands=[(_leaf(i), r) for i, r in op.operands]
                        + [(wire.scalar(float(rep)), None) for rep in op.payload])
    elif op.kind == "diag":
        root = wire.Ast(res.name, wire.OP_DIAG, shape=res.shape, dtype=dt,
                        operands=[(_leaf(i), r) for i, r in op.operands]
                        + [(wire.scalar(float(op.payload)), None)])
    elif op.kind == "xset":
        src, sreg = op.operands[0]
        root = wire.Ast(_state.new_name(), wire.OP_SET_REGION, shape=tuple(op.region.shape()), dtype=dt,
                        region=op.region, operands=[(_leaf(res), None), (_leaf(src), sreg)])
        node = wire.Node(_state.next_node, [root], fusible=False)
        _state.next_node += 1
        return node
    elif op.kind == "randu":
        root = wire.Ast(res.name, wire.OP_RANDU, shape=res.shape, dtype=dt,
                        operands=[(wire.scalar(v), None) for v in op.operands])
    else:
        raise AssertionError(op.kind)
    res.materialised = True
    node = wire.Node(_state.next_node, [root], fusible=False)
    _state.next_node += 1
    return node


def build_nodes(ops):
    """Group a list of recorded ops into DAG nodes (exposed for tests and tools)."""
    # which results are read by an op outside the group that produced them is only known
    # after grouping, so group first and mark temporaries afterwards
    segments = []  # ("group", _Group) | ("single", op) | ("put", op)
    g = _Group()

    def close():
        nonlocal g
        if g.ops:
            segments.append(("group", g))
        g = _Group()

    for op in ops:
        if op.kind in ("ew", "set"):
            if not _can_join(g, op):
                close()
            _join(g, op)
        elif op.kind == "sum":
            src = op.operands[0][0]
            if g.ops and src.name in g.produced and op.operands[0][1] is None:
                g.ops.append(op)       # terminal reduction of the open group
                close()
            else:
                close()
                segments.append(("single", op))
        elif op.kind == "put":
            close()
            segments.append(("put", op))
        else:
            close()
            segments.append(("single", op))
    close()

    # readers per produced name, by segment index
    readers = {}
    for si, (kind, item) in enumerate(segments):
        seg_ops = item.ops if kind == "group" else [item]
        for op in seg_ops:
            for info, _ in _op_views(op):
                readers.setdefault(info.name, set()).add(si)
            if op.kind in ("set", "xset"):
                # the target of an assignment has to exist as an array, even when the program
                # drops its last handle on it before the batch is built
                readers.setdefault(op.result.name, set()).add(si)
    out = []
    for si, (kind, item) in enumerate(segments):
        if kind == "group":
            outside = {op.result.name for op in item.ops
                       if op.kind == "ew" and (readers.get(op.result.name, set()) - {si})}
            out.append(("node", _group_node(item, outside)))
        elif kind == "single":
            out.append(("node", _single_node(item)))
        else:
            out.append(("put", item))
    return out


def execute(interface, mirror=None):
    """Run everything recorded so far on the backend (asynchronously).

    ``mirror`` (optional) is an object with ``run(nodes, deletes)`` and ``put(name, host)``
    that receives exactly what the backend receives, in the same order; the tests pass the
    CPU oracle here so both sides execute one and the same DAG."""
    ops, _state.pending = _state.pending, []
    ctx = getattr(interface, "context", None)
    if mirror is None:
        mirror = getattr(interface, "mirror", None)
    items = build_nodes(ops)
    nodes = []

    def flush(deletes=()):
        if nodes or deletes:
            if ctx is not None:
                ctx.run(nodes, deletes)
            if mirror is not None:
                mirror.run(list(nodes), list(deletes))
            nodes.clear()

    for kind, item in items:
        if kind == "node":
            nodes.append(item)
        else:
            flush()
            if ctx is not None:
                ctx.put(item.result.name, item.payload)
            if mirror is not None:
                mirror.put(item.result.name, item.payload)
            item.result.materialised = True
    # arrays produced but already unreachable are released right after the DAG
    dead = list(_state.dead)
    _state.dead.clear()
    for op in ops:
        res = op.result
        if res is not None and op.kind not in ("set", "xset") and res.materialised and not res.alive \
                and res.name not in dead:
            dead.append(res.name)
    flush(dead)
