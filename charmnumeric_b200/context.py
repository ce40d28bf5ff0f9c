"""Python handle on one backend context (one rank, one GPU) over the C ABI."""
import ctypes as C

import numpy as np

from . import _lib, wire

NP_DTYPES = {wire.F32: np.dtype("float32"), wire.F64: np.dtype("float64"),
             wire.I32: np.dtype("int32"), wire.I64: np.dtype("int64")}
WIRE_DTYPES = {v: k for k, v in NP_DTYPES.items()}


def comm_unique_id():
    """128-byte id created by rank 0 and handed to every rank's ``Context.comm_init``."""
    lib = _lib.load()
    buf = C.create_string_buffer(128)
    _lib.check(None, lib.cn_comm_unique_id(buf))
    return buf.raw


def partition(n0, nranks, rank):
    """Rows [begin, end) of dimension 0 that ``rank`` of ``nranks`` owns (host-only)."""
    lib = _lib.load()
    b = C.c_int64()
    e = C.c_int64()
    _lib.check(None, lib.cn_partition(int(n0), int(nranks), int(rank), C.byref(b), C.byref(e)))
    return b.value, e.value


class Context:
    """One rank of the backend.  ``device`` is the CUDA device index of this process."""

    def __init__(self, device=0, rank=0, nranks=1):
        self._lib = _lib.load()
        self._h = C.c_void_p()
        status = self._lib.cn_context_create(int(device), int(rank), int(nranks), C.byref(self._h))
        if status != 0:
            msg = self._lib.cn_last_error(None)
            raise _lib.CnError(status, msg.decode() if msg else "")
        self.rank = int(rank)
        self.nranks = int(nranks)
        self.epoch = 0

    def close(self):
        if self._h:
            self._lib.cn_context_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status):
        _lib.check(self._h, status)

    # ---- wiring ----
    def comm_init(self, unique_id):
        self._check(self._lib.cn_comm_init(self._h, bytes(unique_id)))

    def mark_rank_failed(self, rank):
        self._check(self._lib.cn_mark_rank_failed(self._h, int(rank)))

    def set_option(self, key, value):
        self._check(self._lib.cn_set_option(self._h, key.encode(), int(value)))

    # ---- execution ----
    def receive_dag(self, blob):
        """Enqueue one DAG blob (bytes); returns without waiting for the GPU."""
        self.epoch += 1
        self._check(self._lib.cn_receive_dag(self._h, self.epoch, len(blob), blob))

    def run(self, nodes, deletes=()):
        self.receive_dag(wire.dag_blob(nodes, deletes, self.epoch + 1))

    def synchronize(self):
        self._check(self._lib.cn_synchronize(self._h))

    def delete_array(self, name):
        self._check(self._lib.cn_delete_array(self._h, int(name)))

    # ---- data movement ----
    def array_info(self, name):
        nd = C.c_int()
        dt = C.c_int()
        shape = (C.c_int64 * 3)()
        rb = C.c_int64()
        re = C.c_int64()
        self._check(self._lib.cn_array_info(self._h, int(name), C.byref(nd), shape, C.byref(dt),
                                            C.byref(rb), C.byref(re)))
        return {"shape": tuple(shape[i] for i in range(nd.value)), "dtype": NP_DTYPES[dt.value],
                "rows": (rb.value, re.value)}

    def get(self, name, shape=None, dtype=None):
        """Whole array as numpy (every rank that calls receives all of it)."""
        if shape is None or dtype is None:
            info = self.array_info(name)
            shape, dtype = info["shape"], info["dtype"]
        dtype = np.dtype(dtype)
        out = np.empty(shape, dtype=dtype)
        self._check(self._lib.cn_get(self._h, len(shape), self.epoch, int(name), out.size,
                                     WIRE_DTYPES[dtype], out.ctypes.data_as(C.c_void_p)))
        return out

    def get_into(self, name, out):
        """Same as ``get`` into a caller-provided (e.g. pinned) contiguous numpy buffer."""
        self._check(self._lib.cn_get(self._h, out.ndim, self.epoch, int(name), out.size,
                                     WIRE_DTYPES[out.dtype], out.ctypes.data_as(C.c_void_p)))
        return out

    def get_root(self, name, root=0, shape=None, dtype=None):
        """Whole array on rank ``root`` only (numpy there, None on the other ranks); every
        rank has to call it."""
        if shape is None or dtype is None:
            info = self.array_info(name)
            shape, dtype = info["shape"], info["dtype"]
        dtype = np.dtype(dtype)
        count = int(np.prod(shape))
        out = np.empty(shape, dtype=dtype) if self.rank == root else None
        ptr = out.ctypes.data_as(C.c_void_p) if out is not None else None
        self._check(self._lib.cn_get_root(self._h, len(shape), self.epoch, int(name), count,
                                          WIRE_DTYPES[dtype], int(root), ptr))
        return out

    def get_local_into(self, name, out):
        """This rank's slab into a caller-provided (e.g. pinned) contiguous numpy buffer."""
        b = C.c_int64()
        e = C.c_int64()
        self._check(self._lib.cn_get_local(self._h, int(name), C.byref(b), C.byref(e), out.size,
                                           out.ctypes.data_as(C.c_void_p)))
        return (b.value, e.value)

    def put_local(self, name, shape, slab):
        """Upload this rank's slab of an array of global ``shape`` from a host buffer that
        holds only those rows."""
        slab = np.ascontiguousarray(slab)
        cshape = (C.c_int64 * len(shape))(*shape)
        self._check(self._lib.cn_put_local(self._h, int(name), len(shape), cshape, WIRE_DTYPES[slab.dtype],
                                           slab.size, slab.ctypes.data_as(C.c_void_p)))

    def execute_node(self, node):
        """Run one node at once (no DAG around it)."""
        blob = node.pack()
        self._check(self._lib.cn_execute_node(self._h, blob, len(blob)))

    def get_local(self, name):
        info = self.array_info(name)
        rb, re = info["rows"]
        shape = (re - rb,) + info["shape"][1:]
        out = np.empty(shape, dtype=info["dtype"])
        b = C.c_int64()
        e = C.c_int64()
        self._check(self._lib.cn_get_local(self._h, int(name), C.byref(b), C.byref(e), out.size,
                                           out.ctypes.data_as(C.c_void_p)))
        return (b.value, e.value), out

    def put(self, name, host):
        """Upload a whole host array; each rank keeps its own slab of dimension 0."""
        host = np.ascontiguousarray(host)
        shape = (C.c_int64 * host.ndim)(*host.shape)
        self._check(self._lib.cn_put(self._h, int(name), host.ndim, shape, WIRE_DTYPES[host.dtype],
                                     host.ctypes.data_as(C.c_void_p)))

    # ---- measurement ----
    def timer_start(self):
        self._check(self._lib.cn_timer_start(self._h))

    def timer_stop(self):
        ms = C.c_float()
        self._check(self._lib.cn_timer_stop(self._h, C.byref(ms)))
        return float(ms.value)

    def profile(self, on=True):
        self.set_option("profile", 1 if on else 0)

    def profile_report(self):
        """Kernels timed since profiling was switched on: list of dicts with label, launches,
        ms (total device time) and bytes (algorithmic bytes moved)."""
        buf = C.create_string_buffer(1 << 16)
        self._check(self._lib.cn_profile_report(self._h, buf, len(buf)))
        rows = []
        for line in buf.value.decode().splitlines():
            label, launches, ms, nbytes = line.split("\t")
            rows.append({"label": label, "launches": int(launches), "ms": float(ms),
                         "bytes": float(nbytes)})
        return rows

    def stats(self):
        s = _lib.Stats()
        self._check(self._lib.cn_get_stats(self._h, C.byref(s)))
        return s.as_dict()

    # ---- kernel-ABI level ----
    def compile_group(self, node):
        h = C.c_uint64()
        blob = node.pack()
        self._check(self._lib.cn_compile_group(self._h, blob, len(blob), C.byref(h)))
        return h.value

    def group_source(self, handle):
        s = C.c_char_p()
        self._check(self._lib.cn_group_source(self._h, handle, C.byref(s)))
        return s.value.decode()


def group_compile_check(node):
    """Host-only: lower + generate + compile one group; returns (source, cubin_bytes)."""
    lib = _lib.load()
    blob = node.pack()
    src = C.create_string_buffer(1 << 18)
    err = C.create_string_buffer(1 << 14)
    nb = C.c_int64(0)
    status = lib.cn_group_compile_check(blob, len(blob), src, len(src), C.byref(nb), err, len(err))
    if status != 0:
        raise _lib.CnError(status, err.value.decode())
    return src.value.decode(), nb.value


def fuse_check(node_a, node_b):
    """Host-only: the CUDA source of the single kernel that runs ``node_a`` (a whole-array
    assignment) and ``node_b`` (a stencil over the assigned array), or None when the pair does
    not fuse."""
    lib = _lib.load()
    a, b = node_a.pack(), node_b.pack()
    src = C.create_string_buffer(1 << 18)
    err = C.create_string_buffer(1 << 14)
    fused = C.c_int(0)
    status = lib.cn_fuse_check(a, len(a), b, len(b), src, len(src), C.byref(fused), err, len(err))
    if status != 0:
        raise _lib.CnError(status, err.value.decode())
    return src.value.decode() if fused.value else None


def tail_check(blob):
    """Host-only: ``blob`` holds a group node, the REDUCE / SUM nodes its kernel takes in and a
    node of size-1 arithmetic; returns the CUDA source of the single kernel when that last node
    runs as the kernel's scalar tail, else None."""
    lib = _lib.load()
    src = C.create_string_buffer(1 << 18)
    err = C.create_string_buffer(1 << 14)
    fused = C.c_int(0)
    status = lib.cn_tail_check(blob, len(blob), src, len(src), C.byref(fused), err, len(err))
    if status != 0:
        raise _lib.CnError(status, err.value.decode())
    return src.value.decode() if fused.value else None


def dag_check(blob):
    """Host-only: parse a DAG blob; returns (n_nodes, n_roots)."""
    lib = _lib.load()
    err = C.create_string_buffer(1024)
    nn = C.c_int()
    nr = C.c_int()
    status = lib.cn_dag_check(blob, len(blob), C.byref(nn), C.byref(nr), err, len(err))
    if status != 0:
        raise _lib.CnError(status, err.value.decode())
    return nn.value, nr.value
