"""ctypes binding of libcnb200.so (the C ABI declared in include/cnb200.h).

The library is the only execution path: if it is missing or fails to load, importing
this module raises instead of falling back to anything else.
"""
import ctypes as C
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("CNB200_LIB", _HERE / "libcnb200.so"))


class CnError(RuntimeError):
    """A non-zero status from the C ABI; `.status` holds the code."""

    def __init__(self, status, message):
        super().__init__(f"cnb200 status {status} ({status_string(status)}): {message}")
        self.status = status
        self.message = message


class Stats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "kernel_launches", "group_launches", "compiles", "halo_exchanges", "allreduces",
        "fused_reductions", "nodes", "bytes_h2d", "bytes_d2h", "plan_hits", "peer_exchanges", "overlapped_sweeps", "deep_halo_sweeps",
        "inlined_producers", "row_fetches", "halo_pushes", "scalar_tails")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class ArrayMeta(C.Structure):
    """cn_array_meta of include/cnb200.h."""
    _fields_ = [("name", C.c_int32), ("ndims", C.c_int32), ("shape", C.c_int64 * 3), ("offset", C.c_int64 * 3),
                ("tile", C.c_int64), ("decomp_final", C.c_int32), ("reserved", C.c_int32)]


# symbol -> (restype, argtypes); must list every function include/cnb200.h declares
_P = C.c_void_p
_I64P = C.POINTER(C.c_int64)
SIGNATURES = {
    "cn_version": (C.c_int, []),
    "cn_status_string": (C.c_char_p, [C.c_int]),
    "cn_context_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(_P)]),
    "cn_context_destroy": (C.c_int, [_P]),
    "cn_last_error": (C.c_char_p, [_P]),
    "cn_comm_unique_id": (C.c_int, [C.c_char_p]),
    "cn_comm_init": (C.c_int, [_P, C.c_char_p]),
    "cn_mark_rank_failed": (C.c_int, [_P, C.c_int]),
    "cn_receive_dag": (C.c_int, [_P, C.c_int, C.c_int64, C.c_char_p]),
    "cn_get": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, _P]),
    "cn_get_local": (C.c_int, [_P, C.c_int, _I64P, _I64P, C.c_int64, _P]),
    "cn_put": (C.c_int, [_P, C.c_int, C.c_int, _I64P, C.c_int, _P]),
    "cn_get_root": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int, _P]),
    "cn_put_local": (C.c_int, [_P, C.c_int, C.c_int, _I64P, C.c_int, C.c_int64, _P]),
    "cn_execute_node": (C.c_int, [_P, C.c_char_p, C.c_int64]),
    "cn_delete_array": (C.c_int, [_P, C.c_int]),
    "cn_array_info": (C.c_int, [_P, C.c_int, C.POINTER(C.c_int), _I64P, C.POINTER(C.c_int),
                                _I64P, _I64P]),
    "cn_synchronize": (C.c_int, [_P]),
    "cn_compile_group": (C.c_int, [_P, C.c_char_p, C.c_int64, C.POINTER(C.c_uint64)]),
    "cn_group_source": (C.c_int, [_P, C.c_uint64, C.POINTER(C.c_char_p)]),
    "cn_launch_group": (C.c_int, [_P, C.c_uint64, C.c_int, C.POINTER(_P), _I64P, _I64P, C.c_int,
                                  C.POINTER(_P), C.c_int, C.POINTER(_P), _I64P, _I64P, _I64P]),
    "cn_dag_check": (C.c_int, [C.c_char_p, C.c_int64, C.POINTER(C.c_int), C.POINTER(C.c_int),
                               C.c_char_p, C.c_int]),
    "cn_group_compile_check": (C.c_int, [C.c_char_p, C.c_int64, C.c_char_p, C.c_int64, _I64P,
                                         C.c_char_p, C.c_int]),
    "cn_fuse_check": (C.c_int, [C.c_char_p, C.c_int64, C.c_char_p, C.c_int64, C.c_char_p, C.c_int64,
                                C.POINTER(C.c_int), C.c_char_p, C.c_int]),
    "cn_tail_check": (C.c_int, [C.c_char_p, C.c_int64, C.c_char_p, C.c_int64, C.POINTER(C.c_int),
                                C.c_char_p, C.c_int]),
    "cn_region_intersect": (C.c_int, [_I64P, _I64P, _I64P]),
    "cn_region_map": (C.c_int, [_I64P, _I64P, _I64P, _I64P]),
    "cn_plan_row_transfers": (C.c_int, [_I64P, C.c_int64, _I64P, C.c_int64, C.c_int, _I64P, C.c_int64,
                                        _I64P, _I64P]),
    "cn_compute_decompositions": (C.c_int, [C.POINTER(ArrayMeta), C.c_int, C.c_char_p, C.c_int64, C.c_int, C.c_int,
                                            _I64P]),
    "cn_partition": (C.c_int, [C.c_int64, C.c_int, C.c_int, _I64P, _I64P]),
    "cn_timer_start": (C.c_int, [_P]),
    "cn_timer_stop": (C.c_int, [_P, C.POINTER(C.c_float)]),
    "cn_profile_report": (C.c_int, [_P, C.c_char_p, C.c_int64]),
    "cn_dot_noalloc": (C.c_int, [_P, _P, C.c_int64, _P, _P]),
    "cn_get_stats": (C.c_int, [_P, C.POINTER(Stats)]),
    "cn_set_option": (C.c_int, [_P, C.c_char_p, C.c_int64]),
}

_lib = None


def load():
    """Load the shared library (once) and attach the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m charmnumeric_b200.build` "
            "(there is no fallback execution path)")
    lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_string(status):
    return load().cn_status_string(int(status)).decode()


def check(ctx, status):
    if status != 0:
        msg = load().cn_last_error(ctx)
        raise CnError(status, msg.decode() if msg else "")
