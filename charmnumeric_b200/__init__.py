"""charmnumeric on B200: the reference's lazy ndarray API over a CUDA (sm_100a) backend.

The public names mirror ``charmnumeric/__init__.py`` of the reference; ``sqrt``, ``abs``,
``sum``, ``dot2d`` and ``random.uniform`` are additions.  Everything executes through
``libcnb200.so`` (see ``include/cnb200.h``); there is no other execution path.
"""
from . import random  # noqa: F401
from .context import Context, comm_unique_id, dag_check, group_compile_check, partition  # noqa: F401
from .frontend import (  # noqa: F401
    Array, ArrayOperation, ArrayView, CharmNumericInterface, DType, LocalCluster, add, arange, array, asarray,
    copy, copyto, create_array, diag, divide, dot, dot2d, empty, empty_like, execute, exp, eye, full,
    full_like, identity, matmul, multiply, norm2, ones, ones_like, reset_frontend_state,
    set_auto_flush, subtract, tanh, tile, sqrt, zeros, zeros_like)
from .frontend import absolute as abs  # noqa: A001,F401
from .frontend import sum_all as sum  # noqa: A001,F401


# module-level names of the reference package (charmnumeric/__init__.py:29-39)
import numpy as _np  # noqa: E402

__version__ = "0.1.dev"
float32 = _np.float32
float64 = _np.float64
int32 = _np.int32
int64 = _np.int64
ndarray = Array
dtype = _np.dtype
newaxis = None
pi = _np.pi
e = _np.e
