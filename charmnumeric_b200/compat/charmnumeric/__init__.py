"""Import shim: ``import charmnumeric as cnp`` resolves to the B200 backend's frontend, so that
programs written against the reference package run without edits.  Put the parent directory
of this package on PYTHONPATH (``PYTHONPATH=charmnumeric_b200/compat python program.py``)."""
from charmnumeric_b200 import *  # noqa: F401,F403
from charmnumeric_b200 import (  # noqa: F401
    Array, ArrayView, CharmNumericInterface, DType, LocalCluster, __version__, abs, dtype, e, float32,
    float64, int32, int64, ndarray, newaxis, pi, random, sum)
