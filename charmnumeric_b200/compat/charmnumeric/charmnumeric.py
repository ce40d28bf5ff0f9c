"""``charmnumeric.charmnumeric`` of the reference: the array classes and constructors."""
from charmnumeric_b200 import (  # noqa: F401
    Array, ArrayOperation, ArrayView, DType, arange, array, asarray, copy, copyto, create_array, empty,
    empty_like, eye, full, full_like, identity, ones, ones_like, zeros, zeros_like)
