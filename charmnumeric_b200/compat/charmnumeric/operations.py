"""``charmnumeric.operations`` of the reference (charmnumeric/operations.py:151-163)."""
from charmnumeric_b200 import (  # noqa: F401
    add, diag, divide, dot, exp, matmul, multiply, norm2, subtract, tanh, tile)
