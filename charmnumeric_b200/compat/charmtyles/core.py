"""``from charmtyles.core import execute, set_auto_flush`` as used by the reference's examples
(examples/multigrid2d.py:15, examples/simple.py:2)."""
from charmnumeric_b200.frontend import execute, reset_frontend_state, set_auto_flush  # noqa: F401
