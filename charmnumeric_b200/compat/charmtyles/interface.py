"""``charmtyles.interface.CCSInterface`` is the base class of the reference's interface
(charmnumeric/interface.py:9-12); here the interface owns the GPU context directly."""
from charmnumeric_b200.frontend import CharmNumericInterface as CCSInterface  # noqa: F401
