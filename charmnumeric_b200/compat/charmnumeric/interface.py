"""``charmnumeric.interface`` of the reference (charmnumeric/interface.py:12-129)."""
from charmnumeric_b200 import CharmNumericInterface, LocalCluster  # noqa: F401
