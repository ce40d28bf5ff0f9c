"""``charmnumeric.random`` of the reference, plus the seeded uniform generator."""
from charmnumeric_b200.random import *  # noqa: F401,F403
