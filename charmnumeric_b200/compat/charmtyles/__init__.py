"""Import shim for the two charmtyles modules that programs written against the reference
import directly (``charmtyles.core``: execute, set_auto_flush; ``charmtyles.interface``)."""
