"""Device ops exposed to Python: the emulated multi-rank NVLink group (all
cross-rank kernels on one GPU) and the landing reduce."""
from .emu import EmuGroup  # noqa: F401
from .reduce import reduce_landing  # noqa: F401
