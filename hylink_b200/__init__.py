"""hylink-b200: a Blackwell-native multipath collective communication library.

Two transports on one 8xB200 node — hand-written sm_100a kernels over
NVLink 5 / NVSwitch peer memory, and a CPU-driven schedule-IR executor that
drives the copy engines through pinned host memory — forked per collective by
an orchestrator that retunes the split online. Public surfaces: the ``hl*`` /
``pccl*`` C API, a drop-in ``nccl*`` symbol layer, and a ``torch.distributed``
backend (``backend="hylink"``).
"""
from ._native import lib, HylinkError, check, DTYPES, OPS  # noqa: F401

__version__ = "0.1.0"
__all__ = ["lib", "HylinkError", "check", "DTYPES", "OPS", "__version__"]
