"""Process-level plumbing: the ``torch.distributed`` backend, a ctypes
communicator for use without torch.distributed, NCCL point-to-point helpers
for pipeline stages, and a DDP wrapper that folds the gradient average into
the all-reduce kernel."""
from .backend import register_backend, backend_stats, set_fused_scale  # noqa: F401
from .comm import Communicator  # noqa: F401
