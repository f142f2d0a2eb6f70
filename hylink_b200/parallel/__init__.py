"""Process-level plumbing: the ``torch.distributed`` backend, a ctypes
communicator for use without torch.distributed, NCCL point-to-point helpers
for pipeline stages, and a DDP wrapper that folds the gradient average into
the all-reduce kernel; and the parallelism schemes that consume the collectives
(tensor / sequence parallel layers, sharded optimizer, expert-parallel MoE,
Ulysses and all-gather context-parallel attention, a GPipe schedule)."""
from .backend import (register_backend, backend_stats, set_fused_scale, set_cta_budget, symmetric_empty,  # noqa: F401
                      is_registered, registered_mem_pool)
from .comm import Communicator  # noqa: F401
