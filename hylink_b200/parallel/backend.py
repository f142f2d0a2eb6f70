"""Registration of the ``hylink`` backend with ``torch.distributed``.

After :func:`register_backend`, ``dist.init_process_group(backend="hylink")``
(or ``"cuda:hylink,cpu:gloo"``) routes all-reduce, broadcast, all-gather,
reduce-scatter, all-to-all and barrier through this library. The C++ side is
``csrc/torch/backend.cpp``.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
from pathlib import Path

_ext = None


def _load_ext():
    global _ext
    if _ext is not None:
        return _ext
    import torch  # noqa: F401  (registers the c10d base classes with pybind)
    import torch.distributed  # noqa: F401

    from .. import _native  # noqa: F401  (loads libhylink_b200.so first)

    path = Path(__file__).resolve().parent.parent / "lib" / "_hylink_c10d.so"
    if not path.exists():
        from .. import _build

        _build.build_torch_ext()
    loader = importlib.machinery.ExtensionFileLoader("_hylink_c10d", str(path))
    spec = importlib.util.spec_from_loader("_hylink_c10d", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    _ext = mod
    return mod


_registered = False


def register_backend() -> None:
    """Make ``backend="hylink"`` known to ``torch.distributed`` (idempotent)."""
    global _registered
    if _registered:
        return
    import torch.distributed as dist

    ext = _load_ext()
    dist.Backend.register_backend("hylink", ext.create_backend, devices=["cuda", "cpu"])
    _registered = True


def _backend_of(group=None):
    import torch
    import torch.distributed as dist

    pg = group if group is not None else dist.group.WORLD
    dev = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    return pg._get_backend(dev)


def backend_stats(group=None) -> dict:
    """Counters of the group's communicator: calls, bytes per path, kernel launches, split ratio."""
    return dict(_load_ext().backend_stats(_backend_of(group)))


def set_fused_scale(scale: float, group=None) -> None:
    """Multiply every all-reduce result by ``scale`` inside the kernel (0 switches it off)."""
    _load_ext().set_fused_scale(_backend_of(group), float(scale))


def set_cta_budget(ctas: int, group=None) -> int:
    """Limit the CTAs a collective of this group may occupy (0 = the library's size table); returns the old limit.

    A collective that overlaps with compute kernels finishes sooner on every SM but holds those kernels back for
    longer than it saves; callers that overlap (a DDP backward pass) therefore give the collectives a budget and
    leave the other SMs to the compute stream. Stand-alone collectives run fastest with no budget.
    """
    return int(_load_ext().set_cta_budget(_backend_of(group), int(ctas)))


def symmetric_empty(shape, dtype=None, group=None, device=None):
    """An uninitialised CUDA tensor in the group's registered memory.

    Registered buffers sit at the same offset of a symmetric heap on every rank; collectives whose buffers are
    registered run zero-copy (peers' inputs read and peers' outputs written in place through NVLink / NVSwitch).
    Every rank must call this in the same order with the same sizes, and release the tensors in the same order.
    """
    import torch

    if isinstance(shape, int):
        shape = (shape,)
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    return _load_ext().symmetric_empty(_backend_of(group), list(shape), dtype or torch.float32, dev)


def is_registered(tensor, group=None) -> bool:
    """Whether the tensor lies in the group's registered memory."""
    return bool(_load_ext().is_registered(_backend_of(group), tensor))


_pool = None


def registered_mem_pool():
    """A ``torch.cuda.MemPool`` whose memory is registered with the group of the ``hylink`` backend.

    Tensors created under ``torch.cuda.use_mem_pool(pool)`` (for instance the gradient buckets of a
    ``DistributedDataParallel`` wrapper built there) come from the symmetric heap, so collectives on them run
    zero-copy. All ranks must allocate in the same order, which any SPMD program does. The process group's
    communicator must exist (one collective has run) before the first allocation.
    """
    global _pool
    if _pool is None:
        import torch
        from torch.cuda.memory import CUDAPluggableAllocator

        from .. import _native

        alloc = CUDAPluggableAllocator(str(_native._LIB_PATH), "hlTorchAlloc", "hlTorchFree")
        _pool = (torch.cuda.MemPool(alloc.allocator()), alloc)
    return _pool[0]
