"""Pipeline point-to-point traffic stays on NCCL.

The collective backend does not re-implement send/recv: a side NCCL process
group carries them on its own stream so that they overlap with this library's
collectives (the reference likewise leaves ``ncclSend``/``ncclRecv`` to the
vendor library: multipath-orchestrator/libampccl/hook/nccl_hook.cc:637-646 and
pcie-ccl-cuda/src/api/nccl_compat/nccl_hook.cpp:730-740).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_p2p_group = None


def p2p_group():
    """The NCCL group used for send/recv (created collectively on first use)."""
    global _p2p_group
    if _p2p_group is None:
        # NCCL between GPUs; gloo when the job runs on CPU tensors (tests on a machine without a GPU)
        _p2p_group = dist.new_group(backend="nccl" if torch.cuda.is_available() else "gloo")
    return _p2p_group


def send(t: torch.Tensor, dst: int):
    return dist.send(t, dst, group=p2p_group())


def recv(t: torch.Tensor, src: int):
    return dist.recv(t, src, group=p2p_group())


def isend(t: torch.Tensor, dst: int):
    return dist.isend(t, dst, group=p2p_group())


def irecv(t: torch.Tensor, src: int):
    return dist.irecv(t, src, group=p2p_group())


def batch_isend_irecv(ops):
    """``ops``: list of ("send"|"recv", tensor, peer)."""
    g = p2p_group()
    reqs = [dist.P2POp(dist.isend if k == "send" else dist.irecv, t, peer, group=g) for k, t, peer in ops]
    return dist.batch_isend_irecv(reqs)
