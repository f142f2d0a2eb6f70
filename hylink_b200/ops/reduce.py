"""Landing reduce: ``dst = scale * op(src_0..src_{k-1})`` in one pass."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from .._native import OPS, check, lib, torch_dtype_code


def reduce_landing(dst: torch.Tensor, srcs: Sequence[torch.Tensor], op: str = "sum", scale: float = 1.0,
                   accumulate: bool = False, blocks: int = 0) -> torch.Tensor:
    """Reduce up to eight same-typed sources into ``dst`` with the sm_100a kernel.

    Sources may be CUDA tensors or pinned host tensors (read over PCIe by the
    kernel itself). With ``accumulate`` the previous content of ``dst`` is the
    first operand.
    """
    if not dst.is_cuda:
        raise ValueError("reduce_landing needs a CUDA destination")
    n = dst.numel()
    arr = (C.c_void_p * len(srcs))()
    for i, s in enumerate(srcs):
        if s.numel() != n or s.dtype != dst.dtype:
            raise ValueError("sources must match the destination's size and dtype")
        if not (s.is_cuda or s.is_pinned()):
            raise ValueError("host sources must be pinned")
        arr[i] = s.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    check(lib.hlReduceLanding(C.c_void_p(dst.data_ptr()), arr, len(srcs), int(accumulate), n,
                              torch_dtype_code(dst.dtype), OPS[op], scale, blocks, C.c_void_p(stream)),
          "hlReduceLanding")
    return dst
