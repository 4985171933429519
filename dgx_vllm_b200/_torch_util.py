"""torch plumbing shared by the op mirrors: argument checks, dtype codes, stream and workspace."""
from __future__ import annotations

import torch

from . import _lib

_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}
_workspaces: dict = {}


def dtype_code(t: torch.dtype) -> int:
    if t not in _DT:
        raise RuntimeError(f"unsupported dtype {t}")
    return _DT[t]


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("b200 nvfp4 ops take CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    return dev


def require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Grow-only scratch buffer per (device, stream).  Calls issued on one stream serialise on the
    GPU, so sharing it between consecutive ops is safe; its address is stable once large enough,
    which CUDA-graph capture relies on."""
    key = (device.index, stream_ptr(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()
