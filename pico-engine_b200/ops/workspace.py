"""Scratch memory of kernels that need global memory beyond their inputs and outputs.

One buffer per purpose and device, allocated on first use and kept; when a purpose needs
more, a larger buffer is added and the old one stays alive, because a captured CUDA graph may
still hold its address.  Kernels of one purpose run one after another on one stream and may
share their buffer.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

_buffers: Dict[Tuple[str, int], List[torch.Tensor]] = {}


def scratch(purpose: str, nbytes: int, device: torch.device, zeroed: bool = False) -> torch.Tensor:
    """A uint8 buffer of at least ``nbytes``.  ``zeroed`` buffers are zero when first handed
    out; their users leave them zero."""
    key = (purpose, device.index or 0)
    have = _buffers.setdefault(key, [])
    if have and have[-1].numel() >= nbytes:
        return have[-1]
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError(f"scratch for {purpose!r} would have to grow to {nbytes} bytes during graph capture; "
                           f"run the step once without capture first")
    size = max(nbytes, 2 * have[-1].numel() if have else 1 << 20)
    buf = torch.zeros(size, dtype=torch.uint8, device=device) if zeroed else \
        torch.empty(size, dtype=torch.uint8, device=device)
    have.append(buf)
    return buf
