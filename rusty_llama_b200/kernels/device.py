"""What the dispatch rules need to know about the GPU they plan for."""

from __future__ import annotations

from functools import lru_cache

import torch

# the part the block targets in `linear.py` and `parts/attention.py` were measured on
B200_SM_COUNT = 148


@lru_cache(maxsize=None)
def _sm_count(index: int) -> int:
    return int(torch.cuda.get_device_properties(index).multi_processor_count)


def sm_count(device=None) -> int:
    """Streaming multiprocessors of `device` (default: the current CUDA device); the B200's count where
    there is no CUDA device to ask (planning on a CPU, as the shape-only tests do)."""
    if not torch.cuda.is_available():
        return B200_SM_COUNT
    if device is None:
        index = torch.cuda.current_device()
    else:
        device = torch.device(device)
        if device.type != "cuda":
            return B200_SM_COUNT
        index = torch.cuda.current_device() if device.index is None else device.index
    return _sm_count(index)
