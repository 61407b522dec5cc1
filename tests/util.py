"""Small helpers shared by the tests."""
from __future__ import annotations

import hashlib

import numpy as np
import torch

MODES = ("fast", "balanced", "accurate", "max", "quality")


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 / fp16 tensor -> uint16 bit patterns, flat."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)


def from_bits(a: np.ndarray, dtype=torch.bfloat16) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(dtype)


def sha(a) -> str:
    if isinstance(a, torch.Tensor):
        a = bits(a) if a.dtype in (torch.bfloat16, torch.float16) else a.detach().cpu().contiguous().numpy()
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
