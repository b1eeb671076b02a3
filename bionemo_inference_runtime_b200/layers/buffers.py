"""Shared pre-allocated buffer dict, as ``bionemo_ir/runtime/buffers.py:38-75`` of the reference."""

from __future__ import annotations

import torch

PreallocatedBuffers = dict[str, torch.Tensor]


def ensure_buffer(buffers: PreallocatedBuffers | None, key: str, shape: tuple, dtype: torch.dtype,
                  device: torch.device) -> torch.Tensor | None:
    """Return the buffer stored under ``key``, reallocating only when shape, dtype or device changed;
    ``None`` when no dict was passed (the caller then allocates for itself)."""
    if buffers is None:
        return None
    buf = buffers.get(key)
    shape = tuple(shape)
    if buf is not None and tuple(buf.shape) == shape and buf.dtype == dtype and buf.device == device:
        return buf
    buf = torch.empty(shape, dtype=dtype, device=device)
    buffers[key] = buf
    return buf
