"""Row-chunking knobs of the pair-track layers.

Mirrors ``bionemo_ir/_torch/utils/auto_chunk.py:42-389`` of the reference (same names, fields and
thresholds) for the two policies this package uses.  Chunking never changes results: pair rows
are independent in both the attention and the transition, so a chunked call only bounds the size
of the workspaces.
"""

from __future__ import annotations

import functools
import math
from collections.abc import Callable, Iterator
from dataclasses import dataclass, replace

import torch

DEFAULT_PAIR_CHUNK_ROWS = 512
_REFERENCE_GPU_GB = 80.0
DEFAULT_AUTOCHUNK_MIN_REF = 2560
_AUTOCHUNK_MIN_FLOOR = 512
AUTOCHUNK_MIN_AUTO = -1

PAIR_TRANSITION = "pair_transition"
TRIANGLE_ATTENTION = "triangle_attention"


@functools.lru_cache(maxsize=8)
def default_autochunk_min(device=None) -> int:
    """Memory-scaled threshold: 2560 tokens on an 80 GB GPU, scaled by sqrt(memory), rounded to 128."""
    try:
        if not torch.cuda.is_available():
            return DEFAULT_AUTOCHUNK_MIN_REF
        if device is None:
            device = torch.cuda.current_device()
        total_gb = torch.cuda.get_device_properties(device).total_memory / (1024**3)
        scaled = DEFAULT_AUTOCHUNK_MIN_REF * math.sqrt(total_gb / _REFERENCE_GPU_GB)
        threshold = max(_AUTOCHUNK_MIN_FLOOR, int(round(scaled / 128) * 128))
        return min(threshold, 1024) if total_gb <= 24 else threshold
    except Exception:
        return DEFAULT_AUTOCHUNK_MIN_REF


def iter_chunks(total: int, chunk: int) -> Iterator[tuple[int, int]]:
    """Yield ``(start, length)`` covering ``range(total)`` in steps of ``chunk``."""
    for start in range(0, total, chunk):
        yield start, min(chunk, total - start)


@dataclass(frozen=True)
class ChunkPolicy:
    """When and how much to chunk: rows per chunk, the size above which chunking starts
    (``-1`` = memory-scaled default), the sliced dimension, the minimum tensor rank and a switch."""

    chunk_size: int = DEFAULT_PAIR_CHUNK_ROWS
    min_size: int = AUTOCHUNK_MIN_AUTO
    dim: int = 1
    min_rank: int = 4
    enabled: bool = True

    def resolved_min_size(self, device=None) -> int:
        return self.min_size if self.min_size >= 0 else default_autochunk_min(device)

    def should_chunk_size(self, n: int, device=None) -> bool:
        return self.enabled and self.chunk_size > 0 and n > self.resolved_min_size(device)

    def should_chunk(self, x: torch.Tensor) -> bool:
        if not (self.enabled and self.chunk_size > 0 and torch.is_tensor(x) and x.dim() >= self.min_rank
                and x.dim() > self.dim):
            return False
        device = x.device if x.is_cuda else None
        return x.shape[self.dim] > self.resolved_min_size(device)

    def replace(self, **changes) -> "ChunkPolicy":
        return replace(self, **changes)


class ChunkRegistry:
    """Name -> :class:`ChunkPolicy` map for chunkable layers."""

    def __init__(self) -> None:
        self._policies: dict[str, ChunkPolicy] = {}

    def register(self, name: str, policy: ChunkPolicy, *, overwrite: bool = True) -> ChunkPolicy:
        if not overwrite and name in self._policies:
            return self._policies[name]
        self._policies[name] = policy
        return policy

    def get(self, name: str, default: ChunkPolicy | None = None) -> ChunkPolicy | None:
        return self._policies.get(name, default)

    def set(self, name: str, **overrides) -> ChunkPolicy:
        policy = (self._policies.get(name) or ChunkPolicy()).replace(**overrides)
        self._policies[name] = policy
        return policy

    def enable(self, name: str) -> ChunkPolicy:
        return self.set(name, enabled=True)

    def disable(self, name: str) -> ChunkPolicy:
        return self.set(name, enabled=False)

    def names(self) -> list[str]:
        return list(self._policies)

    def __contains__(self, name: str) -> bool:
        return name in self._policies

    def __getitem__(self, name: str) -> ChunkPolicy:
        return self._policies[name]


CHUNK_REGISTRY = ChunkRegistry()
CHUNK_REGISTRY.register(PAIR_TRANSITION, ChunkPolicy(chunk_size=DEFAULT_PAIR_CHUNK_ROWS, dim=1, min_rank=4))
CHUNK_REGISTRY.register(TRIANGLE_ATTENTION, ChunkPolicy(chunk_size=DEFAULT_PAIR_CHUNK_ROWS, dim=1, min_rank=4))


def chunk_apply(fn: Callable, *chunked, policy: ChunkPolicy | None = None, cat_dim: int | None = None, **passthrough):
    """Evaluate ``fn(*chunked, **passthrough)`` in slices along ``policy.dim`` and concatenate.

    Tensors whose extent along ``policy.dim`` differs from the first argument's, ``None`` and
    non-tensors pass through unsliced.
    """
    if policy is None:
        policy = CHUNK_REGISTRY.get(PAIR_TRANSITION)
    primary = chunked[0] if chunked else None
    if primary is None or policy is None or not policy.should_chunk(primary):
        return fn(*chunked, **passthrough)
    dim = policy.dim
    total = primary.shape[dim]
    outs = []
    for start, length in iter_chunks(total, policy.chunk_size):
        args = [
            a.narrow(dim, start, length) if torch.is_tensor(a) and a.dim() > dim and a.shape[dim] == total else a
            for a in chunked
        ]
        outs.append(fn(*args, **passthrough))
    cat = dim if cat_dim is None else cat_dim
    if isinstance(outs[0], (tuple, list)):
        return type(outs[0])(torch.cat([o[i] for o in outs], dim=cat) for i in range(len(outs[0])))
    return torch.cat(outs, dim=cat)
