"""Row-chunking knobs of the pair-track layers.

Public names, fields, defaults and thresholds follow the reference's ``bionemo_ir/_torch/utils/auto_chunk.py``
(``ChunkPolicy`` l.108-151, the registry l.154-229, ``chunk_apply`` l.232-389, the memory-scaled threshold
l.42-81), because callers configure the layers through them.  Chunking never changes a result here: pair rows are
independent in the attention (given the triangle bias) and in the transition, so a chunked call only bounds the
size of the workspaces.
"""

from __future__ import annotations

import dataclasses
import functools
import math
from collections.abc import Callable, Iterator

import torch

DEFAULT_PAIR_CHUNK_ROWS = 512
DEFAULT_AUTOCHUNK_MIN_REF = 2560  # tokens above which an 80 GB GPU starts chunking
AUTOCHUNK_MIN_AUTO = -1           # ChunkPolicy.min_size value that selects the memory-scaled threshold

PAIR_TRANSITION = "pair_transition"
TRIANGLE_ATTENTION = "triangle_attention"


def _threshold_for_memory(total_gb: float) -> int:
    """Workspaces grow with the square of the token count, so the threshold grows with the square root of the
    memory: 2560 tokens at 80 GB, in steps of 128, never below 512; small cards (24 GB and less) stop at 1024."""
    steps_of_128 = round(DEFAULT_AUTOCHUNK_MIN_REF * math.sqrt(total_gb / 80.0) / 128)
    tokens = max(512, 128 * int(steps_of_128))
    if total_gb <= 24:
        tokens = min(tokens, 1024)
    return tokens


@functools.lru_cache(maxsize=8)
def default_autochunk_min(device=None) -> int:
    """Token count above which a policy with ``min_size = -1`` chunks, for the given (default: current) GPU."""
    if not torch.cuda.is_available():
        return DEFAULT_AUTOCHUNK_MIN_REF
    try:
        index = torch.cuda.current_device() if device is None else device
        return _threshold_for_memory(torch.cuda.get_device_properties(index).total_memory / 2**30)
    except (RuntimeError, AssertionError, ValueError):
        return DEFAULT_AUTOCHUNK_MIN_REF


def iter_chunks(total: int, chunk: int) -> Iterator[tuple[int, int]]:
    """``(start, length)`` pieces of at most ``chunk`` that cover ``range(total)``."""
    start = 0
    while start < total:
        length = min(chunk, total - start)
        yield start, length
        start += length


@dataclasses.dataclass(frozen=True)
class ChunkPolicy:
    """Rows per chunk, the extent above which chunking starts (``-1``: memory-scaled), the sliced dimension, the
    lowest tensor rank that is chunked at all, and an on/off switch."""

    chunk_size: int = DEFAULT_PAIR_CHUNK_ROWS
    min_size: int = AUTOCHUNK_MIN_AUTO
    dim: int = 1
    min_rank: int = 4
    enabled: bool = True

    def resolved_min_size(self, device=None) -> int:
        return default_autochunk_min(device) if self.min_size < 0 else self.min_size

    def should_chunk_size(self, n: int, device=None) -> bool:
        active = self.enabled and self.chunk_size > 0
        return active and n > self.resolved_min_size(device)

    def should_chunk(self, x: torch.Tensor) -> bool:
        if not torch.is_tensor(x) or x.dim() < max(self.min_rank, self.dim + 1):
            return False
        return self.should_chunk_size(x.shape[self.dim], x.device if x.is_cuda else None)

    def replace(self, **changes) -> "ChunkPolicy":
        return dataclasses.replace(self, **changes)


class ChunkRegistry(dict):
    """Layer kind -> :class:`ChunkPolicy`.  A plain dict plus the three calls callers of the reference use:
    ``register``, ``get`` (inherited) and ``set`` (override fields of a registered policy)."""

    def register(self, name: str, policy: ChunkPolicy, *, overwrite: bool = True) -> ChunkPolicy:
        if overwrite:
            self[name] = policy
        return self.setdefault(name, policy)

    def set(self, name: str, **overrides) -> ChunkPolicy:
        self[name] = self.get(name, ChunkPolicy()).replace(**overrides)
        return self[name]

    def enable(self, name: str) -> ChunkPolicy:
        return self.set(name, enabled=True)

    def disable(self, name: str) -> ChunkPolicy:
        return self.set(name, enabled=False)

    def names(self) -> list[str]:
        return list(self)


CHUNK_REGISTRY = ChunkRegistry()
for _kind in (PAIR_TRANSITION, TRIANGLE_ATTENTION):
    CHUNK_REGISTRY.register(_kind, ChunkPolicy())


def chunk_apply(fn: Callable, *chunked, policy: ChunkPolicy | None = None, cat_dim: int | None = None, **passthrough):
    """``fn(*chunked, **passthrough)`` evaluated piecewise along ``policy.dim`` of the first argument, pieces joined.

    Only tensors that share the first argument's extent along that dimension are sliced; everything else
    (``None``, scalars, tensors of another extent) is handed to every piece whole.  ``fn`` may return one tensor or
    a tuple / list of tensors.
    """
    policy = CHUNK_REGISTRY.get(PAIR_TRANSITION) if policy is None else policy
    lead = chunked[0] if chunked else None
    if lead is None or policy is None or not policy.should_chunk(lead):
        return fn(*chunked, **passthrough)
    dim, extent = policy.dim, lead.shape[policy.dim]

    def piece_of(arg, start, length):
        sliceable = torch.is_tensor(arg) and arg.dim() > dim and arg.shape[dim] == extent
        return arg.narrow(dim, start, length) if sliceable else arg

    pieces = [fn(*(piece_of(a, s, n) for a in chunked), **passthrough) for s, n in iter_chunks(extent, policy.chunk_size)]
    join = dim if cat_dim is None else cat_dim
    if isinstance(pieces[0], (tuple, list)):
        return type(pieces[0])(torch.cat(parts, dim=join) for parts in zip(*pieces))
    return torch.cat(pieces, dim=join)
