"""Attention-backend plug point and pair-mask precompute registry.

Mirrors the reference's ``bionemo_ir/_torch/attention_backend/interface.py:53-95`` (``AttentionBackend``,
``AttentionMetadata``) and ``utils.py:136-391`` (``get_attention_backend``, ``create_attention``,
``PrecomputedPairMasks``, ``precompute_pair_masks``, ``register_precompute_pair_masks``).

The reference selects between six triangle-attention backends by name.  Here every name maps to the one
sm_100a kernel; the names stay valid because callers also hand them to :func:`precompute_pair_masks`,
whose output form depends on the name (additive bias for ``VANILLA``/``SDPA``/``CUEQUIV``, ``int32`` row
lengths for ``CuTeDSL``/``ClaudeKit``/``Heuristic``).  The kernel consumes row lengths, so an additive
bias is converted on the fly (``valid = bias >= 0``), exactly as the reference's router does
(``triangle_attention/heuristic.py:166-189``).
"""

from __future__ import annotations

import enum
import math
import os
from collections.abc import Callable
from dataclasses import dataclass

import torch

from .. import _lib, ops

DEBUG_ASSERTS = os.environ.get("B200TA_DEBUG_ASSERTS", os.environ.get("BIOIR_DEBUG_ASSERTS", "0")) == "1"

TRIANGLE_BACKENDS = ("VANILLA", "SDPA", "CUEQUIV", "CuTeDSL", "ClaudeKit", "Heuristic")
_LENGTH_BACKENDS = ("CuTeDSL", "ClaudeKit", "Heuristic")


@dataclass
class AttentionMetadata:
    bias_cache: dict[str, torch.Tensor] | None = None
    query_to_keys: Callable | None = None
    qkv_packed: bool = True  # accepted for compatibility with the reference's left-mask metadata; unused


class AttentionType(str, enum.Enum):
    TRIANGLE = "triangle"
    PAIRWISE = "pairwise"


def triangle_bias_pad_multiple(backend_name: str) -> int:
    """Keys of the triangle bias are padded to a multiple of 8 (16 bytes) for every backend name here."""
    return 8


def mask_to_lengths(mask_bias: torch.Tensor, batch: int, rows: int) -> torch.Tensor:
    """Row lengths ``[B, R]`` (int32) from any of the accepted mask forms.

    ``int32`` lengths of shape ``[B, R]``, ``[B*R]`` or ``[B]`` pass through (``[B]`` is broadcast over rows);
    an additive bias ``[B, R, 1, 1, S]`` (0 for valid keys, a large negative number otherwise) is reduced
    with ``(bias >= 0).sum(-1)``.  Masks must be left-aligned (``1…1 0…0``); with ``B200TA_DEBUG_ASSERTS=1``
    that is checked (host synchronisation, so not under stream capture).
    """
    if mask_bias.dtype == torch.int32:
        if mask_bias.numel() == batch * rows:
            return mask_bias.reshape(batch, rows)
        if mask_bias.numel() == batch:
            return mask_bias.reshape(batch, 1).expand(batch, rows)
        raise ValueError(f"int32 row lengths must hold B*R={batch * rows} or B={batch} values, got {tuple(mask_bias.shape)}")
    if mask_bias.dim() == 5:
        valid = mask_bias[:, :, 0, 0, :] >= 0
    elif mask_bias.dim() == 3:
        valid = mask_bias >= 0
    else:
        raise ValueError(f"additive mask bias must be [B, R, 1, 1, S] or [B, R, S], got {tuple(mask_bias.shape)}")
    if valid.shape[0] != batch or valid.shape[1] != rows:
        raise ValueError(f"mask bias {tuple(mask_bias.shape)} does not match B={batch}, R={rows}")
    if DEBUG_ASSERTS and not torch.cuda.is_current_stream_capturing():
        if not bool(torch.all(valid[..., :-1] >= valid[..., 1:])):
            raise ValueError("the triangle-attention kernel needs left-aligned (1…1 0…0) key masks")
    return valid.sum(dim=-1).to(torch.int32)


class AttentionBackend:
    """Base class of attention backends (constructor and ``forward`` signature of the reference)."""

    Metadata = AttentionMetadata

    def __init__(self, layer_idx: int, num_heads: int, head_dim: int, num_kv_heads: int | None = None):
        self.layer_idx = layer_idx
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.num_kv_heads = num_kv_heads or num_heads

    def forward(self, q, k, v, biases=None, metadata=None, **kwargs) -> torch.Tensor:
        raise NotImplementedError


class B200TriangleAttention(AttentionBackend):
    """The single triangle-attention backend: ``b200ta_attention`` on strided views of q, k, v.

    ``forward(q, k, v, biases=[mask_bias, triangle_bias], metadata=None, output=None, use_kv_lengths=…,
    output_lse=None)`` with ``q/k/v`` of shape ``[B, I, J, H*D]`` (views of one in-projection buffer are
    fine: only the innermost stride must be 1 and the others multiples of 8 elements) returns
    ``[B, I, J, H, D]`` like the reference's backends
    (``bionemo_ir/_torch/attention_backend/triangle_attention/vanilla.py:29-73``).
    """

    empty_row_mode = _lib.EMPTY_ROW_UNIFORM

    def __init__(self, layer_idx: int, num_heads: int, head_dim: int, num_kv_heads: int | None = None):
        super().__init__(layer_idx, num_heads, head_dim, num_kv_heads)
        if (self.num_heads, self.head_dim, self.num_kv_heads) != (ops.HEADS, ops.HEAD_DIM, ops.HEADS):
            raise ValueError(
                f"the sm_100a triangle-attention kernel is specialised for {ops.HEADS} heads of {ops.HEAD_DIM}; "
                f"got num_heads={num_heads}, head_dim={head_dim}, num_kv_heads={self.num_kv_heads}"
            )

    def forward(self, q, k, v, biases=None, metadata=None, **kwargs) -> torch.Tensor:
        output = kwargs.get("output")
        lse = kwargs.get("output_lse")
        if q.dim() != 4:
            raise ValueError(f"q must be [B, I, J, H*D], got {tuple(q.shape)}")
        B, I, J, HD = q.shape
        if HD != ops.HEADS * ops.HEAD_DIM:
            raise ValueError(f"q last dimension must be {ops.HEADS * ops.HEAD_DIM}")
        for name, t in (("q", q), ("k", k), ("v", v)):
            if not t.is_cuda or t.dtype != torch.bfloat16:
                raise ValueError(f"{name} must be a CUDA bfloat16 tensor")
            if t.shape != q.shape or t.stride() != q.stride() or t.stride(-1) != 1:
                raise ValueError("q, k, v must share shape and strides, with unit innermost stride")
        if q.stride(0) != I * q.stride(1):
            raise ValueError("q, k, v must be contiguous over (B, I)")
        mask_bias, tri_bias = (biases or [None, None])[:2] if biases else (None, None)
        lengths = None if mask_bias is None else mask_to_lengths(mask_bias, B, I).contiguous()
        if tri_bias is None:
            bias2 = torch.zeros((B, ops.HEADS, J, ops.pad8(J)), dtype=torch.bfloat16, device=q.device)
        else:
            if tri_bias.shape[-1] % 8 != 0:
                tri_bias = torch.nn.functional.pad(tri_bias, (0, -tri_bias.shape[-1] % 8))
            bias2 = (tri_bias.float() * ops.BIAS_SCALE).to(torch.bfloat16).contiguous()  # kernel wants bias / scale
        if output is None:
            output = torch.empty((B * I, J, ops.HEADS, ops.HEAD_DIM), dtype=torch.bfloat16, device=q.device)
        o4 = output.view(B * I, J, ops.HEADS, ops.HEAD_DIM)
        ls = (lengths.stride(0), lengths.stride(1)) if lengths is not None else (0, 0)
        _lib.call(
            "b200ta_attention", q.data_ptr(), k.data_ptr(), v.data_ptr(), None,
            q.stride(1), ops.HEAD_DIM, q.stride(2),
            bias2.data_ptr(), bias2.stride(0), bias2.stride(1), bias2.stride(2),
            None if lengths is None else lengths.data_ptr(), *ls,
            o4.data_ptr(), o4.stride(0), o4.stride(1), o4.stride(2),
            None if lse is None else lse.data_ptr(), 1.0 / math.sqrt(self.head_dim), int(self.empty_row_mode),
            B, I, J, bias2.shape[-1], torch.cuda.current_stream().cuda_stream,
        )
        return o4.view(B, I, J, ops.HEADS, ops.HEAD_DIM)


def get_attention_backend(backend_name: str, attention_type: AttentionType = AttentionType.TRIANGLE):
    if attention_type != AttentionType.TRIANGLE:
        raise ValueError(f"only triangle attention is provided here, not {attention_type}")
    if backend_name not in TRIANGLE_BACKENDS:
        raise ValueError(f"Invalid triangle attention backend {backend_name!r}; available: {sorted(TRIANGLE_BACKENDS)}")
    return B200TriangleAttention


def create_attention(backend_name: str, layer_idx: int, num_heads: int, head_dim: int,
                     num_kv_heads: int | None = None, attention_type: AttentionType = AttentionType.TRIANGLE):
    return get_attention_backend(backend_name, attention_type)(layer_idx, num_heads, head_dim, num_kv_heads)


# ---------------------------------------------------------------------------- pair-mask precompute


@dataclass
class PrecomputedPairMasks:
    """Per-row masks computed once per stack: the original ``[B, I, J]`` mask, its row payload for the
    starting node and the payload of the transposed mask for the ending node."""

    pair_mask: torch.Tensor
    mask_bias: torch.Tensor
    mask_bias_transposed: torch.Tensor
    value_mask: torch.Tensor | None = None


PrecomputePairMasksFn = Callable[[torch.Tensor, float, "torch.dtype | None"], PrecomputedPairMasks]
_PRECOMPUTE_PAIR_MASKS_REGISTRY: dict[str, PrecomputePairMasksFn] = {}


def register_precompute_pair_masks(backend_name: str, fn: PrecomputePairMasksFn) -> None:
    _PRECOMPUTE_PAIR_MASKS_REGISTRY[backend_name] = fn


def precompute_pair_masks(backend_name: str, pair_mask: torch.Tensor, inf: float = 1e9,
                          dtype: torch.dtype | None = None, activation_dtype: torch.dtype | None = None):
    fn = _PRECOMPUTE_PAIR_MASKS_REGISTRY.get(backend_name)
    if fn is None:
        raise ValueError(f"No precompute_pair_masks registered for backend '{backend_name}'. "
                         f"Available: {sorted(_PRECOMPUTE_PAIR_MASKS_REGISTRY.keys())}")
    result = fn(pair_mask, inf, dtype)
    if activation_dtype is not None:
        result.value_mask = pair_mask.unsqueeze(-1).to(activation_dtype)
    return result


def _additive_precompute(pair_mask, inf=1e9, dtype=None):
    m = pair_mask.to(dtype) if dtype is not None and pair_mask.dtype != dtype else pair_mask
    bias = (inf * (m - 1))[..., :, None, None, :]
    bias_t = (inf * (m.transpose(-2, -1) - 1))[..., :, None, None, :].contiguous()
    return PrecomputedPairMasks(pair_mask=pair_mask, mask_bias=bias, mask_bias_transposed=bias_t)


def _length_precompute(pair_mask, inf=1e9, dtype=None):
    del inf, dtype
    mb = pair_mask > 0.5
    if DEBUG_ASSERTS and not torch.cuda.is_current_stream_capturing():
        if not (bool(torch.all(mb[..., :-1] >= mb[..., 1:])) and bool(torch.all(mb[..., :-1, :] >= mb[..., 1:, :]))):
            raise ValueError("precompute_pair_masks needs a left-aligned (1…1 0…0) pair_mask along both pair axes")
    return PrecomputedPairMasks(pair_mask=pair_mask, mask_bias=mb.sum(dim=-1).to(torch.int32).contiguous(),
                                mask_bias_transposed=mb.sum(dim=-2).to(torch.int32).contiguous())


for _name in TRIANGLE_BACKENDS:
    register_precompute_pair_masks(_name, _length_precompute if _name in _LENGTH_BACKENDS else _additive_precompute)


# ---- single-track masks (AttentionPairBias) -----------------------------------------------------------------------


@dataclass
class PrecomputedSingleMasks:
    """The single mask ``[*, I]`` in the form the attention consumes, computed once before the layer loop
    (reference: ``PrecomputedSingleMasks``, bionemo_ir/_torch/attention_backend/utils.py:399-426)."""

    single_mask: torch.Tensor
    mask_bias: torch.Tensor
    mask_bias_local: torch.Tensor | None = None
    excluded: torch.Tensor | None = None
    value_mask: torch.Tensor | None = None


PrecomputeSingleMasksFn = Callable[[torch.Tensor, float], PrecomputedSingleMasks]
_PRECOMPUTE_SINGLE_MASKS_REGISTRY: dict[str, PrecomputeSingleMasksFn] = {}


def register_precompute_single_masks(backend_name: str, fn: PrecomputeSingleMasksFn) -> None:
    _PRECOMPUTE_SINGLE_MASKS_REGISTRY[backend_name] = fn


def precompute_single_masks(backend_name: str, single_mask: torch.Tensor, inf: float = 1e9, query_to_keys=None,
                            activation_dtype: torch.dtype | None = None) -> PrecomputedSingleMasks:
    """Same dispatch as the reference (utils.py:441-483).  ``query_to_keys`` (sequence-local attention) is not
    supported by the sm_100a single track and raises."""
    fn = _PRECOMPUTE_SINGLE_MASKS_REGISTRY.get(backend_name)
    if fn is None:
        raise ValueError(f"No precompute_single_masks registered for backend '{backend_name}'. "
                         f"Available: {sorted(_PRECOMPUTE_SINGLE_MASKS_REGISTRY.keys())}")
    if query_to_keys is not None:
        raise ValueError("sequence-local attention (query_to_keys) is not supported by the sm_100a single track")
    result = fn(single_mask, inf)
    if activation_dtype is not None:
        valid = single_mask.unsqueeze(-1)
        result.excluded = ~valid.to(torch.bool)
        result.value_mask = valid.to(activation_dtype)
    return result


def _additive_single(single_mask: torch.Tensor, inf: float = 1e9) -> PrecomputedSingleMasks:
    return PrecomputedSingleMasks(single_mask, ((1 - single_mask.float()) * -inf)[..., None, None, :])


def _length_single(single_mask: torch.Tensor, inf: float = 1e9) -> PrecomputedSingleMasks:
    del inf
    return PrecomputedSingleMasks(single_mask, (single_mask.float() > 0.5).sum(dim=-1, dtype=torch.int32).reshape(-1))


for _name in ("VANILLA", "SDPA"):
    register_precompute_single_masks(_name, _additive_single)
for _name in ("CuTeDSL", "Heuristic"):
    register_precompute_single_masks(_name, _length_single)
