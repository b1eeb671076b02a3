"""Triangle-attention layers with the reference's module API on the sm_100a kernels.

Drop-in counterparts of ``TriangleAttentionNode`` / ``TriangleAttentionStartingNode`` /
``TriangleAttentionEndingNode`` (``bionemo_ir/_torch/layers/triangle_nodes.py:120-292``) and of
``TriangleAttention`` (``bionemo_ir/_torch/layers/attention.py:82-296``): same constructor arguments, forward
signatures, mask forms, chunking knobs and ``state_dict`` keys.  A node forward is three kernel launches
(prologue, attention, epilogue; see ``include/b200ta.h``); the ending node runs the same kernels on the
transposed pair tensor through swapped strides and returns a tensor in the caller's ``[B, I, J, c]`` layout.
"""

from __future__ import annotations

from enum import IntEnum

import torch
import torch.nn as nn

from .. import _lib, ops
from .attention_backend import (AttentionMetadata, AttentionType, create_attention, mask_to_lengths,
                                triangle_bias_pad_multiple)
from .auto_chunk import CHUNK_REGISTRY, TRIANGLE_ATTENTION, ChunkPolicy, iter_chunks
from .buffers import PreallocatedBuffers, ensure_buffer
from .linear import Linear, WeightMode, WeightsLoadingConfig

_EMPTY_ROW_MODES = {"uniform": _lib.EMPTY_ROW_UNIFORM, "zeros": _lib.EMPTY_ROW_ZEROS}


class TriangleAttentionNodeType(IntEnum):
    STARTING = 0
    ENDING = 1


def _weight_state(*params) -> tuple | None:
    """(address, in-place write count) of every parameter; changes when a weight is loaded or edited."""
    try:
        return tuple((p.data_ptr(), p._version, p.device) for p in params if p is not None)
    except RuntimeError:
        return None


def _refold_after_load_state_dict(module, *args) -> None:
    module.post_load_weights()


class TriangleAttention(nn.Module):
    """Gated multi-head attention over the second pair axis with a shared per-head triangle bias.

    Holds the fused in-projection (``in_proj``: q, k, v, gate rows) and ``o_proj`` exactly as the reference does.
    ``forward`` takes already layer-normalised ``hidden_states``; inside a :class:`TriangleAttentionNode` the node
    bypasses it and runs the fused LayerNorm+projection kernel on the raw pair tensor instead.
    """

    def __init__(self, *, hidden_size: int, head_dim: int, num_attention_heads: int,
                 num_key_value_heads: int | None = None, layer_idx: int, bias_flags: dict[str, bool] | None = None,
                 gating: bool = True, chunk_policy: ChunkPolicy | None = None, dtype: torch.dtype = None,
                 skip_create_weights: bool = False, attn_backend: str = "VANILLA"):
        super().__init__()
        if bias_flags is None:
            bias_flags = {"q": False, "k": False, "v": False, "g": False, "o": False}
        self.layer_idx = layer_idx
        self.hidden_size = hidden_size
        self.num_heads = num_attention_heads
        self.head_dim = head_dim
        self.num_key_value_heads = num_key_value_heads or num_attention_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_key_value_heads * self.head_dim
        self.gating = gating
        self.chunk_policy = chunk_policy
        if not gating:
            raise ValueError("the sm_100a triangle-attention path is built for gated attention (gating=True)")
        if (hidden_size, self.num_heads, head_dim) != (ops.C, ops.HEADS, ops.HEAD_DIM):
            raise ValueError(
                f"the sm_100a kernels are specialised for hidden_size={ops.C}, {ops.HEADS} heads of {ops.HEAD_DIM}; "
                f"got hidden_size={hidden_size}, num_attention_heads={self.num_heads}, head_dim={head_dim}")
        self._in_proj_sizes = [self.q_size, self.kv_size, self.kv_size, self.q_size]
        self.in_proj = Linear(
            hidden_size, sum(self._in_proj_sizes),
            bias=bias_flags["q"] or bias_flags["k"] or bias_flags["v"] or bias_flags["g"], dtype=dtype,
            weights_loading_config=WeightsLoadingConfig(weight_mode=WeightMode.FUSED_SEGMENTS_LINEAR,
                                                        segment_sizes=tuple(self._in_proj_sizes)),
            skip_create_weights=skip_create_weights)
        self.o_proj = Linear(self.q_size, hidden_size, bias=bias_flags["o"], dtype=dtype,
                             skip_create_weights=skip_create_weights)
        self.attn = create_attention(attn_backend, layer_idx, self.num_heads, head_dim, self.num_key_value_heads,
                                     attention_type=AttentionType.TRIANGLE)
        self._pack = None
        self._pack_state = None
        self._zero_bias = None

    def _packed(self, device) -> torch.Tensor:
        """Packed weights for the stand-alone path (no LayerNorm, zero triangle-bias rows)."""
        state = _weight_state(self.in_proj.weight, self.in_proj.bias, self.o_proj.weight, self.o_proj.bias)
        if self._pack is None or self._pack.device != device or state != self._pack_state:
            zero_bias_rows = torch.zeros((ops.HEADS, ops.C), dtype=self.in_proj.weight.dtype, device=device)
            pack = ops.pack_node_weights(None, None, self.in_proj.weight, self.in_proj.bias, zero_bias_rows,
                                         self.o_proj.weight, self.o_proj.bias)
            if not torch.cuda.is_current_stream_capturing():
                self._pack, self._pack_state = pack, state
            return pack
        return self._pack

    def forward(self, hidden_states: torch.Tensor, mask_bias: torch.Tensor, triangle_bias: torch.Tensor | None = None,
                attn_metadata: AttentionMetadata | None = None, buffers: PreallocatedBuffers | None = None,
                use_kv_lengths: bool = False, residual: torch.Tensor | None = None,
                inplace_residual: bool = False) -> torch.Tensor:
        """``hidden_states`` [B, I, J, F] (normalised); ``mask_bias`` additive [B, I, 1, 1, J] or int32 lengths;
        ``triangle_bias`` [B, H, J, J(+pad)].  Returns the update, or ``residual + update`` (written into
        ``residual`` when ``inplace_residual``)."""
        x = hidden_states
        B, R, S, _ = x.shape
        packed = self._packed(x.device)
        lengths = mask_to_lengths(mask_bias, B, R).contiguous()
        if triangle_bias is None:
            key = (B, S, x.device)
            if self._zero_bias is None or self._zero_bias[0] != key:  # kept per shape: no allocation per call
                self._zero_bias = (key, torch.zeros((B, ops.HEADS, S, ops.pad8(S)), dtype=torch.bfloat16, device=x.device))
            bias2 = self._zero_bias[1]
        else:
            pad = -triangle_bias.shape[-1] % 8
            tb = torch.nn.functional.pad(triangle_bias, (0, pad)) if pad else triangle_bias
            bias2 = (tb.float() * ops.BIAS_SCALE).to(torch.bfloat16).contiguous()
        out = residual if (residual is not None and inplace_residual) else None
        if out is None:
            out = torch.empty((B, R, S, ops.C), dtype=torch.bfloat16, device=x.device)
        policy = self.chunk_policy
        chunk = policy.chunk_size if (policy is not None and policy.should_chunk(x)) else R
        for start, length in iter_chunks(R, chunk):
            xs = x.narrow(1, start, length)
            qkvg, _ = ops.prologue(xs, packed, want_bias=False)
            og = ensure_buffer(buffers, "tri_attn_output", (B * length, S, ops.HEADS, ops.HEAD_DIM), x.dtype, x.device)
            og = ops.attention(qkvg, bias2, lengths.narrow(1, start, length), B, length, S,
                               out=None if og is None else og.view(B, length, S, ops.C),
                               empty_row_mode=self.attn.empty_row_mode)
            ops.epilogue(og, packed, None if residual is None else residual.narrow(1, start, length),
                         out.narrow(1, start, length))
        return out


class TriangleAttentionNode(nn.Module):
    def __init__(self, c_in: int, c_hidden: int, num_heads: int,
                 node_type: TriangleAttentionNodeType = TriangleAttentionNodeType.STARTING, inf: float = 1e9,
                 layer_idx: int = 0, dtype: torch.dtype = None, chunk_policy: ChunkPolicy | None = None,
                 skip_create_weights: bool = False, attn_backend: str = "VANILLA",
                 mha_bias_flags: dict[str, bool] | None = None, pair_mask_left_aligned: bool = True,
                 transposed_bias: bool = False, empty_row_mode: str = "uniform"):
        """Same arguments as the reference node.  ``empty_row_mode`` is the one addition: what a pair row
        without any valid key produces — ``"uniform"`` (the mean of V over all keys, what the reference's
        eager path computes because its additive -1e9 swamps the logits) or ``"zeros"`` (what the reference's
        fused GPU kernels write)."""
        super().__init__()
        if mha_bias_flags is None:
            mha_bias_flags = {"q": False, "k": False, "v": False, "g": False, "o": False}
        if empty_row_mode not in _EMPTY_ROW_MODES:
            raise ValueError(f"empty_row_mode must be one of {sorted(_EMPTY_ROW_MODES)}")
        self.c_in = c_in
        self.c_hidden = c_hidden
        self.num_heads = num_heads
        self.node_type = TriangleAttentionNodeType(node_type)
        self.inf = inf
        self.dtype = dtype
        self.attn_backend = attn_backend
        self.pair_mask_left_aligned = pair_mask_left_aligned
        self.transposed_bias = transposed_bias
        self.empty_row_mode = empty_row_mode
        self.layer_norm = nn.LayerNorm(c_in, dtype=dtype)
        self.pair_bias_proj = Linear(c_in, num_heads, bias=False, dtype=dtype, skip_create_weights=skip_create_weights)
        self._bias_pad_multiple = triangle_bias_pad_multiple(attn_backend)
        self.mha = TriangleAttention(
            layer_idx=layer_idx, hidden_size=c_in, head_dim=c_hidden, num_attention_heads=num_heads,
            num_key_value_heads=num_heads, gating=True, bias_flags=mha_bias_flags,
            chunk_policy=chunk_policy if chunk_policy is not None else CHUNK_REGISTRY.get(TRIANGLE_ATTENTION),
            dtype=dtype, skip_create_weights=skip_create_weights, attn_backend=attn_backend)
        self.mha.attn.empty_row_mode = _EMPTY_ROW_MODES[empty_row_mode]
        self._pack = None
        self._pack_state = None
        self.register_load_state_dict_post_hook(_refold_after_load_state_dict)

    # ---- weights -----------------------------------------------------------------------------
    def _params(self):
        return (self.layer_norm.weight, self.layer_norm.bias, self.mha.in_proj.weight, self.mha.in_proj.bias,
                self.pair_bias_proj.weight, self.mha.o_proj.weight, self.mha.o_proj.bias)

    @torch.no_grad()
    def post_load_weights(self) -> None:
        """Refold the LayerNorm-folded projection weights from the (re)loaded parameters."""
        params = self._params()
        if not (self.mha.in_proj._weights_created and self.mha.o_proj._weights_created
                and self.pair_bias_proj._weights_created) or not params[2].is_cuda:
            self._pack = self._pack_state = None
            return
        dev = params[2].device
        self._pack = ops.pack_node_weights(*[None if p is None else p.to(dev) for p in params])
        self._pack_state = _weight_state(*params)

    def _packed(self, device) -> torch.Tensor:
        state = _weight_state(*self._params())
        if self._pack is None or self._pack.device != device or state != self._pack_state:
            pack = ops.pack_node_weights(*[None if p is None else p.to(device) for p in self._params()])
            # a fold recorded during graph capture is only filled at replay: use it for this call only
            if not torch.cuda.is_current_stream_capturing():
                self._pack, self._pack_state = pack, state
            return pack
        return self._pack

    # ---- forward -------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None, mask_bias: torch.Tensor | None = None,
                attn_metadata: AttentionMetadata | None = None, buffers: PreallocatedBuffers | None = None, *,
                residual: bool = False, inplace_residual: bool = False) -> torch.Tensor:
        """``x`` [B, I, J, c_in]; ``mask`` [B, I, J] (ignored when ``mask_bias`` is given); ``mask_bias`` is the
        per-row payload of :func:`precompute_pair_masks` for this node (for the ending node: of the transposed
        mask).  Returns the update or ``x + update`` in ``[B, I, J, c_in]``; ``inplace_residual`` writes into ``x``."""
        if self.dtype not in (None, torch.bfloat16) or (self.dtype is None and x.dtype != torch.bfloat16):
            raise ValueError("the sm_100a triangle-attention kernels compute in bfloat16; construct the layer with "
                             "dtype=torch.bfloat16")
        if not x.is_cuda:
            raise ValueError("this layer runs on a CUDA device only (no CPU path)")
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
            inplace_residual = False
        if x.dim() != 4 or x.shape[1] != x.shape[2] or x.shape[3] != ops.C:
            raise ValueError(f"expected a square pair tensor [B, N, N, {ops.C}], got {tuple(x.shape)}")
        ending = self.node_type == TriangleAttentionNodeType.ENDING
        B, N = x.shape[0], x.shape[1]
        R = S = N
        key_mask = None
        if not self.pair_mask_left_aligned and (mask is not None or mask_bias is not None):
            # keys may be switched off anywhere in a row: the kernel takes one bit per key beside the row lengths
            if mask_bias is None:
                valid = (mask.transpose(1, 2) if ending else mask) > 0.5
            elif mask_bias.dtype == torch.int32:
                raise ValueError("a node built with pair_mask_left_aligned=False takes the pair mask or its additive "
                                 "form ([B, R, 1, 1, S]); int32 row lengths describe left-aligned masks only")
            else:
                valid = (mask_bias[:, :, 0, 0, :] if mask_bias.dim() == 5 else mask_bias) >= 0
            if tuple(valid.shape) != (B, R, S):
                raise ValueError(f"mask of shape {tuple(valid.shape)} does not match the pair tensor [B={B}, {R}, {S}]")
            lengths, key_mask = ops.key_mask_bits(valid)
        elif mask_bias is None:
            if mask is None:
                lengths = None
            else:
                m = mask.transpose(1, 2) if ending else mask
                lengths = (m > 0.5).sum(dim=-1).to(torch.int32).contiguous()
        else:
            lengths = mask_to_lengths(mask_bias, B, R).contiguous()
        packed = self._packed(x.device)
        eps = self.layer_norm.eps
        out = x if (residual and inplace_residual) else torch.empty_like(x, memory_format=torch.contiguous_format)
        xk = x.transpose(1, 2) if ending else x      # kernel-order views [B, R, S, c]
        outk = out.transpose(1, 2) if ending else out
        mode = _EMPTY_ROW_MODES[self.empty_row_mode]

        policy = self.mha.chunk_policy
        chunked = policy is not None and policy.should_chunk(xk) and policy.chunk_size < R
        if not chunked and not self.transposed_bias and key_mask is None:
            # common case: one library call for the whole node, intermediates in one workspace
            ws = ensure_buffer(buffers, "tri_attn_workspace", (ops.node_workspace_bytes(B, N),), torch.uint8, x.device)
            return ops.node_forward(x, packed, lengths, eps, ending=ending, residual=residual, out=out, workspace=ws,
                                    empty_row_mode=mode)
        bias = ensure_buffer(buffers, "tri_attn_bias", (B, ops.HEADS, S, ops.pad8(S)), torch.bfloat16, x.device)
        if self.transposed_bias and bias is None:
            bias = torch.zeros((B, ops.HEADS, S, ops.pad8(S)), dtype=torch.bfloat16, device=x.device)
        elif self.transposed_bias and ops.pad8(S) != S:
            bias[..., S:].zero_()  # the transposed write covers keys < S only: keep the key padding of a caller's buffer defined
        # xk is already in kernel order, so the prologue is always called in its "starting" form here
        if chunked:
            # the bias of every row is needed before any row can attend: one bias-only pass first
            _, bias = ops.prologue(xk, packed, eps, want_qkvg=False, bias=bias, transposed_bias=self.transposed_bias)
        step = policy.chunk_size if chunked else R
        for start, length in iter_chunks(R, step):
            xs = xk.narrow(1, start, length)
            qkvg = ensure_buffer(buffers, "tri_attn_qkvg", (4, B * length, ops.HEADS, S, ops.HEAD_DIM),
                                 torch.bfloat16, x.device)
            if chunked:
                qkvg, _ = ops.prologue(xs, packed, eps, qkvg=qkvg, want_bias=False)
            else:
                qkvg, bias = ops.prologue(xs, packed, eps, qkvg=qkvg, bias=bias, transposed_bias=self.transposed_bias)
            og = ensure_buffer(buffers, "tri_attn_output", (B * length, S, ops.HEADS, ops.HEAD_DIM), torch.bfloat16,
                               x.device)
            og = ops.attention(qkvg, bias, None if lengths is None else lengths.narrow(1, start, length), B, length, S,
                               out=None if og is None else og.view(B, length, S, ops.C), empty_row_mode=mode,
                               key_mask=None if key_mask is None else key_mask.narrow(1, start, length))
            ops.epilogue(og, packed, xs if residual else None, outk.narrow(1, start, length))
        return out


class TriangleAttentionStartingNode(TriangleAttentionNode):
    def __init__(self, *args, **kwargs):
        kwargs["node_type"] = TriangleAttentionNodeType.STARTING
        super().__init__(*args, **kwargs)


class TriangleAttentionEndingNode(TriangleAttentionNode):
    def __init__(self, *args, **kwargs):
        kwargs["node_type"] = TriangleAttentionNodeType.ENDING
        super().__init__(*args, **kwargs)


_TRI_ATTN_IN_PROJ_KEYS = ("tri_attn_start.mha.in_proj", "tri_attn_end.mha.in_proj")


def split_pair_bias_proj(weights: dict) -> dict:
    """Move the legacy fifth in-projection segment (the bias heads) of each node to ``pair_bias_proj``,
    as the reference's loader does (``bionemo_ir/_torch/layers/triangle_nodes.py:271-280``)."""
    for key in [k for k in weights if k.endswith(_TRI_ATTN_IN_PROJ_KEYS)]:
        node = key.removesuffix(".mha.in_proj")
        if f"{node}.pair_bias_proj" in weights:
            continue
        *in_proj, bias = weights[key]
        weights[key] = in_proj
        weights[f"{node}.pair_bias_proj"] = [{"weight": bias["weight"]}]
    return weights
