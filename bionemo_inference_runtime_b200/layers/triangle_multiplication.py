"""Triangle multiplication (outgoing / incoming) with the reference's module API on the sm_100a kernels.

Drop-in counterpart of ``TriangleMultiplicationNode`` (``bionemo_ir/_torch/layers/triangle_nodes.py:326-755``), of
``TriangleMultiplicationMetadata`` / ``precompute_trimul_metadata`` (lines 62-117) and of
``set_trimul_token_padding`` (lines 758-764): same constructor arguments, forward signature and ``state_dict`` keys
(``norm_in``, ``p_in``, ``g_in``, ``norm_out``, ``p_out``, ``g_out``).  A forward is three kernel launches (input
projection, contraction, output stage; see ``include/b200ta.h``); the incoming node runs the same kernels with the
input stage reading the pair tensor through swapped strides.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum

import torch
import torch.nn as nn

from .. import ops
from .buffers import ensure_buffer
from .linear import Linear, WeightMode, WeightsLoadingConfig
from .triangle_nodes import _refold_after_load_state_dict, _weight_state

_GEMM_TOKEN_ALIGN = 8


class TriangleMultiplicationNodeType(IntEnum):
    OUTGOING = 0
    INCOMING = 1


@dataclass
class TriangleMultiplicationMetadata:
    """Token alignment and row lengths shared by a stack of nodes (reference lines 62-69).  The kernels here take
    any token count and read the mask itself, so only the presence of row lengths matters: it selects, as in the
    reference, the masked form of the fused residual output."""

    token_pad_multiple: int = -1
    outgoing_actual_seqlen: torch.Tensor | None = None
    incoming_actual_seqlen: torch.Tensor | None = None
    padded_outgoing_actual_seqlen: torch.Tensor | None = None
    padded_incoming_actual_seqlen: torch.Tensor | None = None


def precompute_trimul_metadata(x: torch.Tensor, outgoing_actual_seqlen: torch.Tensor | None,
                               incoming_actual_seqlen: torch.Tensor | None, *,
                               enabled: bool = True) -> TriangleMultiplicationMetadata:
    """Same signature as the reference helper (lines 79-117).  No padded copies of the lengths are made: these
    kernels need no token padding."""
    if not enabled:
        outgoing_actual_seqlen = incoming_actual_seqlen = None
    return TriangleMultiplicationMetadata(-1, outgoing_actual_seqlen, incoming_actual_seqlen, None, None)


class TriangleMultiplicationNode(nn.Module):
    def __init__(self, layer_idx: int = 0, dim: int = 128, hidden_dim: int | None = None, eps: float = 1e-5,
                 multiplication_type: TriangleMultiplicationNodeType = TriangleMultiplicationNodeType.OUTGOING,
                 bias_flags: dict[str, bool] | None = None, dtype: torch.dtype = None, skip_create_weights: bool = False,
                 high_precision: bool = True, mean_normalization: bool = False, pair_mask_left_aligned: bool = True,
                 align_contraction_tokens: bool = True, pad_tokens: bool = False, norm_bias: bool = True):
        """Same arguments as the reference node.  ``high_precision`` keeps ``norm_out`` / ``p_out`` / ``g_out`` in
        fp32 as the reference does; the kernels fold them to bf16 operands with fp32 constants and accumulate in
        fp32, and the result is returned in fp32 in that case (bf16 precision), otherwise in the module dtype.
        ``pair_mask_left_aligned``, ``align_contraction_tokens`` and ``pad_tokens`` are accepted and unused: the
        kernels read the mask itself and take any token count."""
        super().__init__()
        if hidden_dim is None:
            hidden_dim = dim
        if bias_flags is None:
            bias_flags = {"p_in": False, "g_in": False, "p_out": False, "g_out": False}
        if dim != ops.C or hidden_dim != ops.TRI_HIDDEN:
            raise ValueError(f"the sm_100a triangle-multiplication kernels are built for dim={ops.C}, "
                             f"hidden_dim={ops.TRI_HIDDEN}; got dim={dim}, hidden_dim={hidden_dim}")
        if dtype not in (None, torch.bfloat16):
            raise ValueError(f"the sm_100a triangle-multiplication kernels compute in bfloat16; got dtype={dtype}")
        self.layer_idx = layer_idx
        self.dim, self.hidden_dim, self.eps = dim, hidden_dim, eps
        self.dtype = dtype
        self.multiplication_type = TriangleMultiplicationNodeType(multiplication_type)
        self.high_precision = high_precision
        self.mean_normalization = mean_normalization
        self.pair_mask_left_aligned = pair_mask_left_aligned
        self.align_contraction_tokens = align_contraction_tokens
        self.pad_tokens = pad_tokens
        self.high_precision_dtype = torch.float32 if high_precision else dtype
        self.norm_in = nn.LayerNorm(dim, dtype=dtype, eps=eps, bias=norm_bias)
        fused = WeightsLoadingConfig(weight_mode=WeightMode.FUSED_KV_LINEAR)
        self.p_in = Linear(dim, 2 * hidden_dim, bias=bias_flags["p_in"], dtype=dtype, weights_loading_config=fused,
                           skip_create_weights=skip_create_weights)
        self.g_in = Linear(dim, 2 * hidden_dim, bias=bias_flags["g_in"], dtype=dtype, weights_loading_config=fused,
                           skip_create_weights=skip_create_weights)
        hp = self.high_precision_dtype
        self.norm_out = nn.LayerNorm(hidden_dim, dtype=hp, eps=eps, bias=norm_bias)
        self.p_out = Linear(hidden_dim, dim, bias=bias_flags["p_out"], dtype=hp, skip_create_weights=skip_create_weights)
        self.g_out = Linear(dim, dim, bias=bias_flags["g_out"], dtype=hp, skip_create_weights=skip_create_weights)
        self._pack = None
        self._pack_state = None
        self.register_load_state_dict_post_hook(_refold_after_load_state_dict)

    # ---- weights -----------------------------------------------------------------------------
    def set_token_padding(self, enabled: bool) -> None:
        """Kept for callers of the reference API (lines 463-472): these kernels need no token padding."""
        self.pad_tokens = enabled

    def _params(self):
        return (self.norm_in.weight, self.norm_in.bias, self.p_in.weight, self.p_in.bias, self.g_in.weight,
                self.g_in.bias, self.norm_out.weight, self.norm_out.bias, self.p_out.weight, self.p_out.bias,
                self.g_out.weight, self.g_out.bias)

    def _fold(self, device) -> torch.Tensor:
        params = list(self._params())
        for idx in (1, 7):  # a LayerNorm built without bias (norm_bias=False)
            if params[idx] is None:
                params[idx] = torch.zeros_like(params[idx - 1])
        # one dtype for the fold: fp32 when the output layers are kept in fp32
        common = torch.float32 if any(p is not None and p.dtype == torch.float32 for p in params) else torch.bfloat16
        return ops.pack_trimul_weights(*[None if p is None else p.to(device=device, dtype=common) for p in params])

    @torch.no_grad()
    def post_load_weights(self) -> None:
        """Refold the LayerNorm-folded weights from the (re)loaded parameters (reference lines 548-550)."""
        layers = (self.p_in, self.g_in, self.p_out, self.g_out)
        if not all(layer._weights_created for layer in layers) or not self.p_in.weight.is_cuda:
            self._pack = self._pack_state = None
            return
        self._pack = self._fold(self.p_in.weight.device)
        self._pack_state = _weight_state(*self._params())

    def _packed(self, device) -> torch.Tensor:
        state = _weight_state(*self._params())
        if self._pack is None or self._pack.device != device or state != self._pack_state:
            pack = self._fold(device)
            # a fold recorded during graph capture is only filled at replay: use it for this call only
            if not torch.cuda.is_current_stream_capturing():
                self._pack, self._pack_state = pack, state
            return pack
        return self._pack

    def can_fuse_residual(self, x: torch.Tensor) -> bool:
        """Whether ``residual=True`` produces the masked form ``(x + update) * mask`` (reference lines 614-620:
        the fused residual kernel needs token counts that are multiples of 8)."""
        return (self.pair_mask_left_aligned and x.shape[1] % _GEMM_TOKEN_ALIGN == 0
                and x.shape[2] % _GEMM_TOKEN_ALIGN == 0)

    # ---- forward ------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None,
                trimul_metadata: TriangleMultiplicationMetadata | None = None, *, residual: bool = False,
                buffers: dict | None = None) -> torch.Tensor:
        """``x``: pair tensor ``[B, I, J, dim]``; ``mask``: pair mask ``[B, I, J]`` (1 = valid) or ``None``.
        Returns the update, or with ``residual`` ``x + update`` - multiplied by the mask when the metadata carries
        the outgoing row lengths and the token counts are multiples of 8, which is where the reference takes its
        fused masked-residual kernel (lines 706-722).  ``buffers`` (optional dict) keeps the two channel-major
        intermediates between calls."""
        if x.dim() != 4 or x.shape[-1] != self.dim or x.shape[1] != x.shape[2]:
            raise ValueError(f"expected a square pair tensor [B, N, N, {self.dim}], got {tuple(x.shape)}")
        if not x.is_cuda:
            raise ValueError("the sm_100a triangle-multiplication path needs a CUDA tensor (there is no CPU fallback)")
        residual_pair = x
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        B, N = x.shape[0], x.shape[1]
        incoming = self.multiplication_type == TriangleMultiplicationNodeType.INCOMING
        mask_f = None
        if mask is not None:
            if tuple(mask.shape) != (B, N, N):
                raise ValueError(f"mask must have shape {(B, N, N)}, got {tuple(mask.shape)}")
            mask_f = mask.to(torch.float32)
        b_scale = None
        if self.mean_normalization:
            n_valid = mask_f[:, 0, :].sum(dim=-1) if mask_f is not None else x.new_full((B,), float(N), dtype=torch.float32)
            b_scale = (1.0 / (n_valid + 1e-3)).contiguous()
        packed = self._packed(x.device)
        pitch = ops.pad16(N)
        ab = ensure_buffer(buffers, "trimul_ab", (B, 2 * self.hidden_dim, N, pitch), torch.bfloat16, x.device)
        t = ensure_buffer(buffers, "trimul_contracted", (B, self.hidden_dim, N, pitch), torch.bfloat16, x.device)
        ab = ops.trimul_project(x, mask_f, packed, self.eps, incoming=incoming, b_scale=b_scale, ab=ab)
        t = ops.trimul_contract(ab, N, x=t)
        metadata = trimul_metadata if trimul_metadata is not None else TriangleMultiplicationMetadata()
        fuse_mask = (residual and mask_f is not None and metadata.outgoing_actual_seqlen is not None
                     and self.can_fuse_residual(x))
        out = ops.trimul_output(x, t, packed, self.eps, residual=residual, mask=mask_f if fuse_mask else None)
        if self.high_precision:
            out = out.to(torch.float32)
        elif residual and residual_pair.dtype != out.dtype:
            out = out.to(torch.promote_types(residual_pair.dtype, out.dtype))
        return out


def set_trimul_token_padding(module: nn.Module, enabled: bool) -> None:
    """Propagate a model's token-padding setting to every triangle multiplication under ``module``."""
    for child in module.modules():
        if isinstance(child, TriangleMultiplicationNode):
            child.set_token_padding(enabled)
