"""Single-track attention with pair bias on the sm_100a kernels.

Counterpart of ``AttentionPairBias`` (``bionemo_ir/_torch/layers/attention.py:420-1196``) in the form the pairformer
builds it (``bionemo_ir/_torch/layers/transformers/pairformer.py:93-106``): 16 heads over the single representation
``s [B, N, c_s]``, an additive bias projected from the pair representation ``z [B, N, N, 128]``, a sigmoid gate and
an output projection.  Constructor arguments, ``forward`` signature and ``state_dict`` keys (``norm_s``,
``in_proj``, ``proj_z.0``, ``proj_z.1``, ``proj_o``) are the reference's; options of the reference that belong to
other models (AdaLN, separate query/key norms, QK norm, key gathering, windowed attention, output gate, RMS norm)
raise ``ValueError`` when requested.

A forward is five launches: row statistics of ``s``; the in-projection GEMM writing head-major q, k, v and gate
planes (heads padded to 32 columns); the pair-bias pass over ``z`` (LayerNorm + projection + move of the head axis
+ key padding in one kernel); the attention core (the triangle-attention kernel, which sees the 16 heads as 4
items of 4 heads per batch entry); and the output-projection GEMM that reads the attention output in place and
adds bias and residual.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import _lib, ops
from .buffers import ensure_buffer
from .linear import Linear, WeightMode, WeightsLoadingConfig
from .triangle_nodes import _refold_after_load_state_dict, _weight_state

_HEADS = ops.SINGLE_HEADS
_PAD = ops.HEAD_DIM  # head width of the attention kernel


def fold_linear(weight: torch.Tensor, bias: torch.Tensor | None, gamma: torch.Tensor | None,
                beta: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
    """``(w_bf16 [N, K], sc fp32 [N, 2])`` for ``ops.linear``: LayerNorm(gamma, beta) folded into ``weight`` so that
    ``LN(x) · wᵀ + bias = rstd * (x · w_bf16ᵀ) - mean * rstd * rowsum + const`` (rows centred before the bf16
    rounding, the rounding residue kept in ``rowsum``)."""
    w = weight.float()
    if gamma is not None:
        wg = w * gamma.float()
        wq = (wg - wg.mean(dim=1, keepdim=True)).to(torch.bfloat16)
        rowsum = wq.float().sum(dim=1)
        const = (w * beta.float()).sum(dim=1) if beta is not None else torch.zeros_like(rowsum)
    else:
        wq = w.to(torch.bfloat16)
        rowsum = torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
        const = torch.zeros_like(rowsum)
    if bias is not None:
        const = const + bias.float()
    return wq.contiguous(), torch.stack([rowsum, const], dim=1).contiguous()


class AttentionPairBias(nn.Module):
    def __init__(self, layer_idx: int, c_s: int, c_z: int, num_heads: int, initial_norm: bool = True,
                 bias_proj: bool = False, pair_norm: bool = True, dtype: torch.dtype = None, inf: float = 1e6,
                 eps: float = 1e-5, use_initial_ada_layer_norm: bool = False, use_separate_layer_norm: bool = False,
                 use_ada_layer_norm: bool = True, chain_kv_norm: bool = False, norm_type: str = "layer_norm",
                 use_qk_norm: bool = False, kv_bias: bool = False, out_bias: bool = False,
                 pair_norm_type: str = "layer_norm", output_gate_dim: int | None = None,
                 skip_create_weights: bool = False, attn_backend: str = "VANILLA", mask_left_aligned: bool = True):
        super().__init__()
        head_dim = c_s // num_heads
        if num_heads != _HEADS or c_z != ops.C or c_s % 128 or c_s != num_heads * head_dim or head_dim > _PAD:
            raise ValueError(f"the sm_100a single-track attention is built for {_HEADS} heads of at most {_PAD} "
                             f"channels, c_s a multiple of 128 and c_z={ops.C}; got c_s={c_s}, c_z={c_z}, "
                             f"num_heads={num_heads}")
        unsupported = {"bias_proj=False": not bias_proj, "use_initial_ada_layer_norm": use_initial_ada_layer_norm,
                       "use_separate_layer_norm": use_separate_layer_norm, "chain_kv_norm": chain_kv_norm,
                       "use_qk_norm": use_qk_norm, "output_gate_dim": output_gate_dim is not None,
                       "norm_type != layer_norm": norm_type != "layer_norm",
                       "pair_norm_type != layer_norm": pair_norm_type != "layer_norm",
                       "mask_left_aligned=False": not mask_left_aligned}
        bad = [k for k, v in unsupported.items() if v]
        if bad:
            raise ValueError(f"not supported by the sm_100a single-track attention: {', '.join(bad)}")
        if dtype not in (None, torch.bfloat16):
            raise ValueError(f"the sm_100a single-track attention computes in bfloat16; got dtype={dtype}")
        self.layer_idx = layer_idx
        self.c_s, self.c_z, self.num_heads, self.head_dim = c_s, c_z, num_heads, head_dim
        self.initial_norm, self.bias_proj, self.kv_bias = initial_norm, bias_proj, kv_bias
        self.inf, self.eps, self.dtype = inf, eps, dtype
        self.attn_backend = attn_backend
        self.mask_left_aligned = mask_left_aligned
        self.norm_s = nn.LayerNorm(c_s, eps=eps, dtype=dtype) if initial_norm else None
        self._in_proj_sizes = (c_s, c_s, c_s, c_s)  # q, gate, k, v
        self.in_proj = Linear(c_s, 4 * c_s, bias=True, dtype=dtype, skip_create_weights=skip_create_weights,
                              weights_loading_config=WeightsLoadingConfig(weight_mode=WeightMode.FUSED_SEGMENTS_LINEAR,
                                                                          segment_sizes=self._in_proj_sizes))
        linear_z = Linear(c_z, num_heads, bias=False, dtype=dtype, skip_create_weights=skip_create_weights)
        self.proj_z = (nn.Sequential(nn.LayerNorm(c_z, eps=eps, dtype=dtype), linear_z) if pair_norm
                       else nn.Sequential(linear_z))
        self.proj_o = Linear(c_s, c_s, bias=out_bias, dtype=dtype, skip_create_weights=skip_create_weights)
        self._folded = None
        self._folded_state = None
        self._input_norm: list[nn.LayerNorm] = []  # a caller's LayerNorm of s folded into in_proj (not a submodule)
        self.register_load_state_dict_post_hook(_refold_after_load_state_dict)

    # ---- weights -----------------------------------------------------------------------------
    def set_input_norm(self, norm: nn.LayerNorm | None) -> None:
        """Fold a LayerNorm that the caller applies to ``s`` before this layer (the v2 pairformer layer's
        ``pre_norm_s``) into the in-projection: ``forward`` then takes the un-normalised ``s``.  Only for layers
        built without ``initial_norm``; the norm stays the caller's module (its parameters are read at fold time)."""
        if norm is not None and self.norm_s is not None:
            raise ValueError("a layer with initial_norm cannot fold a second LayerNorm")
        self._input_norm = [] if norm is None else [norm]
        self._folded = self._folded_state = None

    def _norm_of_s(self) -> nn.LayerNorm | None:
        return self.norm_s if self.norm_s is not None else (self._input_norm[0] if self._input_norm else None)

    def _params(self):
        norm = self._norm_of_s()
        norm_s = (norm.weight, norm.bias) if norm is not None else (None, None)
        norm_z = (self.proj_z[0].weight, self.proj_z[0].bias) if len(self.proj_z) > 1 else (None, None)
        return (*norm_s, self.in_proj.weight, self.in_proj.bias, *norm_z, self.proj_z[-1].weight, self.proj_o.weight,
                self.proj_o.bias)

    def _fold(self, device) -> dict:
        ns_w, ns_b, w_in, b_in, nz_w, nz_b, w_z, w_o, b_o = [None if p is None else p.detach().to(device)
                                                              for p in self._params()]
        c_s, d = self.c_s, self.head_dim
        # in_proj rows (q, gate, k, v) x (head, d) -> kernel columns (q, k, v, gate) x (head, 32), pad rows zero
        w4 = w_in.float().reshape(4, _HEADS, d, c_s)[[0, 2, 3, 1]]
        b4 = b_in.float().reshape(4, _HEADS, d)[[0, 2, 3, 1]]
        w_pad = torch.zeros(4, _HEADS, _PAD, c_s, dtype=torch.float32, device=device)
        b_pad = torch.zeros(4, _HEADS, _PAD, dtype=torch.float32, device=device)
        w_pad[:, :, :d], b_pad[:, :, :d] = w4, b4
        w_in_f, sc_in = fold_linear(w_pad.reshape(-1, c_s), b_pad.reshape(-1), ns_w, ns_b)
        # proj_o columns (head, d) -> (head, 32): the attention output's padded columns meet zero weights
        wo_pad = torch.zeros(c_s, _HEADS, _PAD, dtype=torch.float32, device=device)
        wo_pad[:, :, :d] = w_o.float().reshape(c_s, _HEADS, d)
        w_o_f, sc_o = fold_linear(wo_pad.reshape(c_s, -1), b_o, None, None)
        # the attention kernel adds the bias to q·k before the softmax scale: keep bias / scale
        packed_z = ops.pack_pair_bias_weights(nz_w, nz_b, w_z, math.sqrt(d))
        return {"w_in": w_in_f, "sc_in": sc_in, "w_o": w_o_f, "sc_o": sc_o, "packed_z": packed_z}

    @torch.no_grad()
    def post_load_weights(self) -> None:
        """Refold the kernel-side weights from the (re)loaded parameters (reference lines 1134-1154 pad its heads
        at the same point)."""
        layers = (self.in_proj, self.proj_z[-1], self.proj_o)
        if not all(layer._weights_created for layer in layers) or not self.in_proj.weight.is_cuda:
            self._folded = self._folded_state = None
            return
        self._folded = self._fold(self.in_proj.weight.device)
        self._folded_state = _weight_state(*self._params())

    @torch.no_grad()
    def _weights(self, device) -> dict:
        state = _weight_state(*self._params())
        if self._folded is None or self._folded["w_in"].device != device or state != self._folded_state:
            folded = self._fold(device)
            if not torch.cuda.is_current_stream_capturing():
                self._folded, self._folded_state = folded, state
            return folded
        return self._folded

    def project_pair_bias(self, z: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        """``[B, H, N_q, pad8(N_k)]`` pair bias of ``z [B, N_q, N_k, 128]``, multiplied by ``sqrt(head_dim)`` (the
        form the attention kernel adds to q·k before its softmax scale); the padding keys are zero."""
        if z.dtype != torch.bfloat16:
            z = z.to(torch.bfloat16)
        return ops.pair_bias(z, self._weights(z.device)["packed_z"], self.num_heads, self.eps, bias=bias)

    # ---- forward ------------------------------------------------------------------------------
    def _lengths(self, mask: torch.Tensor | None, mask_bias: torch.Tensor | None, B: int, N: int, device) -> torch.Tensor:
        """Valid keys per batch entry (int32 ``[B]``) from the reference's mask forms: the ``[B, N]`` mask
        (left-aligned), an additive ``[B, 1, 1, N]`` bias, or int32 lengths."""
        if mask_bias is not None:
            if mask_bias.dtype == torch.int32:
                lengths = mask_bias.reshape(-1)
            else:
                lengths = (mask_bias.reshape(B, -1)[:, -N:] >= 0).sum(dim=-1).to(torch.int32)
        elif mask is not None:
            if tuple(mask.shape) != (B, N):
                raise ValueError(f"mask must have shape {(B, N)}, got {tuple(mask.shape)}")
            lengths = (mask > 0).sum(dim=-1).to(torch.int32)
        else:
            return torch.full((B,), N, dtype=torch.int32, device=device)
        if lengths.numel() != B:
            raise ValueError(f"expected one key count per batch entry, got {lengths.numel()} for B={B}")
        return lengths.to(device)

    def forward(self, s: torch.Tensor, z: torch.Tensor | None, mask: torch.Tensor | None,
                single_embedding: torch.Tensor | None = None, attn_metadata=None,
                mask_bias: torch.Tensor | None = None, mask_bias_local: torch.Tensor | None = None,
                buffers: dict | None = None, residual: torch.Tensor | None = None,
                output_gate_logits: torch.Tensor | None = None, adaln_conditioning=None) -> torch.Tensor:
        """``s``: ``[B, N, c_s]``; ``z``: ``[B, N, N, 128]``; ``mask``: ``[B, N]`` (1 = valid key, left-aligned).
        Returns the update of ``s`` (``residual + update`` when ``residual`` is given), in the dtype of ``s``."""
        if single_embedding is not None or output_gate_logits is not None or adaln_conditioning is not None:
            raise ValueError("AdaLN conditioning and the output gate are not supported by the sm_100a single track")
        if mask_bias_local is not None or (attn_metadata is not None and getattr(attn_metadata, "query_to_keys", None) is not None):
            raise ValueError("sequence-local attention (query_to_keys) is not supported by the sm_100a single track")
        if s.dim() != 3 or s.shape[-1] != self.c_s:
            raise ValueError(f"expected s of shape [B, N, {self.c_s}], got {tuple(s.shape)}")
        if z is None or z.dim() != 4 or tuple(z.shape[:3]) != (s.shape[0], s.shape[1], s.shape[1]) or z.shape[-1] != self.c_z:
            raise ValueError(f"expected z of shape [B, N, N, {self.c_z}] matching s {tuple(s.shape)}")
        if not s.is_cuda:
            raise ValueError("the sm_100a single-track attention needs CUDA tensors (there is no CPU fallback)")
        B, N, c_s = s.shape
        out_dtype = s.dtype
        s16 = s.to(torch.bfloat16).contiguous()
        w = self._weights(s.device)
        lengths = self._lengths(mask, mask_bias, B, N, s.device)

        norm = self._norm_of_s()
        stats = ops.row_stats(s16, norm.eps) if norm is not None else None
        planes = ensure_buffer(buffers, "pw_qkvg", (4, B, _HEADS, N, _PAD), torch.bfloat16, s.device)
        planes = ops.linear(s16, w["w_in"], w["sc_in"], ops.LINEAR_PLANES, B=B, rows=N, stats=stats, out=planes)
        bias = ensure_buffer(buffers, "pw_pair_bias", (B, _HEADS, N, ops.pad8(N)), torch.bfloat16, s.device)
        bias = self.project_pair_bias(z, bias=bias)
        # the attention kernel handles 4 heads per item: batch entry b becomes the 4 items 4b .. 4b+3
        attn = ensure_buffer(buffers, "pw_attn_output", (4 * B, 1, N, ops.C), torch.bfloat16, s.device)
        attn = ops.attention(planes.view(4, 4 * B, ops.HEADS, N, _PAD), bias.view(4 * B, ops.HEADS, N, bias.shape[-1]),
                             lengths.repeat_interleave(4), 4 * B, 1, N, out=attn, scale=1.0 / math.sqrt(self.head_dim),
                             empty_row_mode=_lib.EMPTY_ROW_UNIFORM)
        res16 = None if residual is None else residual.to(torch.bfloat16).contiguous()
        out = ops.linear(attn, w["w_o"], w["sc_o"], ops.LINEAR_ROWS, B=B, rows=N,
                         a_strides=(4 * N * ops.C, ops.C, N * ops.C), residual=res16)
        return out if out.dtype == out_dtype else out.to(out_dtype)
