"""SwiGLU pair transition with the reference's module API on the fused sm_100a kernel.

Drop-in counterpart of ``Transition`` (``bionemo_ir/_torch/layers/transition.py:187-336``): same constructor,
``forward(x, mask=None, *, residual=False, inplace=False)``, ``post_load_weights()`` and ``state_dict`` keys
(``norm.{weight,bias}``, ``fused_fc2_fc1.weight`` with value rows first and gate rows second, ``fc3.weight``).
The reference picks between three paths per call; here every call is the one fused kernel
(``b200ta_transition``), which already does what the reference's ``transition_mlp_w_norm`` path does:
LayerNorm folded into the first linear, hidden activation kept on chip, mask and residual in the epilogue.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from .auto_chunk import ChunkPolicy
from .linear import Linear, WeightMode, WeightsLoadingConfig
from .triangle_nodes import _refold_after_load_state_dict, _weight_state


def _row_mask(x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """One value per row of ``x`` (``[*x.shape[:-1]]``), accepting a trailing axis of size 1 and broadcasting."""
    rows = x.shape[:-1]
    if mask.dim() == x.dim() and mask.shape[-1] == 1:
        mask = mask.squeeze(-1)
    if mask.dim() != len(rows) or any(s not in (1, c) for s, c in zip(mask.shape, rows, strict=True)):
        raise ValueError(f"mask {tuple(mask.shape)} does not hold one value per row of x {tuple(x.shape)}")
    return mask.expand(rows)


class Transition(nn.Module):
    def __init__(self, dim: int, hidden: int, out_dim: int | None = None, layer_idx: int = 0, eps: float = 1e-5,
                 dtype: torch.dtype = None, skip_create_weights: bool = False,
                 auto_chunk_policy: ChunkPolicy | None = None, normalize: bool = True):
        super().__init__()
        if out_dim is None:
            out_dim = dim
        if (dim, hidden, out_dim) != (ops.C, ops.HIDDEN, ops.C):
            raise ValueError(f"the sm_100a transition kernel is specialised for dim={ops.C}, hidden={ops.HIDDEN}, "
                             f"out_dim={ops.C}; got ({dim}, {hidden}, {out_dim})")
        self.auto_chunk_policy = auto_chunk_policy  # accepted; the fused kernel holds no activation beyond its output
        self.normalize = normalize
        self.dtype = dtype
        self.hidden = hidden
        self.layer_idx = layer_idx
        self.norm = nn.LayerNorm(dim, eps=eps, dtype=dtype) if normalize else None
        self.eps = eps
        self.fused_fc2_fc1 = Linear(dim, 2 * hidden, dtype=dtype, bias=False, skip_create_weights=skip_create_weights,
                                    weights_loading_config=WeightsLoadingConfig(weight_mode=WeightMode.FUSED_KV_LINEAR))
        self.fc3 = Linear(hidden, out_dim, dtype=dtype, bias=False, skip_create_weights=skip_create_weights)
        self._pack = None
        self._pack_state = None
        self.register_load_state_dict_post_hook(_refold_after_load_state_dict)

    def _params(self):
        norm = (self.norm.weight, self.norm.bias) if self.norm is not None else (None, None)
        return (*norm, self.fused_fc2_fc1.weight, self.fc3.weight)

    @torch.no_grad()
    def post_load_weights(self) -> None:
        """Refold the LayerNorm-folded weights from the (re)loaded parameters."""
        if not (self.fused_fc2_fc1._weights_created and self.fc3._weights_created) or not self.fc3.weight.is_cuda:
            self._pack = self._pack_state = None
            return
        dev = self.fc3.weight.device
        self._pack = ops.pack_transition_weights(*[None if p is None else p.to(dev) for p in self._params()])
        self._pack_state = _weight_state(*self._params())

    def _packed(self, device) -> torch.Tensor:
        state = _weight_state(*self._params())
        if self._pack is None or self._pack.device != device or state != self._pack_state:
            pack = ops.pack_transition_weights(*[None if p is None else p.to(device) for p in self._params()])
            if not torch.cuda.is_current_stream_capturing():
                self._pack, self._pack_state = pack, state
            return pack
        return self._pack

    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None, *, residual: bool = False,
                inplace: bool = False) -> torch.Tensor:
        """The SwiGLU update ``mask * fc3(silu(gate) * value)``, or ``x`` plus it with ``residual``;
        ``inplace`` (with ``residual``) writes the sum into ``x``."""
        if self.dtype not in (None, torch.bfloat16) or (self.dtype is None and x.dtype != torch.bfloat16):
            raise ValueError("the sm_100a transition kernel computes in bfloat16; construct the layer with "
                             "dtype=torch.bfloat16")
        if not x.is_cuda:
            raise ValueError("this layer runs on a CUDA device only (no CPU path)")
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
            inplace = False
        xc = x if x.is_contiguous() else x.contiguous()
        out = xc if (residual and inplace and xc is x) else None
        row_mask = None if mask is None else _row_mask(xc, mask)
        y = ops.transition(xc, self._packed(x.device), row_mask, self.eps if self.norm is None else self.norm.eps,
                           residual=residual, out=out)
        if residual and inplace and y is not x:
            x.copy_(y)
            return x
        return y
