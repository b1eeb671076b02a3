"""SwiGLU pair transition with the reference's module API on the fused sm_100a kernel.

Drop-in counterpart of ``Transition`` (``bionemo_ir/_torch/layers/transition.py:187-336``): same constructor,
``forward(x, mask=None, *, residual=False, inplace=False)``, ``post_load_weights()`` and ``state_dict`` keys
(``norm.{weight,bias}``, ``fused_fc2_fc1.weight`` with value rows first and gate rows second, ``fc3.weight``).
The reference picks between three paths per call; here every call of the pair transition (dim 128, hidden 512) is
the one fused kernel (``b200ta_transition``), which already does what the reference's ``transition_mlp_w_norm``
path does: LayerNorm applied on chip (the normalised rows, rounded to bf16 as the eager LayerNorm's output is, feed
the first GEMM from tensor memory), hidden activation kept on chip, mask and residual in the epilogue.  Other widths (the single-track transition, dim 384 and hidden 1536) run as row statistics plus two
tensor-core GEMMs (``b200ta_linear``): LayerNorm folded into the first, SwiGLU in its epilogue, the residual in
the epilogue of the second.
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


def _storage_order(x: torch.Tensor) -> list[int] | None:
    """The permutation of dimensions that makes ``x`` contiguous (channels stay last), or None when ``x`` is not a
    permuted view of a dense tensor."""
    if x.stride(-1) != 1:
        return None
    lead = sorted(range(x.dim() - 1), key=lambda d: (-x.stride(d), d))
    order = lead + [x.dim() - 1]
    return order if x.permute(order).is_contiguous() else None


class Transition(nn.Module):
    def __init__(self, dim: int, hidden: int, out_dim: int | None = None, layer_idx: int = 0, eps: float = 1e-5,
                 dtype: torch.dtype = None, skip_create_weights: bool = False,
                 auto_chunk_policy: ChunkPolicy | None = None, normalize: bool = True):
        super().__init__()
        if out_dim is None:
            out_dim = dim
        self._fused = (dim, hidden, out_dim) == (ops.C, ops.HIDDEN, ops.C)
        if not self._fused and (out_dim != dim or dim % 128 or hidden % 128 or dim > 2048):
            raise ValueError(f"the sm_100a transition kernels take dim={ops.C}, hidden={ops.HIDDEN} (fused) or "
                             f"multiples of 128 with dim <= 2048 and out_dim == dim; got ({dim}, {hidden}, {out_dim})")
        self.dim = dim
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
        self._pack = self._fold(self.fc3.weight.device)
        self._pack_state = _weight_state(*self._params())

    @torch.no_grad()
    def _fold(self, device):
        params = [None if p is None else p.detach().to(device) for p in self._params()]
        if self._fused:
            return ops.pack_transition_weights(*params)
        from .attention_pair_bias import fold_linear

        ln_w, ln_b, w1, w2 = params
        # value rows first, gate rows second -> groups of 32 rows: 16 values followed by their 16 gates
        value, gate = w1.float().reshape(2, self.hidden // 16, 16, self.dim)
        w1_f, sc1 = fold_linear(torch.cat([value, gate], dim=1).reshape(2 * self.hidden, self.dim), None, ln_w, ln_b)
        w2_f, sc2 = fold_linear(w2, None, None, None)
        return {"w1": w1_f, "sc1": sc1, "w2": w2_f, "sc2": sc2}

    def _packed(self, device) -> torch.Tensor:
        state = _weight_state(*self._params())
        held = self._pack["w1"] if isinstance(self._pack, dict) else self._pack
        if held is None or held.device != device or state != self._pack_state:
            pack = self._fold(device)
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
        if not x.is_contiguous():
            # The transition is position-wise, so a permuted view (an ending node's transposed pair tensor, say) is
            # processed in its storage order and the result handed back under the same permutation: no copy, and
            # ``inplace`` still writes the caller's storage.
            order = _storage_order(x)
            if order is None:
                raise ValueError("Transition takes a contiguous tensor or a permuted view of one (channels last, "
                                 f"unit stride); got shape {tuple(x.shape)} with strides {x.stride()}")
            inverse = [order.index(d) for d in range(x.dim())]
            mask_p = None if mask is None else _row_mask(x, mask).permute(order[:-1])
            y = self.forward(x.permute(order), mask_p, residual=residual, inplace=inplace)
            return x if (residual and inplace) else y.permute(inverse)
        xc = x
        if not self._fused:
            return self._forward_gemms(x, xc, mask, residual, inplace)
        out = xc if (residual and inplace) else None
        row_mask = None if mask is None else _row_mask(xc, mask)
        return ops.transition(xc, self._packed(x.device), row_mask, self.eps if self.norm is None else self.norm.eps,
                              residual=residual, out=out)

    def _forward_gemms(self, x, xc, mask, residual: bool, inplace: bool) -> torch.Tensor:
        if mask is not None:
            raise ValueError("a row mask is only supported by the fused pair transition (dim 128, hidden 512)")
        w = self._packed(x.device)
        rows = xc.numel() // self.dim
        eps = self.eps if self.norm is None else self.norm.eps
        stats = ops.row_stats(xc, eps) if self.norm is not None else None
        h = ops.linear(xc, w["w1"], w["sc1"], ops.LINEAR_SWIGLU, B=1, rows=rows, stats=stats)
        x3 = xc.view(1, rows, self.dim)
        y = ops.linear(h, w["w2"], w["sc2"], ops.LINEAR_ROWS, B=1, rows=rows, residual=x3 if residual else None,
                       out=x3 if (residual and inplace) else None).view(xc.shape)
        if residual and inplace and xc is not x:
            x.copy_(y)
            return x
        return y


class PairTransition(nn.Module):
    """ReLU pair transition ``linear_2(relu(linear_1(LayerNorm(z))))`` over ``[*, N, N, c_z]``, both linears with
    biases, on the fused sm_100a kernel (``b200ta_transition_relu``).

    Drop-in counterpart of ``PairTransition`` (``bionemo_ir/_torch/layers/transition.py:591-656``, body
    ``_ReluTransition`` l.540-588): same constructor, ``forward(z, mask=None, *, residual=False)`` and
    ``state_dict`` keys (``layer_norm.{weight,bias}``, ``linear_1.{weight,bias}`` ``[n*c_z, c_z]``,
    ``linear_2.{weight,bias}`` ``[c_z, n*c_z]``).  The kernel is specialised for ``c_z = 128`` and ``n = 4``.
    """

    def __init__(self, c_z: int, n: int, eps: float = 1e-5, dtype: torch.dtype = None, skip_create_weights: bool = False,
                 auto_chunk_policy: ChunkPolicy | None = None):
        super().__init__()
        if (c_z, n * c_z) != (ops.C, ops.HIDDEN):
            raise ValueError(f"the sm_100a ReLU transition kernel takes c_z={ops.C}, n={ops.HIDDEN // ops.C}; got c_z={c_z}, n={n}")
        self.c_z, self.n, self.dtype = c_z, n, dtype
        self.auto_chunk_policy = auto_chunk_policy  # accepted; the fused kernel holds no activation beyond its output
        self.layer_norm = nn.LayerNorm(c_z, eps=eps, dtype=dtype)
        self.linear_1 = Linear(c_z, n * c_z, bias=True, dtype=dtype, skip_create_weights=skip_create_weights)
        self.linear_2 = Linear(n * c_z, c_z, bias=True, dtype=dtype, skip_create_weights=skip_create_weights)
        self._pack = None
        self._pack_state = None
        self.register_load_state_dict_post_hook(_refold_after_load_state_dict)

    def _params(self):
        return (self.layer_norm.weight, self.layer_norm.bias, self.linear_1.weight, self.linear_1.bias,
                self.linear_2.weight, self.linear_2.bias)

    @torch.no_grad()
    def post_load_weights(self) -> None:
        """Refold the LayerNorm-folded weights from the (re)loaded parameters."""
        if not (self.linear_1._weights_created and self.linear_2._weights_created) or not self.linear_2.weight.is_cuda:
            self._pack = self._pack_state = None
            return
        device = self.linear_2.weight.device  # LayerNorm's parameters may still sit on the host at load time
        self._pack = ops.pack_relu_transition_weights(*[t.to(device) for t in self._params()])
        self._pack_state = _weight_state(*self._params())

    def _packed(self, device) -> torch.Tensor:
        state = _weight_state(*self._params())
        if self._pack is None or self._pack.device != device or state != self._pack_state:
            pack = ops.pack_relu_transition_weights(*[t.to(device) for t in self._params()])
            if not torch.cuda.is_current_stream_capturing():
                self._pack, self._pack_state = pack, state
            return pack
        return self._pack

    def forward(self, z: torch.Tensor, mask: torch.Tensor | None = None, *, residual: bool = False) -> torch.Tensor:
        """``[z +] mask * (linear_2(relu(linear_1(LayerNorm(z)))))``; ``mask`` holds one value per pair position."""
        if self.dtype not in (None, torch.bfloat16) or (self.dtype is None and z.dtype != torch.bfloat16):
            raise ValueError("the sm_100a transition kernel computes in bfloat16; construct the layer with "
                             "dtype=torch.bfloat16")
        if not z.is_cuda:
            raise ValueError("this layer runs on a CUDA device only (no CPU path)")
        z = z.to(torch.bfloat16)
        if not z.is_contiguous():
            order = _storage_order(z)
            if order is None:
                raise ValueError("PairTransition takes a contiguous tensor or a permuted view of one (channels last, "
                                 f"unit stride); got shape {tuple(z.shape)} with strides {z.stride()}")
            inverse = [order.index(d) for d in range(z.dim())]
            mask_p = None if mask is None else _row_mask(z, mask).permute(order[:-1])
            return self.forward(z.permute(order), mask_p, residual=residual).permute(inverse)
        row_mask = None if mask is None else _row_mask(z, mask)
        return ops.transition(z, self._packed(z.device), row_mask, self.layer_norm.eps, residual=residual, relu=True)
