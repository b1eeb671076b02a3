"""``Linear`` parameter holder with the reference's fused-segment weight loading.

Mirrors ``bionemo_ir/_torch/layers/linear.py:71-198``: ``weight[out, in]`` (+ optional ``bias``) are
``requires_grad=False`` parameters created at construction unless ``skip_create_weights`` is set;
``load_weights`` concatenates checkpoint segments in order.  In this package the node and
transition layers never call ``forward`` on their Linear children (the kernels read the packed
weights); ``forward`` exists for callers that use a Linear on its own and is a plain ``F.linear``.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.parameter import Parameter


class WeightMode(str, enum.Enum):
    VANILLA = "vanilla"
    FUSED_QKV_LINEAR = "fused_qkv_linear"
    FUSED_KV_LINEAR = "fused_kv_linear"
    FUSED_SEGMENTS_LINEAR = "fused_segments_linear"


@dataclass(frozen=True)
class WeightsLoadingConfig:
    weight_mode: WeightMode = WeightMode.VANILLA
    segment_sizes: tuple[int, ...] = ()


class Linear(nn.Module):
    """``weight[out_features, in_features]`` and an optional ``bias[out_features]``, both frozen.  The tensors are
    allocated (uninitialised, on the GPU when there is one) at construction unless ``skip_create_weights`` defers
    that to a later ``create_weights()``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype: torch.dtype = None,
                 weights_loading_config: WeightsLoadingConfig | None = None, skip_create_weights: bool = False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.has_bias, self.dtype = bias, dtype
        self.weights_loading_config = WeightsLoadingConfig() if weights_loading_config is None else weights_loading_config
        self._weights_created = False
        if not skip_create_weights:
            self.create_weights()

    def _frozen(self, *shape: int) -> Parameter:
        device = "cuda" if torch.cuda.is_available() else "cpu"
        return Parameter(torch.empty(shape, dtype=self.dtype, device=device), requires_grad=False)

    def create_weights(self):
        if not self._weights_created:
            self.weight = self._frozen(self.out_features, self.in_features)
            self.register_parameter("bias", self._frozen(self.out_features) if self.has_bias else None)
            self._weights_created = True

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return F.linear(input, self.weight, self.bias)

    @torch.no_grad()
    def load_weights(self, weights: list[dict]):
        """Copy checkpoint segments (dicts with ``weight`` and optional ``bias``) into the fused parameters."""
        assert self._weights_created
        mode = self.weights_loading_config.weight_mode
        dev = self.weight.device

        def cat(key):
            return torch.cat([w[key].to(dev) for w in weights])

        if mode == WeightMode.VANILLA:
            assert len(weights) == 1
            self.weight.data.copy_(weights[0]["weight"].to(dev).to(self.weight.dtype))
            if self.bias is not None:
                self.bias.data.copy_(weights[0]["bias"].to(dev).to(self.bias.dtype))
        elif mode in (WeightMode.FUSED_QKV_LINEAR, WeightMode.FUSED_KV_LINEAR):
            assert len(weights) == (3 if mode == WeightMode.FUSED_QKV_LINEAR else 2)
            self.weight.data.copy_(cat("weight").to(self.weight.dtype))
            if self.bias is not None:
                self.bias.data.copy_(cat("bias").to(self.bias.dtype))
        elif mode == WeightMode.FUSED_SEGMENTS_LINEAR:
            sizes = self.weights_loading_config.segment_sizes
            assert len(weights) == len(sizes) and sum(sizes) == self.out_features
            self.weight.data.zero_()
            if self.bias is not None:
                self.bias.data.zero_()
            start = 0
            for size, segment in zip(sizes, weights, strict=True):
                w = segment["weight"].to(dev)
                rows = w.shape[0]
                assert rows <= size, f"a {rows}-row weight does not fit its {size}-row segment"
                self.weight.data[start:start + rows].copy_(w.to(self.weight.dtype))
                if self.bias is not None and segment.get("bias") is not None:
                    self.bias.data[start:start + rows].copy_(segment["bias"].to(dev).to(self.bias.dtype))
                start += size
        else:
            raise ValueError(f"unsupported weight mode: {mode}")
