"""Checkpoint key mappings from Boltz-style pair-track sublayers to this package's layers.

Same three functions as the reference's ``bionemo_ir/models/convert_utils.py:29-98`` (names, arguments, returned
keys), so a converter written against the reference keeps working:

* triangle attention: ``linear`` -> ``pair_bias_proj``; ``mha.linear_q/k/v/g`` concatenated in that order into
  ``mha.in_proj``; ``mha.linear_o`` -> ``mha.o_proj``
* triangle multiplication: the eight tensors keep their names; the input side is cast, the output side
  (``norm_out``, ``p_out``, ``g_out``) keeps the checkpoint dtype, because the node may hold it in fp32
* transition: ``fc2`` (value) rows first, then ``fc1`` (gate) rows, into ``fused_fc2_fc1``

``get_attention_pair_bias_weights`` adds the single-track attention in the same style, with the mapping the
reference's Boltz converter applies per layer (``bionemo_ir/models/boltz1/convert.py:64-98``): ``proj_q`` (weight
and bias), ``proj_g``, ``proj_k``, ``proj_v`` concatenated in that order into ``in_proj`` (the bias of the three
bias-free segments is zero); ``norm_s``, ``proj_z.0``, ``proj_z.1`` and ``proj_o`` keep their names.
"""

from __future__ import annotations

import torch

__all__ = ["get_attention_pair_bias_weights", "get_transition_weights", "get_tri_attn_node_weights",
           "get_tri_mul_node_weights"]

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "float": torch.float32, "bfloat16": torch.bfloat16,
           "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16, "half": torch.float16}


def _dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"unknown dtype name {name!r}; expected one of {sorted(_DTYPES)}") from None


def _remap(state_dict: dict, prefix: str, bioir_prefix: str, table, dtype: torch.dtype) -> dict:
    """``table``: (target suffix, source suffixes to concatenate along dim 0, cast?)."""
    out = {}
    for target, sources, cast in table:
        parts = [state_dict[f"{prefix}.{name}"] for name in sources]
        tensor = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        out[f"{bioir_prefix}.{target}"] = tensor.to(dtype) if cast else tensor
    return out


_TRI_ATTN = (
    ("layer_norm.weight", ("layer_norm.weight",), True),
    ("layer_norm.bias", ("layer_norm.bias",), True),
    ("pair_bias_proj.weight", ("linear.weight",), True),
    ("mha.in_proj.weight", ("mha.linear_q.weight", "mha.linear_k.weight", "mha.linear_v.weight", "mha.linear_g.weight"), True),
    ("mha.o_proj.weight", ("mha.linear_o.weight",), True),
)
_TRI_MUL = (
    ("norm_in.weight", ("norm_in.weight",), True),
    ("norm_in.bias", ("norm_in.bias",), True),
    ("p_in.weight", ("p_in.weight",), True),
    ("g_in.weight", ("g_in.weight",), True),
    ("norm_out.weight", ("norm_out.weight",), False),
    ("norm_out.bias", ("norm_out.bias",), False),
    ("p_out.weight", ("p_out.weight",), False),
    ("g_out.weight", ("g_out.weight",), False),
)
_TRANSITION = (
    ("norm.weight", ("norm.weight",), True),
    ("norm.bias", ("norm.bias",), True),
    ("fused_fc2_fc1.weight", ("fc2.weight", "fc1.weight"), True),
    ("fc3.weight", ("fc3.weight",), True),
)


def get_tri_attn_node_weights(state_dict: dict, prefix: str, bioir_prefix: str, dtype: str = "float32") -> dict:
    return _remap(state_dict, prefix, bioir_prefix, _TRI_ATTN, _dtype(dtype))


def get_tri_mul_node_weights(state_dict: dict, prefix: str, bioir_prefix: str, dtype: str = "float32") -> dict:
    return _remap(state_dict, prefix, bioir_prefix, _TRI_MUL, _dtype(dtype))


def get_transition_weights(state_dict: dict, prefix: str, bioir_prefix: str, dim: int = 128,
                           dtype: str = "float32") -> dict:
    del dim  # kept for signature compatibility; the widths come from the tensors
    return _remap(state_dict, prefix, bioir_prefix, _TRANSITION, _dtype(dtype))


def get_attention_pair_bias_weights(state_dict: dict, prefix: str, bioir_prefix: str, dtype: str = "float32") -> dict:
    dt = _dtype(dtype)
    q_w = state_dict[f"{prefix}.proj_q.weight"]
    segments = [q_w] + [state_dict[f"{prefix}.proj_{name}.weight"] for name in ("g", "k", "v")]
    q_b = state_dict.get(f"{prefix}.proj_q.bias")
    bias = torch.zeros(sum(w.shape[0] for w in segments), dtype=q_w.dtype, device=q_w.device)
    if q_b is not None:
        bias[:q_w.shape[0]] = q_b
    out = {f"{bioir_prefix}.in_proj.weight": torch.cat(segments, dim=0).to(dt), f"{bioir_prefix}.in_proj.bias": bias.to(dt)}
    for name in ("norm_s.weight", "norm_s.bias", "proj_z.0.weight", "proj_z.0.bias", "proj_z.1.weight", "proj_o.weight",
                 "proj_o.bias"):
        if f"{prefix}.{name}" in state_dict:
            out[f"{bioir_prefix}.{name}"] = state_dict[f"{prefix}.{name}"].to(dt)
    return out
