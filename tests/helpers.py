"""Test helpers: golden-fixture loading and oracle weight conversion."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from oracle import triangle_oracle as orc

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz") as f:
        return {k: (torch.from_numpy(f[k]) if f[k].ndim else f[k].item()) for k in f.files}


def golden_node_weights(g: dict, dtype=torch.float32) -> orc.NodeWeights:
    return orc.NodeWeights(
        ln_w=g["w_ln_w"], ln_b=g["w_ln_b"], w_bias=g["w_w_bias"], w_in=g["w_w_in"],
        b_in=g["w_b_in"] if g["gate_bias"] else None, w_out=g["w_w_out"],
        b_out=g["w_b_out"] if g["out_bias"] else None,
    ).to(dtype)


def golden_transition_weights(g: dict, dtype=torch.float32) -> orc.TransitionWeights:
    return orc.TransitionWeights(g["w_ln_w"], g["w_ln_b"], g["w_w1"], g["w_w2"]).to(dtype)


def golden_trimul_weights(g: dict, dtype=torch.float32) -> orc.TriMulWeights:
    return orc.TriMulWeights(g["w_ln_in_w"], g["w_ln_in_b"], g["w_w_p_in"], g["w_w_g_in"], g["w_ln_out_w"],
                             g["w_ln_out_b"], g["w_w_p_out"], g["w_w_g_out"]).to(dtype)


def _checksum(weights) -> float:
    return float(sum(t.double().abs().sum() for t in weights.__dict__.values() if t is not None))


def golden_single_attention_weights(g: dict, case: str) -> orc.PairBiasAttentionWeights:
    """The seeded weights of a single-track fixture case (bf16-rounded, as fp32), checked against its checksum."""
    w = orc.make_pair_bias_attention_weights(int(g[f"{case}_seed"]), initial_norm=bool(g[f"{case}_initial_norm"]),
                                             out_bias=bool(g[f"{case}_out_bias"])).to(torch.bfloat16).to(torch.float32)
    assert abs(_checksum(w) - g[f"{case}_checksum"]) < 1e-6 * g[f"{case}_checksum"], "weight recipe changed"
    return w


def golden_single_transition_weights(g: dict) -> orc.TransitionWeights:
    w = orc.make_transition_weights(int(g["t_seed"]), c=384, hidden=1536, std=0.05, identity_ln=False)
    w = w.to(torch.bfloat16).to(torch.float32)
    assert abs(_checksum(w) - g["t_checksum"]) < 1e-6 * g["t_checksum"], "weight recipe changed"
    return w
