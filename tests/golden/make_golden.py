"""Generates the golden fixtures in this directory from the reference's own modules.

Run where the reference checkout is available (it is not on the GPU machine):

    BIOIR_REFERENCE=/path/to/reference python tests/golden/make_golden.py

The reference package cannot be imported normally without its compiled kernel
library, so this script pre-registers an empty ``bionemo_ir`` package object
that points at the checkout, stubs the optional ``lru`` module, constructs the
layers with ``skip_create_weights=True`` and assigns CPU parameters.  Only the
reference's eager path runs (``attn_backend="VANILLA"``); the Transition's
Triton SwiGLU, which has no CPU implementation, is replaced by the equivalent
two PyTorch lines, and ``transition_mlp_w_norm_reference`` is called as is.

Every fixture stores its inputs, weights and the reference outputs, so the
tests need nothing but numpy to read them.
"""

from __future__ import annotations

import collections
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = Path(os.environ["BIOIR_REFERENCE"]) if "BIOIR_REFERENCE" in os.environ else None
sys.dont_write_bytecode = True


def install_shim() -> None:
    pkg = types.ModuleType("bionemo_ir")
    pkg.__path__ = [str(REF / "bionemo_ir")]
    pkg.CACHE_DIR = "/tmp/bioir_cache"
    pkg.EXAMPLES_DIR = str(REF / "examples")
    sys.modules["bionemo_ir"] = pkg
    lru = types.ModuleType("lru")

    class LRU(collections.OrderedDict):
        def __init__(self, size, callback=None):
            super().__init__()

    lru.LRU = LRU
    sys.modules["lru"] = lru


def set_linear(linear, weight: torch.Tensor, bias: torch.Tensor | None) -> None:
    linear.weight = torch.nn.Parameter(weight.clone(), requires_grad=False)
    if bias is not None:
        linear.bias = torch.nn.Parameter(bias.clone(), requires_grad=False)
    else:
        linear.register_parameter("bias", None)
    linear._weights_created = True


def build_node(cls, w: dict, dtype: torch.dtype, gate_bias: bool, out_bias: bool, **kw):
    flags = {"q": False, "k": False, "v": False, "g": gate_bias, "o": out_bias}
    node = cls(128, 32, 4, dtype=dtype, skip_create_weights=True, attn_backend="VANILLA", mha_bias_flags=flags, **kw)
    node.layer_norm.weight.data.copy_(w["ln_w"])
    node.layer_norm.bias.data.copy_(w["ln_b"])
    set_linear(node.pair_bias_proj, w["w_bias"].to(dtype), None)
    set_linear(node.mha.in_proj, w["w_in"].to(dtype), w["b_in"].to(dtype) if gate_bias else None)
    set_linear(node.mha.o_proj, w["w_out"].to(dtype), w["b_out"].to(dtype) if out_bias else None)
    return node.to(dtype)


def node_weights(seed: int, identity_ln: bool) -> dict:
    g = torch.Generator().manual_seed(seed)
    w = {
        "w_bias": torch.randn(4, 128, generator=g) * 0.02,
        "w_in": torch.randn(512, 128, generator=g) * 0.02,
        "w_out": torch.randn(128, 128, generator=g) * 0.02,
        "ln_w": torch.ones(128) if identity_ln else 1 + 0.2 * torch.randn(128, generator=g),
        "ln_b": torch.zeros(128) if identity_ln else 0.2 * torch.randn(128, generator=g),
        "b_in": torch.zeros(512),
        "b_out": 0.1 * torch.randn(128, generator=g),
    }
    w["b_in"][384:] = 1.0  # gate bias = 1
    # keep everything exactly representable in bf16 so bf16 and fp32 runs share inputs
    return {k: v.bfloat16().float() for k, v in w.items()}


def save(name: str, **arrays) -> None:
    out = {k: (v.float().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in arrays.items()}
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(f"wrote {name}.npz ({(HERE / f'{name}.npz').stat().st_size / 1024:.0f} KiB)")


def main() -> None:
    if REF is None:
        raise SystemExit("set BIOIR_REFERENCE to the reference checkout")
    install_shim()
    from bionemo_ir._torch.custom_ops.transition_mlp_w_norm import transition_mlp_w_norm_reference
    from bionemo_ir._torch.layers.transition import Transition
    from bionemo_ir._torch.layers.triangle_nodes import TriangleAttentionEndingNode, TriangleAttentionStartingNode

    torch.manual_seed(0)
    # ---- case 1: starting node, all-ones mask, gate bias 1, identity LayerNorm (the reference's CPU benchmark case, shrunk)
    g = torch.Generator().manual_seed(1000)
    N = 24
    z = torch.randn(1, N, N, 128, generator=g).bfloat16().float()
    w = node_weights(1, identity_ln=True)
    node = build_node(TriangleAttentionStartingNode, w, torch.float32, gate_bias=True, out_bias=False)
    mask = torch.ones(1, N, N)
    out_update = node(z, mask=mask)
    out_res = node(z, mask=mask, residual=True)
    save("node_start_fullmask", z=z, mask=mask, out_update=out_update, out_residual=out_res,
         **{f"w_{k}": v for k, v in w.items()}, gate_bias=1, out_bias=0, node_type=0)

    # ---- case 2: ending node, batch of 2 with different valid lengths (padded rows present), affine LayerNorm,
    #      o_proj bias; fp32 and bf16 runs of the reference
    g = torch.Generator().manual_seed(1001)
    N = 20
    z = torch.randn(2, N, N, 128, generator=g).bfloat16().float()
    w = node_weights(2, identity_ln=False)
    m = torch.zeros(2, N)
    m[0, :13] = 1
    m[1, :N] = 1
    mask = m[:, :, None] * m[:, None, :]
    node = build_node(TriangleAttentionEndingNode, w, torch.float32, gate_bias=True, out_bias=True)
    out32 = node(z, mask=mask, residual=True)
    node16 = build_node(TriangleAttentionEndingNode, w, torch.bfloat16, gate_bias=True, out_bias=True)
    out16 = node16(z.bfloat16(), mask=mask.bfloat16(), residual=True)
    start = build_node(TriangleAttentionStartingNode, w, torch.float32, gate_bias=True, out_bias=True)
    out_start = start(z, mask=mask, residual=True)
    save("node_end_padded", z=z, mask=mask, out_residual=out32, out_residual_bf16=out16, out_start_residual=out_start,
         **{f"w_{k}": v for k, v in w.items()}, gate_bias=1, out_bias=1, node_type=1)

    # ---- case 3: transposed triangle bias (OpenFold-3 ending node)
    node_t = build_node(TriangleAttentionEndingNode, w, torch.float32, gate_bias=True, out_bias=True, transposed_bias=True)
    out_t = node_t(z, mask=mask, residual=False)
    save("node_end_transposed_bias", z=z, mask=mask, out_update=out_t, **{f"w_{k}": v for k, v in w.items()},
         gate_bias=1, out_bias=1, node_type=1)

    # ---- case 4: transition
    g = torch.Generator().manual_seed(1002)
    x = torch.randn(2, 12, 12, 128, generator=g).bfloat16().float()
    tw = {
        "w1": (torch.randn(1024, 128, generator=g) * 0.02).bfloat16().float(),
        "w2": (torch.randn(128, 512, generator=g) * 0.02).bfloat16().float(),
        "ln_w": (1 + 0.2 * torch.randn(128, generator=g)).bfloat16().float(),
        "ln_b": (0.2 * torch.randn(128, generator=g)).bfloat16().float(),
    }
    tmask = (torch.rand(2, 12, 12, generator=g) > 0.3).float()
    ref_res = transition_mlp_w_norm_reference(x, tmask, tw["ln_w"], tw["ln_b"], tw["w1"], None, tw["w2"], None, 1e-5,
                                              activation="silu_gate", residual=True)
    ref_upd = transition_mlp_w_norm_reference(x, None, tw["ln_w"], tw["ln_b"], tw["w1"], None, tw["w2"], None, 1e-5,
                                              activation="silu_gate", residual=False)
    layer = Transition(128, 512, dtype=torch.float32, skip_create_weights=True)
    layer.norm.weight.data.copy_(tw["ln_w"])
    layer.norm.bias.data.copy_(tw["ln_b"])
    set_linear(layer.fused_fc2_fc1, tw["w1"], None)
    set_linear(layer.fc3, tw["w2"], None)
    layer._swiglu = lambda t: torch.nn.functional.silu(t[..., 512:]) * t[..., :512]
    mod_upd = layer._forward_impl(x, tmask)
    layer16 = Transition(128, 512, dtype=torch.bfloat16, skip_create_weights=True)
    layer16.norm.weight.data.copy_(tw["ln_w"])
    layer16.norm.bias.data.copy_(tw["ln_b"])
    layer16 = layer16.to(torch.bfloat16)
    set_linear(layer16.fused_fc2_fc1, tw["w1"].bfloat16(), None)
    set_linear(layer16.fc3, tw["w2"].bfloat16(), None)
    layer16._swiglu = lambda t: torch.nn.functional.silu(t[..., 512:].float()).to(t.dtype) * t[..., :512]
    mod_upd16 = layer16._forward_impl(x.bfloat16(), tmask.bfloat16())
    save("transition", x=x, mask=tmask, out_residual_masked=ref_res, out_update=ref_upd, out_module_update_masked=mod_upd,
         out_module_update_masked_bf16=mod_upd16, **{f"w_{k}": v for k, v in tw.items()})

    relu_transition_case()
    trimul_cases()
    single_track_cases()


def relu_transition_case() -> None:
    """ReLU pair transition: the reference's fused-kernel reference function (activation="relu") and the eager body
    of its PairTransition module (``_forward_impl``), fp32 and bf16.  The module's FusedLayerNorm takes CUDA tensors
    only, so its ``layer_norm`` attribute is replaced by a plain ``torch.nn.LayerNorm`` with the same parameters."""
    from bionemo_ir._torch.custom_ops.transition_mlp_w_norm import transition_mlp_w_norm_reference
    from bionemo_ir._torch.layers.transition import PairTransition

    g = torch.Generator().manual_seed(1005)
    x = torch.randn(2, 12, 12, 128, generator=g).bfloat16().float()
    w = {
        "w1": (torch.randn(512, 128, generator=g) * 0.05).bfloat16().float(),
        "b1": (0.1 * torch.randn(512, generator=g)).bfloat16().float(),
        "w2": (torch.randn(128, 512, generator=g) * 0.05).bfloat16().float(),
        "b2": (0.1 * torch.randn(128, generator=g)).bfloat16().float(),
        "ln_w": (1 + 0.2 * torch.randn(128, generator=g)).bfloat16().float(),
        "ln_b": (0.2 * torch.randn(128, generator=g)).bfloat16().float(),
    }
    mask = (torch.rand(2, 12, 12, generator=g) > 0.3).float()
    ref_res = transition_mlp_w_norm_reference(x, mask, w["ln_w"], w["ln_b"], w["w1"], w["b1"], w["w2"], w["b2"], 1e-5,
                                              activation="relu", residual=True)
    ref_upd = transition_mlp_w_norm_reference(x, None, w["ln_w"], w["ln_b"], w["w1"], w["b1"], w["w2"], w["b2"], 1e-5,
                                              activation="relu", residual=False)
    out = {}
    for name, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        layer = PairTransition(128, 4, dtype=dtype, skip_create_weights=True)
        layer.layer_norm = torch.nn.LayerNorm(128, eps=1e-5)
        layer.layer_norm.weight.data.copy_(w["ln_w"])
        layer.layer_norm.bias.data.copy_(w["ln_b"])
        layer = layer.to(dtype)
        set_linear(layer.linear_1, w["w1"].to(dtype), w["b1"].to(dtype))
        set_linear(layer.linear_2, w["w2"].to(dtype), w["b2"].to(dtype))
        out[f"out_module_residual_masked_{name}"] = layer._forward_impl(x.to(dtype), mask.to(dtype), residual=True)
    save("pair_transition_relu", x=x, mask=mask, out_residual_masked=ref_res, out_update=ref_upd, **out,
         **{f"w_{k}": v for k, v in w.items()})


def single_track_cases() -> None:
    """Single-track attention with pair bias and the single-track transition.  The reference's AttentionPairBias runs
    in eager mode on CPU except for its pair-bias projection (LNProjMoveaxisPad launches Triton kernels): that one
    submodule is replaced by the three PyTorch operations it documents (LayerNorm + Linear through the layer's own
    ``proj_z``, moveaxis(-1, -3), no padding); everything else is the reference's code."""
    from bionemo_ir._torch.layers.attention import AttentionPairBias
    from bionemo_ir._torch.layers.transition import Transition

    class EagerPairBias(torch.nn.Module):
        def forward(self, z, **kw):
            return kw["proj_z"](z).movedim(-1, -3).contiguous()

    def build(dtype, w, initial_norm, out_bias):
        layer = AttentionPairBias(layer_idx=0, c_s=384, c_z=128, num_heads=16, dtype=dtype, bias_proj=True, inf=1e9,
                                  skip_create_weights=True, attn_backend="VANILLA", initial_norm=initial_norm,
                                  out_bias=out_bias)
        if initial_norm:
            layer.norm_s.weight.data.copy_(w["norm_s_w"])
            layer.norm_s.bias.data.copy_(w["norm_s_b"])
        layer.proj_z[0].weight.data.copy_(w["norm_z_w"])
        layer.proj_z[0].bias.data.copy_(w["norm_z_b"])
        layer = layer.to(dtype)
        set_linear(layer.in_proj, w["w_in"].to(dtype), w["b_in"].to(dtype))
        set_linear(layer.proj_z[1], w["w_z"].to(dtype), None)
        set_linear(layer.proj_o, w["w_o"].to(dtype), w["b_o"].to(dtype) if out_bias else None)
        layer._ln_proj_moveaxis_pad = EagerPairBias()
        return layer

    # The weights (2.5 M values) are not stored: both this script and the tests rebuild them from the seeded recipes
    # in oracle/triangle_oracle.py; the fixture keeps a checksum of every tensor to detect a change of generator.
    sys.path.insert(0, str(HERE.parent.parent))
    from oracle import triangle_oracle as orc

    def checksum(weights) -> float:
        return float(sum(t.double().abs().sum() for t in weights.__dict__.values() if t is not None))

    g = torch.Generator().manual_seed(77)
    out = {}
    for case, (B, N, valid, initial_norm, out_bias, seed) in {"a": (1, 40, (33,), True, False, 501),
                                                               "b": (2, 24, (24, 17), False, True, 502)}.items():
        # weights, activations and mask rounded to bf16 so that the bf16 run and the kernels see the same numbers
        wo = orc.make_pair_bias_attention_weights(seed, initial_norm=initial_norm, out_bias=out_bias).to(torch.bfloat16).to(torch.float32)
        w = dict(wo.__dict__)
        s = torch.randn(B, N, 384, generator=g).bfloat16().float()
        z = torch.randn(B, N, N, 128, generator=g).bfloat16().float()
        mask = torch.zeros(B, N)
        for b, n_valid in enumerate(valid):
            mask[b, :n_valid] = 1
        upd32 = build(torch.float32, w, initial_norm, out_bias)(s, z, mask)
        upd16 = build(torch.bfloat16, w, initial_norm, out_bias)(s.bfloat16(), z.bfloat16(), mask)
        out.update({f"{case}_s": s, f"{case}_z": z, f"{case}_mask": mask, f"{case}_update": upd32,
                    f"{case}_update_bf16": upd16, f"{case}_initial_norm": int(initial_norm),
                    f"{case}_out_bias": int(out_bias), f"{case}_seed": seed, f"{case}_checksum": checksum(wo)})

    two = orc.make_transition_weights(503, c=384, hidden=1536, std=0.05, identity_ln=False).to(torch.bfloat16).to(torch.float32)
    tw = {"ln_w": two.ln_w, "ln_b": two.ln_b, "w1": two.w1, "w2": two.w2}
    x = torch.randn(1, 40, 384, generator=g).bfloat16().float()
    for name, dtype in (("t_update", torch.float32), ("t_update_bf16", torch.bfloat16)):
        layer = Transition(384, 1536, dtype=dtype, skip_create_weights=True)
        layer.norm.weight.data.copy_(tw["ln_w"])
        layer.norm.bias.data.copy_(tw["ln_b"])
        layer = layer.to(dtype)
        set_linear(layer.fused_fc2_fc1, tw["w1"].to(dtype), None)
        set_linear(layer.fc3, tw["w2"].to(dtype), None)
        layer._swiglu = lambda t: torch.nn.functional.silu(t[..., 1536:].float()).to(t.dtype) * t[..., :1536]
        out[name] = layer._forward_impl(x.to(dtype), None)
    save("single_track", t_x=x, t_seed=503, t_checksum=checksum(two), **out)


def trimul_cases() -> None:
    """Triangle multiplication.  The reference module itself needs CUDA to construct (it probes the SM version and
    its LayerNorm-transpose op takes CUDA tensors only), so the fixtures come from (i) the pure-PyTorch mirror the
    reference's own tests compare against, RefTriangleMultiplicationNode (tests/common/test_utils/boltz/ref_layers.py),
    and (ii) the reference's unfused dual-GEMM functions chained exactly as TriangleMultiplicationNode._forward_impl
    chains them (bf16 run, including the mean-normalised variant)."""
    sys.path.insert(0, str(REF / "tests" / "common"))
    from test_utils.boltz.ref_layers import RefTriangleMultiplicationNode
    from bionemo_ir._torch.custom_ops.dual_gemm_x0_x1.ops import _invoke_vanilla_dual_gemm_x0_x1
    from bionemo_ir._torch.custom_ops.dual_gemm_x_x.ops import _invoke_vanilla_dual_gemm_x_x

    g = torch.Generator().manual_seed(1003)
    N = 20
    z = torch.randn(2, N, N, 128, generator=g).bfloat16().float()
    m = torch.zeros(2, N)
    m[0, :13] = 1
    m[1, :N] = 1
    mask = m[:, :, None] * m[:, None, :]
    w = {
        "ln_in_w": 1 + 0.2 * torch.randn(128, generator=g), "ln_in_b": 0.2 * torch.randn(128, generator=g),
        "w_p_in": torch.randn(256, 128, generator=g) * 0.02, "w_g_in": torch.randn(256, 128, generator=g) * 0.02,
        "ln_out_w": 1 + 0.2 * torch.randn(128, generator=g), "ln_out_b": 0.2 * torch.randn(128, generator=g),
        "w_p_out": torch.randn(128, 128, generator=g) * 0.02, "w_g_out": torch.randn(128, 128, generator=g) * 0.02,
    }
    w = {k: v.bfloat16().float() for k, v in w.items()}
    outs = {}
    for name, outgoing in (("outgoing", True), ("incoming", False)):
        ref = RefTriangleMultiplicationNode(128, outgoing=outgoing)
        ref.norm_in.weight.data.copy_(w["ln_in_w"]), ref.norm_in.bias.data.copy_(w["ln_in_b"])
        ref.norm_out.weight.data.copy_(w["ln_out_w"]), ref.norm_out.bias.data.copy_(w["ln_out_b"])
        ref.p_in.weight.data.copy_(w["w_p_in"]), ref.g_in.weight.data.copy_(w["w_g_in"])
        ref.p_out.weight.data.copy_(w["w_p_out"]), ref.g_out.weight.data.copy_(w["w_g_out"])
        outs[f"update_{name}"] = ref(z, mask)

        # the module's own chain of unfused ops in bf16 (high_precision=False): triangle_nodes.py:680-722
        wb = {k: v.bfloat16() for k, v in w.items()}
        x_in = torch.nn.functional.layer_norm(z.bfloat16(), (128,), wb["ln_in_w"], wb["ln_in_b"], 1e-5)
        for mean_norm in (False, True):
            proj = _invoke_vanilla_dual_gemm_x_x(x_in, wb["w_g_in"], wb["w_p_in"], None, None, mask.bfloat16(),
                                                 transpose_out=True)
            a, b = torch.chunk(proj, 2, dim=0)
            if mean_norm:
                n_valid = mask.bfloat16()[:, 0, :].sum(dim=-1)
                b = b / (n_valid[None, :, None, None] + 1e-3)
            t = torch.einsum("dbik,dbjk->dbij", a, b) if outgoing else torch.einsum("dbki,dbkj->dbij", a, b)
            t = torch.nn.functional.layer_norm(t.permute(1, 2, 3, 0), (128,), wb["ln_out_w"], wb["ln_out_b"], 1e-5)
            upd = _invoke_vanilla_dual_gemm_x0_x1(x_in, t, wb["w_g_out"], wb["w_p_out"])
            outs[f"update_{name}_bf16{'_meannorm' if mean_norm else ''}"] = upd
    save("trimul", z=z, mask=mask, **outs, **{f"w_{k}": v for k, v in w.items()})


if __name__ == "__main__":
    with torch.no_grad():
        main()
