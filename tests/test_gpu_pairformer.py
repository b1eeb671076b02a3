"""The pair-track Pairformer stack (triangle multiplication, triangle attention, transition per block)."""

import pytest
import torch

import bionemo_inference_runtime_b200 as b200
from bionemo_inference_runtime_b200 import _lib
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _clean_device_status():
    _lib.reset_device_status()
    yield
    assert _lib.device_status() == 0, "a kernel abandoned a bounded wait"


def _q(w):
    return w.to(torch.bfloat16).to(torch.float32)


def _block_weights(seed):
    return {"mo": _q(orc.make_trimul_weights(seed, identity_ln=False)), "mi": _q(orc.make_trimul_weights(seed + 1, identity_ln=False)),
            "as": _q(orc.make_node_weights(seed + 2, identity_ln=False)), "ae": _q(orc.make_node_weights(seed + 3, identity_ln=False)),
            "tr": _q(orc.make_transition_weights(seed + 4, identity_ln=False))}


def _state_dict(blocks):
    sd = {}
    for i, w in enumerate(blocks):
        for name, m in (("tri_mul_out", w["mo"]), ("tri_mul_in", w["mi"])):
            sd.update({f"layers.{i}.{name}.norm_in.weight": m.ln_in_w, f"layers.{i}.{name}.norm_in.bias": m.ln_in_b,
                       f"layers.{i}.{name}.p_in.weight": m.w_p_in, f"layers.{i}.{name}.g_in.weight": m.w_g_in,
                       f"layers.{i}.{name}.norm_out.weight": m.ln_out_w, f"layers.{i}.{name}.norm_out.bias": m.ln_out_b,
                       f"layers.{i}.{name}.p_out.weight": m.w_p_out, f"layers.{i}.{name}.g_out.weight": m.w_g_out})
        for name, a in (("tri_attn_start", w["as"]), ("tri_attn_end", w["ae"])):
            sd.update({f"layers.{i}.{name}.layer_norm.weight": a.ln_w, f"layers.{i}.{name}.layer_norm.bias": a.ln_b,
                       f"layers.{i}.{name}.pair_bias_proj.weight": a.w_bias, f"layers.{i}.{name}.mha.in_proj.weight": a.w_in,
                       f"layers.{i}.{name}.mha.o_proj.weight": a.w_out})
        t = w["tr"]
        sd.update({f"layers.{i}.transition_z.norm.weight": t.ln_w, f"layers.{i}.transition_z.norm.bias": t.ln_b,
                   f"layers.{i}.transition_z.fused_fc2_fc1.weight": t.w1, f"layers.{i}.transition_z.fc3.weight": t.w2})
    return sd


def _oracle(z, mask, blocks):
    dev = lambda w: type(w)(*[None if t is None else t.to(DEV) for t in (w.fields() if hasattr(w, "fields") else  # noqa: E731
                                                                        w.__dict__.values())])
    z, mask = z.float().to(DEV), mask.to(DEV)
    for w in blocks:
        z = orc.trimul_forward(z, mask, dev(w["mo"]), orc.OUTGOING, residual=True)
        z = orc.trimul_forward(z, mask, dev(w["mi"]), orc.INCOMING, residual=True)
        z = orc.node_forward(z, mask, dev(w["as"]), orc.STARTING, residual=True)
        z = orc.node_forward(z, mask, dev(w["ae"]), orc.ENDING, residual=True)
        z = orc.transition_forward(z, None, dev(w["tr"]), residual=True)
    return z


@pytest.mark.parametrize("backend", ["Heuristic", "VANILLA"])
def test_two_blocks_match_the_oracle_and_the_graph_replay_matches_eager(backend):
    torch.manual_seed(31)
    n, valid = 72, 72  # all tokens valid: the masked fused-residual form and the plain one coincide
    blocks = [_block_weights(100), _block_weights(200)]
    stack = b200.PairformerNoSeqModule(num_blocks=2, dtype=torch.bfloat16, triangle_attn_backend=backend,
                                       trimul_high_precision=False)
    stack.load_state_dict(_state_dict(blocks), strict=True)
    stack = stack.to(DEV)
    z = torch.randn(1, n, n, 128).bfloat16()
    m = (torch.arange(n) < valid).float()
    mask = (m[:, None] * m[None, :]).unsqueeze(0)
    out = stack(z.to(DEV), mask.to(DEV))
    want = _oracle(z, mask, blocks)
    torch.testing.assert_close(out.float(), want, rtol=3e-2, atol=3e-2)

    graphed = b200.PairformerNoSeqModule(num_blocks=2, dtype=torch.bfloat16, triangle_attn_backend=backend,
                                         trimul_high_precision=False, use_cuda_graph=True)
    graphed.load_state_dict(_state_dict(blocks), strict=True)
    graphed = graphed.to(DEV)
    first = graphed(z.to(DEV), mask.to(DEV))
    again = graphed(z.to(DEV), mask.to(DEV))  # replay
    assert torch.equal(first, out) and torch.equal(again, out)
    z2 = torch.randn(1, n, n, 128).bfloat16().to(DEV)
    assert torch.equal(graphed(z2, mask.to(DEV)), stack(z2, mask.to(DEV)))
    # new weights after the graph was recorded: the next call must not replay kernels that hold the old packs
    other = _state_dict([_block_weights(300), _block_weights(400)])
    graphed.load_state_dict(other, strict=True)
    stack.load_state_dict(other, strict=True)
    fresh = stack(z2, mask.to(DEV))
    assert not torch.equal(fresh, out)
    assert torch.equal(graphed(z2, mask.to(DEV)), fresh)


def test_padded_tokens_stay_finite_and_valid_region_matches():
    torch.manual_seed(32)
    n, valid = 64, 50
    blocks = [_block_weights(300)]
    stack = b200.PairformerNoSeqModule(num_blocks=1, dtype=torch.bfloat16, triangle_attn_backend="Heuristic",
                                       trimul_high_precision=False)
    stack.load_state_dict(_state_dict(blocks), strict=True)
    stack = stack.to(DEV)
    z = torch.randn(1, n, n, 128).bfloat16()
    m = (torch.arange(n) < valid).float()
    mask = (m[:, None] * m[None, :]).unsqueeze(0)
    out = stack(z.to(DEV), mask.to(DEV)).float()
    assert torch.isfinite(out).all()
    # inside the valid square the masked residual form ((x + update) * mask) equals the plain one
    want = _oracle(z, mask, blocks)
    torch.testing.assert_close(out[:, :valid, :valid], want[:, :valid, :valid], rtol=3e-2, atol=3e-2)
