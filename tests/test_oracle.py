"""Pins the CPU oracle against outputs of the reference's own modules (tests/golden/*.npz)."""

import pytest
import torch

from oracle import triangle_oracle as orc
from tests.helpers import golden_node_weights, golden_transition_weights, golden_trimul_weights, load_golden


def test_start_node_full_mask_fp32():
    g = load_golden("node_start_fullmask")
    w = golden_node_weights(g)
    upd = orc.node_forward(g["z"], g["mask"], w, orc.STARTING)
    res = orc.node_forward(g["z"], g["mask"], w, orc.STARTING, residual=True)
    assert (upd - g["out_update"]).abs().max() < 1e-6
    assert (res - g["out_residual"]).abs().max() < 1e-6


def test_end_node_padded_rows_fp32():
    g = load_golden("node_end_padded")
    w = golden_node_weights(g)
    res = orc.node_forward(g["z"], g["mask"], w, orc.ENDING, residual=True)
    assert (res - g["out_residual"]).abs().max() < 1e-6
    start = orc.node_forward(g["z"], g["mask"], w, orc.STARTING, residual=True)
    assert (start - g["out_start_residual"]).abs().max() < 1e-6


def test_end_node_padded_rows_bf16_matches_eager_rounding():
    g = load_golden("node_end_padded")
    w = golden_node_weights(g, torch.bfloat16)
    res = orc.node_forward(g["z"].bfloat16(), g["mask"].bfloat16(), w, orc.ENDING, residual=True)
    # same ops in the same order on the same machine type; allow one bf16 ulp at |x| < 8
    assert (res.float() - g["out_residual_bf16"]).abs().max() <= 2 ** -5


def test_ending_is_transposed_starting():
    g = load_golden("node_end_padded")
    w = golden_node_weights(g)
    end = orc.node_forward(g["z"], g["mask"], w, orc.ENDING)
    start_t = orc.node_forward(g["z"].transpose(1, 2), g["mask"].transpose(1, 2), w, orc.STARTING).transpose(1, 2)
    assert torch.equal(end, start_t)


def test_transposed_bias():
    g = load_golden("node_end_transposed_bias")
    w = golden_node_weights(g)
    upd = orc.node_forward(g["z"], g["mask"], w, orc.ENDING, transposed_bias=True)
    assert (upd - g["out_update"]).abs().max() < 1e-6


def test_empty_rows_are_uniform_in_the_eager_path():
    """A row without a valid key averages V over every key (the additive -1e9 swamps the logits)."""
    g = load_golden("node_end_padded")
    w = golden_node_weights(g)
    st = orc.node_stages(g["z"], g["mask"], w, orc.ENDING)
    B, R, S, _ = st["v"].shape
    lengths = orc.row_lengths(st["mask"])
    assert (lengths == 0).any()
    v = st["v"].reshape(B * R, S, 4, 32)
    o_uniform, _ = orc.attention_core(st["q"].reshape(B * R, S, 4, 32), st["k"].reshape(B * R, S, 4, 32), v,
                                      st["tri_bias"], lengths.reshape(-1), 32 ** -0.5, empty_rows="uniform")
    assert (o_uniform.reshape(B, R, S, 128) - st["o"]).abs().max() < 1e-5


def test_transition_fp32():
    g = load_golden("transition")
    w = golden_transition_weights(g)
    res = orc.transition_forward(g["x"], g["mask"], w, residual=True)
    upd = orc.transition_forward(g["x"], None, w)
    mod = orc.transition_forward(g["x"], g["mask"], w)
    assert (res - g["out_residual_masked"]).abs().max() < 1e-5
    assert (upd - g["out_update"]).abs().max() < 1e-5
    assert (mod - g["out_module_update_masked"]).abs().max() < 1e-5


def test_transition_bf16_matches_eager_rounding():
    g = load_golden("transition")
    w = golden_transition_weights(g, torch.bfloat16)
    mod = orc.transition_forward(g["x"].bfloat16(), g["mask"].bfloat16(), w)
    assert (mod.float() - g["out_module_update_masked_bf16"]).abs().max() <= 2 ** -8


@pytest.mark.parametrize("name,direction", [("outgoing", orc.OUTGOING), ("incoming", orc.INCOMING)])
def test_triangle_multiplication_fp32_matches_the_reference_tests_mirror(name, direction):
    g = load_golden("trimul")
    w = golden_trimul_weights(g)
    upd = orc.trimul_forward(g["z"], g["mask"], w, direction)
    assert (upd - g[f"update_{name}"]).abs().max() < 2e-6
    res = orc.trimul_forward(g["z"], g["mask"], w, direction, residual=True)
    assert (res - (g["z"] + g[f"update_{name}"])).abs().max() < 2e-6


@pytest.mark.parametrize("name,direction", [("outgoing", orc.OUTGOING), ("incoming", orc.INCOMING)])
@pytest.mark.parametrize("mean_norm", [False, True])
def test_triangle_multiplication_bf16_matches_the_unfused_reference_ops(name, direction, mean_norm):
    g = load_golden("trimul")
    w = golden_trimul_weights(g, torch.bfloat16)
    upd = orc.trimul_forward(g["z"].bfloat16(), g["mask"].bfloat16(), w, direction, mean_normalization=mean_norm)
    want = g[f"update_{name}_bf16{'_meannorm' if mean_norm else ''}"]
    # same ops in the same order; einsum summation order may differ by an ulp of the bf16 contraction result
    assert (upd.float() - want).abs().max() <= 2 ** -7 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("case", ["a", "b"])
def test_single_track_attention_matches_the_reference_module(case):
    """AttentionPairBias as the pairformer builds it: with and without initial norm / output bias, one and two
    batch entries with different key counts."""
    from tests.helpers import golden_single_attention_weights

    g = load_golden("single_track")
    w = golden_single_attention_weights(g, case)
    got = orc.pair_bias_attention_forward(g[f"{case}_s"], g[f"{case}_z"], g[f"{case}_mask"], w)
    torch.testing.assert_close(got, g[f"{case}_update"], rtol=1e-4, atol=1e-5)
    got16 = orc.pair_bias_attention_forward(g[f"{case}_s"].bfloat16(), g[f"{case}_z"].bfloat16(), g[f"{case}_mask"],
                                            w.to(torch.bfloat16))
    torch.testing.assert_close(got16.float(), g[f"{case}_update_bf16"], rtol=2e-2, atol=2e-2)


def test_single_track_transition_matches_the_reference_module():
    from tests.helpers import golden_single_transition_weights

    g = load_golden("single_track")
    w = golden_single_transition_weights(g)
    torch.testing.assert_close(orc.transition_forward(g["t_x"], None, w), g["t_update"], rtol=1e-4, atol=1e-5)
    got16 = orc.transition_forward(g["t_x"].bfloat16(), None, w.to(torch.bfloat16))
    torch.testing.assert_close(got16.float(), g["t_update_bf16"], rtol=2e-2, atol=4e-2)


def test_relu_transition_matches_reference_outputs():
    g = load_golden("pair_transition_relu")
    w = orc.ReluTransitionWeights(g["w_ln_w"], g["w_ln_b"], g["w_w1"], g["w_b1"], g["w_w2"], g["w_b2"])
    torch.testing.assert_close(orc.relu_transition_forward(g["x"], g["mask"], w, residual=True), g["out_residual_masked"],
                               rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(orc.relu_transition_forward(g["x"], None, w), g["out_update"], rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(orc.relu_transition_forward(g["x"], g["mask"], w, residual=True),
                               g["out_module_residual_masked_fp32"], rtol=1e-6, atol=1e-6)
    got16 = orc.relu_transition_forward(g["x"].bfloat16(), g["mask"].bfloat16(), w.to(torch.bfloat16), residual=True)
    assert (got16.float() - g["out_module_residual_masked_bf16"]).abs().max() <= 0.03125  # one bf16 ulp at |z| < 8
