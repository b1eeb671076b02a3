"""Parity of the CUDA path (modules -> C ABI -> sm_100a kernels) with the CPU oracle and the golden fixtures.

Tolerances: the full-output bar of the bf16 path is rtol = atol = 2e-2 against the fp32 reference; stage-level
checks use tighter bounds scaled to the bf16 spacing of the values involved.
"""

import math

import pytest
import torch

import bionemo_inference_runtime_b200 as b200
from bionemo_inference_runtime_b200 import _lib, ops
from oracle import triangle_oracle as orc
from tests.helpers import golden_node_weights, golden_transition_weights, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"
RTOL = ATOL = 2e-2


@pytest.fixture(autouse=True)
def _clean_device_status():
    _lib.reset_device_status()
    yield
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "a kernel abandoned a bounded wait"


def build_node(w: orc.NodeWeights, node_type: int, **kw) -> b200.TriangleAttentionNode:
    flags = {"q": False, "k": False, "v": False, "g": w.b_in is not None, "o": w.b_out is not None}
    cls = b200.TriangleAttentionEndingNode if node_type == orc.ENDING else b200.TriangleAttentionStartingNode
    node = cls(128, 32, 4, dtype=torch.bfloat16, mha_bias_flags=flags, **kw)
    sd = {"layer_norm.weight": w.ln_w, "layer_norm.bias": w.ln_b, "pair_bias_proj.weight": w.w_bias,
          "mha.in_proj.weight": w.w_in, "mha.o_proj.weight": w.w_out}
    if w.b_in is not None:
        sd["mha.in_proj.bias"] = w.b_in
    if w.b_out is not None:
        sd["mha.o_proj.bias"] = w.b_out
    node.load_state_dict({k: v.to(torch.bfloat16) for k, v in sd.items()}, strict=True)
    return node.to(DEV)


def build_transition(w: orc.TransitionWeights, **kw) -> b200.Transition:
    t = b200.Transition(128, 512, dtype=torch.bfloat16, **kw)
    sd = {"fused_fc2_fc1.weight": w.w1, "fc3.weight": w.w2}
    if t.norm is not None:
        sd.update({"norm.weight": w.ln_w, "norm.bias": w.ln_b})
    t.load_state_dict({k: v.to(torch.bfloat16) for k, v in sd.items()}, strict=True)
    return t.to(DEV)


def bf16_weights(w):
    """The weights as the bf16 module holds them, widened back to fp32 for the oracle."""
    return w.to(torch.bfloat16).to(torch.float32)


def left_mask(valid: list[int], n: int) -> torch.Tensor:
    m = torch.zeros(len(valid), n)
    for b, v in enumerate(valid):
        m[b, :v] = 1
    return m[:, :, None] * m[:, None, :]


# ------------------------------------------------------------------------------------------ golden fixtures


@pytest.mark.parametrize("name,key,residual", [("node_start_fullmask", "out_residual", True),
                                               ("node_start_fullmask", "out_update", False),
                                               ("node_end_padded", "out_residual", True),
                                               ("node_end_padded", "out_start_residual", True)])
def test_node_matches_reference_outputs(name, key, residual):
    g = load_golden(name)
    node_type = orc.STARTING if "start" in key or name.startswith("node_start") else g["node_type"]
    node = build_node(golden_node_weights(g), node_type)
    out = node(g["z"].to(DEV).bfloat16(), mask=g["mask"].to(DEV), residual=residual)
    torch.testing.assert_close(out.float().cpu(), g[key], rtol=RTOL, atol=ATOL)


def test_node_transposed_bias_matches_reference_output():
    g = load_golden("node_end_transposed_bias")
    node = build_node(golden_node_weights(g), orc.ENDING, transposed_bias=True)
    out = node(g["z"].to(DEV).bfloat16(), mask=g["mask"].to(DEV))
    torch.testing.assert_close(out.float().cpu(), g["out_update"], rtol=RTOL, atol=ATOL)


def test_node_is_closer_to_fp32_reference_than_twice_the_bf16_eager_reference():
    """The reference's own acceptance pattern (tests/_torch/test_triangle_nodes.py:147-157 there)."""
    g = load_golden("node_end_padded")
    node = build_node(golden_node_weights(g), orc.ENDING)
    out = node(g["z"].to(DEV).bfloat16(), mask=g["mask"].to(DEV), residual=True).float().cpu()
    ours = (out - g["out_residual"]).abs().max()
    eager_bf16 = (g["out_residual_bf16"] - g["out_residual"]).abs().max()
    assert ours <= 2 * eager_bf16 + 1e-3


def test_transition_matches_reference_outputs():
    g = load_golden("transition")
    t = build_transition(golden_transition_weights(g))
    x = g["x"].to(DEV).bfloat16()
    torch.testing.assert_close(t(x).float().cpu(), g["out_update"], rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(t(x, g["mask"].to(DEV), residual=True).float().cpu(), g["out_residual_masked"],
                               rtol=RTOL, atol=ATOL)
    upd = t(x, g["mask"].to(DEV)).float().cpu()
    # update alone is small (|u| < 0.1): hold it to the bf16 spacing of that range
    assert (upd - g["out_module_update_masked"]).abs().max() < 2e-3


# ------------------------------------------------------------------------------------------ oracle sweeps


@pytest.mark.parametrize("n", [1, 7, 8, 31, 33, 127, 128, 129, 255, 257])
@pytest.mark.parametrize("node_type", [orc.STARTING, orc.ENDING])
def test_node_shape_sweep(n, node_type):
    torch.manual_seed(n)
    w = bf16_weights(orc.make_node_weights(n, identity_ln=False, gate_bias=1.0, out_bias=True))
    valid = [n, max(1, (2 * n) // 3)]
    mask = left_mask(valid, n)
    z = torch.randn(2, n, n, 128).bfloat16()
    want = orc.node_forward(z.float().to(DEV), mask.to(DEV), orc.NodeWeights(*[None if t is None else t.to(DEV) for t in
                            (w.ln_w, w.ln_b, w.w_bias, w.w_in, w.b_in, w.w_out, w.b_out)]), node_type, residual=True)
    node = build_node(w, node_type)
    out = node(z.to(DEV), mask=mask.to(DEV), residual=True)
    torch.testing.assert_close(out.float(), want, rtol=RTOL, atol=ATOL)


def test_config2_shape_with_padding():
    """[1, 512, 512, 128], 475 valid tokens, start then end; sampled rows checked against the oracle."""
    torch.manual_seed(1001)
    n, valid = 512, 475
    w1 = bf16_weights(orc.make_node_weights(11))
    w2 = bf16_weights(orc.make_node_weights(12))
    z = torch.randn(1, n, n, 128).bfloat16().to(DEV)
    mask = left_mask([valid], n).to(DEV)
    start, end = build_node(w1, orc.STARTING), build_node(w2, orc.ENDING)
    z1 = start(z, mask=mask, residual=True)
    z2 = end(z1, mask=mask, residual=True)

    def dev(w):
        return orc.NodeWeights(*[None if t is None else t.to(DEV) for t in
                                 (w.ln_w, w.ln_b, w.w_bias, w.w_in, w.b_in, w.w_out, w.b_out)])

    want1 = orc.node_forward(z.float(), mask, dev(w1), orc.STARTING, residual=True)
    torch.testing.assert_close(z1.float(), want1, rtol=RTOL, atol=ATOL)
    want2 = orc.node_forward(z1.float(), mask, dev(w2), orc.ENDING, residual=True)
    torch.testing.assert_close(z2.float(), want2, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("node_type", [orc.STARTING, orc.ENDING])
def test_masks_that_are_not_left_aligned(node_type):
    """``pair_mask_left_aligned=False``: keys switched off anywhere in a row (holes, a first key tile without any
    valid key, a single valid key at the end, rows without a valid key), as the 0/1 mask and in its additive form."""
    torch.manual_seed(15 + node_type)
    n = 200
    w = bf16_weights(orc.make_node_weights(37, identity_ln=False, gate_bias=1.0))
    z = torch.randn(2, n, n, 128).bfloat16()
    mask = (torch.rand(2, n, n) > 0.4).float()
    rows = mask if node_type == orc.STARTING else mask.transpose(1, 2)  # [b, pair row of the node, key]
    rows[0, 3, :130] = 0      # no valid key in the first key tile
    rows[0, 4] = 0
    rows[0, 4, n - 1] = 1     # a single valid key, the last one
    rows[0, 5] = 0            # no valid key at all
    rows[1, 7, :] = 1
    rows[1, 8, 64:128] = 0
    dev_w = orc.NodeWeights(*[None if t is None else t.to(DEV) for t in
                              (w.ln_w, w.ln_b, w.w_bias, w.w_in, w.b_in, w.w_out, w.b_out)])
    want = orc.node_forward(z.float().to(DEV), mask.to(DEV), dev_w, node_type, residual=True)
    node = build_node(w, node_type, pair_mask_left_aligned=False)
    out = node(z.to(DEV), mask=mask.to(DEV), residual=True)
    torch.testing.assert_close(out.float(), want, rtol=RTOL, atol=ATOL)
    pre = b200.precompute_pair_masks("VANILLA", mask.to(DEV), dtype=torch.bfloat16)
    bias = pre.mask_bias if node_type == orc.STARTING else pre.mask_bias_transposed
    assert torch.equal(node(z.to(DEV), mask_bias=bias, residual=True), out)
    chunky = build_node(w, node_type, pair_mask_left_aligned=False, chunk_policy=b200.ChunkPolicy(chunk_size=64, min_size=1))
    assert torch.equal(chunky(z.to(DEV), mask=mask.to(DEV), residual=True), out)
    with pytest.raises(ValueError, match="left-aligned"):
        node(z.to(DEV), mask_bias=torch.full((2, n), n, dtype=torch.int32, device=DEV))


def test_ending_equals_transposed_starting_bit_for_bit():
    torch.manual_seed(3)
    w = bf16_weights(orc.make_node_weights(3, identity_ln=False))
    z = torch.randn(2, 150, 150, 128).bfloat16().to(DEV)
    mask = left_mask([150, 97], 150).to(DEV)
    end = build_node(w, orc.ENDING)(z, mask=mask, residual=True)
    start = build_node(w, orc.STARTING)(z.transpose(1, 2).contiguous(), mask=mask.transpose(1, 2).contiguous(),
                                        residual=True)
    assert torch.equal(end, start.transpose(1, 2))


def test_chunked_rows_are_identical_and_mask_forms_agree():
    torch.manual_seed(4)
    w = bf16_weights(orc.make_node_weights(4, identity_ln=False))
    z = torch.randn(1, 72, 72, 128).bfloat16().to(DEV)
    mask = left_mask([60], 72).to(DEV)
    dense = build_node(w, orc.ENDING)(z, mask=mask, residual=True)
    for rows in (8, 16, 50):
        node = build_node(w, orc.ENDING, chunk_policy=b200.ChunkPolicy(chunk_size=rows, min_size=1))
        assert torch.equal(node(z, mask=mask, residual=True), dense)
    node = build_node(w, orc.ENDING)
    for backend in ("VANILLA", "Heuristic"):
        pre = b200.precompute_pair_masks(backend, mask, dtype=torch.bfloat16)
        assert torch.equal(node(z, mask_bias=pre.mask_bias_transposed, residual=True), dense)


def test_inplace_residual_buffers_and_no_mask():
    torch.manual_seed(5)
    w = bf16_weights(orc.make_node_weights(5))
    node = build_node(w, orc.STARTING)
    z = torch.randn(1, 96, 96, 128).bfloat16().to(DEV)
    want = node(z, residual=True)
    upd = node(z)
    torch.testing.assert_close((z.float() + upd.float()), want.float(), rtol=0, atol=2e-2)
    bufs: dict = {}
    zc = z.clone()
    got = node(zc, buffers=bufs, residual=True, inplace_residual=True)
    assert got is zc and torch.equal(zc, want)
    assert "tri_attn_workspace" in bufs
    assert torch.equal(node(z, buffers=bufs, residual=True), want)  # buffers reused
    chunky = build_node(w, orc.STARTING, chunk_policy=b200.ChunkPolicy(chunk_size=40, min_size=1))
    cb: dict = {}
    assert torch.equal(chunky(z, buffers=cb, residual=True), want)
    assert {"tri_attn_output", "tri_attn_qkvg", "tri_attn_bias"} <= set(cb)


def test_single_call_node_equals_the_three_stage_calls():
    torch.manual_seed(14)
    n = 90
    w = bf16_weights(orc.make_node_weights(36, identity_ln=False, out_bias=True))
    packed = ops.pack_node_weights(*[None if t is None else t.bfloat16().to(DEV) for t in
                                     (w.ln_w, w.ln_b, w.w_in, w.b_in, w.w_bias, w.w_out, w.b_out)])
    z = torch.randn(2, n, n, 128).bfloat16().to(DEV)
    lens = torch.randint(0, n + 1, (2, n), dtype=torch.int32, device=DEV)
    for ending in (False, True):
        qkvg, bias = ops.prologue(z, packed, ending=ending)
        og = ops.attention(qkvg, bias, lens, 2, n, n)
        want = ops.epilogue(og, packed, z, ending=ending)
        got = ops.node_forward(z, packed, lens, ending=ending, residual=True)
        assert torch.equal(got, want)
    with pytest.raises(ValueError, match="workspace"):
        ops.node_forward(z, packed, lens, workspace=torch.empty(1024, dtype=torch.uint8, device=DEV))


def test_empty_rows_zeros_mode_and_lengths_beyond_every_boundary():
    """Boundary lengths of the reference's tail test (N, N-1, a multiple of 128, 1, 0), LSE included."""
    torch.manual_seed(6)
    B, R, S = 1, 6, 300
    lens = torch.tensor([S, S - 1, 256, 128, 1, 0], dtype=torch.int32)
    qkvg = torch.randn(4, B * R, 4, S, 32).bfloat16()
    bias = torch.zeros(B, 4, S, ops.pad8(S))
    bias[..., :S] = torch.randn(B, 4, S, S)
    bias = bias.bfloat16()
    q, k, v = [t.float().permute(0, 2, 1, 3) for t in qkvg[:3]]  # [BR, S, H, d]
    for mode, name in ((_lib.EMPTY_ROW_ZEROS, "zeros"), (_lib.EMPTY_ROW_UNIFORM, "uniform")):
        want, want_lse = orc.attention_core(q, k, v, bias[..., :S].float(), lens, 1 / math.sqrt(32), empty_rows=name)
        lse = torch.full((B * R, S, 4), float("nan"), device=DEV)
        bias_dev = (bias.float() * ops.BIAS_SCALE).bfloat16().to(DEV)
        out = ops.attention(qkvg.to(DEV), bias_dev, lens.to(DEV), B, R, S, gate=False, lse=lse, empty_row_mode=mode)
        torch.testing.assert_close(out.float().cpu().view(B * R, S, 4, 32), want, rtol=2e-2, atol=3e-2)
        valid = lens > 0
        torch.testing.assert_close(lse.cpu()[valid], want_lse[valid], rtol=1e-3, atol=2e-2)
        assert torch.isinf(lse.cpu()[~valid]).all() and (lse.cpu()[~valid] < 0).all()
        if name == "zeros":
            assert (out.cpu().view(B * R, S, 128)[~valid] == 0).all()


def test_scores_far_above_the_first_key_tile_move_the_reference_point():
    """The softmax is anchored at the maximum of a row's first key tile; keys ~180 nats above it (and, in one
    row, back below it) must move that reference point without losing the earlier tiles' contribution."""
    torch.manual_seed(61)
    B, R, S = 1, 3, 512
    for jump_at in (128, 200):
        qkvg = torch.randn(4, B * R, 4, S, 32) * 0.1
        qkvg[0] += 4.0
        qkvg[1, :, :, :jump_at] -= 4.0
        qkvg[1, :, :, jump_at:] += 4.0
        qkvg[1, 1, :, 300:] -= 8.0
        qkvg[2] = torch.randn(B * R, 4, S, 32)
        qkvg[3] = torch.rand(B * R, 4, S, 32)  # gate factors in [0, 1]
        qkvg = qkvg.bfloat16()
        bias = torch.randn(B, 4, S, S).bfloat16()
        q, k, v, g = [t.float().permute(0, 2, 1, 3) for t in qkvg]  # [BR, S, H, d]
        want, want_lse = orc.attention_core(q, k, v, bias.float(), torch.full((B * R,), S, dtype=torch.int32),
                                            1 / math.sqrt(32))
        lse = torch.full((B * R, S, 4), float("nan"), device=DEV)
        out = ops.attention(qkvg.to(DEV), (bias.float() * ops.BIAS_SCALE).bfloat16().to(DEV), None, B, R, S,
                            gate=True, lse=lse)
        assert _lib.device_status() == 0
        torch.testing.assert_close(out.float().cpu().view(B * R, S, 4, 32), want * g, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(lse.cpu(), want_lse, rtol=1e-3, atol=5e-2)


def test_backend_forward_on_packed_views():
    """q, k, v as views of one in-projection buffer, as the reference layer hands them to a backend."""
    torch.manual_seed(7)
    B, I, J = 2, 5, 140
    proj = torch.randn(B, I, J, 512).bfloat16().to(DEV)
    q, k, v, _ = proj.split(128, dim=-1)
    tb = torch.randn(B, 4, J, J).bfloat16().to(DEV)
    lens = torch.tensor([[140, 100, 7, 140, 1], [139, 140, 64, 128, 129]], dtype=torch.int32, device=DEV)
    attn = b200.create_attention("CuTeDSL", 0, 4, 32)
    attn.empty_row_mode = _lib.EMPTY_ROW_ZEROS
    out = attn.forward(q, k, v, biases=[lens, tb])
    assert out.shape == (B, I, J, 4, 32)
    want, _ = orc.attention_core(q.float().cpu().reshape(B * I, J, 4, 32), k.float().cpu().reshape(B * I, J, 4, 32),
                                 v.float().cpu().reshape(B * I, J, 4, 32), tb.float().cpu(), lens.cpu().reshape(-1),
                                 1 / math.sqrt(32))
    torch.testing.assert_close(out.float().cpu().reshape(B * I, J, 4, 32), want, rtol=2e-2, atol=3e-2)


def test_standalone_triangle_attention_module():
    torch.manual_seed(8)
    w = bf16_weights(orc.make_node_weights(8, gate_bias=1.0))
    node = build_node(w, orc.STARTING)
    z = torch.randn(1, 80, 80, 128).bfloat16().to(DEV)
    mask = left_mask([66], 80).to(DEV)
    st = orc.node_stages(z.float(), mask, orc.NodeWeights(*[None if t is None else t.to(DEV) for t in
                         (w.ln_w, w.ln_b, w.w_bias, w.w_in, w.b_in, w.w_out, w.b_out)]), orc.STARTING)
    pre = b200.precompute_pair_masks("VANILLA", mask, dtype=torch.bfloat16)
    out = node.mha(st["normed"].bfloat16(), pre.mask_bias, triangle_bias=st["tri_bias"].bfloat16(), residual=z)
    torch.testing.assert_close(out.float(), z.float() + st["update"], rtol=RTOL, atol=ATOL)


# ------------------------------------------------------------------------------------------ transition


@pytest.mark.parametrize("shape", [(1, 128), (3, 5, 7), (2, 130, 130), (1, 1)])
def test_transition_sweep(shape):
    torch.manual_seed(sum(shape))
    w = bf16_weights(orc.make_transition_weights(21, identity_ln=False))
    t = build_transition(w)
    x = torch.randn(*shape, 128).bfloat16().to(DEV)
    mask = (torch.rand(*shape, device=DEV) > 0.25).float()
    wd = orc.TransitionWeights(*[p.to(DEV) for p in (w.ln_w, w.ln_b, w.w1, w.w2)])
    torch.testing.assert_close(t(x, residual=True).float(), orc.transition_forward(x.float(), None, wd, residual=True),
                               rtol=RTOL, atol=ATOL)
    upd = t(x, mask)
    want = orc.transition_forward(x.float(), mask, wd)
    assert (upd.float() - want).abs().max() < 2e-3
    assert (upd.float()[mask == 0] == 0).all()  # masked rows pass through
    xc = x.clone()
    got = t(xc, mask, residual=True, inplace=True)
    assert got is xc
    torch.testing.assert_close(xc.float(), orc.transition_forward(x.float(), mask, wd, residual=True), rtol=RTOL, atol=ATOL)


def test_transition_large_mean_rows_and_determinism():
    torch.manual_seed(9)
    w = bf16_weights(orc.make_transition_weights(22, identity_ln=False))
    t = build_transition(w)
    x = (torch.randn(4, 64, 128) + 40.0 * torch.randn(4, 64, 1)).bfloat16().to(DEV)
    wd = orc.TransitionWeights(*[p.to(DEV) for p in (w.ln_w, w.ln_b, w.w1, w.w2)])
    upd = t(x)
    assert (upd.float() - orc.transition_forward(x.float(), None, wd)).abs().max() < 4e-3
    assert torch.equal(upd, t(x))


def test_transition_on_a_transposed_view_runs_in_storage_order():
    """A permuted view is processed without a copy; ``inplace`` writes the caller's storage; slices are refused."""
    torch.manual_seed(24)
    w = bf16_weights(orc.make_transition_weights(24, identity_ln=False))
    t = build_transition(w)
    x = torch.randn(2, 40, 56, 128).bfloat16().to(DEV)
    mask = (torch.rand(2, 56, 40, device=DEV) > 0.3).float()
    view = x.transpose(1, 2)  # [2, 56, 40, 128], not contiguous
    want = t(view.contiguous(), mask, residual=True)
    assert torch.equal(t(view, mask, residual=True), want)
    xc = x.clone()
    got = t(xc.transpose(1, 2), mask, residual=True, inplace=True)
    assert got.data_ptr() == xc.data_ptr() and torch.equal(xc.transpose(1, 2), want)
    with pytest.raises(ValueError, match="permuted view"):
        t(x[:, ::2])


def test_transition_without_norm():
    torch.manual_seed(10)
    w = bf16_weights(orc.make_transition_weights(23))
    t = build_transition(w, normalize=False)
    x = torch.randn(2, 33, 128).bfloat16().to(DEV)
    h = x.float() @ w.w1.to(DEV).t()
    want = (torch.nn.functional.silu(h[..., 512:]) * h[..., :512]) @ w.w2.to(DEV).t()
    assert (t(x).float() - want).abs().max() < 2e-3


def build_relu_transition(w: orc.ReluTransitionWeights) -> b200.PairTransition:
    t = b200.PairTransition(128, 4, dtype=torch.bfloat16)
    t.load_state_dict({"layer_norm.weight": w.ln_w, "layer_norm.bias": w.ln_b, "linear_1.weight": w.w1,
                       "linear_1.bias": w.b1, "linear_2.weight": w.w2, "linear_2.bias": w.b2}, strict=True)
    return t.to(DEV)


def test_relu_pair_transition_matches_reference_outputs():
    g = load_golden("pair_transition_relu")
    w = orc.ReluTransitionWeights(g["w_ln_w"], g["w_ln_b"], g["w_w1"], g["w_b1"], g["w_w2"], g["w_b2"])
    t = build_relu_transition(w)
    x = g["x"].to(DEV).bfloat16()
    torch.testing.assert_close(t(x, g["mask"].to(DEV), residual=True).float().cpu(), g["out_residual_masked"],
                               rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(t(x).float().cpu(), g["out_update"], rtol=RTOL, atol=ATOL)
    assert (t(x).float().cpu() - g["out_update"]).abs().max() < 1e-2  # |update| ~ 1: a bf16 ulp or two


@pytest.mark.parametrize("shape", [(1, 128), (3, 5, 7), (2, 130, 130), (1, 1), (1, 300, 300)])
def test_relu_pair_transition_sweep(shape):
    torch.manual_seed(sum(shape) + 1)
    w = bf16_weights(orc.make_relu_transition_weights(25))
    t = build_relu_transition(w)
    x = torch.randn(*shape, 128).bfloat16().to(DEV)
    mask = (torch.rand(*shape, device=DEV) > 0.25).float()
    wd = orc.ReluTransitionWeights(*[p.to(DEV) for p in w.__dict__.values()])
    torch.testing.assert_close(t(x, residual=True).float(), orc.relu_transition_forward(x.float(), None, wd, residual=True),
                               rtol=RTOL, atol=ATOL)
    upd = t(x, mask)
    torch.testing.assert_close(upd.float(), orc.relu_transition_forward(x.float(), mask, wd), rtol=RTOL, atol=ATOL)
    assert (upd.float()[mask == 0] == 0).all()  # masked rows get no update (bias included)
    assert torch.equal(t(x.transpose(0, 1) if x.dim() > 2 else x, residual=True),
                       t(x, residual=True).transpose(0, 1) if x.dim() > 2 else t(x, residual=True))
    with pytest.raises(ValueError):
        b200.PairTransition(256, 4, dtype=torch.bfloat16)


# ------------------------------------------------------------------------------------------ lifecycle


def test_refold_after_weights_change():
    torch.manual_seed(11)
    w_a = bf16_weights(orc.make_node_weights(31))
    w_b = bf16_weights(orc.make_node_weights(32))
    z = torch.randn(1, 40, 40, 128).bfloat16().to(DEV)
    node = build_node(w_a, orc.STARTING)
    out_a = node(z)
    ref_b = build_node(w_b, orc.STARTING)(z)
    node.load_state_dict(build_node(w_b, orc.STARTING).state_dict(), strict=True)
    assert torch.equal(node(z), ref_b) and not torch.equal(out_a, ref_b)
    node.mha.o_proj.weight.mul_(0.0)  # an in-place edit is picked up through the version counter
    assert (node(z) == 0).all()


def test_cuda_graph_replay_and_two_streams():
    torch.manual_seed(12)
    w = bf16_weights(orc.make_node_weights(33))
    wt = bf16_weights(orc.make_transition_weights(34))
    node, trans = build_node(w, orc.ENDING), build_transition(wt)
    z = torch.randn(1, 64, 64, 128).bfloat16().to(DEV)
    mask = left_mask([50], 64).to(DEV)
    eager = trans(node(z, mask=mask, residual=True), residual=True)  # also folds the weights outside capture
    static_in = z.clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            static_out = trans(node(static_in, mask=mask, residual=True), residual=True)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out, eager)
    static_in.copy_(z.flip(1))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out, trans(node(z.flip(1), mask=mask, residual=True), residual=True))
    # two streams at once
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(s1):
        a = node(z, mask=mask, residual=True)
    with torch.cuda.stream(s2):
        b = node(z, mask=mask, residual=True)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_outputs_stay_inside_their_buffers():
    """Canary words around the output and workspaces must survive (ragged sizes exercise the clipped stores)."""
    torch.manual_seed(13)
    n = 77
    w = bf16_weights(orc.make_node_weights(35))
    packed = ops.pack_node_weights(*[None if t is None else t.bfloat16().to(DEV) for t in
                                     (w.ln_w, w.ln_b, w.w_in, w.b_in, w.w_bias, w.w_out, w.b_out)])
    z = torch.randn(1, n, n, 128).bfloat16().to(DEV)
    pad = 4096

    def guarded(numel):
        buf = torch.full((numel + 2 * pad,), 12345.0, dtype=torch.bfloat16, device=DEV)
        return buf, buf[pad:pad + numel]

    qbuf, qkvg = guarded(4 * n * 4 * n * 32)
    bbuf, bias = guarded(4 * n * ops.pad8(n))
    obuf, og = guarded(n * n * 128)
    fbuf, out = guarded(n * n * 128)
    qkvg, bias = qkvg.view(4, n, 4, n, 32), bias.view(1, 4, n, ops.pad8(n))
    ops.prologue(z, packed, qkvg=qkvg, bias=bias)
    ops.attention(qkvg, bias, None, 1, n, n, out=og.view(1, n, n, 128))
    ops.epilogue(og.view(1, n, n, 128), packed, z, out.view(1, n, n, 128))
    torch.cuda.synchronize()
    for buf in (qbuf, bbuf, obuf, fbuf):
        assert (buf[:pad] == 12345.0).all() and (buf[-pad:] == 12345.0).all()
    assert torch.isfinite(out.float()).all()
