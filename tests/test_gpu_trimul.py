"""Triangle multiplication on the GPU against the reference-generated fixture and the oracle."""

import pytest
import torch

import bionemo_inference_runtime_b200 as b200
from bionemo_inference_runtime_b200 import _lib, ops
from oracle import triangle_oracle as orc
from tests.helpers import golden_trimul_weights, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"
RTOL = ATOL = 2e-2
OUT, INC = b200.TriangleMultiplicationNodeType.OUTGOING, b200.TriangleMultiplicationNodeType.INCOMING


@pytest.fixture(autouse=True)
def _clean_device_status():
    _lib.reset_device_status()
    yield
    assert _lib.device_status() == 0, "a kernel abandoned a bounded wait"


def build(w: orc.TriMulWeights, direction, *, high_precision=False, **kw) -> b200.TriangleMultiplicationNode:
    flags = {"p_in": w.b_p_in is not None, "g_in": w.b_g_in is not None, "p_out": w.b_p_out is not None,
             "g_out": w.b_g_out is not None}
    node = b200.TriangleMultiplicationNode(multiplication_type=direction, dtype=torch.bfloat16, bias_flags=flags,
                                           high_precision=high_precision, **kw)
    sd = {"norm_in.weight": w.ln_in_w, "norm_in.bias": w.ln_in_b, "p_in.weight": w.w_p_in, "g_in.weight": w.w_g_in,
          "norm_out.weight": w.ln_out_w, "norm_out.bias": w.ln_out_b, "p_out.weight": w.w_p_out,
          "g_out.weight": w.w_g_out}
    for name, bias in (("p_in", w.b_p_in), ("g_in", w.b_g_in), ("p_out", w.b_p_out), ("g_out", w.b_g_out)):
        if bias is not None:
            sd[f"{name}.bias"] = bias
    node.load_state_dict(sd, strict=True)
    return node.to(DEV)


def left_mask(valid, n):
    m = (torch.arange(n)[None, :] < torch.tensor(valid)[:, None]).float()
    return m[:, :, None] * m[:, None, :]


def bf16(w: orc.TriMulWeights) -> orc.TriMulWeights:
    return w.to(torch.bfloat16).to(torch.float32)


@pytest.mark.parametrize("name,direction", [("outgoing", OUT), ("incoming", INC)])
def test_matches_reference_outputs(name, direction):
    g = load_golden("trimul")
    node = build(golden_trimul_weights(g), direction)
    z, mask = g["z"].to(DEV).bfloat16(), g["mask"].to(DEV)
    upd = node(z, mask)
    torch.testing.assert_close(upd.float().cpu(), g[f"update_{name}"], rtol=RTOL, atol=ATOL)
    res = node(z, mask, residual=True)
    torch.testing.assert_close(res.float().cpu(), g["z"] + g[f"update_{name}"], rtol=RTOL, atol=ATOL)
    # not further from the fp32 reference than twice the reference's own unfused bf16 chain
    ours = (upd.float().cpu() - g[f"update_{name}"]).abs().max()
    eager = (g[f"update_{name}_bf16"] - g[f"update_{name}"]).abs().max()
    assert ours <= 2 * eager + 1e-3


@pytest.mark.parametrize("name,direction", [("outgoing", OUT), ("incoming", INC)])
def test_mean_normalization_matches_reference_chain(name, direction):
    g = load_golden("trimul")
    node = build(golden_trimul_weights(g), direction, mean_normalization=True)
    upd = node(g["z"].to(DEV).bfloat16(), g["mask"].to(DEV))
    torch.testing.assert_close(upd.float().cpu(), g[f"update_{name}_bf16_meannorm"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("n", [1, 7, 16, 33, 128, 129, 257])
@pytest.mark.parametrize("direction", [OUT, INC])
def test_shape_sweep_with_padding_and_biases(n, direction):
    torch.manual_seed(n)
    w = bf16(orc.make_trimul_weights(n, identity_ln=False, biases=True))
    valid = [n, max(1, (2 * n) // 3)]
    mask = left_mask(valid, n)
    z = torch.randn(2, n, n, 128).bfloat16()
    want = orc.trimul_forward(z.float().to(DEV), mask.to(DEV),
                              orc.TriMulWeights(*[None if t is None else t.to(DEV) for t in w.fields()]), int(direction),
                              residual=True)
    out = build(w, direction)(z.to(DEV), mask.to(DEV), residual=True)
    torch.testing.assert_close(out.float(), want, rtol=RTOL, atol=ATOL)


def test_config4_token_count_and_unmasked_call():
    """N = 768 (the token count of the 48-block trunk benchmark), no mask; checked against the oracle on the GPU."""
    torch.manual_seed(4)
    n = 768
    w = bf16(orc.make_trimul_weights(44))
    z = torch.randn(1, n, n, 128).bfloat16().to(DEV)
    wd = orc.TriMulWeights(*[None if t is None else t.to(DEV) for t in w.fields()])
    for direction in (OUT, INC):
        out = build(w, direction)(z, None, residual=True)
        want = orc.trimul_forward(z.float(), None, wd, int(direction), residual=True)
        torch.testing.assert_close(out.float(), want, rtol=RTOL, atol=ATOL)


def test_incoming_equals_outgoing_on_the_transposed_pair_tensor_bit_for_bit():
    torch.manual_seed(5)
    w = bf16(orc.make_trimul_weights(5, identity_ln=False))
    z = torch.randn(2, 150, 150, 128).bfloat16().to(DEV)
    mask = left_mask([150, 97], 150).to(DEV)
    inc = build(w, INC)(z, mask)
    out = build(w, OUT)(z.transpose(1, 2).contiguous(), mask.transpose(1, 2).contiguous())
    # sum_k a[k,i] b[k,j] on z equals sum_k a'[i,k] b'[j,k] on zᵀ; the output stage of the incoming node works at
    # (i, j) of z, whose gate and residual are those of zᵀ at (j, i) - so compare the contraction, not the gate
    t_inc = ops.trimul_contract(ops.trimul_project(z, mask, build(w, INC)._packed(z.device), incoming=True), 150)
    zt = z.transpose(1, 2).contiguous()
    t_out = ops.trimul_contract(ops.trimul_project(zt, mask.transpose(1, 2).contiguous(),
                                                   build(w, OUT)._packed(z.device)), 150)
    assert torch.equal(t_inc, t_out)
    assert inc.shape == out.shape


def test_fused_residual_masks_the_output_when_row_lengths_are_given():
    """(x + update) * mask, the semantics of the reference's fused residual kernel
    (tests/_torch/test_triangle_nodes.py:272-311); without row lengths the residual is added unmasked."""
    torch.manual_seed(6)
    n, valid = 256, 249
    w = bf16(orc.make_trimul_weights(6))
    z = (torch.randn(1, n, n, 128) * 0.5).bfloat16().to(DEV)
    mask = left_mask([valid], n).to(DEV)
    node = build(w, OUT)
    lens = (mask > 0).sum(-1, dtype=torch.int32)
    meta = b200.precompute_trimul_metadata(z, lens, (mask > 0).sum(-2, dtype=torch.int32))
    update = node(z, mask, meta)
    fused = node(z, mask, meta, residual=True)
    torch.testing.assert_close(fused.float(), (z.float() + update.float()) * mask.unsqueeze(-1), rtol=1e-2, atol=1e-2)
    assert torch.count_nonzero(fused[:, valid:]) == 0 and torch.count_nonzero(fused[:, :, valid:]) == 0
    plain = node(z, mask, residual=True)
    torch.testing.assert_close(plain.float(), z.float() + update.float(), rtol=1e-2, atol=1e-2)
    assert not node.can_fuse_residual(torch.empty(1, n + 1, n + 1, 128, device="meta"))


def test_high_precision_parameters_fp32_output_and_buffers():
    torch.manual_seed(7)
    w = orc.make_trimul_weights(7, identity_ln=False)
    node = b200.TriangleMultiplicationNode(dtype=torch.bfloat16, high_precision=True)
    assert node.norm_out.weight.dtype == torch.float32 and node.p_out.weight.dtype == torch.float32
    assert node.g_out.weight.dtype == torch.float32 and node.p_in.weight.dtype == torch.bfloat16
    node.load_state_dict({"norm_in.weight": w.ln_in_w, "norm_in.bias": w.ln_in_b, "p_in.weight": w.w_p_in,
                          "g_in.weight": w.w_g_in, "norm_out.weight": w.ln_out_w, "norm_out.bias": w.ln_out_b,
                          "p_out.weight": w.w_p_out, "g_out.weight": w.w_g_out}, strict=True)
    node = node.to(DEV)
    z = torch.randn(1, 96, 96, 128).bfloat16().to(DEV)
    bufs: dict = {}
    out = node(z, None, buffers=bufs)
    assert out.dtype == torch.float32 and {"trimul_ab", "trimul_contracted"} <= set(bufs)
    wq = orc.TriMulWeights(*[None if t is None else t.to(DEV) for t in w.fields()])
    wq.ln_in_w, wq.ln_in_b = wq.ln_in_w.bfloat16().float(), wq.ln_in_b.bfloat16().float()
    wq.w_p_in, wq.w_g_in = wq.w_p_in.bfloat16().float(), wq.w_g_in.bfloat16().float()
    want = orc.trimul_forward(z.float(), None, wq, orc.OUTGOING)
    torch.testing.assert_close(out, want, rtol=RTOL, atol=ATOL)
    again = node(z, None, buffers=bufs)
    assert torch.equal(out, again)


def test_cuda_graph_replay_and_refold_after_load():
    torch.manual_seed(8)
    w = bf16(orc.make_trimul_weights(8))
    node = build(w, INC)
    z = torch.randn(1, 64, 64, 128).bfloat16().to(DEV)
    mask = left_mask([50], 64).to(DEV)
    bufs: dict = {}
    eager = node(z, mask, residual=True, buffers=bufs)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        node(z, mask, residual=True, buffers=bufs)
        with torch.cuda.graph(graph, stream=side):
            captured = node(z, mask, residual=True, buffers=bufs)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, eager)
    # new weights through load_state_dict change the result (the fold is redone)
    w2 = bf16(orc.make_trimul_weights(9))
    node.load_state_dict({"p_out.weight": w2.w_p_out.bfloat16()}, strict=False)
    assert not torch.equal(node(z, mask, residual=True), eager)


def test_rejects_unsupported_configurations():
    with pytest.raises(ValueError):
        b200.TriangleMultiplicationNode(dim=384, hidden_dim=256, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        b200.TriangleMultiplicationNode(dtype=torch.float32)
    node = build(bf16(orc.make_trimul_weights(1)), OUT)
    with pytest.raises(ValueError):
        node(torch.zeros(1, 8, 9, 128, dtype=torch.bfloat16, device=DEV), None)
    with pytest.raises(ValueError):
        node(torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16), None)
    with pytest.raises(ValueError):
        node(torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16, device=DEV), torch.ones(1, 8, 7, device=DEV))
