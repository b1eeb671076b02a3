"""Parity of the CUDA path with the oracle at the sizes the benchmark configurations are quoted on.

* 768 tokens, all valid: both attention nodes and the transition on the whole tensor (48-block trunk shape);
* 4096 tokens, 3900 valid: both attention nodes on the whole tensor, a sample of pair rows checked against the
  oracle (rows are independent given the triangle bias of all rows, so sampled rows are exact);
* batched small complexes: 8 items of 256 tokens with valid lengths drawn from {160..256}, both ends included.

Tolerance: rtol = atol = 2e-2 on the full output (bf16 path against the fp32 restatement).  The oracle runs on the
GPU as plain fp32 PyTorch ops so that these sizes finish in seconds.
"""

import pytest
import torch

from bionemo_inference_runtime_b200 import _lib
from oracle import triangle_oracle as orc
from tests.test_gpu_parity import ATOL, DEV, RTOL, bf16_weights, build_node, build_transition, left_mask

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean_device_status():
    _lib.reset_device_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "a kernel abandoned a bounded wait"
    torch.cuda.empty_cache()


def _dev(w):
    return type(w)(*[None if t is None else t.to(DEV) for t in w.__dict__.values()])


def _randn_bf16(shape, seed):
    """N(0, 1) in bf16, generated on the device in slabs (the fp32 temporary of a 4096-token tensor is 8.6 GB)."""
    gen = torch.Generator(device=DEV).manual_seed(seed)
    out = torch.empty(shape, dtype=torch.bfloat16, device=DEV)
    for r0 in range(0, shape[1], 256):
        out[:, r0:r0 + 256] = torch.randn((shape[0], min(256, shape[1] - r0)) + tuple(shape[2:]), generator=gen,
                                          device=DEV).bfloat16()
    return out


def test_768_tokens_all_valid_both_nodes_and_transition():
    n = 768
    w1 = bf16_weights(orc.make_node_weights(41, identity_ln=False))
    w2 = bf16_weights(orc.make_node_weights(42, identity_ln=False))
    wt = bf16_weights(orc.make_transition_weights(43, identity_ln=False))
    z = _randn_bf16((1, n, n, 128), 4001)
    mask = torch.ones(1, n, n, device=DEV)
    z1 = build_node(w1, orc.STARTING)(z, mask=mask, residual=True)
    want1 = orc.node_forward(z.float(), mask, _dev(w1), orc.STARTING, residual=True)
    torch.testing.assert_close(z1.float(), want1, rtol=RTOL, atol=ATOL)
    del want1
    z2 = build_node(w2, orc.ENDING)(z1, mask=mask, residual=True)
    want2 = orc.node_forward(z1.float(), mask, _dev(w2), orc.ENDING, residual=True)
    torch.testing.assert_close(z2.float(), want2, rtol=RTOL, atol=ATOL)
    del want2
    z3 = build_transition(wt)(z2, residual=True)
    want3 = orc.transition_forward(z2.float(), None, _dev(wt), residual=True)
    torch.testing.assert_close(z3.float(), want3, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("node_type", [orc.STARTING, orc.ENDING])
def test_4096_tokens_3900_valid_sampled_rows(node_type):
    n, valid = 4096, 3900
    w = bf16_weights(orc.make_node_weights(51 + node_type, identity_ln=False))
    z = _randn_bf16((1, n, n, 128), 4002 + node_type)
    m = (torch.arange(n, device=DEV) < valid).float()
    mask = (m[:, None] * m[None, :])[None]
    lengths = torch.where(torch.arange(n, device=DEV) < valid, valid, 0).to(torch.int32).reshape(1, n)
    node = build_node(w, node_type)
    out = node(z, mask_bias=lengths, residual=True)  # m (x) m is symmetric: the same counts serve both nodes
    rows = torch.tensor([0, 1, 127, 128, 1000, 2047, 2048, 3000, 3898, 3899, 3900, 3901, 4000, 4095], device=DEV)
    want = orc.node_forward_rows(z, mask, _dev(w), node_type, rows, residual=True)  # fp32 (the weights' dtype)
    got = (out.transpose(1, 2) if node_type == orc.ENDING else out)[:, rows]
    torch.testing.assert_close(got.float(), want, rtol=RTOL, atol=ATOL)


def test_batched_small_complexes_with_ragged_lengths():
    n = 256
    lens = [160, 256, 161, 255, 192, 200, 233, 177]
    w1 = bf16_weights(orc.make_node_weights(61))
    w2 = bf16_weights(orc.make_node_weights(62))
    wt = bf16_weights(orc.make_transition_weights(63))
    z = _randn_bf16((len(lens), n, n, 128), 4003)
    mask = left_mask(lens, n).to(DEV)
    z1 = build_node(w1, orc.STARTING)(z, mask=mask, residual=True)
    want1 = orc.node_forward(z.float(), mask, _dev(w1), orc.STARTING, residual=True)
    torch.testing.assert_close(z1.float(), want1, rtol=RTOL, atol=ATOL)
    del want1
    z2 = build_node(w2, orc.ENDING)(z1, mask=mask, residual=True)
    want2 = orc.node_forward(z1.float(), mask, _dev(w2), orc.ENDING, residual=True)
    torch.testing.assert_close(z2.float(), want2, rtol=RTOL, atol=ATOL)
    del want2
    z3 = build_transition(wt)(z2, residual=True)
    torch.testing.assert_close(z3.float(), orc.transition_forward(z2.float(), None, _dev(wt), residual=True),
                               rtol=RTOL, atol=ATOL)
