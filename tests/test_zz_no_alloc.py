"""The allocation-free node entry point (``b200ta_node_forward_static``) against the regular one.

Some hosts cannot give this library a workspace: a trunk that is being captured into a CUDA graph must not call
cudaMalloc, and a server whose own pool owns the GPU wants no allocation on the request path.  For them the
library keeps a fixed scratch array inside its own image.  These tests call that entry point through the C ABI
and require bit-identical results to ``b200ta_node_forward`` (same kernels, same inputs), twice in a row because
every call reuses the one array and finds the previous call's intermediates in it.

The file name sorts last on purpose: a run that stops at the first failure has already run everything else.
"""

import pytest
import torch

from bionemo_inference_runtime_b200 import _lib, ops
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _packed(seed: int) -> torch.Tensor:
    w = orc.make_node_weights(seed, identity_ln=False, gate_bias=1.0, out_bias=True).to(torch.bfloat16)
    return ops.pack_node_weights(*[None if t is None else t.to(DEV) for t in
                                   (w.ln_w, w.ln_b, w.w_in, w.b_in, w.w_bias, w.w_out, w.b_out)])


def test_static_scratch_node_matches_workspace_node_on_two_calls_in_a_row():
    torch.manual_seed(2024)
    _lib.reset_device_status()
    assert ops.node_static_max_positions() == 4096
    packed = _packed(41)
    # two different problems back to back: the second finds the first one's intermediates in the scratch
    cases = [(1, 64, False), (3, 33, True)]
    for B, n, ending in cases:
        z = torch.randn(B, n, n, 128).bfloat16().to(DEV)
        lens = torch.randint(0, n + 1, (B, n), dtype=torch.int32, device=DEV)
        want = ops.node_forward(z, packed, lens, ending=ending, residual=True)
        got = torch.empty_like(z)
        before = torch.cuda.memory_allocated()
        ops.node_forward_static(z, packed, lens, got, ending=ending, residual=True)
        assert torch.cuda.memory_allocated() == before  # the call itself took nothing from torch's allocator
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        # same problem again, this time in place on a copy of z
        zc = z.clone()
        ops.node_forward_static(zc, packed, lens, zc, ending=ending, residual=True)
        torch.cuda.synchronize()
        assert torch.equal(zc, want)
    assert _lib.device_status() == 0


def test_static_scratch_node_refuses_problems_beyond_its_limit():
    packed = _packed(42)
    z = torch.randn(1, 65, 65, 128).bfloat16().to(DEV)  # 4225 positions > 4096
    with pytest.raises(_lib.B200TAError, match="4096"):
        ops.node_forward_static(z, packed, None, torch.empty_like(z))
    z = torch.randn(2, 48, 48, 128).bfloat16().to(DEV)  # 4608 positions
    with pytest.raises(_lib.B200TAError, match="exceed"):
        ops.node_forward_static(z, packed, None, torch.empty_like(z))
