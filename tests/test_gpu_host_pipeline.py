"""HostPipeline: pinned host tensors streamed through the nodes give the same results as one-by-one calls."""

import pytest
import torch

from oracle import triangle_oracle as orc
from tests.test_gpu_parity import bf16_weights, build_node, left_mask

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_pipelined_batches_equal_serial_calls():
    import bionemo_inference_runtime_b200 as b200
    from bionemo_inference_runtime_b200 import _lib

    torch.manual_seed(17)
    n = 96
    start = build_node(bf16_weights(orc.make_node_weights(41, identity_ln=False)), orc.STARTING)
    end = build_node(bf16_weights(orc.make_node_weights(42, identity_ln=False)), orc.ENDING)
    mask = left_mask([80], n).to(DEV)
    bufs = [{}, {}, {}]

    def step(z, slot):
        z1 = start(z, mask=mask, buffers=bufs[slot], residual=True)
        return end(z1, mask=mask, buffers=bufs[slot], residual=True, inplace_residual=True)

    inputs = [torch.randn(1, n, n, 128).bfloat16().pin_memory() for _ in range(7)]
    outputs = [torch.empty_like(t).pin_memory() for t in inputs]
    want = [step(t.to(DEV), 2).cpu() for t in inputs]
    for depth in (1, 2):
        for t in outputs:
            t.zero_()
        b200.HostPipeline(step, inputs[0], DEV, depth=depth).run(inputs, outputs)
        assert _lib.device_status() == 0
        for got, ref in zip(outputs, want):
            assert torch.equal(got, ref)


def test_function_that_updates_its_slot_in_place():
    """``fn`` may return the slot tensor itself: the next copy into the slot must wait for the copy-out too."""
    import bionemo_inference_runtime_b200 as b200

    torch.manual_seed(18)
    n = 128
    node = build_node(bf16_weights(orc.make_node_weights(43)), orc.STARTING)
    bufs = [{}, {}, {}]

    def step(z, slot):
        return node(z, buffers=bufs[slot], residual=True, inplace_residual=True)  # returns z (the slot)

    inputs = [torch.randn(1, n, n, 128).bfloat16().pin_memory() for _ in range(9)]
    outputs = [torch.empty_like(t).pin_memory() for t in inputs]
    want = [step(t.to(DEV), 2).cpu() for t in inputs]
    b200.HostPipeline(step, inputs[0], DEV, depth=2).run(inputs, outputs)
    for got, ref in zip(outputs, want):
        assert torch.equal(got, ref)


def test_pipeline_rejects_pageable_or_mismatched_tensors():
    import bionemo_inference_runtime_b200 as b200

    example = torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16).pin_memory()
    pipe = b200.HostPipeline(lambda z, slot: z, example, DEV)
    with pytest.raises(ValueError):
        pipe.run([torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16)], [example])
    with pytest.raises(ValueError):
        pipe.run([example], [torch.zeros(1, 4, 4, 128, dtype=torch.bfloat16).pin_memory()])
    with pytest.raises(ValueError):
        pipe.run([example, example], [example])
