"""The transposing output kernels of the row-sharded mode on ONE GPU: the "peers" are buffers of the same device, so
the addressing of b200ta_epilogue_scatter and b200ta_transition_scatter is checked without a second GPU (the
2-GPU test in test_gpu_sharded.py covers the NVLink stores and the ordering)."""

import ctypes

import pytest
import torch

import bionemo_inference_runtime_b200 as b200
from bionemo_inference_runtime_b200 import _lib, ops
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("world,N", [(2, 256), (4, 256), (8, 256), (2, 192)])
def test_epilogue_scatter_writes_every_ranks_rows_into_the_column_shards(world, N):
    w = orc.make_node_weights(21, identity_ln=False, out_bias=True)
    node = b200.TriangleAttentionStartingNode(128, 32, 4, dtype=torch.bfloat16,
                                             mha_bias_flags={"q": False, "k": False, "v": False, "g": False, "o": True})
    node.load_state_dict({"layer_norm.weight": w.ln_w, "layer_norm.bias": w.ln_b, "pair_bias_proj.weight": w.w_bias,
                          "mha.in_proj.weight": w.w_in, "mha.o_proj.weight": w.w_out, "mha.o_proj.bias": w.b_out})
    node = node.to(DEV)
    packed = node._packed(torch.device(DEV))
    g = torch.Generator().manual_seed(N + world)
    og = torch.randn(1, N, N, 128, generator=g).bfloat16().to(DEV)
    res = torch.randn(1, N, N, 128, generator=g).bfloat16().to(DEV)
    want = ops.epilogue(og, packed, res)  # [1, N, N, 128], the plain kernel
    n = N // world
    shards = [torch.full((1, N, n, 128), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    for rank in range(world):
        rows = slice(rank * n, (rank + 1) * n)
        og_r, res_r = og[:, rows].contiguous(), res[:, rows].contiguous()
        _lib.call("b200ta_epilogue_scatter", og_r.data_ptr(), *og_r.stride()[:3], packed.data_ptr(), res_r.data_ptr(),
                  *res_r.stride()[:3], _ptrs(shards), world, rank, 1, n, N, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for p, shard in enumerate(shards):
        assert torch.equal(shard, want[:, :, p * n:(p + 1) * n])


@pytest.mark.parametrize("world,N", [(2, 256), (4, 128), (8, 256), (2, 192)])
def test_transition_scatter_writes_every_ranks_columns_into_the_row_shards(world, N):
    wt = orc.make_transition_weights(22, identity_ln=False)
    layer = b200.Transition(128, 512, dtype=torch.bfloat16)
    layer.load_state_dict({"norm.weight": wt.ln_w, "norm.bias": wt.ln_b, "fused_fc2_fc1.weight": wt.w1, "fc3.weight": wt.w2})
    layer = layer.to(DEV)
    packed = layer._packed(torch.device(DEV))
    g = torch.Generator().manual_seed(N * world)
    z = torch.randn(1, N, N, 128, generator=g).bfloat16().to(DEV)
    want = layer(z.clone(), residual=True)
    n = N // world
    shards = [torch.full((1, n, N, 128), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    for rank in range(world):
        cols = z[:, :, rank * n:(rank + 1) * n].contiguous()  # this rank's column shard [1, N, n, 128]
        _lib.call("b200ta_transition_scatter", cols.data_ptr(), None, packed.data_ptr(), layer.norm.eps, _ptrs(shards),
                  world, rank, 1, N, n, 1, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for p, shard in enumerate(shards):
        assert torch.equal(shard, want[:, p * n:(p + 1) * n])


def test_scatter_entry_points_refuse_shapes_they_cannot_address():
    buf = torch.zeros(1, 64, 32, 128, dtype=torch.bfloat16, device=DEV)
    layer = b200.Transition(128, 512, dtype=torch.bfloat16).to(DEV)
    packed = layer._packed(torch.device(DEV))
    with pytest.raises(ValueError):  # 24 columns per GPU: not a multiple of 32
        _lib.call("b200ta_transition_scatter", buf.data_ptr(), None, packed.data_ptr(), 1e-5, _ptrs([buf, buf]), 2, 0, 1,
                  48, 24, 1, torch.cuda.current_stream().cuda_stream)
    with pytest.raises(ValueError):  # rank outside the peer list
        _lib.call("b200ta_transition_scatter", buf.data_ptr(), None, packed.data_ptr(), 1e-5, _ptrs([buf, buf]), 2, 2, 1,
                  64, 32, 1, torch.cuda.current_stream().cuda_stream)
