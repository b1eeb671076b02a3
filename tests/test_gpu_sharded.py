"""The row-sharded pair block on 2 GPUs (NCCL) against the same block on one GPU.  Skipped with fewer than 2 GPUs."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
WORLD = 2
N = 256
VALID = 230


def _modules(device):
    import bionemo_inference_runtime_b200 as b200
    from oracle import triangle_oracle as orc

    def node(cls, seed):
        w = orc.make_node_weights(seed, identity_ln=False)
        layer = cls(128, 32, 4, dtype=torch.bfloat16)
        layer.load_state_dict({"layer_norm.weight": w.ln_w, "layer_norm.bias": w.ln_b, "pair_bias_proj.weight": w.w_bias,
                               "mha.in_proj.weight": w.w_in, "mha.o_proj.weight": w.w_out}, strict=True)
        return layer.to(device)

    wt = orc.make_transition_weights(93, identity_ln=False)
    trans = b200.Transition(128, 512, dtype=torch.bfloat16)
    trans.load_state_dict({"norm.weight": wt.ln_w, "norm.bias": wt.ln_b, "fused_fc2_fc1.weight": wt.w1,
                           "fc3.weight": wt.w2}, strict=True)
    return node(b200.TriangleAttentionStartingNode, 91), node(b200.TriangleAttentionEndingNode, 92), trans.to(device)


def _worker(rank: int, port: int, fused: bool, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=device)
    try:
        from bionemo_inference_runtime_b200 import _lib, sharded

        g = torch.Generator().manual_seed(5)
        z = torch.randn(1, N, N, 128, generator=g).bfloat16().to(device)
        start, end, trans = _modules(device)
        n = N // WORLD
        idx = torch.arange(rank * n, (rank + 1) * n, device=device)
        lengths = torch.where(idx < VALID, VALID, 0).to(torch.int32).reshape(1, n)
        block = sharded.ShardedPairBlock(start, end, trans, fused_transpose=fused)
        out_rows = block(sharded.shard(z, rank, WORLD), lengths, lengths)
        if fused:  # a second call reuses the symmetric-memory column shard
            out_rows = block(sharded.shard(z, rank, WORLD), lengths, lengths)
        gathered = [torch.empty_like(out_rows) for _ in range(WORLD)]
        dist.all_gather(gathered, out_rows)
        torch.cuda.synchronize()
        status = _lib.device_status()
        if rank == 0:
            full_len = torch.where(torch.arange(N, device=device) < VALID, VALID, 0).to(torch.int32).reshape(1, N)
            want = start(z, mask_bias=full_len, residual=True)
            want = end(want, mask_bias=full_len, residual=True)
            want = trans(want, residual=True)
            got = torch.cat(gathered, dim=1)
            results.put((bool(torch.equal(got, want)), float((got.float() - want.float()).abs().max()), status))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < WORLD, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", [False, True], ids=["all_to_all", "peer_stores"])
def test_sharded_block_on_two_gpus_equals_single_gpu(fused):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, port + int(fused), fused, results)) for r in range(WORLD)]
    for p in procs:
        p.start()
    equal, max_diff, status = results.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert status == 0
    assert equal, f"sharded result differs from the single-GPU result (max abs diff {max_diff})"
