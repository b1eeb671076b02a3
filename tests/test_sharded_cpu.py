"""The sharded driver's orchestration on CPU ranks (gloo, world size 2): with the oracle as compute stages, the
bias all-gather, the ROWS<->COLS all-to-all and the strided ending-node view must reproduce the unsharded result."""

import math
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from bionemo_inference_runtime_b200 import sharded
from oracle import triangle_oracle as orc

WORLD = 2
N, B = 12, 2


class OracleStages:
    """CPU stand-ins for the kernels, built from the oracle's formulas (test infrastructure only)."""

    def prologue(self, w: orc.NodeWeights, xk):
        normed = F.layer_norm(xk, (128,), w.ln_w, w.ln_b, 1e-5)
        bias = F.linear(normed, w.w_bias).permute(0, 3, 1, 2)  # [B, H, R, S]
        bias = F.pad(bias, (0, -bias.shape[-1] % 8))
        return F.linear(normed, w.w_in, w.b_in), bias.contiguous()

    def attention(self, w, proj, bias_full, lengths, B, R, S):
        q, k, v, g = proj.split(128, dim=-1)
        hf = lambda t: t.reshape(B, R, S, 4, 32).permute(0, 1, 3, 2, 4)  # noqa: E731
        a = torch.matmul(hf(q), hf(k).transpose(-1, -2)) / math.sqrt(32)
        valid = torch.arange(S)[None, None, :] < lengths[..., None]
        a = a + 1e9 * (valid.float() - 1)[:, :, None, None, :] + bias_full[..., :S].unsqueeze(1)
        o = torch.matmul(torch.softmax(a, dim=-1), hf(v)).transpose(-3, -2).reshape(B, R, S, 128)
        return o * torch.sigmoid(g)

    def epilogue(self, w, og, residual, out):
        out.copy_(residual + F.linear(og, w.w_out, w.b_out))
        return out

    def transition(self, w_t, x):
        x.copy_(orc.transition_forward(x, None, w_t, residual=True))
        return x

    # The fused-transpose stages: on CPU ranks the "peer stores" are an exchange into the local shard buffer, so
    # the driver's ordering of stages and buffers is what gets tested.
    class _Shard:
        def __init__(self, shape):
            self.tensor, self.shape, self.ptrs = torch.full(shape, float("nan")), tuple(shape), None

    def peer_shard(self, shape, device, group):
        return self._Shard(shape)

    def transition_scatter_ok(self, cols_per_rank):
        return True

    def epilogue_scatter(self, w, og, residual, cols_shard, rank):
        cols_shard.tensor.copy_(sharded.exchange(residual + F.linear(og, w.w_out, w.b_out), sharded.COLS))

    def transition_scatter(self, w_t, x_cols, rows_shard, rank):
        rows_shard.tensor.copy_(sharded.exchange(orc.transition_forward(x_cols, None, w_t, residual=True), sharded.ROWS))


def _inputs():
    g = torch.Generator().manual_seed(7)
    z = torch.randn(B, N, N, 128, generator=g)
    m = torch.zeros(B, N)
    m[0, :N] = 1
    m[1, :9] = 1
    mask = m[:, :, None] * m[:, None, :]
    w1 = orc.make_node_weights(71, identity_ln=False, gate_bias=1.0, out_bias=True)
    w2 = orc.make_node_weights(72, identity_ln=False)
    wt = orc.make_transition_weights(73, identity_ln=False)
    return z, mask, w1, w2, wt


def _worker(rank: int, port: int, fused: bool, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        z, mask, w1, w2, wt = _inputs()
        block = sharded.ShardedPairBlock(w1, w2, wt, stages=OracleStages(), fused_transpose=fused)
        z_rows = sharded.shard(z, rank, WORLD, sharded.ROWS)
        lengths_rows = orc.row_lengths(sharded.shard(mask.unsqueeze(-1), rank, WORLD, sharded.ROWS).squeeze(-1))
        lengths_cols = orc.row_lengths(sharded.shard(mask.unsqueeze(-1), rank, WORLD, sharded.COLS).squeeze(-1).transpose(1, 2))
        out_rows = block(z_rows.clone(), lengths_rows, lengths_cols)
        if fused:  # a second call reuses the shard buffers
            out_rows = block(z_rows.clone(), lengths_rows, lengths_cols).clone()
        # the exchange round trip must be the identity
        rt = sharded.exchange(sharded.exchange(z_rows.clone(), sharded.COLS), sharded.ROWS)
        gathered = [torch.empty_like(out_rows) for _ in range(WORLD)]
        dist.all_gather(gathered, out_rows)
        if rank == 0:
            results.put((torch.cat(gathered, dim=1), bool(torch.equal(rt, z_rows))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fused", [False, True], ids=["all_to_all", "fused_transpose"])
def test_sharded_block_matches_unsharded_oracle(fused):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + int(fused)
    procs = [ctx.Process(target=_worker, args=(r, port, fused, results)) for r in range(WORLD)]
    for p in procs:
        p.start()
    got, roundtrip_ok = results.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    z, mask, w1, w2, wt = _inputs()
    want = orc.node_forward(z, mask, w1, orc.STARTING, residual=True)
    want = orc.node_forward(want, mask, w2, orc.ENDING, residual=True)
    want = orc.transition_forward(want, None, wt, residual=True)
    assert roundtrip_ok
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)


def test_shard_rejects_indivisible_sizes():
    with pytest.raises(ValueError):
        sharded.shard(torch.zeros(1, 10, 10, 4), 0, 3)
