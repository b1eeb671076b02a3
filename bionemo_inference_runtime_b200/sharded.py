"""Row-sharded pair track for one multi-GPU box: one pair tensor split over the ranks of a process group.

The reference has no distributed compute (its multi-GPU mode is whole-model replicas); this module adds the
DAP-style partition its long-complex case needs.  One process per GPU, ``torch.distributed`` (NCCL) for the
exchanges, the library's kernels for everything else.

Layouts of the local shard of ``z[B, N, N, c]`` on rank ``g`` of ``G`` (``N % G == 0``, ``n = N / G``):

* ``ROWS``: ``z[:, g*n:(g+1)*n, :, :]``  -> tensor ``[B, n, N, c]``
* ``COLS``: ``z[:, :, g*n:(g+1)*n, :]``  -> tensor ``[B, N, n, c]``

Per block:

1. starting node on the ROWS shard.  Pair rows attend independently *given* the triangle bias, and the bias row
   ``bias[h, q, :]`` is a projection of pair row ``q``: every rank projects the bias rows of its own pair rows and
   one all-gather (1/32 of the bytes of ``z``) completes the ``[H, N, N]`` bias everywhere.
2. all-to-all ROWS -> COLS (the transpose between the nodes).
3. ending node on the COLS shard: it works on the transposed pair tensor, so pair *columns* are its independent
   rows; the kernels read the shard through swapped strides, and the same bias all-gather applies.
4. transition on the COLS shard (position-wise, layout does not matter).
5. all-to-all COLS -> ROWS for the next block (``keep_layout=True`` skips it for a caller that continues in COLS).

With ``fused_transpose`` (NCCL groups, CUDA tensors) step 2 is not a collective at all: the starting node's output
kernel (o_proj + residual) stores every result row straight into the column shard of the GPU that owns it, through
peer mappings of a symmetric-memory buffer (NVLink stores from inside the kernel), followed by one barrier.  The way
back (step 5) is fused the same way into the transition, whose TMA stores go to the row shard of the owning GPU
(column counts per GPU that are multiples of 32; otherwise, and without a transition, it stays an all-to-all).

The compute stages are looked up on a small ``stages`` object so that the orchestration (what is gathered, what
is exchanged, which strides are used) can be exercised with CPU tensors and the ``gloo`` backend.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, ops

ROWS = "rows"
COLS = "cols"


class KernelStages:
    """The library's kernels as the four stages the driver composes (CUDA tensors only)."""

    def prologue(self, node, x_kernel_order: torch.Tensor):
        """``x`` in kernel order ``[B, R, S, c]`` (any strides) -> (qkvg planes, local bias rows ``[B, H, R, S_pad]``)."""
        B, R, S, _ = x_kernel_order.shape
        bias = torch.empty((B, ops.HEADS, R, ops.pad8(S)), dtype=torch.bfloat16, device=x_kernel_order.device)
        return ops.prologue(x_kernel_order, node._packed(x_kernel_order.device), node.layer_norm.eps, bias=bias)

    def attention(self, node, qkvg, bias_full, lengths, B, R, S):
        mode = _lib.EMPTY_ROW_UNIFORM if node.empty_row_mode == "uniform" else _lib.EMPTY_ROW_ZEROS
        return ops.attention(qkvg, bias_full, lengths, B, R, S, empty_row_mode=mode)

    def epilogue(self, node, og, residual_kernel_order, out_kernel_order):
        B, R, S, _ = og.shape
        packed = node._packed(og.device)
        r, o = residual_kernel_order, out_kernel_order
        _lib.call("b200ta_epilogue", og.data_ptr(), og.stride(0), og.stride(1), og.stride(2), packed.data_ptr(),
                  None if r is None else r.data_ptr(), *((0, 0, 0) if r is None else r.stride()[:3]),
                  o.data_ptr(), *o.stride()[:3], B, R, S, torch.cuda.current_stream().cuda_stream)
        return out_kernel_order

    def transition(self, layer, x: torch.Tensor) -> torch.Tensor:
        return layer(x, residual=True, inplace=True)

    def peer_shard(self, shape, device, group) -> "_PeerShard":
        """A bf16 shard buffer of this rank that the other ranks' kernels can store into."""
        return _PeerShard(shape, device, group)

    def transition_scatter_ok(self, cols_per_rank: int) -> bool:
        return cols_per_rank % 32 == 0  # the transition's TMA stores move 32 rows at a time

    def epilogue_scatter(self, node, og, residual_kernel_order, cols_shard: "_PeerShard", rank: int):
        """o_proj + residual of the ROWS shard, written transposed into every GPU's COLS shard (peer stores)."""
        B, R, S, _ = og.shape
        packed = node._packed(og.device)
        r = residual_kernel_order
        peer_ptrs = cols_shard.ptrs
        ptrs = (ctypes.c_void_p * len(peer_ptrs))(*peer_ptrs)
        _lib.call("b200ta_epilogue_scatter", og.data_ptr(), og.stride(0), og.stride(1), og.stride(2), packed.data_ptr(),
                  r.data_ptr(), *r.stride()[:3], ptrs, len(peer_ptrs), rank, B, R, S,
                  torch.cuda.current_stream().cuda_stream)


    def transition_scatter(self, layer, x_cols, rows_shard: "_PeerShard", rank: int):
        """The transition (+ residual) of the COLS shard, written into every GPU's ROWS shard (peer TMA stores)."""
        B, N, n, _ = x_cols.shape
        peer_ptrs = rows_shard.ptrs
        ptrs = (ctypes.c_void_p * len(peer_ptrs))(*peer_ptrs)
        eps = layer.eps if layer.norm is None else layer.norm.eps
        _lib.call("b200ta_transition_scatter", x_cols.data_ptr(), None, layer._packed(x_cols.device).data_ptr(), eps,
                  ptrs, len(peer_ptrs), rank, B, N, n, 1, torch.cuda.current_stream().cuda_stream)


class _PeerShard:
    """A shard of this rank (``[B, N, n, c]`` COLS or ``[B, n, N, c]`` ROWS) in symmetric memory, with every rank's
    mapping of it."""

    def __init__(self, shape, device, group):
        import torch.distributed._symmetric_memory as symm_mem

        self.tensor = symm_mem.empty(shape, dtype=torch.bfloat16, device=device)
        handle = symm_mem.rendezvous(self.tensor, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in handle.buffer_ptrs]
        self.shape = tuple(shape)


def shard(z: torch.Tensor, rank: int, world: int, layout: str = ROWS) -> torch.Tensor:
    """A contiguous copy of the local shard of a full pair tensor (for tests and for loading inputs); never a view
    of ``z``, because the sharded block updates its shard in place."""
    n = z.shape[1] // world
    if z.shape[1] % world or z.shape[1] != z.shape[2]:
        raise ValueError(f"need a square pair tensor whose side is divisible by the world size, got {tuple(z.shape)}")
    part = z[:, rank * n:(rank + 1) * n] if layout == ROWS else z[:, :, rank * n:(rank + 1) * n]
    return part.clone(memory_format=torch.contiguous_format)


def exchange(x: torch.Tensor, to_layout: str, group=None) -> torch.Tensor:
    """All-to-all between the ROWS shard ``[B, n, N, c]`` and the COLS shard ``[B, N, n, c]``.

    Rank ``g`` sends the block (its rows, columns of rank ``p``) to rank ``p`` and receives (rows of rank ``p``, its
    columns): ``(G-1)/G`` of the shard crosses the links once.  One staging copy packs the outgoing blocks per peer;
    the received blocks already are the target layout.
    """
    world = dist.get_world_size(group)
    B = x.shape[0]
    c = x.shape[-1]
    if to_layout == COLS:
        n, N = x.shape[1], x.shape[2]
        send = x.view(B, n, world, n, c).permute(2, 0, 1, 3, 4).contiguous()      # [G][B, n(i), n(j), c]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)                            # [G(src p)][B, n(i of p), n(j), c]
        return recv.permute(1, 0, 2, 3, 4).reshape(B, N, n, c)                     # i = p*n + i_local: contiguous view
    if to_layout == ROWS:
        N, n = x.shape[1], x.shape[2]
        send = x.view(B, world, n, n, c).permute(1, 0, 2, 3, 4).contiguous()      # [G(dst p)][B, n(i of p), n(j), c]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)                            # [G(src p)][B, n(i), n(j of p), c]
        return recv.permute(1, 2, 0, 3, 4).reshape(B, n, N, c)                     # j = p*n + j_local (one copy)
    raise ValueError(f"unknown layout {to_layout!r}")


def gather_bias(bias_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of the locally projected bias rows ``[B, H, n, S_pad]`` into the full ``[B, H, N, S_pad]``."""
    world = dist.get_world_size(group)
    B, H, n, sp = bias_local.shape
    gathered = torch.empty((world, B, H, n, sp), dtype=bias_local.dtype, device=bias_local.device)
    dist.all_gather_into_tensor(gathered.view(-1), bias_local.contiguous().view(-1), group=group)
    return gathered.permute(1, 2, 0, 3, 4).reshape(B, H, world * n, sp)


class ShardedPairBlock:
    """start node -> exchange -> end node -> transition (-> exchange back) on a sharded pair tensor."""

    def __init__(self, start_node, end_node, transition=None, group=None, stages=None, fused_transpose: bool = False):
        self.start_node = start_node
        self.end_node = end_node
        self.transition = transition
        self.group = group
        self.stages = stages if stages is not None else KernelStages()
        self.fused_transpose = fused_transpose
        self._cols: _PeerShard | None = None
        self._rows: _PeerShard | None = None
        self._flag: torch.Tensor | None = None

    def _barrier(self, device) -> None:
        """Orders the peer stores against the other ranks' reads: a one-element all-reduce on the current stream."""
        if self._flag is None or self._flag.device != torch.device(device):
            self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        dist.all_reduce(self._flag, group=self.group)

    def _start_node_into_column_shards(self, z_rows: torch.Tensor, lengths_rows) -> torch.Tensor:
        """The starting node on the ROWS shard with its output written directly into every rank's COLS shard."""
        rank = dist.get_rank(self.group)
        B, n, N, c = z_rows.shape
        if self._cols is None or self._cols.shape != (B, N, n, c):
            self._cols = self.stages.peer_shard((B, N, n, c), z_rows.device, self.group)
        node = self.start_node
        qkvg, bias_local = self.stages.prologue(node, z_rows)
        bias_full = gather_bias(bias_local, self.group)
        og = self.stages.attention(node, qkvg, bias_full, lengths_rows, B, n, N)
        # Every rank's last read of its column shard lies before a collective this rank has already completed: the
        # barrier after the previous call's transition, or its exchange back to rows, and the bias all-gather above.
        self.stages.epilogue_scatter(node, og, z_rows, self._cols, rank)
        self._barrier(z_rows.device)  # every rank's stores into this rank's column shard have landed
        return self._cols.tensor

    def _node(self, node, x_shard: torch.Tensor, layout: str, lengths_local: torch.Tensor | None) -> torch.Tensor:
        """One node on the shard whose independent rows are local: ROWS for the starting node, COLS for the ending
        node.  ``lengths_local`` holds the valid-key count of each local kernel row, ``[B, n]`` int32."""
        xk = x_shard if layout == ROWS else x_shard.transpose(1, 2)  # kernel order [B, R = n, S = N, c]
        B, R, S, _ = xk.shape
        qkvg, bias_local = self.stages.prologue(node, xk)
        bias_full = gather_bias(bias_local, self.group)
        og = self.stages.attention(node, qkvg, bias_full, lengths_local, B, R, S)
        self.stages.epilogue(node, og, xk, xk)  # in place: z += update
        return x_shard

    def forward(self, z_rows: torch.Tensor, lengths_rows: torch.Tensor | None = None,
                lengths_cols: torch.Tensor | None = None, keep_layout: bool = False) -> torch.Tensor:
        """``z_rows``: ROWS shard ``[B, n, N, c]`` (updated in place where possible).  ``lengths_rows[b, i_local]`` =
        valid keys of local pair row i (starting node); ``lengths_cols[b, j_local]`` = valid keys of local pair column
        j (ending node).  Returns the ROWS shard of the block output (the COLS shard with ``keep_layout``); with
        ``fused_transpose`` the result is one of the block's symmetric-memory buffers, valid until the next call
        (it may be passed back in as the next call's ``z_rows``)."""
        if self.fused_transpose:
            z_cols = self._start_node_into_column_shards(z_rows, lengths_rows)
        else:
            z_rows = self._node(self.start_node, z_rows, ROWS, lengths_rows)
            z_cols = exchange(z_rows, COLS, self.group)
        z_cols = self._node(self.end_node, z_cols, COLS, lengths_cols)
        B, N, n, c = z_cols.shape
        if (self.fused_transpose and self.transition is not None and not keep_layout
                and self.stages.transition_scatter_ok(n)):
            if self._rows is None or self._rows.shape != (B, n, N, c):
                self._rows = self.stages.peer_shard((B, n, N, c), z_cols.device, self.group)
            # every rank has read its row shard of the previous call (prologue and residual of the starting node)
            # before the barrier that follows the starting node of this call
            self.stages.transition_scatter(self.transition, z_cols, self._rows, dist.get_rank(self.group))
            self._barrier(z_cols.device)  # every rank's stores into this rank's row shard have landed
            return self._rows.tensor
        if self.transition is not None:
            z_cols = self.stages.transition(self.transition, z_cols)
        return z_cols if keep_layout else exchange(z_cols, ROWS, self.group)

    __call__ = forward
