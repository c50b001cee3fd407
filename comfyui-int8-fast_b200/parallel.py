"""Multi-GPU forms of the quantised linear: one process per GPU (torch.distributed).

The path shards without changing any kernel:

* token / batch parallel -- weights replicated, every rank runs its own rows; the per-token
  quantisation is row-local, so there is nothing to communicate (see `shard_rows`);
* column parallel -- rank p owns the output channels [p*N/P, (p+1)*N/P): its int8 weight rows, its
  per-channel scales and its bias slice.  Every rank quantises the full activation itself (50 MB of
  traffic at M = K = 4096, cheaper than exchanging int8), runs the GEMM on its slice and the bf16
  [M, N/P] blocks are all-gathered (NCCL over NVLink).  Per-token scales are identical on all ranks
  (same bits in, same bits out), so the gathered result equals the unsharded one bit for bit,
  provided a tensorwise weight scale is the global one computed before sharding.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor


def shard_bounds(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous [begin, end) of `total` items for `rank`; the first total % world ranks get one more."""
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_rows(x: Tensor, world: int, rank: int) -> Tensor:
    """Token-parallel split of a [M, K] activation (no communication follows)."""
    b, e = shard_bounds(x.shape[0], world, rank)
    return x[b:e]


@dataclass
class ColumnShard:
    """One rank's slice of a quantised linear layer."""
    weight: Tensor            # int8 [n_local, K]
    weight_scale: object      # python float / 1-element tensor (global) or fp32 [n_local, 1]
    bias: Tensor | None       # [n_local]
    begin: int
    end: int
    out_features: int


def shard_columns(weight: Tensor, weight_scale, bias: Tensor | None, world: int, rank: int) -> ColumnShard:
    """Slice of W [N,K], its scales and bias owned by `rank`.  A tensorwise scale is passed through
    unchanged: it has to stay the global scale for the sharded result to equal the unsharded one."""
    n = weight.shape[0]
    b, e = shard_bounds(n, world, rank)
    per_channel = isinstance(weight_scale, Tensor) and weight_scale.numel() > 1
    ws = weight_scale.reshape(n, 1)[b:e].contiguous() if per_channel else weight_scale
    return ColumnShard(weight[b:e].contiguous(), ws, None if bias is None else bias[b:e].contiguous(), b, e, n)


def all_gather_columns(y_local: Tensor, out_features: int, group=None) -> Tensor:
    """[M, n_local] blocks of every rank -> [M, N].  Uneven splits are padded to the widest block for the
    collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    m = y_local.shape[0]
    widths = [shard_bounds(out_features, world, r) for r in range(world)]
    widest = max(e - b for b, e in widths)
    send = y_local
    if y_local.shape[1] != widest:
        send = y_local.new_zeros((m, widest))
        send[:, : y_local.shape[1]] = y_local
    flat = y_local.new_empty((world * m, widest))          # rank r's block lands in rows [r*m, (r+1)*m)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    gathered = flat.view(world, m, widest)
    out = y_local.new_empty((m, out_features))
    for r, (b, e) in enumerate(widths):
        out[:, b:e] = gathered[r, :, : e - b]
    return out


def column_parallel_linear(x: Tensor, shard: ColumnShard, out_dtype: torch.dtype, hadamard: bool = False,
                           group=None, linear_fn=None) -> Tensor:
    """Full [M, N] output of a column-parallel quantised linear.

    `linear_fn(x, weight, weight_scale, bias, out_dtype, hadamard=...)` computes the local block; it
    defaults to the CUDA path (functional.linear_forward) and exists as a parameter so the sharding and
    gathering logic can be exercised with CPU ranks.
    """
    if linear_fn is None:
        from . import functional as F
        linear_fn = F.linear_forward
    y_local = linear_fn(x, shard.weight, shard.weight_scale, shard.bias, out_dtype, hadamard=hadamard)
    return all_gather_columns(y_local, shard.out_features, group=group)


class FusedColumnParallelOutput:
    """Every rank's copy of the full [M, N] activation in symmetric memory, for the fused form of the
    column-parallel linear: the GEMM epilogue stores each finished tile of this rank's column block into all
    ranks' copies (TMA stores to this GPU's memory and, over NVLink, to the peers' mapped buffers), so there is
    no separate all-gather pass and the transfer overlaps the tensor-core main loop.  Only stores cross GPUs.

    After `forward` returns, the local copy holds all columns once every rank's kernel has finished; `forward`
    ends with a barrier over the symmetric-memory signal pads, stream-ordered on the current stream.
    """

    def __init__(self, rows: int, out_features: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.out_features = out_features
        self.buffer = symm_mem.empty((rows, out_features), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        # own buffer first: the local store is the cheap one
        self.dest_ptrs = [self.peer_ptrs[self.rank]] + [p for r, p in enumerate(self.peer_ptrs) if r != self.rank]

    def forward(self, x: Tensor, shard: ColumnShard, hadamard: bool = False) -> Tensor:
        from . import functional as F
        if (shard.end - shard.begin) % 32:
            raise ValueError("the fused column-parallel path needs a block width that is a multiple of 32")
        q, xs = F.quantize_rowwise(x, hadamard=hadamard)
        self.handle.barrier(channel=0)        # nobody still reads the previous step's result
        F.linear_w8a8_scatter(q, xs, shard.weight, shard.weight_scale, shard.bias, self.dest_ptrs, self.out_features,
                              shard.begin, self.buffer.dtype)
        self.handle.barrier(channel=1)        # every rank's block has landed everywhere
        return self.buffer[: x.shape[0]]
