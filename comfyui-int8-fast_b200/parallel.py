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

    The ranks meet twice per `forward` in the library's own barrier kernel (`i8f_peer_barrier`): once before the
    stores (nobody still reads the previous result) and once after them (every block has landed everywhere).
    Its wait is BOUNDED: if a peer never arrives -- it raised on the host, it was killed -- the kernel gives up
    after about a second and leaves code 105 in the device status word, which `check()` turns into an exception;
    no rank is left spinning on the GPU.  Everything that can raise on one rank only (argument checks, the
    activation quantiser) runs before the first meeting, and the width rule is evaluated for ALL ranks' blocks, so
    the ranks either all pass it or all raise.
    """
    WAIT_LIMIT_CYCLES = 4_000_000_000       # about two seconds of SM clocks

    def __init__(self, rows: int, out_features: int, dtype: torch.dtype, device: torch.device, group=None):
        import os
        # plain peer stores only: the buffers need no NVLink multicast binding
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device
        self.out_features = out_features
        widths = [e - b for b, e in (shard_bounds(out_features, self.world, r) for r in range(self.world))]
        if any(w % 32 for w in widths):     # the same verdict on every rank
            raise ValueError(f"the fused column-parallel path needs every rank's block width to be a multiple of 32, got {widths}")
        self.buffer = symm_mem.empty((rows, out_features), dtype=dtype, device=device)
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.flag_handle = symm_mem.rendezvous(self.flags, self.group)
        dist.barrier(self.group)            # every rank's flags are zero before anyone publishes an epoch
        torch.cuda.synchronize(device)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.flag_ptrs = [int(p) for p in self.flag_handle.buffer_ptrs]
        # own buffer first: the local store is the cheap one
        self.dest_ptrs = [self.peer_ptrs[self.rank]] + [p for r, p in enumerate(self.peer_ptrs) if r != self.rank]
        self.epoch = 0

    def _meet(self) -> None:
        from . import functional as F
        self.epoch += 1
        F.peer_barrier(self.flag_ptrs, self.rank, self.epoch, self.device, self.WAIT_LIMIT_CYCLES)

    def forward(self, x: Tensor, shard: ColumnShard, hadamard: bool = False) -> Tensor:
        from . import functional as F
        if shard.out_features != self.out_features or (shard.begin, shard.end) != shard_bounds(self.out_features, self.world, self.rank):
            raise ValueError("the shard does not belong to this output buffer")
        if x.shape[0] > self.buffer.shape[0]:
            raise ValueError(f"{x.shape[0]} rows do not fit the buffer of {self.buffer.shape[0]}")
        q, xs = F.quantize_rowwise(x, hadamard=hadamard)
        self._meet()                          # nobody still reads the previous step's result
        F.linear_w8a8_scatter(q, xs, shard.weight, shard.weight_scale, shard.bias, self.dest_ptrs, self.out_features,
                              shard.begin, self.buffer.dtype)
        self._meet()                          # every rank's block has landed everywhere
        return self.buffer[: x.shape[0]]

    def check(self) -> None:
        """Synchronises the device and raises if a bounded wait of this library ran out since the last check (a peer
        that did not arrive at a meeting, or a stalled pipeline inside a kernel)."""
        from . import _native as nat
        with torch.cuda.device(self.device):
            status = nat.device_status()
        if status != 0:
            raise nat.NativeLibraryError(
                f"device status {status}: a bounded device-side wait ran out"
                + (" (a peer rank did not reach the column-parallel meeting point)" if status == 105 else ""))
