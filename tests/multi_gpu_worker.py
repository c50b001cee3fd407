"""Worker for test_gpu_multi.py: one process per GPU (launched with torch.distributed.run)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import __graft_entry__ as g
    pkg = g.load_package()
    F, par, wl = pkg.functional, pkg.parallel, pkg.workloads
    M, K, N = 520, 512, 256 * world
    x = wl.activation(M, K, seed=3).to(dev)                        # identical on every rank
    w = wl.weight_fp32(N, K, seed=3).to(dev)
    bias = wl.bias_fp32(N, seed=3).to(dev)
    ok = True
    for per_channel in (True, False):
        wq, ws = F.quantize_weight_rows(w) if per_channel else F.quantize_tensorwise(w)
        full = F.linear_forward(x, wq, ws, bias, torch.bfloat16)    # unsharded result
        shard = par.shard_columns(wq, ws if per_channel else ws.reshape(1), bias, world, rank)
        y_nccl = par.column_parallel_linear(x, shard, torch.bfloat16)
        ok &= bool(torch.equal(y_nccl, full))
        fused = par.FusedColumnParallelOutput(M, N, torch.bfloat16, dev)
        for _ in range(3):                                         # repeated steps reuse the symmetric buffer
            y = fused.forward(x, shard)
        torch.cuda.synchronize()
        ok &= bool(torch.equal(y, full))
        rows = par.shard_rows(x, world, rank)                      # token-parallel: no communication at all
        b, e = par.shard_bounds(M, world, rank)
        ok &= bool(torch.equal(F.linear_forward(rows, wq, ws, bias, torch.bfloat16), full[b:e]))
    ok &= pkg._native.device_status() == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    if rank == 0:
        print("MULTI_GPU_OK" if int(flag.item()) == 1 else "MULTI_GPU_MISMATCH")
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
