"""Sharding bookkeeping of the multi-GPU paths with two CPU ranks (gloo).

The local block is computed by the CPU oracle here (the CUDA path cannot run without a GPU); what is
under test is the partitioning, the scale / bias slicing and the all-gather, including an uneven
split, and that the gathered result equals the unsharded computation bit for bit.
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_linear(x, weight, weight_scale, bias, out_dtype, hadamard=False):
    from oracle import bitspec as bs
    ws = weight_scale.numpy() if isinstance(weight_scale, torch.Tensor) else np.float32(weight_scale)
    y = bs.linear_w8a8(x.float().numpy(), weight.numpy(), ws, None if bias is None else bias.numpy(), hadamard=hadamard)
    return torch.from_numpy(y).to(out_dtype)


def _worker(rank, world, port, per_channel, n_out, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests" / "fake_comfy"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import __graft_entry__ as g
        from oracle import bitspec as bs
        pkg = g.load_package()
        par, wl = pkg.parallel, pkg.workloads
        M, K = 24, 256
        x = wl.activation(M, K, seed=1)
        w = wl.weight_fp32(n_out, K, seed=1).numpy()
        wq, ws = bs.quantize_rowwise(w) if per_channel else bs.quantize_tensorwise(w)
        bias = wl.bias_fp32(n_out, seed=1)
        ws_t = torch.from_numpy(np.asarray(ws))
        shard = par.shard_columns(torch.from_numpy(wq), ws_t if per_channel else float(ws), bias, world, rank)
        y = par.column_parallel_linear(x, shard, torch.bfloat16, linear_fn=_oracle_linear)
        full = _oracle_linear(x, torch.from_numpy(wq), ws_t if per_channel else float(ws), bias, torch.bfloat16)
        rows = par.shard_rows(x, world, rank)
        q.put((rank, bool(torch.equal(y, full)), tuple(y.shape), shard.begin, shard.end, rows.shape[0]))
    except Exception as e:  # noqa: BLE001 - report instead of leaving the parent waiting
        q.put((rank, repr(e), (), -1, -1, -1))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("per_channel,n_out", [(True, 96), (False, 96), (True, 101)])
def test_column_parallel_equals_unsharded(per_channel, n_out):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, per_channel, n_out, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1] for r in results] == [True, True]
    assert all(r[2] == (24, n_out) for r in results)
    assert results[0][3] == 0 and results[0][4] == results[1][3] and results[1][4] == n_out
    assert sum(r[5] for r in results) == 24


def test_shard_bounds_cover_everything(pkg):
    par = pkg.parallel
    for total, world in [(16384, 8), (101, 2), (7, 8), (0, 4)]:
        spans = [par.shard_bounds(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1
