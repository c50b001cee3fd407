"""The allocation-free forward, i8f_linear_forward_static, against the ordinary i8f_linear_forward.

Some callers may not allocate device memory at all: a host program that handed the whole GPU to its
own pool, a latency-critical loop that keeps away from the allocator, a sandboxed plugin that is only
allowed to launch on a stream it was given.  For them the library carries a fixed workspace inside
its own image; this test drives that entry point through the C ABI and checks that it gives the
same bits as the workspace-taking entry point -- twice in a row, the second time on a smaller
problem, so the array still holds the first call's data when the second call starts.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

from oracle import bitspec as bs
from oracle import torch_path as tp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(pkg, M, K, N, seed, per_channel, hadamard, with_bias):
    F, wl = pkg.functional, pkg.workloads
    x = wl.activation(M, K, seed=seed).to(DEV)
    w = wl.weight_fp32(N, K, seed=seed).to(DEV)
    if per_channel:
        wq, ws = F.quantize_weight_rows(w, hadamard=hadamard)
        ws = ws.reshape(-1).contiguous()
    else:
        wq, ws = F.quantize_tensorwise(w, hadamard=hadamard)
        ws = ws.reshape(1)
    bias = wl.bias_fp32(N, seed=seed).to(DEV).bfloat16() if with_bias else None
    return x, wq, ws, bias


def test_static_workspace_forward_matches_twice_in_a_row(cuda_pkg):
    F, nat = cuda_pkg.functional, cuda_pkg._native
    cases = [(1024, 2048, 1536, 21, True, False, True),     # first call fills a large part of the array
             (200, 512, 328, 22, False, True, False)]       # second, smaller call runs over the leftovers
    warmed = False
    for M, K, N, seed, per_channel, hadamard, with_bias in cases:
        x, wq, ws, bias = _case(cuda_pkg, M, K, N, seed, per_channel, hadamard, with_bias)
        want = F.linear_forward(x, wq, ws, bias, torch.bfloat16, hadamard=hadamard)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)   # the caller owns the output
        if not warmed:
            # The FIRST call on a device is where the driver gives the built-in array its memory (lazy module
            # loading), so device memory in use may grow by the array's size here -- once.
            F.linear_forward_static(x, wq, ws, bias, out, hadamard=hadamard)
            warmed = True
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats(DEV)["allocation.all.allocated"]      # running count of allocator requests
        free_before, _ = torch.cuda.mem_get_info(DEV)                           # what the DRIVER has left
        got = F.linear_forward_static(x, wq, ws, bias, out, hadamard=hadamard)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(DEV)
        after = torch.cuda.memory_stats(DEV)["allocation.all.allocated"]
        assert after == before, f"the wrapper must not allocate through torch either ({after - before} new blocks)"
        # torch's counter cannot see allocations made behind its back; the driver's free-memory figure can
        assert free_after >= free_before, f"device memory in use grew by {free_before - free_after} bytes during the call"
        assert got is out
        # and against the CPU oracle directly, not only against the sibling entry point
        x_cpu = x.cpu()
        if hadamard:
            x_cpu = torch.from_numpy(bs.rotate_activation(x_cpu.float().numpy(), "bf16")).bfloat16()
        oracle = tp.linear_w8a8(x_cpu, wq.cpu(), ws.cpu().reshape(-1, 1) if per_channel else float(ws.cpu()[0]),
                                None if bias is None else bias.cpu(), torch.bfloat16)
        assert torch.equal(got.cpu().view(torch.int16), oracle.view(torch.int16))
        # tolerance used by the linear tests: 1e-2 * RMS in max-abs; the two entry points share every
        # kernel, so they are in fact bit-identical
        rms = want.float().pow(2).mean().sqrt().item()
        assert (got.float() - want.float()).abs().max().item() <= 1e-2 * rms
        assert torch.equal(got, want)
    assert nat.device_status() == 0


def test_static_workspace_limit_is_enforced(cuda_pkg):
    """A problem beyond the built-in workspace is refused with a clear message and nothing is launched."""
    nat = cuda_pkg._native
    lib = nat.load()
    limit = nat.STATIC_WORKSPACE_BYTES
    assert lib.i8f_linear_workspace_bytes(4096, 4096) <= limit            # the stated example fits
    K = 4096
    M = limit // K + 1
    x = torch.empty(1, dtype=torch.bfloat16, device=DEV)                   # never dereferenced: the size check comes first
    rc = lib.i8f_linear_forward_static(nat.ptr(x), nat.I8F_BF16, K, 0, nat.ptr(x), K, nat.ptr(x), 0, None, 0, nat.ptr(x),
                                       nat.I8F_BF16, 16, M, 16, K, 0, ctypes.c_void_p(0))
    assert rc == -6
    msg = nat.last_error()
    assert "built-in" in msg and "i8f_linear_forward" in msg
    torch.cuda.synchronize()
    assert nat.device_status() == 0
