"""Randomised larger shapes (several waves of 256 x 256 pair tiles, ragged edges) checked against independent paths:
the plain linear against the library int8 matmul + the reference's PyTorch epilogue expression, the fused-LoRA GEMM
against the two-kernel form (LoRA up projection, then GEMM with add) -- bit for bit in both cases."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_linear_matches_library_int_mm_and_torch_epilogue_on_large_ragged_shapes(cuda_pkg):
    F = cuda_pkg.functional
    rng = random.Random(7)
    for _ in range(24):
        M = rng.choice([17, 129, 255, 257, 513, 777, 1500, 2049, 4097])
        N, K = 8 * rng.randint(1, 800), 16 * rng.randint(1, 300)
        a = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=DEV)
        w = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=DEV)
        acc = torch._int_mm(a, w.t())
        assert torch.equal(F.gemm_i8_i32(a, w), acc)
        xs = torch.rand(M, 1, device=DEV) * 0.02 + 1e-4
        per_ch = rng.random() < 0.5
        ws = (torch.rand(N, device=DEV) * 1e-3 + 1e-5) if per_ch else torch.tensor([3.1e-4], device=DEV)
        bias = (torch.randn(N, device=DEV) * 0.05) if rng.random() < 0.7 else None
        # int8_quant.py:84-88 (scalar scale) and :115-119 (per-row scale)
        ref = (acc.float() * xs * ws.reshape(1, -1)).to(torch.bfloat16) if per_ch else (acc.float() * (ws * xs)).to(torch.bfloat16)
        if bias is not None:
            ref = ref + bias.to(torch.bfloat16)
        assert torch.equal(F.linear_w8a8(a, xs, w, ws, bias, torch.bfloat16), ref), (M, N, K, per_ch)
    torch.cuda.synchronize()
    assert cuda_pkg._native.device_status() == 0


def test_fused_lora_gemm_equals_two_kernel_form_on_ragged_shapes(cuda_pkg):
    F = cuda_pkg.functional
    rng = random.Random(11)
    for _ in range(20):
        M = rng.choice([129, 257, 300, 513, 777, 1500, 2049, 3000])
        N, K, r = 8 * rng.randint(17, 500), 16 * rng.randint(1, 200), rng.choice([8, 16, 24, 64, 128])
        a = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=DEV)
        w = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=DEV)
        xs = torch.rand(M, 1, device=DEV) * 0.02 + 1e-4
        ws = (torch.rand(N, device=DEV) * 1e-3 + 1e-5) if rng.random() < 0.5 else torch.tensor([3.1e-4], device=DEV)
        bias = (torch.randn(N, device=DEV) * 0.05).bfloat16() if rng.random() < 0.7 else None
        t = (torch.randn(M, r, device=DEV) * 0.5).bfloat16()
        lb = (torch.randn(N, r, device=DEV) * 0.1).bfloat16()
        fused = F.linear_w8a8_lora(a, xs, w, ws, bias, t, lb, torch.bfloat16)
        two = F.lora_up(t, lb)
        F.linear_w8a8(a, xs, w, ws, bias, torch.bfloat16, add_into=two)
        assert torch.equal(fused, two), (M, N, K, r)
    torch.cuda.synchronize()
    assert cuda_pkg._native.device_status() == 0
