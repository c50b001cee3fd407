"""Seeded synthetic inputs for the benchmark configurations.

No checkpoint, LoRA file or dataset is available offline, so every workload is
synthetic: shapes and value distributions follow the benchmark definitions
(activations ~N(0,1) with 1 % of the K channels scaled x20 as outliers,
weights ~N(0,0.02), bias ~N(0,0.01)).  Tensors are generated on the CPU with
one torch.Generator per tensor (seed * 1000 + tag), so the CPU oracle and the
GPU kernels see identical bits regardless of generation order.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

TAG_X, TAG_W, TAG_BIAS, TAG_LORA_A, TAG_LORA_B, TAG_UNIFORM, TAG_OUTLIER = 1, 2, 3, 4, 5, 6, 7


def _gen(seed: int, tag: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed * 1000 + tag)
    return g


def activation(M: int, K: int, seed: int, dtype: torch.dtype = torch.bfloat16, outlier_frac: float = 0.01,
               outlier_gain: float = 20.0) -> torch.Tensor:
    x = torch.randn(M, K, generator=_gen(seed, TAG_X))
    n_out = int(round(K * outlier_frac))
    if n_out > 0:
        idx = torch.randperm(K, generator=_gen(seed, TAG_OUTLIER))[:n_out]
        x[:, idx] *= outlier_gain
    return x.to(dtype)


def weight_fp32(N: int, K: int, seed: int, std: float = 0.02) -> torch.Tensor:
    return torch.randn(N, K, generator=_gen(seed, TAG_W)) * std


def bias_fp32(N: int, seed: int, std: float = 0.01) -> torch.Tensor:
    return torch.randn(N, generator=_gen(seed, TAG_BIAS)) * std


def lora_factors(N: int, K: int, r: int, seed: int, dtype: torch.dtype = torch.bfloat16):
    """lora_A [r,K] ~ N(0, 1/r) (variance), lora_B [N,r] ~ N(0, 0.01) (std), in the reference's layout."""
    a = torch.randn(r, K, generator=_gen(seed, TAG_LORA_A)) * (1.0 / r) ** 0.5
    b = torch.randn(N, r, generator=_gen(seed, TAG_LORA_B)) * 0.01
    return a.to(dtype), b.to(dtype)


def uniforms(N: int, K: int, seed: int) -> torch.Tensor:
    return torch.rand(N, K, generator=_gen(seed, TAG_UNIFORM), dtype=torch.float32)


@dataclass(frozen=True)
class LinearShape:
    name: str
    M: int
    K: int
    N: int
    hadamard: bool
    per_channel: bool
    bias: bool
    lora_rank: int = 0


# The benchmark configurations of the quantised linear (single GPU).
CONFIGS = {
    "c0_cpu_linear": LinearShape("c0_cpu_linear", 256, 3072, 3072, False, True, True),
    "c1_quarot_mlp_up": LinearShape("c1_quarot_mlp_up", 4096, 4096, 12288, True, False, False),
    "c2_dynamic_lora": LinearShape("c2_dynamic_lora", 8192, 4096, 4096, False, True, True, 64),
}
