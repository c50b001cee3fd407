"""Block-diagonal Walsh-Hadamard rotation (QuaRot) in groups of 128 channels.

Same entry points as the node pack's quarot.py.  The rotation itself runs in
the CUDA kernels as a register/shuffle butterfly (natural Sylvester order), in
the hot path fused into the activation quantiser; the functions here are the
stand-alone forms.  `H` arguments are accepted for signature compatibility and
ignored: the kernels implement exactly the normalised Sylvester matrix of
order 128.
"""
from __future__ import annotations

import torch

from . import functional as F

GROUP_SIZE = 128
_CACHE: dict = {}


def build_hadamard(size: int, device="cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Normalised Sylvester-Hadamard matrix, H[i,j] = (-1)^popcount(i&j) / sqrt(size).   quarot.py:18-39"""
    key = (size, str(device), dtype)
    if key not in _CACHE:
        if size <= 0 or size & (size - 1):
            raise ValueError(f"Hadamard size must be power of 2, got {size}")
        idx = torch.arange(size)
        bits = idx[:, None] & idx[None, :]
        parity = torch.zeros_like(bits)
        while bool(bits.any()):
            parity ^= bits & 1
            bits = bits >> 1
        _CACHE[key] = ((1 - 2 * parity).to(dtype) / (size ** 0.5)).to(device)
    return _CACHE[key]


def _rotate(t: torch.Tensor, group_size: int) -> torch.Tensor:
    if group_size != GROUP_SIZE:
        raise NotImplementedError("the CUDA kernels implement group_size 128 only")
    if t.shape[-1] % group_size:
        raise ValueError(f"features {t.shape[-1]} not divisible by group_size {group_size}")
    flat = t.reshape(-1, t.shape[-1])
    return F.quantize_rowwise(flat, hadamard=True, return_rotated=True)[2].reshape(t.shape)


def rotate_weight(weight: torch.Tensor, H, group_size: int = GROUP_SIZE) -> torch.Tensor:
    """W @ H_block^T for a weight [out, in] (H is symmetric); computed in fp32.   quarot.py:42-70"""
    return _rotate(weight.float(), group_size).to(weight.dtype)


def rotate_activation(x: torch.Tensor, H, group_size: int = GROUP_SIZE) -> torch.Tensor:
    """x @ H_block over the last axis, rounded to x's dtype.   quarot.py:73-102"""
    return _rotate(x, group_size)
