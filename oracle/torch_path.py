"""The hot path as multi-threaded CPU PyTorch.  TEST INFRASTRUCTURE ONLY.

This is what the reference executes on a machine without a GPU (CPU tensors
select its non-Triton branch, int8_quant.py:72 and :103).  It is used (1) by
tests, to tie the NumPy bit-spec to PyTorch arithmetic, and (2) by the
benchmark's CPU-baseline arm, which times it on the host cores.

Parity pin: fixtures generated from the reference's own functions
(tests/golden/); the reference itself has no tests.
"""
from __future__ import annotations

import torch

_NORM = {}


def _hadamard128(dtype: torch.dtype) -> torch.Tensor:
    """Normalised Sylvester-Hadamard matrix of order 128 in `dtype`.   quarot.py:18-39

    Entry (i, j) is (-1)^popcount(i & j); the +-1 matrix is built in `dtype`
    and divided by sqrt(128) in that dtype, as the reference does.
    """
    if dtype not in _NORM:
        idx = torch.arange(128)
        bits = idx[:, None] & idx[None, :]
        pop = torch.zeros_like(bits)
        for s in range(7):
            pop += (bits >> s) & 1
        h = (1 - 2 * (pop & 1)).to(dtype)
        _NORM[dtype] = h / (128 ** 0.5)
    return _NORM[dtype]


def rotate_activation(x: torch.Tensor) -> torch.Tensor:
    """Block-diagonal x @ H in x's dtype.   quarot.py:73-102"""
    k = x.shape[-1]
    return torch.matmul(x.reshape(*x.shape[:-1], k // 128, 128), _hadamard128(x.dtype)).reshape(x.shape)


def rotate_weight(w: torch.Tensor) -> torch.Tensor:
    """Block-diagonal W @ H^T.   quarot.py:42-70"""
    n, k = w.shape
    return torch.matmul(w.reshape(n, k // 128, 128), _hadamard128(w.dtype).T).reshape(n, k)


def quantize_rowwise(x: torch.Tensor):
    """int8_quant.py:28-31 with :20-21"""
    amax = x.abs().amax(dim=-1, keepdim=True)
    scale = (amax.float() / 127.0).clamp(min=1e-30)
    q = x.float().mul(1.0 / scale).round_().clamp_(-128.0, 127.0).to(torch.int8)
    return q, scale


def quantize_tensorwise(x: torch.Tensor):
    """int8_quant.py:23-26"""
    scale = (x.abs().max().float() / 127.0).clamp(min=1e-30)
    q = x.float().mul(1.0 / scale).round_().clamp_(-128.0, 127.0).to(torch.int8)
    return q, scale


@torch.no_grad()
def linear_w8a8(x: torch.Tensor, w_q: torch.Tensor, w_scale, bias, out_dtype: torch.dtype,
                hadamard: bool = False, return_parts: bool = False):
    """Forward of one quantised linear on CPU tensors.   int8_quant.py:741-754, :77-88, :107-119

    w_scale: python float / 1-element tensor (tensorwise) or [N,1] tensor (per channel).
    """
    x2 = x.reshape(-1, x.shape[-1])
    if hadamard:
        x2 = rotate_activation(x2)
    q, xs = quantize_rowwise(x2)
    acc = torch._int_mm(q, w_q.T)
    if isinstance(w_scale, torch.Tensor) and w_scale.numel() > 1:
        y = acc.float().mul_(xs).mul_(w_scale.reshape(1, -1)).to(out_dtype)
    else:
        ws = float(w_scale) if not isinstance(w_scale, torch.Tensor) else w_scale.reshape(())
        y = acc.float().mul_(ws * xs).to(out_dtype)
    if bias is not None:
        y = y + bias.to(out_dtype)
    if return_parts:
        return y, q, xs, acc
    return y


@torch.no_grad()
def linear_small_batch(x: torch.Tensor, w_q: torch.Tensor, w_scale, bias):
    """The M <= 16 branch: dequantised weights in the activation dtype, a float matmul.   int8_quant.py:756-760"""
    scale = w_scale.reshape(-1, 1) if isinstance(w_scale, torch.Tensor) and w_scale.numel() > 1 else w_scale
    w_float = (w_q.float() * scale).to(x.dtype)
    return torch.nn.functional.linear(x, w_float, bias.to(x.dtype) if bias is not None else None)


@torch.no_grad()
def lora_dynamic_add(y: torch.Tensor, x2: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor):
    """y + ((x @ A^T) @ B^T) with the adapter-dtype roundings.   int8_quant.py:763-774"""
    t = torch.nn.functional.linear(x2.to(lora_a.dtype), lora_a)
    return y + torch.nn.functional.linear(t, lora_b).to(y.dtype)


@torch.no_grad()
def stochastic_round(x: torch.Tensor, scale, u: torch.Tensor) -> torch.Tensor:
    """int8_quant.py:47-62 with the uniforms passed in instead of drawn at :55."""
    xs = x / scale
    fl = torch.floor(xs)
    up = (u < (xs - fl)).to(xs.dtype)
    return torch.clamp(fl + up, -128, 127).to(torch.int8)


@torch.no_grad()
def lora_merge(w_q: torch.Tensor, w_scale, up: torch.Tensor, down: torch.Tensor, lora_scale: float,
               u: torch.Tensor, hadamard: bool = False) -> torch.Tensor:
    """int8_quant.py:139-155 (delta), :291-316 (round, add, clamp)."""
    delta = torch.mm(up.float(), down.float()) * lora_scale
    if hadamard:
        delta = rotate_weight(delta)
    dq = stochastic_round(delta, w_scale, u)
    return torch.clamp(w_q.to(torch.int32) + dq.to(torch.int32), -128, 127).to(torch.int8)
