"""The forward entry points as `torch.library` custom operators.

The node pack's fast mode runs the diffusion model under `torch.compile`.  A ctypes call is opaque to the
tracer, so the two forwards the Linear layer uses are registered as custom ops with fake (meta) kernels:
dynamo / AOT-autograd then see them as single nodes with known output shapes and do not graph-break, while
the real kernels stay the hand-written CUDA ones (nothing is generated or traced through).

    torch.ops.int8_fast_b200.linear_forward(x, w, w_scale, bias, out_dtype, hadamard, order)
    torch.ops.int8_fast_b200.linear_lora_forward(x, w, w_scale, bias, lora_a, lora_b, out_dtype, hadamard,
                                                 rotated_lora_input, order)
    torch.ops.int8_fast_b200.small_batch_forward(x, w, w_scale, bias, lora_a, lora_b, hadamard)
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import functional as F

NAMESPACE = "int8_fast_b200"


def _impl_linear_forward(x: Tensor, w: Tensor, w_scale: Tensor, bias: Optional[Tensor], out_dtype: torch.dtype,
                   hadamard: bool, order: int) -> Tensor:
    """[M,K] activations -> [M,N]: (rotate) -> per-token int8 -> int8 GEMM -> dequant (+bias)."""
    with torch.cuda.device(x.device):      # the C ABI launches on the current device
        return F.linear_forward(x, w, w_scale, bias, out_dtype, hadamard=hadamard, order=order)


def _fake_linear_forward(x, w, w_scale, bias, out_dtype, hadamard, order):
    return x.new_empty((x.shape[0], w.shape[0]), dtype=out_dtype)


def _impl_linear_lora_forward(x: Tensor, w: Tensor, w_scale: Tensor, bias: Optional[Tensor], lora_a: Tensor, lora_b: Tensor,
                        out_dtype: torch.dtype, hadamard: bool, rotated_lora_input: bool, order: int) -> Tensor:
    """The same with a dynamic LoRA: t = x_lora @ lora_a^T, then the int8 GEMM with t @ lora_b^T fused in.
    `rotated_lora_input` feeds the rotated activations to the LoRA (the reference's behaviour when QuaRot is on)."""
    with torch.cuda.device(x.device):
        if hadamard and rotated_lora_input:
            q, qs, lora_in = F.quantize_rowwise(x, hadamard=True, return_rotated=True)
        else:
            q, qs = F.quantize_rowwise(x, hadamard=hadamard)
            lora_in = x
        return F.linear_w8a8_lora(q, qs, w, w_scale, bias, F.lora_down(lora_in, lora_a), lora_b, out_dtype, order=order)


def _fake_linear_lora_forward(x, w, w_scale, bias, lora_a, lora_b, out_dtype, hadamard, rotated_lora_input, order):
    return x.new_empty((x.shape[0], w.shape[0]), dtype=out_dtype)


def _impl_small_batch_forward(x: Tensor, w: Tensor, w_scale: Tensor, bias: Optional[Tensor], lora_a: Optional[Tensor],
                              lora_b: Optional[Tensor], hadamard: bool) -> Tensor:
    """M <= 16 tokens: the activations stay unquantised and meet the dequantised weights (int8_quant.py:756-760); the
    weights are dequantised inside the kernel, never materialised.  With `hadamard` the activations are rotated
    first (and, as in the reference, the rotated ones feed the dynamic LoRA)."""
    from . import quarot
    with torch.cuda.device(x.device):
        if hadamard:
            x = quarot.rotate_activation(x, None, quarot.GROUP_SIZE)
        if x.dtype in (torch.bfloat16, torch.float16) and x.shape[1] % 16 == 0:
            y = F.linear_small_batch(x, w, w_scale, bias)
        else:   # fp32 activations or an odd K: the reference's expression as it stands
            scale = w_scale.reshape(-1, 1) if w_scale.numel() > 1 else w_scale
            y = torch.nn.functional.linear(x, (w.float() * scale).to(x.dtype), bias.to(x.dtype) if bias is not None else None)
        if lora_a is not None and lora_b is not None:
            F.lora_up_add_(y, F.lora_down(x, lora_a), lora_b)
    return y


def _fake_small_batch_forward(x, w, w_scale, bias, lora_a, lora_b, hadamard):
    return x.new_empty((x.shape[0], w.shape[0]))


def _register():
    """Registers the operators once per process (the package may be imported under more than one module name)."""
    ns = getattr(torch.ops, NAMESPACE)
    if hasattr(ns, "linear_forward") and hasattr(ns, "linear_lora_forward") and hasattr(ns, "small_batch_forward"):
        return ns.linear_forward, ns.linear_lora_forward, ns.small_batch_forward
    op1 = torch.library.custom_op(f"{NAMESPACE}::linear_forward", mutates_args=())(_impl_linear_forward)
    op1.register_fake(_fake_linear_forward)
    op2 = torch.library.custom_op(f"{NAMESPACE}::linear_lora_forward", mutates_args=())(_impl_linear_lora_forward)
    op2.register_fake(_fake_linear_lora_forward)
    op3 = torch.library.custom_op(f"{NAMESPACE}::small_batch_forward", mutates_args=())(_impl_small_batch_forward)
    op3.register_fake(_fake_small_batch_forward)
    return op1, op2, op3


linear_forward, linear_lora_forward, small_batch_forward = _register()
