"""The forward entry points as `torch.library` custom operators.

The node pack's fast mode runs the diffusion model under `torch.compile`.  A ctypes call is opaque to the
tracer, so the two forwards the Linear layer uses are registered as custom ops with fake (meta) kernels:
dynamo / AOT-autograd then see them as single nodes with known output shapes and do not graph-break, while
the real kernels stay the hand-written CUDA ones (nothing is generated or traced through).

    torch.ops.int8_fast_b200.linear_forward(x, w, w_scale, bias, out_dtype, hadamard, order)
    torch.ops.int8_fast_b200.linear_lora_forward(x, w, w_scale, bias, lora_a, lora_b, out_dtype, hadamard,
                                                 rotated_lora_input, order)
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


def _register():
    """Registers both operators once per process (the package may be imported under more than one module name)."""
    ns = getattr(torch.ops, NAMESPACE)
    if hasattr(ns, "linear_forward") and hasattr(ns, "linear_lora_forward"):
        return ns.linear_forward, ns.linear_lora_forward
    op1 = torch.library.custom_op(f"{NAMESPACE}::linear_forward", mutates_args=())(_impl_linear_forward)
    op1.register_fake(_fake_linear_forward)
    op2 = torch.library.custom_op(f"{NAMESPACE}::linear_lora_forward", mutates_args=())(_impl_linear_lora_forward)
    op2.register_fake(_fake_linear_lora_forward)
    return op1, op2


linear_forward, linear_lora_forward = _register()
