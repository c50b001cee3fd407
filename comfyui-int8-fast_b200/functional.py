"""Tensor-level wrappers over the C ABI (one call per kernel).

All functions take CUDA tensors on one sm_100 device, run on the current
stream of that device, never synchronise and never fall back to another
implementation.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _native as nat

HADAMARD_GROUP = 128


def _rows(t: Tensor) -> Tensor:
    """2-D view with unit inner stride (copies only if the layout forces it)."""
    if t.dim() != 2:
        raise ValueError(f"expected a 2-D tensor, got shape {tuple(t.shape)}")
    if t.stride(1) != 1 and t.shape[1] > 1:
        t = t.contiguous()
    if t.shape[0] > 1 and t.stride(0) < t.shape[1]:
        t = t.contiguous()
    return t


def _ld(t: Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 else max(t.shape[1], 1)


def _code(dtype: torch.dtype) -> int:
    try:
        return nat.DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; expected bf16, fp16 or fp32") from None


_WORKSPACE_BYTES: dict = {}


def _workspace_need(M: int, K: int) -> int:
    need = _WORKSPACE_BYTES.get((M, K))
    if need is None:
        need = _WORKSPACE_BYTES[(M, K)] = int(nat.load().i8f_linear_workspace_bytes(M, K))
    return need


def _wscale_arg(w_scale, device: torch.device, n_rows: int) -> tuple[Tensor, int]:
    """Device fp32 tensor + granularity code from a float, 0-d/1-element tensor or [N,1]/[N] tensor.

    A tensor scale must have exactly one entry or one per weight row: the C ABI cannot see the length, a shorter
    vector would be read past its end by the kernel and a longer one (a block-wise scale, say) would be applied
    with the wrong stride, where the reference's broadcast would raise.
    """
    if not isinstance(w_scale, Tensor):
        return torch.tensor([float(w_scale)], dtype=torch.float32, device=device), nat.WSCALE_TENSOR
    ws = w_scale
    if ws.dtype is not torch.float32 or ws.device != device:
        ws = ws.to(device=device, dtype=torch.float32)
    if ws.numel() == 1:
        return ws, nat.WSCALE_TENSOR        # one element: the pointer is all the library needs, whatever the shape
    if ws.numel() != n_rows:
        raise ValueError(f"weight scale has {ws.numel()} entries; expected 1 or one per weight row ({n_rows})")
    return (ws if ws.is_contiguous() else ws.contiguous()), nat.WSCALE_CHANNEL   # [N] and [N,1] share their memory layout


def _check_weight(w: Tensor, K: int) -> None:
    if w.dtype != torch.int8 or w.shape[1] != K:
        raise ValueError(f"weight must be int8 [N, {K}], got {w.dtype} {tuple(w.shape)}")


def quantize_rowwise(x: Tensor, hadamard: bool = False, return_rotated: bool = False):
    """Per-token absmax int8 quantisation, optionally after the 128-block Hadamard rotation.

    Returns (q int8 [M,K], scale fp32 [M,1]) and, if asked, the rotated activations in x's dtype.
    """
    nat.require_device(x.device)
    x = _rows(x)
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    scale = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    xrot = torch.empty_like(x, memory_format=torch.contiguous_format) if (hadamard and return_rotated) else None
    if xrot is not None and _ld(x) != K:
        x = x.contiguous()
    if M > 0:
        nat.check(nat.load().i8f_quant_rowwise(nat.ptr(x), _code(x.dtype), M, K, _ld(x), nat.ptr(q), K, nat.ptr(scale),
                                               1 if hadamard else 0, nat.ptr(xrot), nat.current_stream(x.device)),
                  "i8f_quant_rowwise")
    if return_rotated:
        return q, scale, (xrot if hadamard else x)
    return q, scale


def quantize_rowwise_ln_modulate(x: Tensor, shift: Tensor, scale: Tensor, eps: float = 1e-5, return_y: bool = False):
    """Per-token int8 of LayerNorm(x) * (1 + scale) + shift in one pass over x [M,K] (bf16 / fp16; shift, scale [K]).

    Returns (q, row_scale) and, if asked, the modulated activations y in x's dtype (the tensor the unfused model
    code would have handed to the linear)."""
    nat.require_device(x.device)
    x = _rows(x)
    M, K = x.shape
    shift = shift.reshape(-1).to(device=x.device, dtype=x.dtype).contiguous()
    scale = scale.reshape(-1).to(device=x.device, dtype=x.dtype).contiguous()
    if shift.numel() != K or scale.numel() != K:
        raise ValueError(f"shift and scale must have {K} elements")
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    rs = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    y = torch.empty((M, K), dtype=x.dtype, device=x.device) if return_y else None
    if M > 0:
        nat.check(nat.load().i8f_quant_rowwise_ln_modulate(nat.ptr(x), _code(x.dtype), M, K, _ld(x), nat.ptr(shift), nat.ptr(scale),
                                                           float(eps), nat.ptr(q), K, nat.ptr(rs), nat.ptr(y), K,
                                                           nat.current_stream(x.device)), "i8f_quant_rowwise_ln_modulate")
    return (q, rs, y) if return_y else (q, rs)


def quantize_rowwise_gelu(x_gelu: Tensor, x_plain: Tensor | None = None, return_y: bool = False):
    """Per-token int8 of the row [ x_plain | GELU_tanh(x_gelu) ] in one pass (x_plain may be None).  The two parts may
    be column slices of wider matrices (unit inner stride, 16-byte aligned)."""
    nat.require_device(x_gelu.device)
    if x_gelu.dim() != 2 or x_gelu.stride(1) != 1 or (x_plain is not None and (x_plain.dim() != 2 or x_plain.stride(1) != 1)):
        raise ValueError("inputs must be 2-D with unit inner stride")
    M, K1 = x_gelu.shape
    K0 = 0 if x_plain is None else x_plain.shape[1]
    if x_plain is not None and (x_plain.shape[0] != M or x_plain.dtype != x_gelu.dtype):
        raise ValueError("the two parts must have the same rows and dtype")
    q = torch.empty((M, K0 + K1), dtype=torch.int8, device=x_gelu.device)
    rs = torch.empty((M, 1), dtype=torch.float32, device=x_gelu.device)
    y = torch.empty((M, K0 + K1), dtype=x_gelu.dtype, device=x_gelu.device) if return_y else None
    if M > 0:
        nat.check(nat.load().i8f_quant_rowwise_gelu(nat.ptr(x_plain), K0, x_plain.stride(0) if x_plain is not None else 0,
                                                    nat.ptr(x_gelu), K1, x_gelu.stride(0), _code(x_gelu.dtype), M, nat.ptr(q),
                                                    K0 + K1, nat.ptr(rs), nat.ptr(y), K0 + K1,
                                                    nat.current_stream(x_gelu.device)), "i8f_quant_rowwise_gelu")
    return (q, rs, y) if return_y else (q, rs)


def rmsnorm_heads_(x: Tensor, eps: float = 1e-6) -> Tensor:
    """In place RMS norm of every 128-column block of every row of x [rows, cols] (per attention head)."""
    nat.require_device(x.device)
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be 2-D with unit inner stride")
    rows, cols = x.shape
    if rows and cols:
        nat.check(nat.load().i8f_rmsnorm_heads(nat.ptr(x), _code(x.dtype), rows, cols, x.stride(0), float(eps),
                                               nat.current_stream(x.device)), "i8f_rmsnorm_heads")
    return x


def quantize_weight_rows(w: Tensor, hadamard: bool = False):
    """Per-output-channel weight quantisation in fp32 (rotation, if any, also in fp32)."""
    nat.require_device(w.device)
    w = _rows(w)
    N, K = w.shape
    q = torch.empty((N, K), dtype=torch.int8, device=w.device)
    scale = torch.empty((N, 1), dtype=torch.float32, device=w.device)
    if N > 0:
        nat.check(nat.load().i8f_quant_weight_rows(nat.ptr(w), _code(w.dtype), N, K, _ld(w), nat.ptr(q), K, nat.ptr(scale),
                                                   1 if hadamard else 0, nat.current_stream(w.device)),
                  "i8f_quant_weight_rows")
    return q, scale


def quantize_tensorwise(w: Tensor, hadamard: bool = False):
    """One-scale quantisation of a whole matrix; returns (q int8, 0-d fp32 scale tensor)."""
    nat.require_device(w.device)
    w = _rows(w)
    N, K = w.shape
    q = torch.empty((N, K), dtype=torch.int8, device=w.device)
    scale = torch.empty((1,), dtype=torch.float32, device=w.device)
    scratch = torch.empty((1,), dtype=torch.float32, device=w.device)
    nat.check(nat.load().i8f_quant_tensorwise(nat.ptr(w), _code(w.dtype), N, K, _ld(w), nat.ptr(q), K, nat.ptr(scale),
                                              1 if hadamard else 0, nat.ptr(scratch), nat.current_stream(w.device)),
              "i8f_quant_tensorwise")
    return q, scale.reshape(())


def gemm_i8_i32(a: Tensor, w: Tensor) -> Tensor:
    """Exact int32 [M,N] = a int8 [M,K] @ w int8 [N,K]^T."""
    nat.require_device(a.device)
    a, w = _rows(a), _rows(w)
    (M, K), (N, K2) = a.shape, w.shape
    if K != K2 or a.dtype != torch.int8 or w.dtype != torch.int8:
        raise ValueError("gemm_i8_i32 expects int8 [M,K] and int8 [N,K]")
    acc = torch.empty((M, N), dtype=torch.int32, device=a.device)
    if M and N:
        nat.check(nat.load().i8f_gemm_i8_i32(nat.ptr(a), _ld(a), nat.ptr(w), _ld(w), nat.ptr(acc), N, M, N, K,
                                             nat.current_stream(a.device)), "i8f_gemm_i8_i32")
    return acc


def linear_w8a8(q: Tensor, q_scale: Tensor, w: Tensor, w_scale, bias: Tensor | None, out_dtype: torch.dtype,
                order: int = nat.EPI_PYTORCH, add_into: Tensor | None = None, out: Tensor | None = None) -> Tensor:
    """Dequantising int8 GEMM from pre-quantised activations.

    With `add_into` ([M,N], out_dtype, unit inner stride) the result is added onto what that tensor holds
    (out = round(round(result) + add_into)), in place, and `add_into` is returned.  With `out` ([M,N], out_dtype,
    unit inner stride, e.g. a row or column slice of a wider buffer) the result is written there.
    """
    nat.require_device(q.device)
    q, w = _rows(q), _rows(w)
    M, K = q.shape
    N = w.shape[0]
    _check_weight(w, K)
    ws, mode = _wscale_arg(w_scale, q.device, N)
    if bias is not None:
        bias = bias.to(q.device).contiguous()
    if add_into is not None:
        if add_into.shape != (M, N) or add_into.dtype != out_dtype or add_into.stride(1) != 1:
            raise ValueError("add_into must be [M,N] in out_dtype with unit inner stride")
        out, fn, what = add_into, nat.load().i8f_linear_w8a8_add, "i8f_linear_w8a8_add"
    else:
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=q.device)
        elif out.shape != (M, N) or out.dtype != out_dtype or out.stride(1) != 1:
            raise ValueError("out must be [M,N] in out_dtype with unit inner stride")
        fn, what = nat.load().i8f_linear_w8a8, "i8f_linear_w8a8"
    if M and N:
        nat.check(fn(nat.ptr(q), _ld(q), nat.ptr(q_scale.reshape(-1)), nat.ptr(w), _ld(w), nat.ptr(ws), mode, nat.ptr(bias),
                     _code(bias.dtype) if bias is not None else 0, nat.ptr(out), _code(out_dtype), _ld(out), M, N, K, order,
                     nat.current_stream(q.device)), what)
    return out


def linear_w8a8_gated_add_(residual: Tensor, gate: Tensor, q: Tensor, q_scale: Tensor, w: Tensor, w_scale,
                           bias: Tensor | None) -> Tensor:
    """In place residual <- round(residual + gate * round(dequant(q @ w^T) (+ bias))): the gated branch of a
    transformer block added to its residual stream inside the GEMM epilogue (torch.addcmul's arithmetic).
    residual [M,N] bf16 / fp16 with unit inner stride, gate [N]."""
    nat.require_device(q.device)
    q, w = _rows(q), _rows(w)
    M, K = q.shape
    N = w.shape[0]
    _check_weight(w, K)
    if residual.shape != (M, N) or residual.stride(1) != 1 or residual.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("residual must be [M,N] bf16 / fp16 with unit inner stride")
    gate = gate.reshape(-1).to(device=q.device, dtype=residual.dtype).contiguous()
    if gate.numel() != N:
        raise ValueError(f"gate must have {N} elements")
    ws, mode = _wscale_arg(w_scale, q.device, N)
    if bias is not None:
        bias = bias.to(q.device).contiguous()
    if M and N:
        nat.check(nat.load().i8f_linear_w8a8_gated_add(nat.ptr(q), _ld(q), nat.ptr(q_scale.reshape(-1)), nat.ptr(w), _ld(w),
                                                       nat.ptr(ws), mode, nat.ptr(bias), _code(bias.dtype) if bias is not None else 0,
                                                       nat.ptr(gate), nat.ptr(residual), _code(residual.dtype), _ld(residual),
                                                       M, N, K, nat.current_stream(q.device)), "i8f_linear_w8a8_gated_add")
    return residual


def linear_w8a8_lora(q: Tensor, q_scale: Tensor, w: Tensor, w_scale, bias: Tensor | None, t: Tensor, lora_b: Tensor,
                     out_dtype: torch.dtype, order: int = nat.EPI_PYTORCH) -> Tensor:
    """Dequantising int8 GEMM with the dynamic-LoRA term round(t @ lora_b^T) added inside the kernel."""
    nat.require_device(q.device)
    q, w = _rows(q), _rows(w)
    t, lora_b = _rows(t.to(out_dtype)), _rows(lora_b.to(out_dtype))
    M, K = q.shape
    N = w.shape[0]
    r = t.shape[1]
    _check_weight(w, K)
    ws, mode = _wscale_arg(w_scale, q.device, N)
    if bias is not None:
        bias = bias.to(q.device).contiguous()
    out = torch.empty((M, N), dtype=out_dtype, device=q.device)
    if M and N:
        nat.check(nat.load().i8f_linear_w8a8_lora(nat.ptr(q), _ld(q), nat.ptr(q_scale.reshape(-1)), nat.ptr(w), _ld(w),
                                                  nat.ptr(ws), mode, nat.ptr(bias), _code(bias.dtype) if bias is not None else 0,
                                                  nat.ptr(t), _ld(t), nat.ptr(lora_b), _ld(lora_b), r, nat.ptr(out),
                                                  _code(out_dtype), N, M, N, K, order, nat.current_stream(q.device)),
                  "i8f_linear_w8a8_lora")
    return out


def linear_w8a8_scatter(q: Tensor, q_scale: Tensor, w: Tensor, w_scale, bias: Tensor | None, dest_ptrs: list[int],
                        n_total: int, col_offset: int, out_dtype: torch.dtype, order: int = nat.EPI_PYTORCH) -> None:
    """Dequantising int8 GEMM whose [M, N] block is stored at column `col_offset` of every destination matrix
    [M, n_total] (row-major, contiguous) given by raw device pointers (this GPU's buffer and peers' mapped buffers)."""
    import ctypes
    nat.require_device(q.device)
    q, w = _rows(q), _rows(w)
    M, K = q.shape
    N = w.shape[0]
    _check_weight(w, K)
    ws, mode = _wscale_arg(w_scale, q.device, N)
    if bias is not None:
        bias = bias.to(q.device).contiguous()
    arr = (ctypes.c_void_p * len(dest_ptrs))(*[ctypes.c_void_p(int(p)) for p in dest_ptrs])
    nat.check(nat.load().i8f_linear_w8a8_scatter(nat.ptr(q), _ld(q), nat.ptr(q_scale.reshape(-1)), nat.ptr(w), _ld(w),
                                                 nat.ptr(ws), mode, nat.ptr(bias), _code(bias.dtype) if bias is not None else 0,
                                                 arr, len(dest_ptrs), n_total, n_total, col_offset, _code(out_dtype), M, N, K,
                                                 order, nat.current_stream(q.device)), "i8f_linear_w8a8_scatter")


def linear_forward(x: Tensor, w: Tensor, w_scale, bias: Tensor | None, out_dtype: torch.dtype, hadamard: bool = False,
                   order: int = nat.EPI_PYTORCH, workspace: Tensor | None = None) -> Tensor:
    """(rotate) -> quantise -> int8 GEMM -> dequant (+bias) through the single fused entry point."""
    device = x.device
    nat.require_device(device)
    x, w = _rows(x), _rows(w)
    M, K = x.shape
    N = w.shape[0]
    _check_weight(w, K)
    ws, mode = _wscale_arg(w_scale, device, N)
    if bias is not None and (bias.device != device or not bias.is_contiguous()):
        bias = bias.to(device).contiguous()
    out = torch.empty((M, N), dtype=out_dtype, device=device)
    if M == 0 or N == 0:
        return out
    need = _workspace_need(M, K)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty((need,), dtype=torch.uint8, device=device)
    rc = nat.load().i8f_linear_forward(x.data_ptr(), _code(x.dtype), _ld(x), 1 if hadamard else 0, w.data_ptr(), _ld(w),
                                       ws.data_ptr(), mode, bias.data_ptr() if bias is not None else None,
                                       _code(bias.dtype) if bias is not None else 0, out.data_ptr(), _code(out_dtype), N, M, N, K,
                                       order, workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                                       nat.current_stream(device))
    if rc:
        nat.check(rc, "i8f_linear_forward")
    return out


def linear_small_batch(x: Tensor, w: Tensor, w_scale, bias: Tensor | None) -> Tensor:
    """M <= 16 rows: y = x @ dt(w.float() * w_scale)^T + dt(bias) in x's dtype (bf16 or fp16), activations not
    quantised; one pass over the int8 weights instead of a dequantised copy of them."""
    nat.require_device(x.device)
    x, w = _rows(x), _rows(w)
    M, K = x.shape
    N = w.shape[0]
    _check_weight(w, K)
    ws, mode = _wscale_arg(w_scale, x.device, N)
    if bias is not None:
        bias = bias.to(x.device).contiguous()
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    if M == 0 or N == 0:
        return out
    nat.check(nat.load().i8f_linear_w8a16_small(nat.ptr(x), _code(x.dtype), _ld(x), nat.ptr(w), _ld(w), nat.ptr(ws), mode,
                                                nat.ptr(bias), _code(bias.dtype) if bias is not None else 0,
                                                nat.ptr(out), N, M, N, K, nat.current_stream(x.device)),
              "i8f_linear_w8a16_small")
    return out


def linear_forward_static(x: Tensor, w: Tensor, w_scale, bias: Tensor | None, out: Tensor, hadamard: bool = False,
                          order: int = nat.EPI_PYTORCH) -> Tensor:
    """linear_forward into a caller-supplied `out`, using the workspace built into the library.

    For callers that must not allocate device memory: the native call allocates nothing, and this
    wrapper allocates nothing either as long as `w_scale` is already a device tensor and `bias` is on
    the device.  Limits and sharing rules are those of i8f_linear_forward_static.
    """
    nat.require_device(x.device)
    if x.dim() != 2 or w.dim() != 2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError("x and w must be 2-D with unit inner stride (this wrapper never copies)")
    M, K = x.shape
    N = w.shape[0]
    _check_weight(w, K)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError(f"out must be [{M},{N}] with unit inner stride")
    if not isinstance(w_scale, Tensor) or w_scale.device != x.device or w_scale.dtype != torch.float32:
        raise ValueError("w_scale must be an fp32 tensor on the device (1 element, or N elements)")
    mode = nat.WSCALE_TENSOR if w_scale.numel() == 1 else nat.WSCALE_CHANNEL
    if mode == nat.WSCALE_CHANNEL and (w_scale.numel() != N or not w_scale.is_contiguous()):
        raise ValueError("per-channel w_scale must be contiguous with N elements")
    if bias is not None and (bias.device != x.device or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous device tensor")
    nat.check(nat.load().i8f_linear_forward_static(nat.ptr(x), _code(x.dtype), _ld(x), 1 if hadamard else 0, nat.ptr(w),
                                                   _ld(w), nat.ptr(w_scale), mode, nat.ptr(bias),
                                                   _code(bias.dtype) if bias is not None else 0, nat.ptr(out),
                                                   _code(out.dtype), _ld(out), M, N, K, order,
                                                   nat.current_stream(x.device)), "i8f_linear_forward_static")
    return out


def lora_down(x: Tensor, lora_a: Tensor) -> Tensor:
    """t [M,r] = x [M,K] @ lora_a [r,K]^T, rounded to x's dtype (bf16 or fp16)."""
    nat.require_device(x.device)
    x, lora_a = _rows(x), _rows(lora_a.to(x.dtype))
    M, K = x.shape
    r = lora_a.shape[0]
    t = torch.empty((M, r), dtype=x.dtype, device=x.device)
    if M and r:
        nat.check(nat.load().i8f_lora_down(nat.ptr(x), _ld(x), nat.ptr(lora_a), _ld(lora_a), nat.ptr(t), r, _code(x.dtype),
                                           M, K, r, nat.current_stream(x.device)), "i8f_lora_down")
    return t


def lora_up(t: Tensor, lora_b: Tensor) -> Tensor:
    """y [M,N] = round(t [M,r] @ lora_b [N,r]^T) in t's dtype."""
    nat.require_device(t.device)
    t, lora_b = _rows(t), _rows(lora_b.to(t.dtype))
    M, r = t.shape
    N = lora_b.shape[0]
    y = torch.empty((M, N), dtype=t.dtype, device=t.device)
    if M and N and r:
        nat.check(nat.load().i8f_lora_up(nat.ptr(t), _ld(t), nat.ptr(lora_b), _ld(lora_b), nat.ptr(y), N, _code(t.dtype),
                                         M, N, r, nat.current_stream(t.device)), "i8f_lora_up")
    elif M and N:
        y.zero_()
    return y


def lora_up_add_(y: Tensor, t: Tensor, lora_b: Tensor) -> Tensor:
    """In place y [M,N] += round(t [M,r] @ lora_b [N,r]^T) with the reference's two roundings."""
    nat.require_device(y.device)
    if y.dim() != 2 or y.stride(1) != 1:
        raise ValueError("y must be a 2-D tensor with unit inner stride")
    t, lora_b = _rows(t), _rows(lora_b.to(y.dtype))
    M, N = y.shape
    r = t.shape[1]
    if M and N and r:
        nat.check(nat.load().i8f_lora_up_add(nat.ptr(t), _ld(t), nat.ptr(lora_b), _ld(lora_b), nat.ptr(y), _ld(y),
                                             _code(y.dtype), M, N, r, nat.current_stream(y.device)), "i8f_lora_up_add")
    return y


def lora_merge_sr_(w: Tensor, w_scale, up: Tensor, down: Tensor, lora_scale: float, hadamard: bool = False,
                   uniforms: Tensor | None = None, seed: int = 0) -> Tensor:
    """In place stochastic-rounding merge of (up @ down) * lora_scale into int8 weights."""
    nat.require_device(w.device)
    if w.dtype != torch.int8 or w.dim() != 2 or w.stride(1) != 1:
        raise ValueError("w must be a 2-D int8 tensor with unit inner stride")
    N, K = w.shape
    if up.numel() == 0 or down.numel() == 0:   # rank 0: nothing to merge
        return w
    up = _rows(up.reshape(up.shape[0], -1).to(w.device))
    down = _rows(down.reshape(down.shape[0], -1).to(w.device))
    if up.dtype != down.dtype:
        down = down.to(up.dtype)
    r = up.shape[1]
    if up.shape[0] != N or down.shape != (r, K):
        raise ValueError(f"factor shapes {tuple(up.shape)} x {tuple(down.shape)} do not give [{N},{K}]")
    ws, mode = _wscale_arg(w_scale, w.device, N)
    if uniforms is not None:
        uniforms = uniforms.to(device=w.device, dtype=torch.float32).contiguous()
        if uniforms.shape != (N, K):
            raise ValueError("uniforms must have the shape of w")
    limit = lora_merge_max_rank(up.dtype, uniforms is not None)
    if r > limit:
        raise ValueError(f"rank {r} exceeds the one-pass limit {limit} of the fused merge for {up.dtype} factors; "
                         "build the delta and use stochastic_round instead")
    nat.check(nat.load().i8f_lora_merge_sr(nat.ptr(w), _ld(w), nat.ptr(ws), mode, nat.ptr(up), _ld(up), nat.ptr(down),
                                           _ld(down), _code(up.dtype), N, K, r, float(lora_scale), 1 if hadamard else 0,
                                           nat.ptr(uniforms), int(seed) & 0xFFFFFFFFFFFFFFFF,
                                           nat.current_stream(w.device)), "i8f_lora_merge_sr")
    return w


def gemm_plan(M: int, N: int, K: int, elem_bytes: int = 1, sm_count: int = 0) -> dict:
    """The tile configuration the GEMM entry points choose for this shape (host-side decision, no device needed):
    {'tile': (rows, cols), 'ctas_per_tile': n, 'k_split': 1 | 2}."""
    import ctypes
    out = [ctypes.c_int(0) for _ in range(4)]
    nat.check(nat.load().i8f_gemm_plan(M, N, K, elem_bytes, sm_count, *[ctypes.byref(o) for o in out]), "i8f_gemm_plan")
    return {"tile": (out[0].value, out[1].value), "ctas_per_tile": out[2].value, "k_split": out[3].value}


def lora_merge_max_rank(factor_dtype: torch.dtype, with_uniforms: bool = False) -> int:
    """Largest rank the fused merge kernel takes in one launch for factors of this dtype."""
    return int(nat.load().i8f_lora_merge_max_rank(_code(factor_dtype), 1 if with_uniforms else 0))


def peer_barrier(flag_ptrs: list[int], rank: int, epoch: int, device: torch.device, limit_cycles: int = 2_000_000_000) -> None:
    """Enqueue a meeting of the ranks on the current stream: publish `epoch` in every rank's flag array (raw device
    pointers, this rank's own included), wait -- bounded -- until all ranks have published it in this rank's array."""
    import ctypes
    nat.require_device(device)
    arr = (ctypes.c_void_p * len(flag_ptrs))(*[ctypes.c_void_p(int(p)) for p in flag_ptrs])
    nat.check(nat.load().i8f_peer_barrier(arr, len(flag_ptrs), rank, epoch & 0xFFFFFFFF, limit_cycles,
                                          nat.current_stream(device)), "i8f_peer_barrier")


def stochastic_round(delta: Tensor, w_scale, uniforms: Tensor | None = None, seed: int = 0) -> Tensor:
    """int8 = clamp(floor(delta/scale) + [u < frac]) for an fp32 [N,K] delta."""
    nat.require_device(delta.device)
    delta = _rows(delta.float())
    N, K = delta.shape
    ws, mode = _wscale_arg(w_scale, delta.device, N)
    out = torch.empty((N, K), dtype=torch.int8, device=delta.device)
    if uniforms is not None:
        uniforms = uniforms.to(device=delta.device, dtype=torch.float32).contiguous()
    if N and K:
        nat.check(nat.load().i8f_stochastic_round(nat.ptr(delta), _ld(delta), nat.ptr(ws), mode, nat.ptr(out), K, N, K,
                                                  nat.ptr(uniforms), int(seed) & 0xFFFFFFFFFFFFFFFF,
                                                  nat.current_stream(delta.device)), "i8f_stochastic_round")
    return out
