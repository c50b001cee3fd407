"""ctypes binding of libi8f.so, the C ABI declared in include/i8f.h.

There is no fallback: if the shared library is missing or the device is not
sm_100, every call raises.  Build it with ``python build_native.py`` in this
directory (nvcc cross-compiles without a GPU).
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_uint64, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libi8f.so"

I8F_BF16, I8F_F16, I8F_F32 = 0, 1, 2
WSCALE_TENSOR, WSCALE_CHANNEL = 0, 1
EPI_PYTORCH, EPI_SINGLE = 0, 1
STATIC_WORKSPACE_BYTES = 16 * 1024 * 1024 + 256 * 1024

DTYPE_CODE = {torch.bfloat16: I8F_BF16, torch.float16: I8F_F16, torch.float32: I8F_F32}


class NativeLibraryError(RuntimeError):
    """libi8f.so is missing, stale, or reported an error."""


_PROTOTYPES = {
    "i8f_version": (c_int, []),
    "i8f_last_error": (c_char_p, []),
    "i8f_device_check": (c_int, []),
    "i8f_device_status": (c_int, [ctypes.POINTER(c_int), c_int]),
    "i8f_selftest_bounded_wait": (c_int, [c_int64, c_void_p]),
    "i8f_quant_rowwise": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int,
                                  c_void_p, c_void_p]),
    "i8f_quant_rowwise_ln_modulate": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_float, c_void_p,
                                              c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "i8f_quant_rowwise_gelu": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int64, c_void_p, c_int64,
                                       c_void_p, c_void_p, c_int64, c_void_p]),
    "i8f_rmsnorm_heads": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_float, c_void_p]),
    "i8f_quant_tensorwise": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int,
                                     c_void_p, c_void_p]),
    "i8f_quant_weight_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int,
                                      c_void_p]),
    "i8f_gemm_i8_i32": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                c_void_p]),
    "i8f_linear_w8a8": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int,
                                c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "i8f_linear_w8a8_add": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int,
                                    c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "i8f_linear_w8a8_gated_add": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int,
                                          c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "i8f_linear_w8a8_lora": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int,
                                     c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64, c_int64,
                                     c_int64, c_int, c_void_p]),
    "i8f_linear_w8a8_scatter": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int,
                                        ctypes.POINTER(c_void_p), c_int, c_int64, c_int64, c_int64, c_int, c_int64, c_int64,
                                        c_int64, c_int, c_void_p]),
    "i8f_launch_count": (ctypes.c_uint64, []),
    "i8f_gemm_plan": (c_int, [c_int64, c_int64, c_int64, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                              ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "i8f_linear_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "i8f_linear_forward": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int, c_void_p,
                                   c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p,
                                   c_size_t, c_void_p]),
    "i8f_linear_forward_static": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int, c_void_p,
                                          c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "i8f_linear_w8a16_small": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int,
                                       c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "i8f_lora_down": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64, c_int64,
                              c_int64, c_void_p]),
    "i8f_lora_up": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64, c_int64,
                            c_int64, c_void_p]),
    "i8f_lora_up_add": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64, c_int64,
                                c_int64, c_void_p]),
    "i8f_lora_merge_sr": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int,
                                  c_int64, c_int64, c_int64, c_float, c_int, c_void_p, c_uint64, c_void_p]),
    "i8f_lora_merge_max_rank": (c_int64, [c_int, c_int]),
    "i8f_peer_barrier": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, ctypes.c_uint32, c_int64, c_void_p]),
    "i8f_stochastic_round": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64,
                                     c_void_p, c_uint64, c_void_p]),
}

_lock = threading.Lock()
_lib = None
_device_ok: set[int] = set()


def exported_symbols() -> list[str]:
    """Names this binding expects the library to export."""
    return list(_PROTOTYPES)


def load() -> ctypes.CDLL:
    """Load libi8f.so once; raises NativeLibraryError when it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise NativeLibraryError(
                    f"{LIB_PATH} not found. This package has no CPU or Triton fallback; build the CUDA "
                    f"library with `python {LIB_PATH.parent / 'build_native.py'}`.")
            lib = ctypes.CDLL(str(LIB_PATH))
            for name, (res, args) in _PROTOTYPES.items():
                try:
                    fn = getattr(lib, name)
                except AttributeError as e:
                    raise NativeLibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from e
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def last_error() -> str:
    msg = load().i8f_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeLibraryError(f"{what} failed with code {rc}: {last_error()}")


@torch.compiler.disable
def require_device(device: torch.device) -> None:
    """Hard requirement: a CUDA device of compute capability 10.0."""
    if device.type != "cuda":
        raise NativeLibraryError(f"INT8 Fast (B200) kernels need CUDA tensors, got a tensor on {device}")
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _device_ok:
        return
    with torch.cuda.device(idx):
        check(load().i8f_device_check(), "i8f_device_check")
    _device_ok.add(idx)


def device_status(reset: bool = True) -> int:
    out = c_int(0)
    check(load().i8f_device_status(ctypes.byref(out), 1 if reset else 0), "i8f_device_status")
    return out.value


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def current_stream(device: torch.device) -> c_void_p:
    """The current CUDA stream of `device` as a raw handle (the library enqueues on it and nowhere else)."""
    if _raw_stream is not None:   # no Stream object is built: this call sits in front of every kernel launch
        return c_void_p(_raw_stream(device.index if device.index is not None else torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)
