"""The C ABI: header, shared library and ctypes binding agree (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "i8f.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(i8f_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_symbols()
    for must in ("i8f_quant_rowwise", "i8f_gemm_i8_i32", "i8f_linear_w8a8", "i8f_linear_forward",
                 "i8f_lora_down", "i8f_lora_up_add", "i8f_lora_merge_sr", "i8f_last_error", "i8f_version"):
        assert must in names


def test_library_builds_and_exports_every_declared_symbol():
    import __graft_entry__ as g
    g.build()
    lib = ctypes.CDLL(str(g.PKG_DIR / "libi8f.so"))
    for name in declared_symbols():
        assert hasattr(lib, name), f"libi8f.so does not export {name}"
    lib.i8f_version.restype = ctypes.c_int
    m = re.search(r"#define\s+I8F_VERSION\s+(\d+)", HEADER.read_text())
    assert lib.i8f_version() == int(m.group(1))


def test_binding_covers_the_header(pkg):
    assert sorted(pkg._native.exported_symbols()) == declared_symbols()
    pkg._native.load()


def test_argument_errors_are_reported_not_raised_as_faults(pkg):
    """Host-side validation runs before any CUDA call, so it can be exercised without a GPU."""
    nat = pkg._native
    lib = nat.load()
    rc = lib.i8f_quant_rowwise(None, 7, 4, 64, 64, None, 64, None, 0, None, None)
    assert rc == -1 and "dtype" in nat.last_error()
    rc = lib.i8f_quant_rowwise(ctypes.c_void_p(16), nat.I8F_BF16, 4, 60, 64, ctypes.c_void_p(16), 64,
                               ctypes.c_void_p(16), 0, None, None)
    assert rc == -3 and "multiple of 8" in nat.last_error()
    rc = lib.i8f_quant_rowwise(ctypes.c_void_p(16), nat.I8F_BF16, 4, 64, 64, ctypes.c_void_p(16), 64,
                               ctypes.c_void_p(16), 1, None, None)
    assert rc == -3 and "128" in nat.last_error()
    rc = lib.i8f_gemm_i8_i32(ctypes.c_void_p(16), 40, ctypes.c_void_p(16), 40, ctypes.c_void_p(16), 8, 4, 8, 40, None)
    assert rc == -2 and "16 bytes" in nat.last_error()
    rc = lib.i8f_linear_forward(ctypes.c_void_p(16), nat.I8F_BF16, 64, 0, ctypes.c_void_p(16), 64, ctypes.c_void_p(16),
                                0, None, 0, ctypes.c_void_p(16), nat.I8F_BF16, 8, 4, 8, 64, 0, None, 0, None)
    assert rc == -6 and "workspace" in nat.last_error()
    assert lib.i8f_linear_workspace_bytes(4, 64) == 256 + 256


def test_gemm_tile_plan_is_a_host_decision_and_pinned(pkg):
    """Which tiles a GEMM runs on, and whether two CTAs of a cluster split a tile's K range, is decided on the host
    from the shape and the SM count alone: pinned here for the benchmark shapes on 148 SMs."""
    plan = pkg.functional.gemm_plan
    # the headline linear and the DiT's image-stream linears: full-rate 256 x 256 tiles of a CTA pair, never split
    assert plan(4096, 12288, 4096, sm_count=148) == {"tile": (256, 256), "ctas_per_tile": 2, "k_split": 1}
    assert plan(4608, 24576, 4096, sm_count=148)["tile"] == (256, 256)
    # configuration 0 of the baseline (96 CTAs of 128 x 64 fill most of the GPU: the split would not pay)
    assert plan(256, 3072, 3072, sm_count=148) == {"tile": (128, 64), "ctas_per_tile": 1, "k_split": 1}
    # the DiT's text-stream linears at K = 4096: 128 CTAs already
    assert plan(512, 4096, 4096, sm_count=148) == {"tile": (128, 128), "ctas_per_tile": 1, "k_split": 1}
    # few tiles and a long K: two CTAs per tile
    assert plan(64, 4096, 4096, sm_count=148) == {"tile": (128, 64), "ctas_per_tile": 2, "k_split": 2}
    assert plan(17, 4096, 4096, sm_count=148)["k_split"] == 2
    assert plan(512, 4096, 12288, sm_count=148) == {"tile": (128, 256), "ctas_per_tile": 2, "k_split": 2}
    # the LoRA down projection (16-bit operands, N = rank): 64 tiles -> 128 CTAs
    assert plan(8192, 64, 4096, elem_bytes=2, sm_count=148) == {"tile": (128, 64), "ctas_per_tile": 2, "k_split": 2}
    assert plan(4608, 16, 4096, elem_bytes=2, sm_count=148) == {"tile": (128, 32), "ctas_per_tile": 2, "k_split": 2}
    # a short K never splits; a smaller GPU changes the decision
    assert plan(64, 4096, 512, sm_count=148)["k_split"] == 1
    assert plan(64, 4096, 4096, sm_count=64)["k_split"] == 1
    with pytest.raises(pkg._native.NativeLibraryError):
        plan(0, 64, 64)


def test_cpu_tensors_are_rejected(pkg):
    import torch
    with pytest.raises(pkg._native.NativeLibraryError, match="CUDA"):
        pkg.functional.quantize_rowwise(torch.zeros(4, 64, dtype=torch.bfloat16))
