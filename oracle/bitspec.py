"""Bit-level NumPy definition of the W8A8 linear hot path.  TEST INFRASTRUCTURE ONLY.

Every function states the arithmetic the CUDA kernels must reproduce and cites
the reference lines it follows (paths are relative to the reference project).
All floating point work is IEEE binary32 with round-to-nearest-even unless a
narrower type is named; no fused multiply-add is assumed anywhere.

Parity pin: the reference ships no tests or vectors; this file is pinned by
fixtures produced from the reference's own functions (see tests/golden/).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
HADAMARD_GROUP = 128
# 1/sqrt(128) as the reference materialises it:
#   bf16 activations: the matrix is built directly in bf16 (quarot.py:35-36
#   with dtype=x.dtype, int8_quant.py:743) -> bf16(1/sqrt(128)).
#   fp32 weights: built in fp32 (int8_quant.py:605) -> fp32(1)/fp32(sqrt(128)).
HADAMARD_NORM_BF16 = F32(0.08837890625)
HADAMARD_NORM_F16 = F32(np.float16(1.0) / np.float16(128 ** 0.5))
HADAMARD_NORM_F32 = F32(1.0) / F32(128 ** 0.5)
SCALE_FLOOR = F32(1e-30)  # clamp(min=1e-30), int8_quant.py:25, :30


# --------------------------------------------------------------------------
# bf16 helpers (NumPy has no bfloat16; values travel as uint16 bit patterns)
# --------------------------------------------------------------------------
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(F32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (NaN stays quiet NaN)."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    rounded = (u + np.uint32(0x7FFF) + lsb) >> np.uint32(16)
    nan = np.isnan(x)
    out = rounded.astype(np.uint16)
    if np.any(nan):
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def round_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 values rounded to bf16 precision, returned as fp32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round fp32 to 'bf16' / 'f16' / 'f32' precision, returned as fp32."""
    if dtype == "bf16":
        return round_bf16(x)
    if dtype == "f16":
        return np.asarray(x, dtype=F32).astype(np.float16).astype(F32)
    if dtype == "f32":
        return np.asarray(x, dtype=F32)
    raise ValueError(dtype)


# --------------------------------------------------------------------------
# Quantisation                                     int8_quant.py:20-31
# --------------------------------------------------------------------------
def quantize_with_scale(x: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """q = clamp(rint(x * (1/scale)), -128, 127)      int8_quant.py:20-21

    The reciprocal is a correctly rounded fp32 division, the product a plain
    fp32 multiply, the rounding is half-to-even.
    """
    inv = F32(1.0) / np.asarray(scale, dtype=F32)
    y = np.rint(np.asarray(x, dtype=F32) * inv)
    return np.clip(y, F32(-128.0), F32(127.0)).astype(np.int8)


def quantize_rowwise(x: np.ndarray):
    """Per-token absmax quantisation.                 int8_quant.py:28-31

    x: [M, K] fp32 holding the exact values of the bf16/fp16/fp32 input.
    Returns q int8 [M, K] and scale fp32 [M, 1] with
    scale = max(absmax / 127, 1e-30) (true fp32 division).
    """
    x = np.asarray(x, dtype=F32)
    absmax = np.max(np.abs(x), axis=-1, keepdims=True) if x.shape[-1] else np.zeros(x.shape[:-1] + (1,), F32)
    scale = np.maximum(absmax / F32(127.0), SCALE_FLOOR).astype(F32)
    return quantize_with_scale(x, scale), scale


def quantize_tensorwise(x: np.ndarray):
    """One scale for the whole tensor.                int8_quant.py:23-26"""
    x = np.asarray(x, dtype=F32)
    absmax = np.max(np.abs(x)) if x.size else F32(0)
    scale = np.maximum(F32(absmax) / F32(127.0), SCALE_FLOOR).astype(F32)
    return quantize_with_scale(x, scale), scale


def dequantize(q: np.ndarray, scale) -> np.ndarray:
    """int8_quant.py:33-34"""
    return q.astype(F32) * np.asarray(scale, dtype=F32)


# --------------------------------------------------------------------------
# Block Walsh-Hadamard rotation                     quarot.py:18-102
# --------------------------------------------------------------------------
def wht128_sums(x: np.ndarray) -> np.ndarray:
    """Un-normalised 128-point Walsh-Hadamard transform of every 128-block of
    the last axis, natural (Sylvester) order: out[j] = sum_i (-1)^popcount(i&j) x[i],
    which is x_block @ scipy.linalg.hadamard(128) (quarot.py:35, symmetric).

    The fp32 summation order is part of the definition: an in-place butterfly
    with strides 1, 2, 4, ..., 64 in that order, the element whose index has
    the stride bit clear receiving a+b and its partner a-b.
    """
    x = np.asarray(x, dtype=F32)
    K = x.shape[-1]
    if K % HADAMARD_GROUP:
        raise ValueError(f"features {K} not divisible by {HADAMARD_GROUP}")
    lead = x.shape[:-1]
    v = x.reshape(-1, K // HADAMARD_GROUP, HADAMARD_GROUP).copy()
    h = 1
    while h < HADAMARD_GROUP:
        w = v.reshape(v.shape[0], v.shape[1], HADAMARD_GROUP // (2 * h), 2, h)
        a = w[..., 0, :].copy()
        b = w[..., 1, :].copy()
        w[..., 0, :] = a + b
        w[..., 1, :] = a - b
        h *= 2
    return v.reshape(*lead, K)


def rotate_activation(x: np.ndarray, dtype: str = "bf16") -> np.ndarray:
    """x @ H per 128-block in the activation dtype.  quarot.py:73-102, int8_quant.py:741-744

    Canonical form: dtype_round(fp32 butterfly sums * dtype(1/sqrt(128))).
    The reference runs a library matmul whose accumulation order is backend
    specific; the two agree except for rare last-place differences.
    """
    norm = {"bf16": HADAMARD_NORM_BF16, "f16": HADAMARD_NORM_F16, "f32": HADAMARD_NORM_F32}[dtype]
    return round_to(wht128_sums(x) * norm, dtype)


def rotate_weight(w: np.ndarray) -> np.ndarray:
    """W @ H^T per 128-block of each row in fp32.   quarot.py:42-70, int8_quant.py:597-608"""
    return (wht128_sums(w) * HADAMARD_NORM_F32).astype(F32)


# --------------------------------------------------------------------------
# Integer matmul                                    int8_quant.py:80, :110
# --------------------------------------------------------------------------
def int_mm(a_q: np.ndarray, w_q: np.ndarray) -> np.ndarray:
    """Exact int32 = a_q [M,K] (int8) times w_q [N,K]^T (int8).

    Evaluated in float64 BLAS (every partial sum is an integer below 2^53, so
    the result is exact) and cast back.
    """
    acc = a_q.astype(np.float64) @ w_q.astype(np.float64).T
    return acc.astype(np.int64).astype(np.int32)


# --------------------------------------------------------------------------
# Dequantising epilogue                             int8_quant.py:84-88, :115-119
# --------------------------------------------------------------------------
def epilogue(acc: np.ndarray, x_scale: np.ndarray, w_scale, bias, out_dtype: str = "bf16",
             order: str = "pytorch") -> np.ndarray:
    """int32 accumulators -> output dtype (returned as fp32 values).

    order="pytorch" follows the reference's PyTorch path:
      scalar weight scale : out = rnd(f32(acc) * (ws * xs))          :84
      per-channel [N,1]   : out = rnd((f32(acc) * xs) * ws[n])       :115
      bias                : out = rnd(out + rnd(bias))               :86-87, :117-118
    order="single" rounds once: rnd(f32(acc) * (xs * ws) + f32(bias)), the
    form of the reference's fused GPU kernel (int8_fused_kernel.py:146-173).
    """
    accf = acc.astype(F32)  # int32 -> fp32, round-to-nearest-even
    xs = np.asarray(x_scale, dtype=F32).reshape(-1, 1)
    ws = np.asarray(w_scale, dtype=F32)
    per_channel = ws.size > 1
    if order == "pytorch":
        if per_channel:
            y = (accf * xs) * ws.reshape(1, -1)
        else:
            y = accf * (ws.reshape(()) * xs)
        y = round_to(y, out_dtype)
        if bias is not None:
            y = round_to(y + round_to(np.asarray(bias, dtype=F32), out_dtype).reshape(1, -1), out_dtype)
        return y
    if order == "single":
        total = xs * (ws.reshape(1, -1) if per_channel else ws.reshape(()))
        y = accf * total
        if bias is not None:
            y = y + np.asarray(bias, dtype=F32).reshape(1, -1)
        return round_to(y, out_dtype)
    raise ValueError(order)


def linear_w8a8(x: np.ndarray, w_q: np.ndarray, w_scale, bias=None, *, act_dtype: str = "bf16",
                hadamard: bool = False, order: str = "pytorch", return_parts: bool = False):
    """Whole forward of one quantised linear for M > 16.   int8_quant.py:741-754

    x holds the exact values of the activation tensor (already representable
    in act_dtype).  Output dtype equals act_dtype for bf16/f16, bf16 for f32
    (int8_quant.py:736).
    """
    out_dtype = act_dtype if act_dtype in ("bf16", "f16") else "bf16"
    xr = rotate_activation(x, act_dtype) if hadamard else np.asarray(x, dtype=F32)
    q, xs = quantize_rowwise(xr)
    acc = int_mm(q, w_q)
    y = epilogue(acc, xs, w_scale, bias, out_dtype, order)
    if return_parts:
        return y, q, xs, acc
    return y


# --------------------------------------------------------------------------
# Tiny-batch branch (M <= 16)                       int8_quant.py:756-760
# --------------------------------------------------------------------------
def linear_small_batch(x: np.ndarray, w_q: np.ndarray, w_scale, bias=None, dtype: str = "bf16") -> np.ndarray:
    """y = rnd(x @ rnd(w.float() * scale)^T + rnd(bias)): the weights are dequantised to the activation dtype
    (`dequantize(weight, w_scale).to(x.dtype)`, :757), the activations are NOT quantised, the matmul accumulates
    in wider precision and rounds once (F.linear, :760).  Accumulated here in float64."""
    scale = np.asarray(w_scale, dtype=F32)
    if scale.ndim == 1 and scale.size > 1:
        scale = scale.reshape(-1, 1)
    w_f = round_to(dequantize(w_q, scale), dtype)
    acc = np.asarray(x, dtype=F32).astype(np.float64) @ w_f.astype(np.float64).T
    if bias is not None:
        acc = acc + round_to(np.asarray(bias, dtype=F32), dtype).astype(np.float64)
    return round_to(acc.astype(F32), dtype)


# --------------------------------------------------------------------------
# Dynamic LoRA                                      int8_quant.py:763-774
# --------------------------------------------------------------------------
def lora_down(x: np.ndarray, lora_a: np.ndarray, dtype: str = "bf16") -> np.ndarray:
    """t = rnd(x [M,K] @ lora_a[r,K]^T) in the adapter dtype.   int8_quant.py:768"""
    t = np.asarray(x, dtype=F32).astype(np.float64) @ np.asarray(lora_a, dtype=F32).astype(np.float64).T
    return round_to(t.astype(F32), dtype)


def lora_up_add(y: np.ndarray, t: np.ndarray, lora_b: np.ndarray, dtype: str = "bf16") -> np.ndarray:
    """y + rnd(t [M,r] @ lora_b[N,r]^T), both roundings in the output dtype.   :769, :774"""
    d = np.asarray(t, dtype=F32).astype(np.float64) @ np.asarray(lora_b, dtype=F32).astype(np.float64).T
    return round_to(np.asarray(y, dtype=F32) + round_to(d.astype(F32), dtype), dtype)


# --------------------------------------------------------------------------
# Stochastic rounding and the LoRA merge            int8_quant.py:36-62, :274-323
# --------------------------------------------------------------------------
def stochastic_round(x: np.ndarray, scale, u: np.ndarray) -> np.ndarray:
    """int8 = clamp(floor(x/scale) + [u < frac]).     int8_quant.py:47-62

    u are the uniforms in [0,1) the reference draws with torch.rand at :55;
    they are an input here so both sides can be fed the same stream.
    """
    xs = np.asarray(x, dtype=F32) / np.asarray(scale, dtype=F32)
    fl = np.floor(xs)
    fr = xs - fl
    r = np.where(np.asarray(u, dtype=F32) < fr, fl + F32(1.0), fl)
    return np.clip(r, F32(-128.0), F32(127.0)).astype(np.int8)


def lora_delta(up: np.ndarray, down: np.ndarray, lora_scale) -> np.ndarray:
    """delta = (up [N,r] @ down [r,K]) * scale in fp32.   int8_quant.py:139-155, :291

    Summation order is part of the definition: j = 0..r-1 ascending, each step
    acc = fp32(acc + fp32(up[n,j] * down[j,k])), starting from 0.
    """
    up = np.asarray(up, dtype=F32)
    down = np.asarray(down, dtype=F32)
    acc = np.zeros((up.shape[0], down.shape[1]), dtype=F32)
    for j in range(up.shape[1]):
        acc = acc + up[:, j:j + 1] * down[j:j + 1, :]
    return acc * F32(lora_scale)


def lora_merge(w_q: np.ndarray, w_scale, up: np.ndarray, down: np.ndarray, lora_scale,
               u: np.ndarray, hadamard: bool = False) -> np.ndarray:
    """W' = clamp(int32(W) + SR(delta / w_scale)).     int8_quant.py:291-316

    w_scale: scalar or [N,1].  With hadamard the delta is rotated like the
    weights were (int8_quant.py:300-306).  Two clamps: the rounded delta first
    (:62), then the sum (:315).
    """
    d = lora_delta(up, down, lora_scale)
    if hadamard:
        d = rotate_weight(d)
    ws = np.asarray(w_scale, dtype=F32)
    ws = ws.reshape(-1, 1) if ws.size > 1 else ws.reshape(())
    dq = stochastic_round(d, ws, u).astype(np.int32)
    return np.clip(w_q.astype(np.int32) + dq, -128, 127).astype(np.int8)


# --------------------------------------------------------------------------
# Philox4x32-10 counter RNG (in-kernel uniform source of the merge kernel)
# --------------------------------------------------------------------------
_PHILOX_M0 = np.uint64(0xD2511F53)
_PHILOX_M1 = np.uint64(0xCD9E8D57)
_PHILOX_W0 = np.uint32(0x9E3779B9)
_PHILOX_W1 = np.uint32(0xBB67AE85)


def philox4x32_10(counter: np.ndarray, key: np.ndarray) -> np.ndarray:
    """Philox4x32-10 (Salmon et al., SC'11).  counter [...,4] u32, key [...,2] u32 -> [...,4] u32."""
    c = [np.asarray(counter[..., i], dtype=np.uint32).copy() for i in range(4)]
    k0 = np.asarray(key[..., 0], dtype=np.uint32).copy()
    k1 = np.asarray(key[..., 1], dtype=np.uint32).copy()
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = _PHILOX_M0 * c[0].astype(np.uint64)
        p1 = _PHILOX_M1 * c[2].astype(np.uint64)
        hi0 = (p0 >> np.uint64(32)).astype(np.uint32)
        lo0 = (p0 & mask).astype(np.uint32)
        hi1 = (p1 >> np.uint64(32)).astype(np.uint32)
        lo1 = (p1 & mask).astype(np.uint32)
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0 = (k0 + _PHILOX_W0).astype(np.uint32)
        k1 = (k1 + _PHILOX_W1).astype(np.uint32)
    return np.stack(c, axis=-1)


def philox_uniforms(seed: int, n_rows: int, n_cols: int) -> np.ndarray:
    """Uniforms in [0,1) for an [n_rows, n_cols] matrix.

    Element (n, k) uses Philox4x32-10 with counter = (n, k // 8, 0, 0) and key = (seed low 32 bits, seed high 32
    bits): 16-bit half (k % 8) % 2 (low half first) of word (k % 8) // 2; u = half * 2^-16, so u is exactly
    representable and below 1.  One generator block serves eight elements.
    """
    groups = (n_cols + 7) // 8
    ctr = np.zeros((n_rows, groups, 4), dtype=np.uint32)
    ctr[..., 0] = np.arange(n_rows, dtype=np.uint32)[:, None]
    ctr[..., 1] = np.arange(groups, dtype=np.uint32)[None, :]
    key = np.zeros((n_rows, groups, 2), dtype=np.uint32)
    key[..., 0] = np.uint32(seed & 0xFFFFFFFF)
    key[..., 1] = np.uint32((seed >> 32) & 0xFFFFFFFF)
    words = philox4x32_10(ctr, key)                                    # [n_rows, groups, 4]
    halves = np.stack([words & np.uint32(0xFFFF), words >> np.uint32(16)], axis=-1)   # [..., 4, 2]: low half first
    halves = halves.reshape(n_rows, groups * 8)[:, :n_cols]
    return halves.astype(F32) * F32(2.0 ** -16)


# --------------------------------------------------------------------------
# Quantiser prologues (no counterpart in the reference: the model's own element-wise steps in front of a
# quantised linear, folded into the activation quantiser; defined by comfyui-int8-fast_b200/csrc/quant_prologue.cu)
# --------------------------------------------------------------------------
def rowsum_tree(v: np.ndarray, threads: int = 128) -> np.ndarray:
    """Sum of every row of v [M, K] (K % 8 == 0) in the quantiser kernels' fixed order.

    A row belongs to `threads` threads (128: four warps; 32: one warp); thread t holds the 8-element vectors
    t, t + threads, ...  Order of the fp32 additions: the 8 elements of a vector left to right; a thread's vector
    sums in slot order; the 32 lanes of a warp as a balanced binary tree (neighbours first); the warps left to
    right.  Vectors past the end count as zeros.
    """
    v = np.asarray(v, dtype=F32)
    M, K = v.shape
    nvec = K // 8
    vpt = max(1, -(-nvec // threads))
    pad = np.zeros((M, vpt * threads * 8), dtype=F32)
    pad[:, :K] = v
    e = pad.reshape(M, vpt, threads, 8)
    s = e[..., 0] + e[..., 1]
    for j in range(2, 8):
        s = s + e[..., j]
    t = s[:, 0, :]
    for i in range(1, vpt):
        t = t + s[:, i, :]
    w = t.reshape(M, threads // 32, 32)
    while w.shape[-1] > 1:
        w = w[..., 0::2] + w[..., 1::2]
    w = w[..., 0]
    total = w[:, 0]
    for k in range(1, w.shape[1]):
        total = total + w[:, k]
    return total


def rowsum128(v: np.ndarray) -> np.ndarray:
    return rowsum_tree(v, 128)


def round_f64_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """float64 values rounded ONCE (nearest even) to 'bf16' / 'f16', returned as fp32.  For values in the normal
    range of the target type (what the tests produce); used where a kernel rounds an exact result directly to the
    16-bit type (a fused multiply-add in that type) instead of through fp32."""
    x = np.asarray(x, dtype=np.float64)
    if dtype == "f16":
        return x.astype(np.float16).astype(F32)
    if dtype != "bf16":
        raise ValueError(dtype)
    bits = np.ascontiguousarray(x).view(np.uint64)
    lsb = (bits >> np.uint64(45)) & np.uint64(1)
    rounded = ((bits + np.uint64((1 << 44) - 1) + lsb) >> np.uint64(45)) << np.uint64(45)
    out = rounded.view(np.float64)
    out = np.where(np.isfinite(x), out, x)
    return out.astype(F32)


def layernorm_modulate(x: np.ndarray, shift: np.ndarray, scale: np.ndarray, eps: float = 1e-5, dtype: str = "bf16") -> np.ndarray:
    """y = rnd(rnd((x - mean) * rstd) * rnd(1 + scale) + shift): LayerNorm without affine parameters followed by the
    adaptive modulation of a diffusion transformer block.  The row sums run in the order of `rowsum_tree`, with one
    warp per row for rows of at most 4096 elements and 128 threads per row above; the last step is ONE rounding of the
    exact value ln * gain + shift to the activation dtype (a fused multiply-add in that dtype)."""
    x = np.asarray(x, dtype=F32)
    threads = 32 if x.shape[1] <= 4096 else 128
    K = F32(x.shape[1])
    mean = (rowsum_tree(x, threads) / K).astype(F32)[:, None]
    d = (x - mean).astype(F32)
    var = (rowsum_tree(d * d, threads) / K).astype(F32)[:, None]
    rstd = (F32(1.0) / np.sqrt((var + F32(eps)).astype(F32))).astype(F32)
    ln = round_to(d * rstd, dtype)
    gain = round_to(F32(1.0) + np.asarray(scale, dtype=F32).reshape(1, -1), dtype)
    exact = ln.astype(np.float64) * gain.astype(np.float64) + np.asarray(shift, dtype=F32).reshape(1, -1).astype(np.float64)
    return round_f64_to(exact, dtype)


_GELU_C0 = F32(0.7978845608028654)
_GELU_C1 = F32(0.035677408136300125)
_NEG2_LOG2E = F32(-2.8853900817779268)
_EXP2_A = [F32(0.0013333558146428443), F32(0.009618129107628477), F32(0.05550410866482158), F32(0.2402265069591007),
           F32(0.6931471805599453)]


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """x * sigmoid(2u), u = x * (c0 + c1 x^2): the tanh form of GELU with the exponential written out in correctly
    rounded fp32 multiplications and additions (fp32 result, not yet rounded to the activation dtype)."""
    x = np.asarray(x, dtype=F32)
    with np.errstate(over="ignore", under="ignore"):
        u = x * ((x * x) * _GELU_C1 + _GELU_C0)
        t = np.clip(u * _NEG2_LOG2E, F32(-125.0), F32(125.0)).astype(F32)
        n = np.rint(t).astype(F32)
        f = (t - n).astype(F32)
        p = _EXP2_A[0] * f + _EXP2_A[1]
        for a in _EXP2_A[2:]:
            p = p * f + a
        p = (p * f + F32(1.0)).astype(F32)
        e = np.ldexp(p, n.astype(np.int32)).astype(F32)      # exponent arithmetic: exact, stays normal for |n| <= 125
        return (x * (F32(1.0) / (F32(1.0) + e))).astype(F32)


def quantize_rowwise_ln_modulate(x, shift, scale, eps: float = 1e-5, dtype: str = "bf16"):
    y = layernorm_modulate(x, shift, scale, eps, dtype)
    q, s = quantize_rowwise(y)
    return q, s, y


def quantize_rowwise_gelu(x_gelu, x_plain=None, dtype: str = "bf16"):
    y = round_to(gelu_tanh(x_gelu), dtype)
    if x_plain is not None:
        y = np.concatenate([np.asarray(x_plain, dtype=F32), y], axis=1)
    q, s = quantize_rowwise(y)
    return q, s, y


def rmsnorm_heads(x: np.ndarray, eps: float = 1e-6, dtype: str = "bf16") -> np.ndarray:
    """Per-head RMS norm: every 128-column block of every row, y = rnd(x * (1 / sqrt(sum(x^2) / 128 + eps))).
    Sum order: 16 lanes of 8 elements, squares summed left to right per lane, lanes as a balanced binary tree."""
    x = np.asarray(x, dtype=F32)
    rows, cols = x.shape
    e = (x * x).astype(F32).reshape(rows, cols // 128, 16, 8)
    s = e[..., 0] + e[..., 1]
    for j in range(2, 8):
        s = s + e[..., j]
    while s.shape[-1] > 1:
        s = s[..., 0::2] + s[..., 1::2]
    ms = (s * F32(0.0078125) + F32(eps)).astype(F32)
    rstd = (F32(1.0) / np.sqrt(ms)).astype(F32)
    return round_to(x.reshape(rows, cols // 128, 128) * rstd, dtype).reshape(rows, cols)


def gated_add(residual: np.ndarray, gate: np.ndarray, y: np.ndarray, dtype: str = "bf16") -> np.ndarray:
    """rnd(residual + gate[n] * y): a gated branch added to the residual stream (torch.addcmul's arithmetic).  All
    three operands hold values of the 16-bit type, so gate * y is exact in fp32 and the sum is rounded once."""
    prod = np.asarray(gate, dtype=F32).reshape(1, -1).astype(np.float64) * np.asarray(y, dtype=F32).astype(np.float64)
    return round_to((np.asarray(residual, dtype=F32).astype(np.float64) + prod).astype(F32), dtype)
