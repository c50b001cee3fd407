"""Property tests over ragged shapes: every M >= 1, K a multiple of 16 (the TMA pitch rule), any N, both weight-scale
granularities, with and without bias / rotation -- int8, scales and int32 stay bit-exact, outputs match the oracle."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from oracle import bitspec as bs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
COMMON = dict(max_examples=30, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])


def to_np(t):
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


@settings(**COMMON)
@given(M=st.integers(1, 300), kb=st.integers(1, 40), N=st.integers(1, 600), seed=st.integers(0, 2 ** 16))
def test_gemm_any_shape(cuda_pkg, M, kb, N, seed):
    K = 16 * kb
    gen = torch.Generator().manual_seed(seed)
    a = torch.randint(-128, 128, (M, K), generator=gen, dtype=torch.int8)
    w = torch.randint(-128, 128, (N, K), generator=gen, dtype=torch.int8)
    got = cuda_pkg.functional.gemm_i8_i32(a.to(DEV), w.to(DEV))
    assert np.array_equal(to_np(got), bs.int_mm(a.numpy(), w.numpy()))


@settings(**COMMON)
@given(M=st.integers(1, 200), kv=st.integers(1, 96), had=st.booleans(), dt=st.sampled_from(["bf16", "f16"]),
       seed=st.integers(0, 2 ** 16))
def test_quant_any_shape(cuda_pkg, M, kv, had, dt, seed):
    K = 128 * ((kv + 15) // 16) if had else 8 * kv
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    x = cuda_pkg.workloads.activation(M, K, seed=seed, dtype=tdt)
    xr = bs.rotate_activation(to_np(x), dt) if had else to_np(x)
    q_want, s_want = bs.quantize_rowwise(xr)
    q, s = cuda_pkg.functional.quantize_rowwise(x.to(DEV), hadamard=had)
    assert np.array_equal(to_np(q), q_want) and np.array_equal(to_np(s), s_want)


@settings(**COMMON)
@given(M=st.integers(1, 280), kb=st.integers(1, 24), N=st.integers(1, 400), per_ch=st.booleans(), use_bias=st.booleans(),
       order=st.integers(0, 1), seed=st.integers(0, 2 ** 16))
def test_linear_any_shape(cuda_pkg, M, kb, N, per_ch, use_bias, order, seed):
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    K = 16 * kb
    x = wl.activation(M, K, seed=seed)
    w = wl.weight_fp32(N, K, seed=seed).numpy()
    wq, ws = bs.quantize_rowwise(w) if per_ch else bs.quantize_tensorwise(w)
    b = wl.bias_fp32(N, seed=seed) if use_bias else None
    want = bs.linear_w8a8(to_np(x), wq, ws, None if b is None else b.numpy(), order="pytorch" if order == 0 else "single")
    y = F.linear_forward(x.to(DEV), torch.from_numpy(wq).to(DEV), torch.from_numpy(np.asarray(ws, dtype=np.float32)).to(DEV),
                         None if b is None else b.to(DEV), torch.bfloat16, order=order)
    assert np.array_equal(to_np(y), want)


@settings(**COMMON)
@given(M=st.integers(1, 16), kb=st.integers(1, 70), N=st.integers(1, 300), per_ch=st.booleans(), use_bias=st.booleans(),
       dt=st.sampled_from(["bf16", "f16"]), seed=st.integers(0, 2 ** 16))
def test_small_batch_linear_any_shape(cuda_pkg, M, kb, N, per_ch, use_bias, dt, seed):
    """The tiny-batch branch over ragged K (any multiple of 16: full chunks, partial chunks, fewer chunks than warps),
    any N (partial feature blocks) and every token count up to 16."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    K = 16 * kb
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    x = wl.activation(M, K, seed=seed, dtype=tdt)
    w = wl.weight_fp32(N, K, seed=seed).numpy()
    wq, ws = bs.quantize_rowwise(w) if per_ch else bs.quantize_tensorwise(w)
    b = wl.bias_fp32(N, seed=seed) if use_bias else None
    want = bs.linear_small_batch(to_np(x), wq, ws, None if b is None else b.numpy(), dt)
    y = F.linear_small_batch(x.to(DEV), torch.from_numpy(wq).to(DEV), torch.from_numpy(np.asarray(ws, dtype=np.float32)).to(DEV),
                             None if b is None else b.to(DEV))
    got = to_np(y)
    scale = float(np.sqrt(np.mean(want.astype(np.float64) ** 2))) + 1e-30
    step = np.abs(want) * (2.0 ** -7 if dt == "bf16" else 2.0 ** -10) + 1e-4 * scale
    assert np.all(np.abs(got - want) <= step)


def test_status_word_is_clean_after_the_property_runs(cuda_pkg):
    torch.cuda.synchronize()
    assert cuda_pkg._native.device_status() == 0
