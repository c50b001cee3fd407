"""Parity of every CUDA kernel with the CPU oracle, through the C ABI, on a B200.

Bars: int8 activations / weights, fp32 scales and int32 accumulators are
bit-exact; bf16 / fp16 outputs are within 1e-2 * RMS(reference output) in
max-abs (they are in fact bit-exact for the plain linear, where no
accumulation order is involved after the exact integer GEMM).
"""
import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import bitspec as bs

from conftest import GOLDEN

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2
NAME = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}


def rms(a):
    return float(np.sqrt(np.mean(np.asarray(a, dtype=np.float64) ** 2)))


def to_np(t):
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def dev_ws(ws):
    return torch.from_numpy(np.asarray(ws, dtype=np.float32)).to(DEV)


@pytest.fixture(autouse=True)
def _status_clean(cuda_pkg):
    yield
    torch.cuda.synchronize()
    assert cuda_pkg._native.device_status() == 0, "a bounded device-side wait ran out"


# ------------------------------------------------------------------ K1 quant
@pytest.mark.parametrize("M,K,had,dt", [
    (200, 512, False, torch.bfloat16), (256, 3072, False, torch.bfloat16), (64, 4096, True, torch.bfloat16),
    (33, 12288, True, torch.bfloat16), (70, 1024, False, torch.float16), (70, 1024, True, torch.float16),
    (70, 1024, True, torch.float32), (5, 16384, False, torch.bfloat16), (300, 128, True, torch.bfloat16),
    (1, 8, False, torch.bfloat16), (17, 24, False, torch.float32), (3, 32768, True, torch.bfloat16),
])
def test_quant_rowwise_bit_exact(cuda_pkg, M, K, had, dt):
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(M, K, seed=3, dtype=dt)
    xr = bs.rotate_activation(to_np(x), NAME[dt]) if had else to_np(x)
    q_want, s_want = bs.quantize_rowwise(xr)
    q, s, xrot = F.quantize_rowwise(x.to(DEV), hadamard=had, return_rotated=True)
    assert np.array_equal(to_np(q), q_want)
    assert np.array_equal(to_np(s), s_want)
    if had:
        assert np.array_equal(to_np(xrot), xr)


@pytest.mark.parametrize("M,K,dt", [
    (2051, 4096, torch.bfloat16), (2048, 8192, torch.float16), (4099, 4096, torch.float16), (2300, 8192, torch.bfloat16),
])
def test_quant_rowwise_rotated_many_rows_bit_exact(cuda_pkg, M, K, dt):
    """Rotated rows of 4096 / 8192 elements, thousands of rows (several waves of CTAs), row counts that are no multiple
    of the rows per CTA, a pitched input."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(M, K, seed=11, dtype=dt)
    xr = bs.rotate_activation(to_np(x), NAME[dt])
    q_want, s_want = bs.quantize_rowwise(xr)
    q, s = F.quantize_rowwise(x.to(DEV), hadamard=True)
    assert np.array_equal(to_np(q), q_want)
    assert np.array_equal(to_np(s), s_want)
    wide = torch.zeros(M, K + 64, dtype=dt, device=DEV)
    wide[:, 32:32 + K] = x.to(DEV)
    q2, s2 = F.quantize_rowwise(wide[:, 32:32 + K], hadamard=True)
    assert torch.equal(q2, q) and torch.equal(s2, s)
    # asking for the rotated copy as well changes nothing
    q3, s3, _ = F.quantize_rowwise(x.to(DEV), hadamard=True, return_rotated=True)
    assert torch.equal(q3, q) and torch.equal(s3, s)


def test_quant_edge_rows(cuda_pkg):
    """All-zero rows take the 1e-30 floor; a strided (pitched) input is read in place."""
    F = cuda_pkg.functional
    x = torch.zeros(6, 256, dtype=torch.bfloat16)
    x[1, 5] = -3.0
    x[2] = 1e-38
    x[3, 200] = 65280.0
    q_want, s_want = bs.quantize_rowwise(to_np(x))
    q, s = F.quantize_rowwise(x.to(DEV))
    assert np.array_equal(to_np(q), q_want) and np.array_equal(to_np(s), s_want)
    assert to_np(s)[0, 0] == np.float32(1e-30)
    big = torch.randn(10, 512, dtype=torch.bfloat16, generator=torch.Generator().manual_seed(1)).to(DEV)
    view = big[:, 128:384]
    q, s = F.quantize_rowwise(view)
    q_want, s_want = bs.quantize_rowwise(to_np(view))
    assert np.array_equal(to_np(q), q_want) and np.array_equal(to_np(s), s_want)
    q, s = F.quantize_rowwise(torch.empty(0, 64, dtype=torch.bfloat16, device=DEV))
    assert q.shape == (0, 64) and s.shape == (0, 1)


def test_quant_golden_fixture(cuda_pkg, golden):
    g = golden("linear_small.npz")
    x = torch.from_numpy(g["x_bits"].view(np.int16)).view(torch.bfloat16).to(DEV)
    q, s = cuda_pkg.functional.quantize_rowwise(x)
    assert np.array_equal(to_np(q), g["xq"]) and np.array_equal(to_np(s), g["xs"])


@pytest.mark.parametrize("N,K,had,dt", [(300, 512, False, torch.float32), (300, 512, True, torch.float32),
                                        (128, 4096, True, torch.bfloat16), (77, 1152, False, torch.float16)])
def test_weight_quant_bit_exact(cuda_pkg, N, K, had, dt):
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    w = wl.weight_fp32(N, K, seed=13).to(dt)
    wr = bs.rotate_weight(to_np(w)) if had else to_np(w)
    q_want, s_want = bs.quantize_rowwise(wr)
    q, s = F.quantize_weight_rows(w.to(DEV), hadamard=had)
    assert np.array_equal(to_np(q), q_want) and np.array_equal(to_np(s), s_want)
    qt_want, st_want = bs.quantize_tensorwise(wr)
    qt, st = F.quantize_tensorwise(w.to(DEV), hadamard=had)
    assert np.array_equal(to_np(qt), qt_want) and float(st.item()) == float(st_want)


# ------------------------------------------------------------------ K2 GEMM
@pytest.mark.parametrize("M,N,K", [
    (128, 256, 128), (128, 256, 4096), (256, 512, 1024), (1024, 2048, 512), (200, 328, 528), (17, 40, 16),
    (1, 8, 64), (129, 100, 144), (300, 64, 272), (16, 16, 16), (4608, 300, 192), (2048, 12288, 256),
    # few tiles and a long K: two CTAs of a cluster share each tile's K range (an odd number of K slabs included)
    (64, 4096, 4096), (17, 4104, 4224), (512, 4096, 12288), (130, 520, 8192),
])
def test_gemm_int32_bit_exact(cuda_pkg, M, N, K):
    gen = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    a = torch.randint(-128, 128, (M, K), generator=gen, dtype=torch.int8)
    w = torch.randint(-128, 128, (N, K), generator=gen, dtype=torch.int8)
    want = bs.int_mm(a.numpy(), w.numpy())
    got = cuda_pkg.functional.gemm_i8_i32(a.to(DEV), w.to(DEV))
    assert np.array_equal(to_np(got), want)


def test_gemm_extreme_values_do_not_saturate(cuda_pkg):
    """-128 * -128 * K stays exact (the MMA must not saturate)."""
    K = 8192
    a = torch.full((130, K), -128, dtype=torch.int8)
    w = torch.full((70, K), -128, dtype=torch.int8)
    w[1] = 127
    got = to_np(cuda_pkg.functional.gemm_i8_i32(a.to(DEV), w.to(DEV)))
    assert np.all(got[:, 0] == 128 * 128 * K) and np.all(got[:, 1] == -128 * 127 * K)


def test_gemm_linearity_at_full_size(cuda_pkg):
    """Size-independent property at the benchmark shape: (A1 + A2) W^T == A1 W^T + A2 W^T, and a
    column checksum against int64 arithmetic."""
    M, K, N = 4096, 4096, 12288
    gen = torch.Generator(device=DEV).manual_seed(5)
    a1 = torch.randint(-60, 61, (M, K), generator=gen, dtype=torch.int8, device=DEV)
    a2 = torch.randint(-60, 61, (M, K), generator=gen, dtype=torch.int8, device=DEV)
    w = torch.randint(-128, 128, (N, K), generator=gen, dtype=torch.int8, device=DEV)
    F = cuda_pkg.functional
    c1, c2, c12 = F.gemm_i8_i32(a1, w), F.gemm_i8_i32(a2, w), F.gemm_i8_i32(a1 + a2, w)
    assert torch.equal(c1 + c2, c12)
    # sum over rows of C equals (sum over rows of A) W^T, computed in float64 on the device
    want = a1.to(torch.float64).sum(0) @ w.to(torch.float64).T
    assert torch.equal(c1.to(torch.float64).sum(0), want)


# ------------------------------------------------------ K2 + epilogue (linear)
@pytest.mark.parametrize("M,K,N,per_ch,use_bias,had,order,dt", [
    (256, 3072, 3072, True, True, False, 0, torch.bfloat16),
    (200, 512, 328, False, True, False, 0, torch.bfloat16),
    (200, 512, 328, True, False, True, 0, torch.bfloat16),
    (130, 256, 520, False, True, True, 1, torch.bfloat16),
    (130, 256, 520, True, True, False, 1, torch.bfloat16),
    (64, 384, 200, True, True, False, 0, torch.float16),
    (64, 4096, 1000, True, True, True, 0, torch.bfloat16), (40, 8192, 520, False, True, False, 1, torch.float16),
    (17, 128, 72, False, False, False, 0, torch.float16),
    (90, 640, 77, True, True, False, 0, torch.bfloat16),     # N not a multiple of 8: scalar store path
])
def test_linear_forward_matches_oracle(cuda_pkg, M, K, N, per_ch, use_bias, had, order, dt):
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(M, K, seed=5, dtype=dt)
    w = wl.weight_fp32(N, K, seed=5)
    b = wl.bias_fp32(N, seed=5) if use_bias else None
    wn = bs.rotate_weight(w.numpy()) if had else w.numpy()
    wq, ws = bs.quantize_rowwise(wn) if per_ch else bs.quantize_tensorwise(wn)
    want = bs.linear_w8a8(to_np(x), wq, ws, None if b is None else b.numpy(), act_dtype=NAME[dt], hadamard=had,
                          order="pytorch" if order == 0 else "single")
    y = F.linear_forward(x.to(DEV), torch.from_numpy(wq).to(DEV), dev_ws(ws), None if b is None else b.to(DEV), dt,
                         hadamard=had, order=order)
    got = to_np(y)
    assert np.max(np.abs(got - want)) <= TOL * rms(want)
    assert np.array_equal(got, want), "the epilogue is deterministic fp32 arithmetic and should be bit-exact"


def test_linear_golden_fixtures(cuda_pkg, golden):
    """Outputs recorded from the reference's int8_forward_dynamic[_per_row] on CPU."""
    F = cuda_pkg.functional
    g = golden("linear_small.npz")
    x = torch.from_numpy(g["x_bits"].view(np.int16)).view(torch.bfloat16).to(DEV)
    b = torch.from_numpy(g["bias"]).to(DEV)
    acc = F.gemm_i8_i32(torch.from_numpy(g["xq"]).to(DEV), torch.from_numpy(g["wq_c"]).to(DEV))
    assert np.array_equal(to_np(acc), g["acc_c"])
    y = F.linear_forward(x, torch.from_numpy(g["wq_c"]).to(DEV), dev_ws(g["ws_c"]), b, torch.bfloat16)
    assert np.array_equal(y.cpu().view(torch.int16).numpy().view(np.uint16), g["y_c_bits"])
    y = F.linear_forward(x, torch.from_numpy(g["wq_c"]).to(DEV), dev_ws(g["ws_c"]), None, torch.bfloat16)
    assert np.array_equal(y.cpu().view(torch.int16).numpy().view(np.uint16), g["y_c_nb_bits"])
    y = F.linear_forward(x, torch.from_numpy(g["wq_t"]).to(DEV), float(g["ws_t"]), b, torch.bfloat16)
    assert np.array_equal(y.cpu().view(torch.int16).numpy().view(np.uint16), g["y_t_bits"])
    y = F.linear_forward(x.half(), torch.from_numpy(g["wq_t"]).to(DEV), float(g["ws_t"]), b, torch.float16)
    assert np.array_equal(y.cpu().view(torch.int16).numpy().view(np.uint16), g["y_t_f16_bits"])


def test_config0_digests_on_gpu(cuda_pkg):
    """The CPU-runnable benchmark configuration at full size against the reference's recorded digests."""
    ref = json.loads((GOLDEN / "config0_digests.json").read_text())
    M, K, N = ref["shape"]
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(M, K, seed=ref["seed"]).to(DEV)
    w = wl.weight_fp32(N, K, seed=ref["seed"]).to(DEV)
    b = wl.bias_fp32(N, seed=ref["seed"]).to(DEV)
    sha = lambda t: hashlib.sha256(np.ascontiguousarray(t.cpu().numpy()).tobytes()).hexdigest()  # noqa: E731
    wq, ws = F.quantize_weight_rows(w)
    assert sha(wq) == ref["wq"] and sha(ws) == ref["ws"]
    q, s = F.quantize_rowwise(x)
    assert sha(q) == ref["xq"] and sha(s) == ref["xs"]
    assert sha(F.gemm_i8_i32(q, wq)) == ref["acc"]
    y = F.linear_forward(x, wq, ws, b, torch.bfloat16)
    assert sha(y.view(torch.int16)) == ref["y_bits"]


def test_quarot_golden_within_rotation_tolerance(cuda_pkg, golden):
    """Against the reference's library-matmul rotation: a few last-place differences are expected."""
    F = cuda_pkg.functional
    g = golden("quarot_small.npz")
    x = torch.from_numpy(g["x_bits"].view(np.int16)).view(torch.bfloat16).to(DEV)
    q, s, xr = F.quantize_rowwise(x, hadamard=True, return_rotated=True)
    ref = bs.bf16_bits_to_f32(g["xr_bits"])
    assert (to_np(xr) != ref).mean() <= 1e-3
    assert (to_np(q) != g["xrq"]).mean() <= 1e-4 and np.array_equal(to_np(s), g["xrs"])
    y = F.linear_forward(x, torch.from_numpy(g["wrq"]).to(DEV), dev_ws(g["wrs"]), None, torch.bfloat16, hadamard=True)
    want = bs.bf16_bits_to_f32(g["y_rot_bits"])
    assert np.max(np.abs(to_np(y) - want)) <= TOL * rms(want)


def test_split_calls_equal_fused_call(cuda_pkg):
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(300, 1024, seed=8).to(DEV)
    wq, ws = F.quantize_weight_rows(wl.weight_fp32(520, 1024, seed=8).to(DEV))
    b = wl.bias_fp32(520, seed=8).to(DEV)
    q, s = F.quantize_rowwise(x)
    y1 = F.linear_w8a8(q, s, wq, ws, b, torch.bfloat16)
    y2 = F.linear_forward(x, wq, ws, b, torch.bfloat16)
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("N", [256, 96])     # 128-byte and 64-byte store boxes
def test_scatter_epilogue_writes_every_destination(cuda_pkg, N):
    """The column-parallel epilogue on one GPU: a [M, N] block goes to column `col_offset` of two destination
    matrices (standing in for this GPU's and a peer's copy of the full output); nothing else is touched."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    M, K, n_total, off = 300, 512, 1024, 512
    x = wl.activation(M, K, seed=14).to(DEV)
    wq, ws = F.quantize_weight_rows(wl.weight_fp32(N, K, seed=14).to(DEV))
    b = wl.bias_fp32(N, seed=14).to(DEV)
    q, s = F.quantize_rowwise(x)
    want = F.linear_w8a8(q, s, wq, ws, b, torch.bfloat16)
    dests = [torch.full((M, n_total), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    F.linear_w8a8_scatter(q, s, wq, ws, b, [d.data_ptr() for d in dests], n_total, off, torch.bfloat16)
    for d in dests:
        assert torch.equal(d[:, off:off + N], want)
        assert bool((d[:, :off] == 7.0).all()) and bool((d[:, off + N:] == 7.0).all())
    nat = cuda_pkg._native
    with pytest.raises(nat.NativeLibraryError, match="multiple of 32"):
        F.linear_w8a8_scatter(q, s, wq[:72], ws[:72], None, [dests[0].data_ptr()], n_total, 0, torch.bfloat16)


# ------------------------------------------------------------ K3 dynamic LoRA
@pytest.mark.parametrize("M,K,N,r,dt", [(256, 512, 384, 64, torch.bfloat16), (200, 1024, 328, 16, torch.bfloat16),
                                        (130, 256, 520, 8, torch.bfloat16), (96, 384, 160, 32, torch.float16),
                                        (300, 512, 264, 136, torch.bfloat16)])
def test_dynamic_lora_matches_oracle(cuda_pkg, M, K, N, r, dt):
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(M, K, seed=9, dtype=dt)
    A, B = wl.lora_factors(N, K, r, seed=9, dtype=dt)
    y0 = torch.randn(M, N, generator=torch.Generator().manual_seed(4)).to(dt)
    t_want = bs.lora_down(to_np(x), to_np(A), NAME[dt])
    t = F.lora_down(x.to(DEV), A.to(DEV))
    assert np.max(np.abs(to_np(t) - t_want)) <= TOL * rms(t_want)
    y_want = bs.lora_up_add(to_np(y0), to_np(t), to_np(B), NAME[dt])
    y = y0.to(DEV).clone()
    F.lora_up_add_(y, t, B.to(DEV))
    assert np.max(np.abs(to_np(y) - y_want)) <= TOL * rms(y_want)


def test_lora_term_added_in_the_gemm_epilogue(cuda_pkg):
    """lora_up writes round(t B^T); linear_w8a8(add_into=...) adds the dequantised GEMM onto it with the
    reference's roundings: y = round(round(dequant + bias) + lora_y)."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    M, K, N, r = 300, 512, 264, 16
    x = wl.activation(M, K, seed=12)
    wq, ws = bs.quantize_rowwise(wl.weight_fp32(N, K, seed=12).numpy())
    b = wl.bias_fp32(N, seed=12).bfloat16()
    A, B = wl.lora_factors(N, K, r, seed=12)
    xd = x.to(DEV)
    t = F.lora_down(xd, A.to(DEV))
    lora_y = F.lora_up(t, B.to(DEV))
    want_ly = bs.round_bf16((to_np(t).astype(np.float64) @ to_np(B).astype(np.float64).T).astype(np.float32))
    assert np.max(np.abs(to_np(lora_y) - want_ly)) <= TOL * rms(want_ly)
    q, s = F.quantize_rowwise(xd)
    kept = lora_y.clone()
    y = F.linear_w8a8(q, s, torch.from_numpy(wq).to(DEV), dev_ws(ws), b.to(DEV), torch.bfloat16, add_into=lora_y)
    assert y is lora_y
    base = bs.linear_w8a8(to_np(x), wq, ws, to_np(b))
    want = bs.round_bf16(base + to_np(kept))               # exact given the stored LoRA term
    assert np.array_equal(to_np(y), want)
    y_rmw = F.linear_w8a8(q, s, torch.from_numpy(wq).to(DEV), dev_ws(ws), b.to(DEV), torch.bfloat16)
    F.lora_up_add_(y_rmw, t, B.to(DEV))
    assert torch.equal(y_rmw, y)                            # same result as the read-modify-write form
    # fully fused: t @ B^T accumulated in tensor memory next to the int32 accumulator
    y_fused = F.linear_w8a8_lora(q, s, torch.from_numpy(wq).to(DEV), dev_ws(ws), b.to(DEV), t, B.to(DEV), torch.bfloat16)
    assert np.max(np.abs(to_np(y_fused) - want)) <= TOL * rms(want)
    assert (to_np(y_fused) != want).mean() <= 1e-2          # fp32 accumulation order of the low-rank product only


@pytest.mark.parametrize("M,K,N,r,per_ch,dt", [(520, 384, 392, 64, True, torch.bfloat16), (4608, 512, 1024, 16, False, torch.bfloat16),
                                               (300, 256, 264, 136, True, torch.float16), (100, 256, 264, 8, True, torch.bfloat16),
                                               (300, 256, 96, 8, False, torch.bfloat16)])
def test_fused_lora_linear_matches_oracle(cuda_pkg, M, K, N, r, per_ch, dt):
    """i8f_linear_w8a8_lora (fused for M, N > 128, two-kernel form below that) against the oracle."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(M, K, seed=15, dtype=dt)
    w = wl.weight_fp32(N, K, seed=15).numpy()
    wq, ws = bs.quantize_rowwise(w) if per_ch else bs.quantize_tensorwise(w)
    b = wl.bias_fp32(N, seed=15).to(dt)
    A, B = wl.lora_factors(N, K, r, seed=15, dtype=dt)
    xd = x.to(DEV)
    q, s = F.quantize_rowwise(xd)
    t = F.lora_down(xd, A.to(DEV))
    y = F.linear_w8a8_lora(q, s, torch.from_numpy(wq).to(DEV), dev_ws(ws), b.to(DEV), t, B.to(DEV), dt)
    base = bs.linear_w8a8(to_np(x), wq, ws, to_np(b), act_dtype=NAME[dt])
    want = bs.lora_up_add(base, to_np(t), to_np(B), NAME[dt])
    assert np.max(np.abs(to_np(y) - want)) <= TOL * rms(want)
    assert (to_np(y) != want).mean() <= 2e-2


def test_module_golden_with_dynamic_lora(cuda_pkg, golden):
    """Output of the reference's Linear.forward with lora_A / lora_B set (CPU run)."""
    F = cuda_pkg.functional
    g = golden("module_small.npz")
    as_bf16 = lambda bits: torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).to(DEV)  # noqa: E731
    x = as_bf16(g["x_bits"])
    y = F.linear_forward(x, torch.from_numpy(g["wq"]).to(DEV), dev_ws(g["ws"]), as_bf16(g["bias_bits"]), torch.bfloat16)
    assert np.array_equal(y.cpu().view(torch.int16).numpy().view(np.uint16), g["y_bits"])
    F.lora_up_add_(y, F.lora_down(x, as_bf16(g["lora_a_bits"])), as_bf16(g["lora_b_bits"]))
    want = bs.bf16_bits_to_f32(g["y_lora_bits"])
    assert np.max(np.abs(to_np(y) - want)) <= TOL * rms(want)


# ------------------------------------------------------ K4 stochastic merge
@pytest.mark.parametrize("N,K,r,per_ch,had,philox,fdt", [
    (256, 512, 64, True, False, False, torch.bfloat16), (200, 384, 16, False, True, False, torch.bfloat16),
    (100, 200, 8, True, False, True, torch.float32), (512, 1024, 64, True, True, True, torch.float16),
    (33, 130, 4, False, False, True, torch.bfloat16), (64, 256, 0, True, False, False, torch.bfloat16),
])
def test_lora_merge_bit_exact(cuda_pkg, N, K, r, per_ch, had, philox, fdt):
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    w = wl.weight_fp32(N, K, seed=11)
    wq, ws = bs.quantize_rowwise(w.numpy()) if per_ch else bs.quantize_tensorwise(w.numpy())
    down, up = wl.lora_factors(N, K, max(r, 1), seed=11, dtype=fdt)
    down, up = down[:r], (up[:, :r].float() * 30).to(fdt)
    u = bs.philox_uniforms(318008, N, K) if philox else wl.uniforms(N, K, seed=11).numpy()
    want = bs.lora_merge(wq, ws, to_np(up), to_np(down), 0.75, u, hadamard=had)
    wd = torch.from_numpy(wq).to(DEV).clone()
    F.lora_merge_sr_(wd, dev_ws(ws), up.to(DEV), down.to(DEV), 0.75, hadamard=had,
                     uniforms=None if philox else torch.from_numpy(u).to(DEV), seed=318008)
    if philox and fdt != torch.float32:
        # 16-bit factors + in-kernel RNG run the rank-r product on the tensor cores: a delta may differ in its last
        # place from the sequential fp32 sum, which can move a handful of weights by one step
        diff = to_np(wd).astype(np.int32) - want.astype(np.int32)
        assert np.abs(diff).max() <= 1 and (diff != 0).mean() <= 1e-4
    else:
        assert np.array_equal(to_np(wd), want)
    if r:
        assert (want != wq).mean() > 0.5, "the case must actually change the weights"
    else:
        assert np.array_equal(want, wq)


def test_merge_golden_fixture(cuda_pkg, golden):
    """Weights produced by the reference's INT8LoRAPatchAdapter.calculate_weight on CPU (uniforms recorded)."""
    F = cuda_pkg.functional
    g = golden("sr_merge_small.npz")
    as_bf16 = lambda bits: torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).to(DEV)  # noqa: E731
    up, down, u = as_bf16(g["up_bits"]), as_bf16(g["down_bits"]), torch.from_numpy(g["u"]).to(DEV)
    for wq, ws, merged in ((g["wq_c"], g["ws_c"], g["merged_c"]), (g["wq_t"], g["ws_t"], g["merged_t"])):
        wd = torch.from_numpy(wq).to(DEV).clone()
        F.lora_merge_sr_(wd, dev_ws(ws), up, down, 0.5, uniforms=u)
        assert np.array_equal(to_np(wd), merged)
    sr = F.stochastic_round(torch.from_numpy(g["delta"]).to(DEV), dev_ws(g["ws_c"]), uniforms=u)
    assert np.array_equal(to_np(sr), g["sr_c"])
    wd = torch.from_numpy(g["wrq"]).to(DEV).clone()
    F.lora_merge_sr_(wd, dev_ws(g["wrs"]), up, down, 0.5, hadamard=True, uniforms=u)
    assert np.max(np.abs(to_np(wd).astype(int) - g["merged_rot"].astype(int))) <= 1
    assert (to_np(wd) != g["merged_rot"]).mean() <= 1e-3


def test_stochastic_rounding_is_unbiased_in_philox_mode(cuda_pkg):
    """E[q * s] == x within 4 sigma and P(round up) == frac, with the in-kernel counter RNG."""
    F = cuda_pkg.functional
    N, K = 512, 2048
    delta = torch.full((N, K), 0.3 * 0.01, device=DEV)
    q = F.stochastic_round(delta, 0.01, seed=1234).float()
    p_up = float((q == 1).float().mean())
    assert set(torch.unique(q).tolist()) <= {0.0, 1.0}
    assert abs(p_up - 0.3) < 4 * (0.3 * 0.7 / (N * K)) ** 0.5 + 1e-6
    q2 = F.stochastic_round(delta, 0.01, seed=1235).float()
    assert not torch.equal(q, q2)
    assert torch.equal(q, F.stochastic_round(delta, 0.01, seed=1234).float())


def test_merge_idempotent_shape_properties_at_full_size(cuda_pkg):
    """Config-2 size: a zero-strength merge leaves W untouched; merging +D then -D with the same
    uniforms restores every weight that did not clamp to within one step."""
    F = cuda_pkg.functional
    N = K = 4096
    gen = torch.Generator(device=DEV).manual_seed(2)
    w0 = torch.randint(-40, 41, (N, K), generator=gen, dtype=torch.int8, device=DEV)
    ws = torch.rand(N, 1, generator=gen, device=DEV) * 1e-3 + 1e-3      # delta/ws has sigma <= 10: no clamping
    up = (torch.randn(N, 64, generator=gen, device=DEV) * 0.01).bfloat16()
    down = (torch.randn(64, K, generator=gen, device=DEV) * 0.125).bfloat16()
    w = w0.clone()
    F.lora_merge_sr_(w, ws, up, down, 0.0, seed=7)
    assert torch.equal(w, w0)
    F.lora_merge_sr_(w, ws, up, down, 1.0, seed=7)
    assert not torch.equal(w, w0)
    F.lora_merge_sr_(w, ws, up, down, -1.0, seed=7)
    assert int((w.int() - w0.int()).abs().max()) <= 1


def test_bounded_wait_times_out_and_reports(cuda_pkg):
    """A device-side wait that can never be satisfied gives up after its limit, the kernel returns, the status word
    carries the code, and the context stays usable."""
    nat = cuda_pkg._native
    assert nat.device_status() == 0
    nat.check(nat.load().i8f_selftest_bounded_wait(20_000_000, nat.current_stream(torch.device(DEV))), "selftest")
    torch.cuda.synchronize()
    assert nat.device_status(reset=True) == 199
    assert nat.device_status() == 0
    got = cuda_pkg.functional.gemm_i8_i32(torch.ones(32, 64, dtype=torch.int8, device=DEV),
                                          torch.ones(16, 64, dtype=torch.int8, device=DEV))
    assert bool((got == 64).all())


def test_peer_barrier_meets_and_times_out_on_one_gpu(cuda_pkg):
    """The column-parallel meeting kernel on ONE GPU, with the second rank played by the host: when the peer's slot
    already holds the epoch the kernel passes at once and publishes its own slot in both arrays; when the peer never
    arrives the wait gives up after its limit, the status word reads 105 and the context stays usable.  (Two ranks
    that really wait on each other never share a GPU; the two-GPU form runs in the multi-GPU test.)"""
    F, nat = cuda_pkg.functional, cuda_pkg._native
    dev = torch.device(DEV)
    mine = torch.zeros(8, dtype=torch.int32, device=DEV)      # rank 0's flag array
    peer = torch.zeros(8, dtype=torch.int32, device=DEV)      # stands in for rank 1's (mapped) array
    mine[1] = 5                                               # "rank 1 has reached epoch 5"
    F.peer_barrier([mine.data_ptr(), peer.data_ptr()], 0, 5, dev, limit_cycles=200_000_000)
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    assert mine.tolist()[:2] == [5, 5] and peer.tolist()[:2] == [5, 0]
    F.peer_barrier([mine.data_ptr(), peer.data_ptr()], 0, 4, dev, limit_cycles=200_000_000)   # an older epoch passes too
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    F.peer_barrier([mine.data_ptr(), peer.data_ptr()], 0, 6, dev, limit_cycles=20_000_000)    # nobody sets slot 1 to 6
    torch.cuda.synchronize()
    assert nat.device_status(reset=True) == 105
    assert nat.device_status() == 0
    assert bool((F.gemm_i8_i32(torch.ones(32, 64, dtype=torch.int8, device=DEV),
                               torch.ones(16, 64, dtype=torch.int8, device=DEV)) == 64).all())
    with pytest.raises(nat.NativeLibraryError):
        F.peer_barrier([mine.data_ptr()] * 9, 0, 1, dev)


# ------------------------------------------------------------------ quantiser prologues
@pytest.mark.parametrize("M,K,dt", [(64, 4096, torch.bfloat16), (33, 256, torch.bfloat16), (7, 1032, torch.float16),
                                    (130, 12288, torch.bfloat16), (5, 16384, torch.float16), (1, 8, torch.bfloat16),
                                    # thousands of rows (several waves of CTAs), row counts that are no multiple of the
                                    # rows per CTA
                                    (2051, 4096, torch.bfloat16), (2300, 2056, torch.float16)])
def test_ln_modulate_quantiser_bit_exact(cuda_pkg, M, K, dt):
    """LayerNorm -> (1 + scale), shift -> per-token int8 in one kernel: int8, scales and the modulated activations
    equal the bit-level definition; the same tensor built from PyTorch's own LayerNorm and addcmul agrees to within
    a bf16 / fp16 step (its reductions run in another order)."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = (wl.activation(M, K, seed=50, dtype=torch.float32) * 0.7 + 0.3).to(dt)
    g = torch.Generator().manual_seed(K + M)
    shift = (torch.randn(K, generator=g) * 0.2).to(dt)
    scale = (torch.randn(K, generator=g) * 0.3).to(dt)
    q, rs, y = F.quantize_rowwise_ln_modulate(x.to(DEV), shift.to(DEV), scale.to(DEV), eps=1e-5, return_y=True)
    q_want, s_want, y_want = bs.quantize_rowwise_ln_modulate(to_np(x), to_np(shift), to_np(scale), 1e-5, NAME[dt])
    assert np.array_equal(to_np(y), y_want)
    assert np.array_equal(to_np(rs), s_want) and np.array_equal(to_np(q), q_want)
    q2, rs2 = F.quantize_rowwise_ln_modulate(x.to(DEV), shift.to(DEV), scale.to(DEV), eps=1e-5)
    assert torch.equal(q2, q) and torch.equal(rs2, rs)
    wide = torch.zeros(M, K + 32, dtype=dt, device=DEV)      # a pitched input (column slice of a wider buffer)
    wide[:, 16:16 + K] = x.to(DEV)
    q3, rs3 = F.quantize_rowwise_ln_modulate(wide[:, 16:16 + K], shift.to(DEV), scale.to(DEV), eps=1e-5)
    assert torch.equal(q3, q) and torch.equal(rs3, rs)
    lib = torch.addcmul(shift.to(DEV), torch.nn.functional.layer_norm(x.to(DEV), (K,)), 1 + scale.to(DEV))
    d = (y.float() - lib.float()).abs()
    # steps of the 16-bit type at the magnitude of the terms (the modulated value can be a small difference of large ones)
    mag = torch.maximum(lib.float().abs(), torch.maximum(shift.to(DEV).float().abs().expand_as(lib), (lib.float() - shift.to(DEV).float()).abs()))
    step = torch.exp2(torch.floor(torch.log2(mag.clamp_min(2.0 ** -14))) - (7 if dt == torch.bfloat16 else 10))
    assert bool((d <= 3 * step).all()) and (d > 0).float().mean().item() <= 0.05, ((d / step).max().item(), (d > 0).float().mean().item())


@pytest.mark.parametrize("M,K0,K1,dt", [(64, 0, 12288, torch.bfloat16), (40, 4096, 12288, torch.bfloat16), (9, 128, 264, torch.float16),
                                        (3, 0, 8, torch.bfloat16), (130, 256, 768, torch.bfloat16),
                                        # large enough for the look-up-table kernel (persistent CTAs, four rows each)
                                        (301, 4096, 12288, torch.bfloat16), (182, 0, 12288, torch.float16), (1027, 0, 2056, torch.bfloat16),
                                        # a thousand rows and more, two sources, row counts that are no multiple of the grid
                                        (1100, 4096, 12288, torch.bfloat16), (1500, 1024, 3080, torch.float16)])
def test_gelu_quantiser_bit_exact(cuda_pkg, M, K0, K1, dt):
    """[ plain | GELU_tanh ] -> per-token int8 in one kernel, the two parts read as column slices of wider matrices."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    wide = (wl.activation(M, K1 + 64, seed=51, dtype=torch.float32) * 1.5).to(dt).to(DEV)
    if K1 >= 8:   # values on and beyond the edges of the look-up table of the large-input kernel, zeros of both signs
        wide[0, 64:72] = torch.tensor([0.0, -0.0, 1e-5, -3e-6, 100.0, -100.0, 2.0 ** -12, 15.9375], dtype=dt, device=DEV)
        wide[M - 1, 64:72] = torch.tensor([-(2.0 ** -12), 16.0, -16.0, 2.0 ** -13, -15.9375, 6e-8, 3e4, -3e4], dtype=dt, device=DEV)
    xg = wide[:, 64:]                                                 # a column slice, as in a fused qkv + mlp buffer
    xp = (wl.activation(M, K0, seed=52, dtype=torch.float32)).to(dt).to(DEV) if K0 else None
    q, rs, y = F.quantize_rowwise_gelu(xg, xp, return_y=True)
    q_want, s_want, y_want = bs.quantize_rowwise_gelu(to_np(xg), None if xp is None else to_np(xp), NAME[dt])
    assert np.array_equal(to_np(y), y_want)
    assert np.array_equal(to_np(rs), s_want) and np.array_equal(to_np(q), q_want)
    lib = torch.nn.functional.gelu(xg, approximate="tanh")
    got = y[:, K0:]
    d = (got.float() - lib.float()).abs()
    step = torch.exp2(torch.floor(torch.log2(lib.float().abs().clamp_min(2.0 ** -14))) - (7 if dt == torch.bfloat16 else 10))
    assert bool((d <= step + 1e-6).all()) and (d > 0).float().mean().item() <= 0.01 + 16.0 / d.numel()   # 16 injected edge values
    # special values: zero, large magnitudes of both signs
    sp = torch.tensor([[0.0, -0.0, 30.0, -30.0, 1e4, -1e4, 1e-3, -1e-3]], dtype=dt, device=DEV)
    _, _, ysp = F.quantize_rowwise_gelu(sp, None, return_y=True)
    assert np.array_equal(to_np(ysp), bs.round_to(bs.gelu_tanh(to_np(sp)), NAME[dt]))
    assert float(ysp[0, 2]) == 30.0 and abs(float(ysp[0, 3])) < 1e-30 and float(ysp[0, 4]) == float(sp[0, 4])


@pytest.mark.parametrize("rows,cols,dt", [(70, 256, torch.bfloat16), (513, 1024, torch.float16), (1, 128, torch.bfloat16)])
def test_rmsnorm_heads_bit_exact(cuda_pkg, rows, cols, dt):
    """Per-head RMS norm in place over the q and k columns of a wider (qkv) buffer."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    buf = wl.activation(rows, cols + 128, seed=53, dtype=torch.float32).to(dt).to(DEV)
    before = buf.clone()
    F.rmsnorm_heads_(buf[:, :cols], eps=1e-6)
    assert np.array_equal(to_np(buf[:, :cols]), bs.rmsnorm_heads(to_np(before[:, :cols]), 1e-6, NAME[dt]))
    assert torch.equal(buf[:, cols:], before[:, cols:])                       # the v columns are untouched
    lib = torch.nn.functional.rms_norm(before[:, :cols].reshape(rows, cols // 128, 128), (128,), eps=1e-6).reshape(rows, cols)
    assert (buf[:, :cols] != lib).float().mean().item() <= 0.01


@pytest.mark.parametrize("M,K,N,per_ch,use_bias,dt", [(300, 512, 392, True, True, torch.bfloat16), (64, 256, 4096, False, False, torch.bfloat16),
                                                      (520, 384, 264, False, True, torch.float16)])
def test_gated_residual_epilogue_bit_exact(cuda_pkg, M, K, N, per_ch, use_bias, dt):
    """residual += gate * linear(x) inside the GEMM epilogue equals round(residual + gate * y) of the separately
    computed linear output y, bit for bit (and so torch.addcmul on the same tensors)."""
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(M, K, seed=60, dtype=dt).to(DEV)
    wq, ws = F.quantize_weight_rows(wl.weight_fp32(N, K, seed=60).to(DEV)) if per_ch else F.quantize_tensorwise(wl.weight_fp32(N, K, seed=60).to(DEV))
    bias = wl.bias_fp32(N, seed=60).to(dt).to(DEV) if use_bias else None
    g = torch.Generator().manual_seed(N)
    residual = torch.randn(M, N, generator=g).to(dt).to(DEV)
    gate = (torch.randn(N, generator=g) * 0.5).to(dt).to(DEV)
    q, xs = F.quantize_rowwise(x)
    y = F.linear_w8a8(q, xs, wq, ws, bias, dt)
    want = bs.gated_add(to_np(residual), to_np(gate), to_np(y), NAME[dt])
    lib = torch.addcmul(residual, gate, y)
    got = F.linear_w8a8_gated_add_(residual.clone(), gate, q, xs, wq, ws, bias)
    assert np.array_equal(to_np(got), want)
    assert torch.equal(got, lib)
    # a row slice of a wider residual buffer is updated in place, its neighbours are not touched
    wide = torch.randn(M + 8, N, generator=g).to(dt).to(DEV)
    keep = wide.clone()
    F.linear_w8a8_gated_add_(wide[4:M + 4], gate, q, xs, wq, ws, bias)
    assert torch.equal(wide[4:M + 4], torch.addcmul(keep[4:M + 4], gate, y))
    assert torch.equal(wide[:4], keep[:4]) and torch.equal(wide[M + 4:], keep[M + 4:])


# ------------------------------------------------------------------ tiny-batch branch (M <= 16)
@pytest.mark.parametrize("M,K,N,per_channel,bias_dt,dt", [
    (1, 4096, 4096, False, torch.bfloat16, torch.bfloat16),     # a modulation-sized call
    (8, 384, 72, True, torch.bfloat16, torch.bfloat16),
    (16, 1024, 1000, True, torch.float32, torch.bfloat16),      # N not a multiple of the feature block
    (9, 208, 333, False, None, torch.bfloat16),                 # K a multiple of 16 but not of 64, odd N
    (3, 3072, 9216, True, torch.float16, torch.float16),
    (13, 16, 5, True, torch.float32, torch.float16),
    (2, 12288, 24576, False, torch.bfloat16, torch.bfloat16),   # widest feature block, several waves
])
def test_small_batch_linear_matches_oracle(cuda_pkg, M, K, N, per_channel, bias_dt, dt):
    F, wl = cuda_pkg.functional, cuda_pkg.workloads
    x = wl.activation(M, K, seed=41, dtype=dt)
    w = wl.weight_fp32(N, K, seed=41).numpy()
    wq, ws = (bs.quantize_rowwise if per_channel else bs.quantize_tensorwise)(w)
    b = wl.bias_fp32(N, seed=41).to(bias_dt) if bias_dt is not None else None
    want = bs.linear_small_batch(to_np(x), wq, ws, to_np(b) if b is not None else None, NAME[dt])
    y = F.linear_small_batch(x.to(DEV), torch.from_numpy(wq).to(DEV), dev_ws(ws), b.to(DEV) if b is not None else None)
    assert y.dtype == dt and y.shape == (M, N)
    got = to_np(y)
    # fp32 accumulation in a fixed order against float64: the rounded outputs differ on a few values, by one step
    # of the output type (which at four sigma is itself above 1e-2 of the RMS for bf16, so the bar is per value),
    # plus the fp32 accumulation error where the sum cancels
    assert np.mean(got != want) <= 2e-2
    step = np.abs(want) * (2.0 ** -7 if dt == torch.bfloat16 else 2.0 ** -10) + 1e-4 * rms(want)
    assert np.all(np.abs(got - want) <= step)
    assert rms(got - want) <= 1e-3 * rms(want)


def test_small_batch_linear_is_deterministic_and_checks_arguments(cuda_pkg):
    F, wl, nat = cuda_pkg.functional, cuda_pkg.workloads, cuda_pkg._native
    x = wl.activation(16, 512, seed=5).to(DEV)
    wq, ws = bs.quantize_rowwise(wl.weight_fp32(260, 512, seed=5).numpy())
    wq, ws = torch.from_numpy(wq).to(DEV), dev_ws(ws)
    a, b = F.linear_small_batch(x, wq, ws, None), F.linear_small_batch(x, wq, ws, None)
    assert torch.equal(a, b)
    # every row of a batch equals the same row computed alone (rows do not interact)
    for m in (0, 7, 8, 15):
        assert torch.equal(F.linear_small_batch(x[m:m + 1], wq, ws, None), a[m:m + 1])
    assert F.linear_small_batch(x[:0], wq, ws, None).shape == (0, 260)
    with pytest.raises(nat.NativeLibraryError):
        F.linear_small_batch(wl.activation(17, 512, seed=5).to(DEV), wq, ws, None)       # M > 16
    with pytest.raises(nat.NativeLibraryError):
        F.linear_small_batch(x[:, :40].contiguous(), wq[:, :40].contiguous(), ws, None)   # K % 16 != 0


def test_launch_counter_counts_kernels(cuda_pkg):
    """The library's own launch counter: a fused forward is two launches (quantise, GEMM), a tiny-batch call one."""
    F, wl, nat = cuda_pkg.functional, cuda_pkg.workloads, cuda_pkg._native
    lib = nat.load()
    x = wl.activation(64, 256, seed=2).to(DEV)
    wq, ws = bs.quantize_rowwise(wl.weight_fp32(96, 256, seed=2).numpy())
    wq, ws = torch.from_numpy(wq).to(DEV), dev_ws(ws)
    before = lib.i8f_launch_count()
    F.linear_forward(x, wq, ws, None, torch.bfloat16)
    assert lib.i8f_launch_count() - before == 2
    before = lib.i8f_launch_count()
    F.linear_small_batch(x[:4], wq, ws, None)
    assert lib.i8f_launch_count() - before == 1
