"""The CPU oracle against the fixtures recorded from the reference's own functions."""
import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import bitspec as bs
from oracle import torch_path as tp

from conftest import GOLDEN


def f32(bits):
    return bs.bf16_bits_to_f32(bits)


def test_rowwise_and_tensorwise_quant_match_reference(golden):
    g = golden("linear_small.npz")
    x = f32(g["x_bits"])
    q, s = bs.quantize_rowwise(x)
    assert np.array_equal(q, g["xq"]) and np.array_equal(s, g["xs"])
    wq, ws = bs.quantize_rowwise(g["w"])
    assert np.array_equal(wq, g["wq_c"]) and np.array_equal(ws, g["ws_c"])
    wq, ws = bs.quantize_tensorwise(g["w"])
    assert np.array_equal(wq, g["wq_t"]) and ws == g["ws_t"]


def test_int_mm_matches_reference(golden):
    g = golden("linear_small.npz")
    assert np.array_equal(bs.int_mm(g["xq"], g["wq_c"]), g["acc_c"])
    assert np.array_equal(bs.int_mm(g["xq"], g["wq_t"]), g["acc_t"])


def test_linear_outputs_bit_exact_vs_reference(golden):
    g = golden("linear_small.npz")
    x = f32(g["x_bits"])
    y = bs.linear_w8a8(x, g["wq_c"], g["ws_c"], g["bias"])
    assert np.array_equal(bs.f32_to_bf16_bits(y), g["y_c_bits"])
    y = bs.linear_w8a8(x, g["wq_c"], g["ws_c"], None)
    assert np.array_equal(bs.f32_to_bf16_bits(y), g["y_c_nb_bits"])
    y = bs.linear_w8a8(x, g["wq_t"], g["ws_t"], g["bias"])
    assert np.array_equal(bs.f32_to_bf16_bits(y), g["y_t_bits"])
    xh = x.astype(np.float16).astype(np.float32)
    y = bs.linear_w8a8(xh, g["wq_t"], g["ws_t"], g["bias"], act_dtype="f16")
    assert np.array_equal(y.astype(np.float16).view(np.uint16), g["y_t_f16_bits"])


def test_hadamard_constants_match_reference(golden):
    g = golden("quarot_small.npz")
    assert f32(g["h_bf16_00_bits"])[0, 0] == bs.HADAMARD_NORM_BF16
    assert g["h_f32_00"][0, 0] == bs.HADAMARD_NORM_F32
    assert bs.HADAMARD_NORM_F16 == bs.HADAMARD_NORM_BF16


def test_wht_is_the_sylvester_matrix():
    eye = np.eye(128, dtype=np.float32)
    h = bs.wht128_sums(eye)
    i = np.arange(128)
    pop = np.array([[bin(a & b).count("1") for b in i] for a in i])
    assert np.array_equal(h, (1 - 2 * (pop & 1)).astype(np.float32))


def test_rotation_matches_reference_up_to_accumulation_order(golden):
    """The reference rotates with a library matmul (order unspecified); the canonical butterfly may
    differ in the last place of a few sums.  Bound the differences and their effect after quantisation."""
    g = golden("quarot_small.npz")
    x = f32(g["x_bits"])
    xr = bs.rotate_activation(x, "bf16")
    ref = f32(g["xr_bits"])
    diff = xr != ref
    assert diff.mean() <= 1e-3
    assert np.max(np.abs(xr - ref) / np.maximum(np.abs(ref), 1e-6)) <= 2 ** -7   # one bf16 ulp
    q, s = bs.quantize_rowwise(xr)
    assert (q != g["xrq"]).mean() <= 1e-4 and np.array_equal(s, g["xrs"])
    wr = bs.rotate_weight(g["w"])
    assert np.max(np.abs(wr - g["wr"])) <= 4 * np.finfo(np.float32).eps * np.max(np.abs(g["wr"]))
    wq, ws = bs.quantize_rowwise(wr)
    assert (wq != g["wrq"]).mean() <= 5e-3
    assert np.max(np.abs(ws - g["wrs"]) / g["wrs"]) <= 8 * np.finfo(np.float32).eps


def test_stochastic_round_and_merge_match_reference(golden):
    g = golden("sr_merge_small.npz")
    assert np.array_equal(bs.stochastic_round(g["delta"], g["ws_c"], g["u"]), g["sr_c"])
    assert np.array_equal(bs.stochastic_round(g["delta"], g["ws_t"], g["u"]), g["sr_t"])
    up, down = f32(g["up_bits"]), f32(g["down_bits"])
    # the reference's adapter was built with alpha = r/2, strength 1 -> scale 0.5
    assert np.array_equal(bs.lora_merge(g["wq_c"], g["ws_c"], up, down, 0.5, g["u"]), g["merged_c"])
    assert np.array_equal(bs.lora_merge(g["wq_t"], g["ws_t"], up, down, 0.5, g["u"]), g["merged_t"])
    rot = bs.lora_merge(g["wrq"], g["wrs"], up, down, 0.5, g["u"], hadamard=True)
    assert (rot != g["merged_rot"]).mean() <= 1e-3      # rotation order, see the rotation test
    assert np.max(np.abs(rot.astype(int) - g["merged_rot"].astype(int))) <= 1


def test_module_forward_with_dynamic_lora_matches_reference(golden):
    g = golden("module_small.npz")
    x = f32(g["x_bits"])
    bias = f32(g["bias_bits"])
    y = bs.linear_w8a8(x, g["wq"], g["ws"], bias)
    assert np.array_equal(bs.f32_to_bf16_bits(y), g["y_bits"])
    a, b = f32(g["lora_a_bits"]), f32(g["lora_b_bits"])
    y2 = bs.lora_up_add(y, bs.lora_down(x, a), b)
    ref = f32(g["y_lora_bits"])
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert np.max(np.abs(y2 - ref)) <= 1e-2 * rms
    assert (bs.f32_to_bf16_bits(y2) != g["y_lora_bits"]).mean() <= 1e-2   # fp32 accumulation order inside the two GEMMs


def test_small_batch_branch_matches_reference(golden):
    """M <= 16: unquantised activations against dequantised weights.  The reference's CPU matmul accumulates in
    its own order, so the bar is the output tolerance, and in fact at most one bf16 step on a few values."""
    g = golden("module_small.npz")
    x = f32(g["x_bits"]).reshape(4, 12, -1)
    bias = f32(g["bias_bits"])
    for xs, key in ((x[0, :8], "y_small_plain_bits"), (x[2, 5:6], "y_one_bits")):
        ref = f32(g[key])
        y = bs.linear_small_batch(xs, g["wq"], g["ws"], bias)
        rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
        assert np.max(np.abs(y - ref)) <= 1e-2 * rms
        assert (bs.f32_to_bf16_bits(y) != g[key]).mean() <= 2e-2
    # with the dynamic LoRA on top (the LoRA sees the same unquantised activations)
    a, b = f32(g["lora_a_bits"]), f32(g["lora_b_bits"])
    y = bs.lora_up_add(bs.linear_small_batch(x[0, :8], g["wq"], g["ws"], bias), bs.lora_down(x[0, :8], a), b)
    ref = f32(g["y_small_bits"])
    assert np.max(np.abs(y - ref)) <= 1e-2 * np.sqrt(np.mean(ref.astype(np.float64) ** 2))


def test_torch_path_equals_bitspec(pkg):
    wl = pkg.workloads
    x = wl.activation(40, 384, seed=3)
    w = wl.weight_fp32(72, 384, seed=3)
    b = wl.bias_fp32(72, seed=3)
    for per_channel in (True, False):
        wq, ws = (bs.quantize_rowwise if per_channel else bs.quantize_tensorwise)(w.numpy())
        y_np, q_np, s_np, acc_np = bs.linear_w8a8(x.float().numpy(), wq, ws, b.numpy(), return_parts=True)
        y, q, s, acc = tp.linear_w8a8(x, torch.from_numpy(wq), torch.from_numpy(np.asarray(ws)), b, torch.bfloat16,
                                      return_parts=True)
        assert np.array_equal(q.numpy(), q_np) and np.array_equal(s.numpy(), s_np)
        assert np.array_equal(acc.numpy(), acc_np)
        assert np.array_equal(y.float().numpy(), y_np)
    u = wl.uniforms(72, 384, seed=3)
    d = torch.randn(72, 384, generator=torch.Generator().manual_seed(5)) * 0.01
    wq, ws = bs.quantize_rowwise(w.numpy())
    assert np.array_equal(tp.stochastic_round(d, torch.from_numpy(ws), u).numpy(),
                          bs.stochastic_round(d.numpy(), ws, u.numpy()))


def test_config0_digests_from_the_oracle(pkg):
    """Full-size CPU configuration: the oracle reproduces the digests of the reference's outputs."""
    ref = json.loads((GOLDEN / "config0_digests.json").read_text())
    M, K, N = ref["shape"]
    wl = pkg.workloads
    x = wl.activation(M, K, seed=ref["seed"])
    w = wl.weight_fp32(N, K, seed=ref["seed"])
    b = wl.bias_fp32(N, seed=ref["seed"])
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()  # noqa: E731
    wq, ws = bs.quantize_rowwise(w.numpy())
    assert sha(wq) == ref["wq"] and sha(ws) == ref["ws"]
    y, q, s, acc = bs.linear_w8a8(x.float().numpy(), wq, ws, b.numpy(), return_parts=True)
    assert sha(q) == ref["xq"] and sha(s) == ref["xs"] and sha(acc) == ref["acc"]
    assert sha(bs.f32_to_bf16_bits(y)) == ref["y_bits"]


def test_philox_known_answers():
    """Random123 known-answer vectors for Philox4x32-10."""
    z = bs.philox4x32_10(np.zeros((1, 4), np.uint32), np.zeros((1, 2), np.uint32))[0]
    assert [int(v) for v in z] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = bs.philox4x32_10(np.full((1, 4), 0xFFFFFFFF, np.uint32), np.full((1, 2), 0xFFFFFFFF, np.uint32))[0]
    assert [int(v) for v in f] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    p = bs.philox4x32_10(np.array([[0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344]], np.uint32),
                         np.array([[0xA4093822, 0x299F31D0]], np.uint32))[0]
    assert [int(v) for v in p] == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]
    u = bs.philox_uniforms(318008, 7, 10)
    assert u.shape == (7, 10) and u.min() >= 0.0 and u.max() < 1.0
    # mapping: element (n, k) <- counter (n, k // 8), word (k % 8) // 2, low half first, times 2^-16
    blk = bs.philox4x32_10(np.array([[5, 1, 0, 0]], np.uint32), np.array([[318008, 0]], np.uint32))[0]
    assert u[5, 8] == np.float32(int(blk[0]) & 0xFFFF) * np.float32(2.0 ** -16)
    assert u[5, 9] == np.float32(int(blk[0]) >> 16) * np.float32(2.0 ** -16)
    blk0 = bs.philox4x32_10(np.array([[5, 0, 0, 0]], np.uint32), np.array([[318008, 0]], np.uint32))[0]
    assert u[5, 7] == np.float32(int(blk0[3]) >> 16) * np.float32(2.0 ** -16)


@pytest.mark.parametrize("rows,cols", [(0, 128), (3, 0)])
def test_empty_inputs(rows, cols):
    q, s = bs.quantize_rowwise(np.zeros((rows, cols), np.float32))
    assert q.shape == (rows, cols) and s.shape == (rows, 1)
    if rows:
        assert np.all(s == bs.SCALE_FLOOR)


def test_zero_rows_use_the_scale_floor():
    x = np.zeros((2, 64), np.float32)
    x[1, 3] = 5.0
    q, s = bs.quantize_rowwise(x)
    assert s[0, 0] == np.float32(1e-30) and np.all(q[0] == 0)
    assert q[1, 3] == 127
