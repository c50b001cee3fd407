"""Generates the golden fixtures in this directory by EXECUTING THE REFERENCE.

    python tests/golden/make_golden.py /path/to/reference

The reference project (a checkout of ComfyUI-INT8-Fast) is imported as a package with
the test-only fake `comfy` on sys.path, and its own functions are run on CPU
tensors built from the seeded recipes in the package's workloads module:

  quantize_int8_axiswise / _tensorwise, int8_forward_dynamic[_per_row],
  quarot.rotate_activation / rotate_weight, stochastic_round_int8_delta (with
  torch.rand patched to return the recorded uniforms),
  INT8LoRAPatchAdapter.calculate_weight, Int8TensorwiseOps.Linear.forward
  (incl. the dynamic-LoRA branch).

Small cases are stored in full (inputs and outputs); the full-size CPU
configuration (M=256, K=3072, N=3072) is stored as SHA-256 digests of the
reference's outputs.  The reference is only needed to regenerate; the tests
read the committed .npz / .json files.
"""
from __future__ import annotations

import hashlib
import importlib.util
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "fake_comfy"))


def load_reference(path: str):
    spec = importlib.util.spec_from_file_location("int8_fast_ref", f"{path}/__init__.py",
                                                  submodule_search_locations=[path])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["int8_fast_ref"] = mod
    spec.loader.exec_module(mod)
    from int8_fast_ref import int8_quant, quarot  # noqa: PLC0415
    return int8_quant, quarot


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16/fp16 tensor -> uint16 bit patterns."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/the/reference/checkout")
    ref_path = sys.argv[1]
    rq, rr = load_reference(ref_path)
    import __graft_entry__ as g  # noqa: PLC0415
    wl = g.load_package().workloads

    # ---- small linear cases, stored in full --------------------------------
    M, K, N = 48, 256, 96
    x = wl.activation(M, K, seed=101)
    w = wl.weight_fp32(N, K, seed=101)
    b = wl.bias_fp32(N, seed=101)
    wq_c, ws_c = rq.quantize_int8_axiswise(w, dim=1)
    wq_t, ws_t = rq.quantize_int8_tensorwise(w)
    xq, xs = rq.quantize_int8_axiswise(x, dim=-1)
    acc_c = torch._int_mm(xq, wq_c.T)
    acc_t = torch._int_mm(xq, wq_t.T)
    y_c = rq.int8_forward_dynamic_per_row(x, wq_c, ws_c, b, torch.bfloat16)
    y_c_nb = rq.int8_forward_dynamic_per_row(x, wq_c, ws_c, None, torch.bfloat16)
    y_t = rq.int8_forward_dynamic(x, wq_t, ws_t.item(), b, torch.bfloat16)
    y_t_f16 = rq.int8_forward_dynamic(x.half(), wq_t, ws_t.item(), b, torch.float16)
    np.savez_compressed(HERE / "linear_small.npz", x_bits=bits(x), w=w.numpy(), bias=b.numpy(),
                        wq_c=wq_c.numpy(), ws_c=ws_c.numpy(), wq_t=wq_t.numpy(), ws_t=ws_t.numpy(),
                        xq=xq.numpy(), xs=xs.numpy(), acc_c=acc_c.numpy(), acc_t=acc_t.numpy(),
                        y_c_bits=bits(y_c), y_c_nb_bits=bits(y_c_nb), y_t_bits=bits(y_t), y_t_f16_bits=bits(y_t_f16))

    # ---- QuaRot -------------------------------------------------------------
    H16 = rr.build_hadamard(128, dtype=torch.bfloat16)
    H32 = rr.build_hadamard(128, dtype=torch.float32)
    xr = rr.rotate_activation(x, H16, 128)
    wr = rr.rotate_weight(w, H32, 128)
    wrq, wrs = rq.quantize_int8_axiswise(wr, dim=1)
    xrq, xrs = rq.quantize_int8_axiswise(xr, dim=-1)
    y_rot = rq.int8_forward_dynamic_per_row(xr, wrq, wrs, None, torch.bfloat16)
    np.savez_compressed(HERE / "quarot_small.npz", x_bits=bits(x), w=w.numpy(), xr_bits=bits(xr), wr=wr.numpy(),
                        wrq=wrq.numpy(), wrs=wrs.numpy(), xrq=xrq.numpy(), xrs=xrs.numpy(), y_rot_bits=bits(y_rot),
                        h_bf16_00_bits=bits(H16[:1, :1]), h_f32_00=H32[:1, :1].numpy())

    # ---- stochastic rounding + merge adapter --------------------------------
    r = 16
    lora_a, lora_b = wl.lora_factors(N, K, r, seed=101)       # down [r,K], up [N,r]
    u = wl.uniforms(N, K, seed=101)
    delta = torch.mm(lora_b.float(), lora_a.float()) * 0.5
    real_rand = torch.rand
    torch.rand = lambda *a, **k: u.clone()
    try:
        sr_c = rq.stochastic_round_int8_delta(delta, ws_c, 318008)
        sr_t = rq.stochastic_round_int8_delta(delta, ws_t.item(), 318008)
        adapter = rq.INT8LoRAPatchAdapter({"k"}, (lora_b, lora_a, float(r) * 0.5, None, None, None), ws_c, seed=318008)
        import comfy.model_management as mm  # noqa: PLC0415
        mm._FORCED_DEVICE = torch.device("cpu")
        rq.Int8TensorwiseOps.enable_quarot = False
        merged_c = adapter.calculate_weight(wq_c.clone(), "k", 1.0, 1.0, None, None)
        adapter_t = rq.INT8LoRAPatchAdapter({"k"}, (lora_b, lora_a, None, None, None, None), ws_t.item(), seed=318008)
        merged_t = adapter_t.calculate_weight(wq_t.clone(), "k", 0.5, 1.0, None, None)
        rq.Int8TensorwiseOps.enable_quarot = True
        adapter_rot = rq.INT8LoRAPatchAdapter({"k"}, (lora_b, lora_a, None, None, None, None), wrs, seed=318008)
        merged_rot = adapter_rot.calculate_weight(wrq.clone(), "k", 0.5, 1.0, None, None)
        rq.Int8TensorwiseOps.enable_quarot = False
    finally:
        torch.rand = real_rand
    np.savez_compressed(HERE / "sr_merge_small.npz", up_bits=bits(lora_b), down_bits=bits(lora_a), u=u.numpy(),
                        delta=delta.numpy(), wq_c=wq_c.numpy(), ws_c=ws_c.numpy(), wq_t=wq_t.numpy(), ws_t=ws_t.numpy(),
                        sr_c=sr_c.numpy(), sr_t=sr_t.numpy(), merged_c=merged_c.numpy(), merged_t=merged_t.numpy(),
                        wrq=wrq.numpy(), wrs=wrs.numpy(), merged_rot=merged_rot.numpy())

    # ---- module forward incl. dynamic LoRA ----------------------------------
    lin = rq.Int8TensorwiseOps.Linear(K, N, bias=True)
    sd = {"weight": wq_c.clone(), "weight_scale": ws_c.clone(), "bias": b.bfloat16()}
    lin._load_from_state_dict(sd, "", {}, True, [], [], [])
    x3 = x.reshape(4, 12, K)
    y_mod = lin(x3)
    y_small_plain = lin(x3[:1, :8])   # M <= 16 without a LoRA: x @ bf16(w.float() * scale)^T + bias
    y_one = lin(x3[2:3, 5:6])         # a single token
    lin.lora_A, lin.lora_B = lora_a, lora_b
    y_mod_lora = lin(x3)
    y_small = lin(x3[:1, :8])     # M <= 16: dequantised-weight branch
    np.savez_compressed(HERE / "module_small.npz", x_bits=bits(x), wq=wq_c.numpy(), ws=ws_c.numpy(),
                        bias_bits=bits(b.bfloat16()), lora_a_bits=bits(lora_a), lora_b_bits=bits(lora_b),
                        y_bits=bits(y_mod.reshape(M, N)), y_lora_bits=bits(y_mod_lora.reshape(M, N)),
                        y_small_bits=bits(y_small.reshape(8, N)), y_small_plain_bits=bits(y_small_plain.reshape(8, N)),
                        y_one_bits=bits(y_one.reshape(1, N)))

    # ---- full-size CPU configuration, digests only ---------------------------
    M, K, N = 256, 3072, 3072
    x = wl.activation(M, K, seed=0)
    w = wl.weight_fp32(N, K, seed=0)
    b = wl.bias_fp32(N, seed=0)
    wq, ws = rq.quantize_int8_axiswise(w, dim=1)
    xq, xs = rq.quantize_int8_axiswise(x, dim=-1)
    acc = torch._int_mm(xq, wq.T)
    y = rq.int8_forward_dynamic_per_row(x, wq, ws, b, torch.bfloat16)
    digests = {"shape": [M, K, N], "seed": 0, "wq": sha(wq.numpy()), "ws": sha(ws.numpy()), "xq": sha(xq.numpy()),
               "xs": sha(xs.numpy()), "acc": sha(acc.numpy()), "y_bits": sha(bits(y)),
               "torch": torch.__version__}
    (HERE / "config0_digests.json").write_text(json.dumps(digests, indent=1) + "\n")
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")), "config0_digests.json")


if __name__ == "__main__":
    main()
