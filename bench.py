#!/usr/bin/env python
"""Benchmark of the W8A8 linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c0|c2|c2merge|c4|dit|smallm|prologue|subwave]
                    [--impl reference]

One "step" is one pass of the hot path over one batch of synthetic input:
(Hadamard rotation +) per-token int8 quantisation, the int8 tensor-core GEMM
and the dequantising epilogue (plus the dynamic-LoRA kernels for c2).  The
default workload is the QuaRot MLP-up linear (M=4096, K=4096, N=12288).  With
N > 1 every rank runs its own batch of tokens against replicated weights
(token-parallel, no data-path collective), so scaling is weak.

Prints ONE JSON line (rank 0).  `value` is aggregate int8 tensor throughput
with inputs resident in HBM, every timed step going through the public fused
call; `roofline` times the GEMM (and the quantiser) alone in a loop of their
own; `e2e` is the same metric through the ops-class module call with host
buffers (pinned host -> device copy of the activations and device -> host copy
of the output inside the timed region), next to the same copies without
kernels.  The default workload also carries, measured in the same process
outside the headline region:
    parity       the timed inputs checked against the CPU oracle
    comparators  torch._int_mm and the library expression of the step on this GPU
    sustained    the step back to back for seconds (power-managed steady state)
    dit          the synthetic 9B-class DiT denoising step (one sample per GPU)
    c4           (N > 1) the column-parallel sweep: fused epilogue scatter vs NCCL
                 all-gather, with equality checks the run fails on
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_INT8_TOPS = 4500.0   # B200 dense INT8, data-sheet
# dram__bytes_read.sum + dram__bytes_write.sum of one GEMM launch from the ncu capture summarised under profiles/
NCU_GEMM_TRAFFIC_BYTES = {"c1_quarot_mlp_up": 184.6e6, "c2_dynamic_lora": 87.0e6}
NCU_SMALL_M_TRAFFIC_BYTES = 104.6e6   # small_m_kernel at M=1, K=4096, N=24576
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
N_BUFFER_SETS = 4


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:  # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU through NVML (read-only queries) from a
    thread while the timed region runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake"}

    def __init__(self, torch_device_index: int, period_s: float = 0.004):
        self.idx = torch_device_index
        self.period = period_s
        self.samples = []
        self.thread = None
        self.stop_flag = False
        self.handle = None
        self.nv = None

    def start(self):
        try:
            import threading
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = str(torch.cuda.get_device_properties(self.idx).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:  # noqa: BLE001
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.thread = None

    def _run(self):
        nv, h = self.nv, self.handle
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag:
            try:
                self.samples.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetPowerUsage(h) / 1e3,
                                     int(reasons_fn(h)), time.perf_counter()))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def stop(self, t_begin: float = 0.0, t_end: float = float("inf")):
        """Summary of the samples taken between the two host timestamps (the timed region)."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is None:
            return out
        self.stop_flag = True
        self.thread.join(timeout=2)
        inside = [s for s in self.samples if t_begin <= s[3] <= t_end]
        if not inside and self.samples:   # a timed region shorter than the sampling period: take the nearest sample
            near = min(self.samples, key=lambda s: min(abs(s[3] - t_begin), abs(s[3] - t_end)))
            out["note"] = (f"timed region shorter than the sampling period; nearest sample, "
                           f"{min(abs(near[3] - t_begin), abs(near[3] - t_end)) * 1e3:.1f} ms away")
            inside = [near]
        self.samples = inside
        try:
            out["sm_max_mhz"] = float(self.nv.nvmlDeviceGetMaxClockInfo(self.handle, self.nv.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            pass
        if self.samples:
            sm = sorted(s[0] for s in self.samples)
            mask = 0
            for s_ in self.samples:
                mask |= s_[2]
            out.update(sm_mhz=float(sm[len(sm) // 2]), sm_min_mhz=float(sm[0]), power_w_max=max(s[1] for s in self.samples),
                       reasons=sorted(name for bit, name in self.REASONS.items() if mask & bit), samples=len(self.samples))
        return out


def workload_shape(name: str):
    import __graft_entry__ as g
    wl = g.load_package().workloads
    key = {"c0": "c0_cpu_linear", "c1": "c1_quarot_mlp_up", "c2": "c2_dynamic_lora"}[name]
    return wl.CONFIGS[key]


def build_cpu_inputs(shape, seed: int, rows: int | None = None):
    """Seeded CPU tensors of one workload (optionally only the first `rows` tokens)."""
    import torch
    import __graft_entry__ as g
    wl = g.load_package().workloads
    M = shape.M if rows is None else rows
    x = wl.activation(M, shape.K, seed=seed)
    w = wl.weight_fp32(shape.N, shape.K, seed=seed)
    if shape.hadamard:
        w = w.bfloat16().float()          # the QuaRot configuration starts from bf16 weights
    b = wl.bias_fp32(shape.N, seed=seed) if shape.bias else None
    lora = wl.lora_factors(shape.N, shape.K, shape.lora_rank, seed=seed) if shape.lora_rank else None
    return x, w, b, lora


def config_dict(shape, world: int):
    working_set_mb = N_BUFFER_SETS * (shape.M * shape.K * 3 + shape.N * shape.K + shape.M * shape.N * 2) / 1e6
    return {"workload": shape.name, "M_per_gpu": shape.M, "K": shape.K, "N": shape.N, "hadamard": shape.hadamard,
            "weight_scale": "per_channel" if shape.per_channel else "tensorwise", "bias": shape.bias,
            "lora_rank": shape.lora_rank, "out_dtype": "bf16", "parallelism": f"token-parallel x{world}",
            "l2": f"inputs rotate over {N_BUFFER_SETS} buffer sets ({working_set_mb:.0f} MB > 126 MB L2)"}


# ----------------------------------------------------------------- CPU arm
def cpu_reference_rate(shape, steps: int, warmup: int, budget_s: float):
    """Times the oracle's CPU PyTorch path (what the reference runs without a GPU) on a bounded sample."""
    import torch
    from oracle import torch_path as tp
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rows = min(shape.M, 512)
    x, w, b, lora = build_cpu_inputs(shape, seed=0, rows=rows)
    if shape.hadamard:
        w = tp.rotate_weight(w)
    wq, ws = tp.quantize_rowwise(w) if shape.per_channel else tp.quantize_tensorwise(w)

    def step():
        y = tp.linear_w8a8(x, wq, ws, b, torch.bfloat16, hadamard=shape.hadamard)
        if lora is not None:
            y = tp.lora_dynamic_add(y, x, lora[0], lora[1])
        return y

    t0 = time.perf_counter()
    step()
    first = time.perf_counter() - t0
    for _ in range(max(0, warmup - 1)):
        step()
    n = max(1, min(steps, int(budget_s / max(first, 1e-4))))
    t0 = time.perf_counter()
    for _ in range(n):
        step()
    dt = (time.perf_counter() - t0) / n
    ops = 2.0 * rows * shape.N * shape.K
    return {"value": ops / dt / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
            "sample": f"first {rows} of {shape.M} tokens of {shape.name}, {n} timed passes of "
                      f"{dt * 1e3:.2f} ms, torch {torch.get_num_threads()} threads"}, dt


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    shape = workload_shape(args.workload)
    base, dt = cpu_reference_rate(shape, args.steps, args.warmup, budget_s=60.0)
    line = {
        "impl": "reference", "metric": "w8a8_linear_int8_throughput", "value": base["value"], "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config_dict(shape, max(1, args.gpus)),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------- GPU arm
def rank_context():
    """(rank, world, local_rank, device, dist-or-None); initialises NCCL when launched with more than one rank."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
    return rank, world, local_rank, dev, dist


def make_sync(dist):
    import torch

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
    return sync_all


def max_over_ranks(values, dev, dist):
    import torch
    if dist is None:
        return [float(v) for v in values]
    t = torch.tensor(list(values), device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def make_module(pkg, s, shape):
    """The public layer object a user of the node pack holds: an ops-class Linear loaded from a pre-quantised
    state dict (int8 weight + weight_scale [+ bias]), QuaRot flag and dynamic-LoRA factors set as the loader /
    the hook would set them."""
    lin = pkg.ops.StandaloneInt8Ops.Linear(shape.K, shape.N, bias=shape.bias, device="meta")
    sd = {"weight": s["wq"], "weight_scale": s["ws"].reshape(-1, 1) if shape.per_channel else s["ws"].reshape(1).clone()}
    if shape.bias:
        sd["bias"] = s["bias"]
    lin._load_from_state_dict(sd, "", {}, True, [], [], [])
    lin._use_quarot = shape.hadamard
    if s["lora"] is not None:
        lin.lora_A, lin.lora_B = s["lora"]
    return lin


def parity_record(pkg, shape, s, dev):
    """The timed configuration's first buffer set against the CPU oracle: int8 activations, scales and int32
    accumulators must be equal, the 16-bit output is compared bit for bit and as max|d| / RMS.  The oracle is the
    checker here, nothing of it is timed.  The rotation on the oracle side is the canonical butterfly of
    oracle/bitspec.py (the reference's own library matmul orders its fp32 sums backend by backend)."""
    import torch
    from oracle import bitspec as bs
    from oracle import torch_path as tp
    F = pkg.functional
    t0 = time.perf_counter()
    x = s["x"].cpu()
    wq, ws = s["wq"].cpu(), s["ws"].cpu()
    bias = None if s["bias"] is None else s["bias"].cpu()
    xr = torch.from_numpy(bs.rotate_activation(x.float().numpy(), "bf16")).bfloat16() if shape.hadamard else x
    want, q_want, xs_want, acc_want = tp.linear_w8a8(xr, wq, ws.reshape(-1, 1) if shape.per_channel else float(ws.reshape(-1)[0]),
                                                     bias, torch.bfloat16, hadamard=False, return_parts=True)
    q, xs = F.quantize_rowwise(s["x"], hadamard=shape.hadamard)
    acc = F.gemm_i8_i32(q, s["wq"])
    y = F.linear_forward(s["x"], s["wq"], s["ws"], s["bias"], torch.bfloat16, hadamard=shape.hadamard)
    rec = {"against": "oracle/torch_path.py (CPU, canonical rotation from oracle/bitspec.py)", "buffer_set": 0,
           "int8_activations_equal": bool(torch.equal(q.cpu(), q_want)),
           "activation_scales_equal": bool(torch.equal(xs.cpu().reshape(-1), xs_want.reshape(-1))),
           "int32_accumulators_equal": bool(torch.equal(acc.cpu(), acc_want))}
    del acc
    yc = y.cpu()
    base = want
    if s["lora"] is not None:
        want = tp.lora_dynamic_add(want, xr, s["lora"][0].cpu(), s["lora"][1].cpu())
        yc = pkg.custom_ops.linear_lora_forward(s["x"], s["wq"], s["ws"], s["bias"], s["lora"][0], s["lora"][1], torch.bfloat16,
                                                shape.hadamard, False, 0).cpu()
    rms = float(want.double().pow(2).mean().sqrt())
    d = (yc.float() - want.float()).abs()
    rec["out_bits_equal"] = bool(torch.equal(yc.view(torch.int16), want.view(torch.int16)))
    rec["out_max_abs_err_over_rms"] = float(d.max()) / rms
    rec["out_tolerance"] = 1e-2
    # where bf16 itself is coarser than 1e-2 RMS (outputs of several RMS in magnitude), two bf16 steps at the magnitude of
    # the terms is the bar instead; only the dynamic-LoRA path (tensor-core float sums) ever needs it
    mag = torch.maximum(torch.maximum(base.float().abs(), (want.float() - base.float()).abs()), want.float().abs())
    step = torch.exp2(torch.floor(torch.log2(mag.clamp_min(2.0 ** -126))) - 7)
    rec["out_elements_outside_bar"] = int((~((d <= 1e-2 * rms) | (d <= 2 * step))).sum())
    rec["ok"] = bool(rec["int8_activations_equal"] and rec["activation_scales_equal"] and rec["int32_accumulators_equal"]
                     and rec["out_elements_outside_bar"] == 0)
    rec["seconds"] = round(time.perf_counter() - t0, 2)
    return rec


def comparators_record(shape, sets, steps: int):
    """The kernels to beat on the same GPU, on the same tensors: the library int8 GEMM (torch._int_mm, cuBLASLt) alone,
    and the whole step as the reference's non-Triton CUDA path expresses it with library kernels
    (rotate_activation quarot.py:73-102 -> quantize_int8_axiswise int8_quant.py:28-31 -> torch._int_mm :80 ->
    scale and cast :84 / :115 -> bias :86-87).  Not the product path; timed for comparison only."""
    import torch
    M, K, N = shape.M, shape.K, shape.N
    dev = sets[0]["x"].device
    h128 = None
    if shape.hadamard:
        idx = torch.arange(128, device=dev)
        bits = idx[:, None] & idx[None, :]
        par = torch.zeros_like(bits)
        for b in range(7):
            par ^= (bits >> b) & 1
        h128 = ((1 - 2 * par).float() / (128 ** 0.5)).to(torch.bfloat16)

    def library_step(s):
        x = s["x"]
        if h128 is not None:
            x = torch.matmul(x.view(M, K // 128, 128), h128).view(M, K)
        absmax = x.abs().amax(dim=-1, keepdim=True)
        xs = (absmax.float() / 127.0).clamp(min=1e-30)
        q = x.float().mul(1.0 / xs).round_().clamp_(-128.0, 127.0).to(torch.int8)
        acc = torch._int_mm(q, s["wq"].T)
        if shape.per_channel:
            y = acc.float().mul_(xs).mul_(s["ws"].reshape(1, -1)).to(torch.bfloat16)
        else:
            y = acc.float().mul_(s["ws"].reshape(()) * xs).to(torch.bfloat16)
        if s["bias"] is not None:
            y = y + s["bias"].to(torch.bfloat16)
        return q, y

    n = len(sets)
    qs = [library_step(s)[0] for s in sets]
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for i in range(3):
        torch._int_mm(qs[i % n], sets[i % n]["wq"].T)
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(ev):
        a.record()
        torch._int_mm(qs[i % n], sets[i % n]["wq"].T)
        b.record()
    torch.cuda.synchronize()
    mm = sorted(a.elapsed_time(b) for a, b in ev[1:])
    for i in range(2):
        library_step(sets[i % n])
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        library_step(sets[i % n])
    b.record()
    torch.cuda.synchronize()
    lib_ms = a.elapsed_time(b) / steps
    ops = 2.0 * M * N * K
    # the int8 counterpart of the driver's bf16 peak measurement (which has no int8 figure): the library GEMM at
    # 8192^3, best of 10 single launches and the average of a loop of about 1.5 s
    peak = {}
    try:
        gen = torch.Generator(device=dev).manual_seed(5)
        pa = torch.randint(-127, 128, (8192, 8192), generator=gen, dtype=torch.int8, device=dev)
        pb = torch.randint(-127, 128, (8192, 8192), generator=gen, dtype=torch.int8, device=dev).t()
        for _ in range(3):
            torch._int_mm(pa, pb)
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            torch._int_mm(pa, pb)
            b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b))
        reps = max(10, int(1500.0 / best))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            torch._int_mm(pa, pb)
        b.record()
        torch.cuda.synchronize()
        sus = a.elapsed_time(b) / reps
        pops = 2.0 * 8192 ** 3
        peak = {"int_mm_8192_burst_tops": pops / (best * 1e-3) / 1e12, "int_mm_8192_sustained_tops": pops / (sus * 1e-3) / 1e12,
                "int_mm_8192_sustained_s": sus * reps * 1e-3}
        del pa, pb
    except Exception as e:      # a comparator only: its absence must not fail the run
        peak = {"int_mm_8192_error": str(e)[:120]}
    return {**peak,
            "int_mm_ms_median": median(mm), "int_mm_ms_best": mm[0], "int_mm_tops": ops / (median(mm) * 1e-3) / 1e12,
            "int_mm_output": "int32 [M,N] (no epilogue)", "library_step_ms": lib_ms,
            "library_step_tops": ops / (lib_ms * 1e-3) / 1e12, "n": steps,
            "what": "torch._int_mm alone; and rotate -> quantise -> _int_mm -> scale -> bf16 (+bias) with library "
                    "kernels, the reference's CUDA path without Triton (its Triton kernels are not on this box)"}


def run_gpu_arm(args):
    import torch
    import __graft_entry__ as g

    rank, world, local_rank, dev, dist = rank_context()
    sync_all = make_sync(dist)
    pkg = g.load_package()
    F, nat = pkg.functional, pkg._native
    nat.require_device(dev)
    shape = workload_shape(args.workload)
    M, K, N = shape.M, shape.K, shape.N
    out_dtype = torch.bfloat16
    extras = args.workload == "c1" and not args.headline_only

    # Weak scaling: rank r owns its own batch of M tokens (seed differs per rank), weights replicated.
    sets = []
    for i in range(N_BUFFER_SETS):
        x, w, b, lora = build_cpu_inputs(shape, seed=100 * rank + i)
        wd = w.to(dev)
        if shape.per_channel:
            wq, ws = F.quantize_weight_rows(wd, hadamard=shape.hadamard)
        else:
            wq, ws = F.quantize_tensorwise(wd, hadamard=shape.hadamard)
            ws = ws.reshape(1)
        del wd
        sets.append({"x": x.to(dev), "x_host": x.pin_memory(), "wq": wq, "ws": ws,
                     "bias": None if b is None else b.to(dev).to(out_dtype),
                     "lora": None if lora is None else (lora[0].to(dev), lora[1].to(dev)),
                     "y_host": torch.empty((M, N), dtype=out_dtype).pin_memory()})
    workspace = torch.empty((nat.load().i8f_linear_workspace_bytes(M, K),), dtype=torch.uint8, device=dev)

    def step(i: int):
        """One pass of the hot path through the public fused call: K1 and K2 back to back on the stream."""
        s = sets[i % N_BUFFER_SETS]
        if s["lora"] is None:
            return F.linear_forward(s["x"], s["wq"], s["ws"], s["bias"], out_dtype, hadamard=shape.hadamard,
                                    workspace=workspace)
        return pkg.custom_ops.linear_lora_forward(s["x"], s["wq"], s["ws"], s["bias"], s["lora"][0], s["lora"][1], out_dtype,
                                                  shape.hadamard, False, nat.EPI_PYTORCH)

    # ---- headline: W warm-up steps, then exactly K timed steps between barriers, max over ranks
    for i in range(args.warmup):
        step(i)
    sync_all()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.15)
    sync_all()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    host_t0 = time.perf_counter()
    launches_before = nat.load().i8f_launch_count()
    t_start.record()
    for i in range(args.steps):
        step(i)
    t_end.record()
    launches_timed = nat.load().i8f_launch_count() - launches_before   # counted by the library itself
    sync_all()
    host_t1 = time.perf_counter()
    elapsed_ms = t_start.elapsed_time(t_end)
    clocks = sampler.stop(host_t0, host_t1) if sampler else None

    # ---- the two kernels on their own: KERNEL_SAMPLES event-bracketed launches each, back to back over the rotating
    # buffer sets (so operands come from HBM, not L2); the first launch after the idle gap is discarded
    KERNEL_SAMPLES = 33
    quantised = [F.quantize_rowwise(s["x"], hadamard=shape.hadamard) for s in sets]
    lora_ts = [F.lora_down(s["x"], s["lora"][0]) if s["lora"] is not None else None for s in sets]

    def gemm_only(i):
        s, (q, xs) = sets[i % N_BUFFER_SETS], quantised[i % N_BUFFER_SETS]
        if s["lora"] is not None:
            return F.linear_w8a8_lora(q, xs, s["wq"], s["ws"], s["bias"], lora_ts[i % N_BUFFER_SETS], s["lora"][1], out_dtype)
        return F.linear_w8a8(q, xs, s["wq"], s["ws"], s["bias"], out_dtype)

    def quant_only(i):
        return F.quantize_rowwise(sets[i % N_BUFFER_SETS]["x"], hadamard=shape.hadamard)

    def bracketed(fn):
        for i in range(4):
            fn(i)
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(KERNEL_SAMPLES)]
        for i, (a, b) in enumerate(evs):
            a.record()
            fn(i)
            b.record()
        torch.cuda.synchronize()
        return sorted(a.elapsed_time(b) for a, b in evs[1:])

    def graph_timed(fn, launches=8, replays=9):
        """Per-launch time of a short kernel: `launches` calls captured into one CUDA graph (so the host's launch
        cost is out of the picture, which an event pair around a 15 us kernel cannot keep out), replayed `replays`
        times; the first replay is discarded.  Returns the sorted per-launch averages of the replays."""
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for i in range(launches):
                fn(i)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(launches):
                    fn(i)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        out = []
        for _ in range(replays):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b) / launches)
        del graph
        return sorted(out[1:])

    gemm_ms = bracketed(gemm_only)
    gemm_graph_ms = graph_timed(gemm_only)
    quant_ms = graph_timed(quant_only)
    del quantised, lora_ts

    # ---- end to end: host buffers through the public MODULE call (the ops-class Linear a ComfyUI model is built
    # from), copies inside the timed region.  The three phases of consecutive steps overlap as a serving loop would
    # run them: host->device copy on one stream, the forward on the current stream, device->host copy of the result
    # on a third (PCIe is full duplex); every step still moves its own input and its own output.
    modules = [make_module(pkg, s, shape) for s in sets]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    cur = torch.cuda.current_stream(dev)
    x_dev = [torch.empty_like(s["x"]) for s in sets]
    y_dev = [torch.empty((M, N), dtype=out_dtype, device=dev) for _ in sets]     # copy-only loop's source
    keep = [None] * N_BUFFER_SETS            # outputs stay referenced until their copy-out has been enqueued again
    fwd_done = [torch.cuda.Event() for _ in range(N_BUFFER_SETS)]
    in_done = [torch.cuda.Event() for _ in range(N_BUFFER_SETS)]
    for ev in fwd_done:
        ev.record(cur)

    def e2e_step(i: int, compute: bool = True):
        k = i % N_BUFFER_SETS
        s = sets[k]
        with torch.cuda.stream(s_in):
            s_in.wait_event(fwd_done[k])     # x_dev[k] was last read by the forward of step i - N_BUFFER_SETS
            x_dev[k].copy_(s["x_host"], non_blocking=True)
            in_done[k].record(s_in)
        cur.wait_event(in_done[k])
        y = modules[k](x_dev[k]) if compute else y_dev[k]
        fwd_done[k].record(cur)
        keep[k] = y
        y.record_stream(s_out)
        with torch.cuda.stream(s_out):
            s_out.wait_event(fwd_done[k])
            s["y_host"].copy_(y, non_blocking=True)

    def e2e_loop(n, compute):
        for i in range(3):
            e2e_step(i, compute)
        cur.wait_stream(s_out)
        sync_all()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            e2e_step(i, compute)
        cur.wait_stream(s_out)
        cur.wait_stream(s_in)
        b.record()
        sync_all()
        return a.elapsed_time(b)

    e2e_steps = max(3, min(args.steps, 40))
    with torch.no_grad():
        e2e_ms = e2e_loop(e2e_steps, True)
    copy_ms = e2e_loop(e2e_steps, False)       # the same copies without any kernel: what the host link allows
    del x_dev, y_dev, keep
    status = nat.device_status()

    elapsed_ms, e2e_ms, copy_ms, gemm_med, quant_med = max_over_ranks(
        [elapsed_ms, e2e_ms, copy_ms, median(gemm_ms), median(quant_ms)], dev, dist)

    sub = {}
    rc = 0
    if extras:
        sub["sustained"] = sustained_record(step, shape, gemm_only, sets, F, local_rank, rank, dev, dist, sync_all, args.sustained_s)
        if rank == 0:
            sub["comparators"] = comparators_record(shape, sets, 20)
        sync_all()
    parity_set = {k: sets[0][k] for k in ("x", "wq", "ws", "bias", "lora")}
    del sets, modules, workspace
    torch.cuda.empty_cache()
    if extras:
        sub["dit"] = dit_record(pkg, args, rank, world, local_rank, dev, dist, steps=10)
        torch.cuda.empty_cache()
        if world > 1:
            sub["c4"] = column_parallel_record(pkg, rank, world, dev, dist, steps=20)
            if rank == 0 and not sub["c4"]["ok"]:
                rc = 1
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    parity = parity_record(pkg, shape, parity_set, dev) if (extras or args.parity) else None
    if parity is not None and not parity["ok"]:
        rc = 1

    ops_step = 2.0 * M * N * K                       # int8 GEMM ops of one rank's step
    value = world * ops_step * args.steps / (elapsed_ms * 1e-3) / 1e12
    e2e_value = world * ops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
    peaks, peak_kind = measured_peaks()
    # int8 tensor throughput is twice the bf16 rate of the same tensor cores; the kernel is timed in a short
    # back-to-back loop of its own, so the burst figure is the denominator
    peak_tops = 2.0 * peaks["bf16_tflops"]
    achieved = ops_step / (gemm_med * 1e-3) / 1e12
    cpu_base, _ = cpu_reference_rate(shape, steps=20, warmup=2, budget_s=12.0)
    k1_bytes = M * K * 3 + 4 * M
    line = {
        "metric": "w8a8_linear_int8_throughput", "value": value, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config_dict(shape, world),
        "frac_of_nominal_int8_peak": value / (world * NOMINAL_INT8_TOPS),
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel<i8, pair" + (", fused LoRA>" if shape.lora_rank else ">"),
                     "achieved": achieved, "peak": peak_tops, "unit": "TOPS", "frac": achieved / peak_tops,
                     "traffic": NCU_GEMM_TRAFFIC_BYTES.get(shape.name),
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the capture "
                                       "summarised in profiles/gemm_tcgen05_i8_pair_c1_quarot_mlp_up.md (not re-measured in this run)",
                     "peak_source": f"2 x bf16_tflops (burst) of {peak_kind} MEASURED_PEAKS.json; int8 ops counted as 2*M*N*K",
                     "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS, "kernel_ms_median": gemm_med,
                     "kernel_ms_best": gemm_ms[0], "kernel_ms_n": len(gemm_ms),
                     "kernel_ms_graph_median": median(gemm_graph_ms),
                     "timing": f"{len(gemm_ms)} event-bracketed launches of the GEMM alone, back to back over the rotating "
                               "buffer sets, after the headline loop; first launch discarded; median (max over ranks)",
                     "quant_kernel": {"kernel": "quant_rows_kernel" + (" (with the Hadamard rotation)" if shape.hadamard else ""),
                                      "bound": "hbm", "kernel_ms_median": quant_med, "kernel_ms_best": quant_ms[0],
                                      "kernel_ms_n": len(quant_ms), "algorithmic_bytes": k1_bytes,
                                      "timing": "8 launches per CUDA-graph replay over the rotating buffer sets, 8 replays, "
                                                "per-launch average of each replay; median (max over ranks)",
                                      "achieved": k1_bytes / (quant_med * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": k1_bytes / (quant_med * 1e-3) / 1e9 / peaks["hbm_gbs"]},
                     "kernels_sum_vs_step_ms": [gemm_med + quant_med, elapsed_ms / args.steps]},
        "cpu_baseline": cpu_base,
        "e2e": {"value": e2e_value, "unit": "TOPS", "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "call": "StandaloneInt8Ops.Linear.forward (the ops-class module) on a device copy of the pinned host input",
                "copy_only_ms_per_step": copy_ms / e2e_steps, "frac_of_copy_roofline": copy_ms / e2e_ms,
                "copy_roofline": "the same pinned H2D + D2H copies on the same three streams with no kernel in between "
                                 "(max over ranks): what the host link delivers to all ranks at once"},
        "gpu_launches": int(launches_timed) * world,
        "clocks": clocks,
        "device_status": status,
    }
    if parity is not None:
        line["parity"] = parity
    line.update(sub)
    cmp_rec = sub.get("comparators") or {}
    if "int_mm_8192_burst_tops" in cmp_rec:
        # the same fraction against the int8 rate the library GEMM reaches on this GPU in this run (burst, 8192^3)
        line["roofline"]["frac_of_library_int8_burst"] = achieved / cmp_rec["int_mm_8192_burst_tops"]
    print(json.dumps(line))
    if rc:
        sys.exit(rc)


def sustained_record(step, shape, gemm_only, sets, F, local_rank, rank, dev, dist, sync_all, seconds: float):
    """The headline step back to back for `seconds` (the chip is power-managed: a 20-step burst runs at the idle
    clock, steady state does not).  The GEMM alone is event-bracketed on every 64th step, which replaces that step's
    fused call by the two separate entry points."""
    import torch
    M, K, N = shape.M, shape.K, shape.N
    n_probe = 200
    sync_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(n_probe):
        step(i)
    b.record()
    torch.cuda.synchronize()
    est_ms = a.elapsed_time(b) / n_probe
    n = int(max(n_probe, min(40000, seconds * 1e3 / est_ms)))
    sampler = ClockSampler(local_rank, period_s=0.02) if rank == 0 else None
    if sampler:
        sampler.start()
    sync_all()
    evs = []
    h0 = time.perf_counter()
    a.record()
    for i in range(n):
        if i % 64 == 63:
            s = sets[i % N_BUFFER_SETS]
            q, xs = F.quantize_rowwise(s["x"], hadamard=shape.hadamard)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            F.linear_w8a8(q, xs, s["wq"], s["ws"], s["bias"], torch.bfloat16)
            e1.record()
            evs.append((e0, e1))
        else:
            step(i)
    b.record()
    sync_all()
    h1 = time.perf_counter()
    ms = a.elapsed_time(b) / n
    clocks = sampler.stop(h0, h1) if sampler else None
    k2 = sorted(x.elapsed_time(y) for x, y in evs) if shape.lora_rank == 0 else [float("nan")]
    ms, k2_med = max_over_ranks([ms, median(k2)], dev, dist)
    peaks, kind = measured_peaks()
    ops = 2.0 * M * N * K
    rec = {"seconds": ms * n / 1e3, "steps": n, "ms_per_step": ms, "tops_per_gpu": ops / (ms * 1e-3) / 1e12,
           "gemm_ms_median": k2_med, "gemm_tops": ops / (k2_med * 1e-3) / 1e12, "gemm_samples": len(k2),
           "frac_of_2x_bf16_sustained": ops / (k2_med * 1e-3) / 1e12 / (2.0 * peaks["bf16_tflops_sustained"]),
           "frac_of_nominal_4500": ops / (k2_med * 1e-3) / 1e12 / NOMINAL_INT8_TOPS,
           "peak_source": f"2 x bf16_tflops_sustained of {kind} MEASURED_PEAKS.json", "clocks": clocks}
    if clocks and clocks.get("sm_mhz"):
        # time x clock = cycles: compares burst and sustained numbers clock for clock
        rec["gemm_ms_times_sm_mhz"] = k2_med * clocks["sm_mhz"]
        rec["step_ms_times_sm_mhz"] = ms * clocks["sm_mhz"]
    return rec


# ------------------------------------------------------------- DiT workload
def dit_config_dict(cfg, world, graph):
    return {"workload": "c3_synthetic_dit_step", "batch_per_gpu": 1, "img_tokens": cfg.img_tokens,
            "txt_tokens": cfg.txt_tokens, "hidden": cfg.hidden, "heads": cfg.heads, "double_blocks": cfg.double_blocks,
            "single_blocks": cfg.single_blocks, "int8_params_B": cfg.int8_params() / 1e9,
            "int8_TOP_per_step": cfg.int8_ops() / 1e12, "attention_TFLOP_per_step": cfg.attention_flops() / 1e12,
            "linears": "int8 tensorwise weights, per-token activation quant", "attention": "bf16 SDPA",
            "parallelism": f"one sample per GPU x{world}", "cuda_graph": graph,
            "l2": "6.7 GB of int8 weights stream through the 126 MB L2 every step"}


def dit_cpu_seconds(cfg, budget_s: float):
    """CPU estimate of one step: the oracle linear timed on 512 tokens of the two MLP shapes, scaled by op count
    (attention and element-wise work are left out, which favours the CPU)."""
    import __graft_entry__ as g
    wl = g.load_package().workloads
    rates = []
    for name in ("c1_quarot_mlp_up",):
        base, _ = cpu_reference_rate(wl.LinearShape(name, 4608, cfg.hidden, cfg.mlp_hidden, False, False, True), 10, 2, budget_s)
        rates.append(base)
    tops = sum(r["value"] for r in rates) / len(rates)
    return cfg.int8_ops() / (tops * 1e12), rates[0]


def dit_record(pkg, args, rank, world, local_rank, dev, dist, steps: int, graph_wanted: bool = True, fused: bool = True):
    """Times the synthetic DiT denoising step on every rank (one sample per GPU, no communication) and returns the
    measurements (max over ranks) as a dict; rank 0's dict is the one that is printed."""
    import importlib
    import torch
    dit = importlib.import_module(pkg.__name__ + ".dit")
    cfg = dit.DiTConfig()
    sync_all = make_sync(dist)
    model = dit.SyntheticDiT(cfg, seed=0, device=dev, fused=fused)
    gen = torch.Generator().manual_seed(1000 + rank)
    img_h = torch.randn(1, cfg.img_tokens, cfg.in_channels, generator=gen).bfloat16().pin_memory()
    txt_h = torch.randn(1, cfg.txt_tokens, cfg.txt_dim, generator=gen).bfloat16().pin_memory()
    out_h = torch.empty(1, cfg.img_tokens, cfg.in_channels, dtype=torch.bfloat16).pin_memory()
    img, txt = img_h.to(dev), txt_h.to(dev)
    t = torch.full((1,), 0.5, device=dev)
    nat = pkg._native

    for _ in range(3):
        out = model(img, txt, t)
    sync_all()
    eager_out = out.clone()
    launches0 = nat.load().i8f_launch_count()
    model(img, txt, t)
    launches_per_step = int(nat.load().i8f_launch_count() - launches0)
    graph = None
    if graph_wanted:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                model(img, txt, t)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = model(img, txt, t)
            graph.replay()
            sync_all()
        except Exception as e:  # noqa: BLE001
            print(f"CUDA graph capture failed ({e!r}); running eagerly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def step():
        nonlocal out
        if graph is not None:
            graph.replay()
        else:
            out = model(img, txt, t)

    for _ in range(3):
        step()
    sync_all()
    replay_equals_eager = bool(torch.equal(out, eager_out)) if graph is not None else None
    sampler = ClockSampler(local_rank, period_s=0.02) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    host_t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    sync_all()
    host_t1 = time.perf_counter()
    ms = e0.elapsed_time(e1) / steps
    clocks = sampler.stop(host_t0, host_t1) if sampler else None

    def e2e_step():
        img.copy_(img_h, non_blocking=True)
        txt.copy_(txt_h, non_blocking=True)
        step()
        out_h.copy_(out, non_blocking=True)

    e2e_step()
    sync_all()
    e0.record()
    for _ in range(steps):
        e2e_step()
    e1.record()
    sync_all()
    e2e_ms = e0.elapsed_time(e1) / steps
    status = nat.device_status()
    finite = bool(torch.isfinite(out.float()).all())
    ms, e2e_ms = max_over_ranks([ms, e2e_ms], dev, dist)
    del model, graph
    peaks, peak_kind = measured_peaks()
    peak_tops = 2.0 * peaks["bf16_tflops_sustained"]
    achieved = cfg.int8_ops() / (ms * 1e-3) / 1e12
    return {"ms_per_step": ms, "s_per_it": ms * 1e-3, "steps": steps,
            "block_code": "fused (LayerNorm+modulate and GELU inside the quantiser, one qkv buffer, per-head RMS-norm kernel)"
                          if fused else "unfused (every element-wise step its own PyTorch call)", "cuda_graph": graph_wanted and replay_equals_eager is not None,
            "graph_replay_equals_eager": replay_equals_eager, "samples_per_s_all_gpus": world / (ms * 1e-3),
            "n_gpus": world, "parallelism": f"one 1024x1024 sample per GPU x{world}, no communication",
            "int8_TOP_per_step": cfg.int8_ops() / 1e12, "attention_TFLOP_per_step": cfg.attention_flops() / 1e12,
            "int8_params_B": cfg.int8_params() / 1e9, "int8_tops_over_whole_step": achieved,
            "frac_of_2x_bf16_sustained_whole_step": achieved / peak_tops, "peak_source": f"{peak_kind} MEASURED_PEAKS.json",
            "e2e_ms_per_step": e2e_ms, "h2d_bytes_per_step": img_h.numel() * 2 + txt_h.numel() * 2,
            "d2h_bytes_per_step": out_h.numel() * 2, "library_launches_per_step": launches_per_step,
            "clocks": clocks, "device_status": status, "output_finite": finite}


def run_dit(args):
    import importlib
    import torch
    import __graft_entry__ as g
    pkg = g.load_package()
    dit = importlib.import_module(pkg.__name__ + ".dit")
    cfg = dit.DiTConfig()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        sec, base = dit_cpu_seconds(cfg, budget_s=40.0)
        base = dict(base, value=sec, unit="s/it", sample=base["sample"] + "; step time = int8 ops / that rate")
        print(json.dumps({"impl": "reference", "metric": "dit_step_time", "value": sec, "unit": "s/it", "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": False,
                          "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                          "config": dit_config_dict(cfg, max(1, args.gpus), False), "cpu_baseline": base,
                          "e2e": {"value": sec, "unit": "s/it", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                          "gpu_launches": 0}))
        return
    rank, world, local_rank, dev, dist = rank_context()
    steps = min(args.steps, 20)
    rec = dit_record(pkg, args, rank, world, local_rank, dev, dist, steps, graph_wanted=not args.no_graph,
                     fused=not args.dit_unfused)
    if dist is not None:
        dist.destroy_process_group()
    if rank != 0:
        return
    ms = rec["ms_per_step"]
    peaks, peak_kind = measured_peaks()
    peak_tops = 2.0 * peaks["bf16_tflops_sustained"]
    achieved = rec["int8_tops_over_whole_step"]
    cpu_sec, cpu_base = dit_cpu_seconds(cfg, budget_s=12.0)
    cpu_base = dict(cpu_base, value=cpu_sec, unit="s/it", sample=cpu_base["sample"] + "; step time = int8 ops / that rate")
    print(json.dumps({
        "metric": "dit_step_time", "value": ms * 1e-3, "unit": "s/it", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic", "config": dit_config_dict(cfg, world, rec["cuda_graph"]),
        "samples_per_s_all_gpus": world / (ms * 1e-3), "graph_replay_equals_eager": rec["graph_replay_equals_eager"],
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel<i8,256> (whole step)", "achieved": achieved,
                     "peak": peak_tops, "unit": "TOPS", "frac": achieved / peak_tops, "traffic": None,
                     "peak_source": f"2 x bf16_tflops_sustained of {peak_kind} MEASURED_PEAKS.json; achieved = int8 linear ops "
                                    "/ WHOLE step time (attention, norms and element-wise work included in the time)",
                     "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS},
        "cpu_baseline": cpu_base,
        "e2e": {"value": rec["e2e_ms_per_step"] * 1e-3, "unit": "s/it", "h2d_bytes_per_step": rec["h2d_bytes_per_step"],
                "d2h_bytes_per_step": rec["d2h_bytes_per_step"], "steps": steps},
        "gpu_launches": rec["library_launches_per_step"] * steps * world, "clocks": rec["clocks"],
        "device_status": rec["device_status"], "output_finite": rec["output_finite"]}))


# ------------------------------------------- column-parallel sweep (config 4)
NVLINK_PEER_GBS = 770.0   # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)


def column_parallel_record(pkg, rank, world, dev, dist, steps: int, m_sweep=(1024, 4096, 16384, 32768)):
    """W8A8 linear K=4096, N=16384 split over the ranks by output channel; every rank quantises the full x and runs
    its slice.  The bf16 [M, N/P] blocks are gathered two ways: NCCL all-gather (blocks as they land, and with the
    row-major re-layout), and the fused form whose GEMM epilogue stores every tile into all ranks' buffers over
    NVLink.  Also checks, on every rank, that the fused result equals the NCCL one and, at M = 1024, that the
    gathered [M, N] equals the unsharded computation of the same inputs bit for bit."""
    import torch
    F, par, wl = pkg.functional, pkg.parallel, pkg.workloads
    K, N = 4096, 16384
    w = wl.weight_fp32(N, K, seed=4)
    b0, e0_ = par.shard_bounds(N, world, rank)
    wq_full, ws_full = F.quantize_weight_rows(w.to(dev))            # per-channel scales: row-local, shard = slice
    shard = par.shard_columns(wq_full, ws_full, None, world, rank)
    wq, ws = shard.weight, shard.weight_scale
    n_local = e0_ - b0
    results = []
    all_ok = True
    fused = par.FusedColumnParallelOutput(max(m_sweep), N, torch.bfloat16, dev)
    for M in m_sweep:
        x = wl.activation(M, K, seed=40).to(dev)          # same bits on every rank
        gathered = torch.empty((world * M, n_local), dtype=torch.bfloat16, device=dev)   # [P, M, N/P] blocks
        full = torch.empty((M, N), dtype=torch.bfloat16, device=dev)

        def step_nccl(relayout: bool):
            q, xs = F.quantize_rowwise(x)
            y = F.linear_w8a8(q, xs, wq, ws, None, torch.bfloat16)
            dist.all_gather_into_tensor(gathered, y)
            if relayout:
                full.view(M, world, n_local).copy_(gathered.view(world, M, n_local).transpose(0, 1))
            return y

        def timed(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                fn()
            b.record()
            torch.cuda.synchronize()
            dist.barrier()
            return max_over_ranks([a.elapsed_time(b) / steps], dev, dist)[0]

        ms_blocks = timed(lambda: step_nccl(False))
        ms_full = timed(lambda: step_nccl(True))
        ms_fused = timed(lambda: fused.forward(x, shard))
        y_all = fused.forward(x, shard)
        step_nccl(True)
        torch.cuda.synchronize()
        flags = [1.0 if torch.equal(y_all, full) else 0.0]
        if M == min(m_sweep):
            unsharded = F.linear_forward(x, wq_full, ws_full, None, torch.bfloat16)
            flags.append(1.0 if torch.equal(full, unsharded) and torch.equal(y_all, unsharded) else 0.0)
            del unsharded
        if dist is not None:
            t = torch.tensor(flags, device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)          # true only if true on every rank
            flags = t.tolist()
        ops = 2.0 * M * N * K
        comm_bytes = 2.0 * M * N * (world - 1) / world
        nvlink_ms = comm_bytes / (NVLINK_PEER_GBS * 1e9) * 1e3
        compute_ms = (ops / world) / (2.0 * measured_peaks()[0]["bf16_tflops"] * 1e12) * 1e3   # this rank's slice of the GEMM
        floor_ms = max(nvlink_ms, compute_ms)
        rec = {"M": M, "compute_floor_ms": compute_ms, "roofline_ms": floor_ms, "frac_of_roofline_fused": floor_ms / ms_fused,
               "ms_fused_epilogue_scatter": ms_fused, "ms_nccl_blocks_layout": ms_blocks,
               "ms_nccl_row_major_layout": ms_full, "fused_equals_nccl_result": bool(flags[0] == 1.0),
               "tops_fused": ops / (ms_fused * 1e-3) / 1e12, "allgather_bytes_in_per_gpu": comm_bytes,
               "nvlink_roofline_ms": nvlink_ms, "frac_of_nvlink_roofline_fused": nvlink_ms / ms_fused,
               "frac_of_nvlink_roofline_nccl_blocks": nvlink_ms / ms_blocks}
        if len(flags) > 1:
            rec["equals_unsharded"] = bool(flags[1] == 1.0)
            all_ok = all_ok and rec["equals_unsharded"]
        all_ok = all_ok and rec["fused_equals_nccl_result"]
        results.append(rec)
        del x, gathered, full, y_all
    torch.cuda.synchronize()
    status = pkg._native.device_status()
    status = int(max_over_ranks([status], dev, dist)[0])
    del fused
    return {"workload": "c4_column_parallel", "K": K, "N": N, "n_gpus": world, "steps": steps,
            "parallelism": f"column-parallel x{world}: NCCL all-gather of bf16 [M, N/P] blocks vs GEMM-epilogue scatter over NVLink",
            "sweep": results, "device_status": status, "ok": bool(all_ok and status == 0),
            "nvlink_peer_gbs": NVLINK_PEER_GBS,
            "note": "communication-bound by construction (bytes per op fixed by K): the roofline is NVLink, "
                    f"{NVLINK_PEER_GBS} GB/s per direction per GPU (measured peer copy); weights (64 MB / P per rank) stay "
                    "L2-resident across steps"}


def run_column_parallel(args):
    """One line with a result per M of the column-parallel sweep (needs more than one rank)."""
    import torch
    import __graft_entry__ as g
    K, N = 4096, 16384
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        wl = g.load_package().workloads
        base, dt = cpu_reference_rate(wl.LinearShape("c4_column_parallel", 4096, K, N, False, True, False), args.steps,
                                      args.warmup, budget_s=40.0)
        print(json.dumps({"impl": "reference", "metric": "w8a8_linear_int8_throughput", "value": base["value"], "unit": "TOPS",
                          "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
                          "data": "synthetic", "config": {"workload": "c4_column_parallel", "K": K, "N": N, "M": 4096},
                          "cpu_baseline": base, "gpu_launches": 0,
                          "e2e": {"value": base["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    rank, world, local_rank, dev, dist = rank_context()
    if world < 2:
        raise SystemExit("the column-parallel sweep needs at least two ranks (torchrun --nproc-per-node N bench.py --workload c4)")
    pkg = g.load_package()
    steps = min(args.steps, 50)
    rec = column_parallel_record(pkg, rank, world, dev, dist, steps)
    dist.barrier()
    dist.destroy_process_group()
    if rank != 0:
        return
    ref = next(r for r in rec["sweep"] if r["M"] == 4096)
    print(json.dumps({"metric": "w8a8_linear_int8_throughput", "value": ref["tops_fused"], "unit": "TOPS", "n_gpus": world,
                      "steps": steps, "warmup": 3, "ms_per_step": ref["ms_fused_epilogue_scatter"], "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                      "config": {"workload": "c4_column_parallel", "K": K, "N": N, "M": 4096, "weight_scale": "per_channel",
                                 "parallelism": rec["parallelism"],
                                 "l2": "weights 64 MB / P per rank stay L2-resident across steps (real layers would not)"},
                      "sweep": rec["sweep"], "gpu_launches": 4 * steps * world, "device_status": rec["device_status"],
                      "ok": rec["ok"], "note": rec["note"]}))
    if not rec["ok"]:
        sys.exit(1)


# ------------------------------------------- stochastic LoRA merge (config 2, second variant)
def run_merge(args):
    """One step = one stochastic-rounding merge of a rank-64 LoRA (bf16 factors, Philox uniforms keyed by the
    node's seed) into int8 weights [4096, 4096] with per-channel scales.  HBM-bound by design: the algorithmic
    traffic is the weights read + written plus the factors and scales."""
    import torch
    import __graft_entry__ as g
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    N = K = 4096
    r = 64
    bytes_step = 2.0 * N * K + 2.0 * r * (N + K) + 4.0 * N
    pkg = g.load_package()
    wl = pkg.workloads
    cfg = {"workload": "c2_stochastic_lora_merge", "N": N, "K": K, "rank": r, "factors": "bf16", "weight_scale": "per_channel",
           "rng": "Philox4x32-10, seed 318008", "parallelism": f"independent layers x{world}",
           "l2": "weights rotate over 8 buffers (134 MB > 126 MB L2)"}
    if args.impl == "reference":
        if rank != 0:
            return
        from oracle import torch_path as tp
        torch.set_num_threads(os.cpu_count() or 1)
        w = wl.weight_fp32(N, K, seed=0)
        wq, ws = tp.quantize_rowwise(w)
        down, up = wl.lora_factors(N, K, r, seed=0)
        u = wl.uniforms(N, K, seed=0)
        tp.lora_merge(wq, ws, up, down, 1.0, u)
        n = max(1, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(n):
            tp.lora_merge(wq, ws, up, down, 1.0, u)
        dt = (time.perf_counter() - t0) / n
        base = {"value": bytes_step / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port",
                "sample": f"the full merge, {n} passes of {dt * 1e3:.1f} ms (uniforms pre-drawn)"}
        print(json.dumps({"impl": "reference", "metric": "lora_merge_sr_bandwidth", "value": base["value"], "unit": "GB/s",
                          "n_gpus": args.gpus, "steps": n, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": cfg,
                          "cpu_baseline": base, "gpu_launches": 0,
                          "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    F = pkg.functional
    wq0, ws = F.quantize_weight_rows(wl.weight_fp32(N, K, seed=rank).to(dev))
    down, up = wl.lora_factors(N, K, r, seed=rank)
    down, up = down.to(dev), up.to(dev)
    bufs = [wq0.clone() for _ in range(8)]
    for i in range(max(3, args.warmup)):
        F.lora_merge_sr_(bufs[i % 8], ws, up, down, 1.0, seed=318008)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0 = time.perf_counter()
    a.record()
    for i in range(args.steps):
        F.lora_merge_sr_(bufs[i % 8], ws, up, down, 1.0, seed=318008)
    b.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    h1 = time.perf_counter()
    ms = a.elapsed_time(b) / args.steps
    clocks = sampler.stop(h0, h1) if sampler else None
    # end to end: int8 weights and factors from pinned host memory, merged weights back to the host
    w_host, out_host = wq0.cpu().pin_memory(), torch.empty((N, K), dtype=torch.int8).pin_memory()
    up_h, down_h = up.cpu().pin_memory(), down.cpu().pin_memory()
    e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        wd = w_host.to(dev, non_blocking=True)
        F.lora_merge_sr_(wd, ws, up_h.to(dev, non_blocking=True), down_h.to(dev, non_blocking=True), 1.0, seed=318008)
        out_host.copy_(wd, non_blocking=True)

    e2e_step()
    torch.cuda.synchronize()
    a.record()
    for _ in range(e_steps):
        e2e_step()
    b.record()
    torch.cuda.synchronize()
    e2e_ms = a.elapsed_time(b) / e_steps
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = (float(v) for v in t.tolist())
        dist.destroy_process_group()
    if rank != 0:
        return
    peaks, kind = measured_peaks()
    achieved = bytes_step / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "lora_merge_sr_bandwidth", "value": world * achieved, "unit": "GB/s", "n_gpus": world,
                      "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": cfg,
                      "roofline": {"bound": "hbm", "kernel": "lora_merge_tc_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"],
                                   "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                                   "peak_source": f"hbm_gbs of {kind} MEASURED_PEAKS.json; time includes host launch gaps "
                                                  "(one launch per step, back to back)"},
                      "e2e": {"value": world * bytes_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                              "h2d_bytes_per_step": N * K + 2 * r * (N + K), "d2h_bytes_per_step": N * K, "steps": e_steps},
                      "gpu_launches": args.steps * world, "clocks": clocks, "device_status": pkg._native.device_status()}))


def run_small_batch(args):
    """One step = one Linear call with M tokens <= 16 (a modulation-sized call: M=1, K=4096, N=24576) through the
    tiny-batch branch: unquantised activations against int8 weights dequantised inside the kernel.  HBM-bound: the
    algorithmic traffic is the int8 weights once, plus activations, bias and output."""
    import torch
    import __graft_entry__ as g
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    M, K, N = 1, 4096, 24576
    bytes_step = float(N * K + 2 * M * K + 2 * N + 2 * M * N + 4)
    pkg = g.load_package()
    wl = pkg.workloads
    n_sets = 8
    cfg = {"workload": "small_batch_modulation_linear", "M_per_gpu": M, "K": K, "N": N, "weight_scale": "tensorwise",
           "bias": True, "out_dtype": "bf16", "parallelism": f"independent calls x{world}",
           "l2": f"weights rotate over {n_sets} buffers ({n_sets * N * K / 1e6:.0f} MB > 126 MB L2)"}
    metric = "small_batch_linear_weight_bandwidth"
    if args.impl == "reference":
        if rank != 0:
            return
        from oracle import torch_path as tp
        torch.set_num_threads(os.cpu_count() or 1)
        x = wl.activation(M, K, seed=0)
        wq, ws = tp.quantize_tensorwise(wl.weight_fp32(N, K, seed=0))
        b = wl.bias_fp32(N, seed=0).bfloat16()
        tp.linear_small_batch(x, wq, ws, b)
        n = max(1, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(n):
            tp.linear_small_batch(x, wq, ws, b)
        dt = (time.perf_counter() - t0) / n
        base = {"value": bytes_step / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port",
                "sample": f"the full call, {n} passes of {dt * 1e3:.1f} ms"}
        print(json.dumps({"impl": "reference", "metric": metric, "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
                          "steps": n, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg, "cpu_baseline": base,
                          "gpu_launches": 0,
                          "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    F = pkg.functional
    wq0, ws = F.quantize_tensorwise(wl.weight_fp32(N, K, seed=rank).to(dev))
    ws = ws.reshape(1)
    weights = [wq0.clone() for _ in range(n_sets)]
    bias = wl.bias_fp32(N, seed=rank).bfloat16().to(dev)
    x = wl.activation(M, K, seed=rank).to(dev)
    steps = max(n_sets, (args.steps // n_sets) * n_sets)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(max(3, args.warmup)):
            y = F.linear_small_batch(x, weights[i % n_sets], ws, bias)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(n_sets):
                y = F.linear_small_batch(x, weights[i], ws, bias)
    graph.replay()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0 = time.perf_counter()
    a.record()
    for _ in range(steps // n_sets):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    h1 = time.perf_counter()
    ms = a.elapsed_time(b) / steps
    clocks = sampler.stop(h0, h1) if sampler else None

    # comparator (not the product path): the reference's expression with library kernels on this GPU
    def torch_expression(w):
        return torch.nn.functional.linear(x, (w.float() * ws).to(x.dtype), bias)
    for i in range(3):
        torch_expression(weights[i])
    a.record()
    for i in range(n_sets):
        torch_expression(weights[i])
    b.record()
    torch.cuda.synchronize()
    lib_ms = a.elapsed_time(b) / n_sets

    # end to end: activations from pinned host memory, output back to the host, every step
    x_host, y_host = x.cpu().pin_memory(), torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    e_steps = max(3, min(args.steps, 50))

    def e2e_step(i):
        y_host.copy_(F.linear_small_batch(x_host.to(dev, non_blocking=True), weights[i % n_sets], ws, bias), non_blocking=True)

    e2e_step(0)
    torch.cuda.synchronize()
    a.record()
    for i in range(e_steps):
        e2e_step(i)
    b.record()
    torch.cuda.synchronize()
    e2e_ms = a.elapsed_time(b) / e_steps
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = (float(v) for v in t.tolist())
        dist.destroy_process_group()
    if rank != 0:
        return
    peaks, kind = measured_peaks()
    achieved = bytes_step / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": metric, "value": world * achieved, "unit": "GB/s", "n_gpus": world, "steps": steps,
                      "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
                      "roofline": {"bound": "hbm", "kernel": "small_m_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"],
                                   "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_SMALL_M_TRAFFIC_BYTES,
                                   "peak_source": f"hbm_gbs of {kind} MEASURED_PEAKS.json; launches replayed from a CUDA "
                                                  f"graph of {n_sets}"},
                      "library_expression_ms": lib_ms,
                      "e2e": {"value": world * bytes_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                              "h2d_bytes_per_step": 2 * M * K, "d2h_bytes_per_step": 2 * M * N, "steps": e_steps},
                      "gpu_launches": steps * world, "clocks": clocks, "device_status": pkg._native.device_status()}))


def run_prologue(args):
    """The quantiser prologues and the per-head RMS norm alone, on the shapes of the synthetic DiT (4608 tokens): one
    JSON line with the time and achieved HBM rate of each.  Inputs rotate over buffer sets larger than L2."""
    import torch
    import __graft_entry__ as g
    rank, world, local_rank, dev, dist = rank_context()
    pkg = g.load_package()
    F = pkg.functional
    T, h, m = 4608, 4096, 12288
    n_sets = 4
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    xs_h = [torch.randn(T, h, generator=gen, device=dev).bfloat16() for _ in range(n_sets * 2)]       # 38 MB each
    ys = [torch.randn(T, 3 * h + m, generator=gen, device=dev).bfloat16() for _ in range(n_sets)]      # 226 MB each
    attn = [torch.randn(T, h, generator=gen, device=dev).bfloat16() for _ in range(n_sets)]
    shift = (torch.randn(h, generator=gen, device=dev) * 0.1).bfloat16()
    scale = (torch.randn(h, generator=gen, device=dev) * 0.1).bfloat16()
    cases = {
        "ln_modulate_quant_kernel [4608 x 4096]": (lambda i: F.quantize_rowwise_ln_modulate(xs_h[i % len(xs_h)], shift, scale), T * h * 3 + 4 * T + 4 * h),
        "gelu_quant (table) [4608 x (4096 plain + 12288 GELU)]": (lambda i: F.quantize_rowwise_gelu(ys[i % n_sets][:, 3 * h:], attn[i % n_sets]), T * (h + m) * 3 + 4 * T),
        "gelu_quant (table) [4608 x 12288]": (lambda i: F.quantize_rowwise_gelu(ys[i % n_sets][:, :m]), T * m * 3 + 4 * T),
        "rmsnorm_heads_kernel [4608 x 8192 of a 24576-wide buffer]": (lambda i: F.rmsnorm_heads_(ys[i % n_sets][:, : 2 * h]), T * 2 * h * 4),
        "quant_rows_kernel [4608 x 4096] (plain quantiser, for comparison)": (lambda i: F.quantize_rowwise(xs_h[i % len(xs_h)]), T * h * 3 + 4 * T),
    }
    peaks, kind = measured_peaks()
    out = {}
    for name, (fn, nbytes) in cases.items():
        side = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(side):
            for i in range(8):
                fn(i)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(8):
                    fn(i)
        torch.cuda.synchronize()
        ts = []
        for _ in range(max(4, min(args.steps, 12))):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / 8)
        ms = median(ts[1:])
        out[name] = {"ms": ms, "algorithmic_bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
                     "frac_of_hbm": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        del graph
    if dist is not None:
        dist.destroy_process_group()
    if rank != 0:
        return
    head = out["gelu_quant (table) [4608 x (4096 plain + 12288 GELU)]"]
    print(json.dumps({"metric": "quantiser_prologue_bandwidth", "value": head["gbs"], "unit": "GB/s", "n_gpus": world,
                      "steps": args.steps, "warmup": 8, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "dit_quantiser_prologues", "tokens": T, "hidden": h, "mlp_hidden": m,
                                 "l2": "inputs rotate over 4 to 8 buffer sets (150 MB to 900 MB > 126 MB L2)"},
                      "roofline": {"bound": "hbm", "kernel": "gelu_quant_table_kernel", "achieved": head["gbs"], "peak": peaks["hbm_gbs"],
                                   "unit": "GB/s", "frac": head["frac_of_hbm"], "traffic": None,
                                   "peak_source": f"hbm_gbs of {kind} MEASURED_PEAKS.json; launches replayed from a CUDA graph of 8"},
                      "kernels": out, "gpu_launches": 8 * len(cases), "device_status": pkg._native.device_status()}))


def run_subwave(args):
    """GEMMs that do not fill one wave of tiles (few tokens, the text stream of the DiT, the LoRA down projection): one
    JSON line with the CUDA-graph-timed launch of each, cuBLAS `torch._int_mm` on the same int8 operands beside the
    int8 ones (no epilogue there), and an equality check of the int32 accumulators against it."""
    import torch
    import __graft_entry__ as g
    rank, world, local_rank, dev, dist = rank_context()
    pkg = g.load_package()
    F = pkg.functional
    gen = torch.Generator(device=dev).manual_seed(11 + rank)

    def timed(fn, n=20, reps=6):
        side = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(n):
                    fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / n)
        del graph
        return median(ts[1:])

    out = {}
    launches = 0
    all_equal = True
    for (M, K, N) in [(17, 4096, 4096), (64, 4096, 4096), (256, 3072, 3072), (512, 4096, 4096), (512, 4096, 12288),
                      (512, 12288, 4096), (1024, 4096, 4096)]:
        q = torch.randint(-127, 128, (M, K), generator=gen, dtype=torch.int8, device=dev)
        w = torch.randint(-127, 128, (N, K), generator=gen, dtype=torch.int8, device=dev)
        qs = torch.rand(M, 1, generator=gen, device=dev) * 0.02 + 0.001
        ws = torch.full((1,), 0.01, device=dev)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: F.linear_w8a8(q, qs, w, ws, None, torch.bfloat16, out=y))
        rec = {"ms": ms, "tops": 2.0 * M * N * K / (ms * 1e-3) / 1e12}
        if M > 16:       # the library routine wants more than 16 rows
            wt = w.t()
            rec["int_mm_ms"] = timed(lambda: torch._int_mm(q, wt))
            equal = bool(torch.equal(F.gemm_i8_i32(q, w), torch._int_mm(q, wt)))
            rec["int32_equals_int_mm"] = equal
            all_equal = all_equal and equal
        out[f"w8a8 M={M} K={K} N={N}"] = rec
        launches += 20
    for (M, K, r) in [(8192, 4096, 64), (4608, 4096, 16)]:
        x = torch.randn(M, K, generator=gen, device=dev).bfloat16()
        a = (torch.randn(r, K, generator=gen, device=dev) * 0.02).bfloat16()
        ms = timed(lambda: F.lora_down(x, a))
        nbytes = 2 * M * K + 2 * r * K + 2 * M * r
        peaks, kind = measured_peaks()
        want = (x.float() @ a.float().t())
        got = F.lora_down(x, a).float()
        # the result is rounded to bf16: allow one step at the value's magnitude (2^-8 relative) on top of the RMS floor
        err = float(((got - want).abs() / (want.abs() + want.pow(2).mean().sqrt())).max())
        out[f"lora_down M={M} K={K} r={r}"] = {"ms": ms, "algorithmic_bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
                                                "frac_of_hbm": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                                "max_err_over_magnitude_vs_fp32": err}
        all_equal = all_equal and err <= 2.0 ** -8
        launches += 20
    status = pkg._native.device_status()
    if dist is not None:
        dist.destroy_process_group()
    if rank != 0:
        return
    head = out["lora_down M=8192 K=4096 r=64"]
    print(json.dumps({"metric": "lora_down_bandwidth", "value": head["gbs"], "unit": "GB/s", "n_gpus": world, "steps": 20,
                      "warmup": 3, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "sub_wave_gemms", "l2": "operands of the int8 cases are L2-resident by design (they "
                                 "are smaller than L2 in the model too); the LoRA input (67 MB) is re-read from HBM"},
                      "roofline": {"bound": "hbm", "kernel": "gemm_tcgen05_kernel<bf16, 64, single, K split>", "achieved": head["gbs"],
                                   "peak": measured_peaks()[0]["hbm_gbs"], "unit": "GB/s", "frac": head["frac_of_hbm"], "traffic": None},
                      "kernels": out, "ok": all_equal, "gpu_launches": launches, "device_status": status}))
    if not all_equal or status != 0:
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", choices=["c0", "c1", "c2", "c2merge", "c4", "dit", "smallm", "prologue", "subwave"], default="c1")
    ap.add_argument("--no-graph", action="store_true", help="dit: run eagerly instead of replaying a CUDA graph")
    ap.add_argument("--dit-unfused", action="store_true",
                    help="dit: the block code without the fused quantiser prologues (every element-wise step a PyTorch call)")
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--headline-only", action="store_true",
                    help="c1: skip the sub-records (sustained loop, comparators, DiT step, column-parallel sweep, parity)")
    ap.add_argument("--parity", action="store_true", help="with --headline-only or another workload: still log the parity record")
    ap.add_argument("--sustained-s", type=float, default=2.5, help="length of the sustained-load loop in seconds")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "dit":
        run_dit(args)
    elif args.workload == "c4":
        run_column_parallel(args)
    elif args.workload == "c2merge":
        run_merge(args)
    elif args.workload == "smallm":
        run_small_batch(args)
    elif args.workload == "prologue":
        run_prologue(args)
    elif args.workload == "subwave":
        run_subwave(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
