#!/usr/bin/env python
"""Benchmark of the W8A8 linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c0|c2] [--impl reference]

One "step" is one pass of the hot path over one batch of synthetic input:
(Hadamard rotation +) per-token int8 quantisation, the int8 tensor-core GEMM
and the dequantising epilogue (plus the dynamic-LoRA kernels for c2).  The
default workload is the QuaRot MLP-up linear (M=4096, K=4096, N=12288).  With
N > 1 every rank runs its own batch of tokens against replicated weights
(token-parallel, no data-path collective), so scaling is weak.

Prints ONE JSON line (rank 0).  `value` is aggregate int8 tensor throughput
with inputs resident in HBM; `e2e` is the same metric through the public
module call with host buffers (pinned host -> device copy of the activations
and device -> host copy of the output inside the timed region).
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
def run_gpu_arm(args):
    import torch
    import __graft_entry__ as g

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
        dist.init_process_group("nccl", device_id=dev)

    pkg = g.load_package()
    F, nat = pkg.functional, pkg._native
    nat.require_device(dev)
    shape = workload_shape(args.workload)
    M, K, N = shape.M, shape.K, shape.N
    out_dtype = torch.bfloat16

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
    gemm_events = []

    workspace = torch.empty((nat.load().i8f_linear_workspace_bytes(M, K),), dtype=torch.uint8, device=dev)
    EVENT_EVERY = 8   # the GEMM launch is bracketed by CUDA events on every 8th step of the timed region

    def step(i: int, timed: bool):
        s = sets[i % N_BUFFER_SETS]
        if s["lora"] is None and not (timed and i % EVENT_EVERY == 0):
            # the public fused call: K1 and K2 back to back on the stream (programmatic dependent launch), no events
            return F.linear_forward(s["x"], s["wq"], s["ws"], s["bias"], out_dtype, hadamard=shape.hadamard,
                                    workspace=workspace)
        if s["lora"] is not None and not (timed and i % EVENT_EVERY == 0):
            # the public fused-LoRA op: K1 and the LoRA down projection overlap on two streams, then the fused GEMM
            return pkg.custom_ops.linear_lora_forward(s["x"], s["wq"], s["ws"], s["bias"], s["lora"][0], s["lora"][1], out_dtype,
                                                      shape.hadamard, False, nat.EPI_PYTORCH)
        timed = timed and i % EVENT_EVERY == 0
        q, xs = F.quantize_rowwise(s["x"], hadamard=shape.hadamard)
        # dynamic LoRA: t = x @ A^T, then the int8 GEMM accumulates t @ B^T in a second tensor-memory accumulator
        lora_t = F.lora_down(s["x"], s["lora"][0]) if s["lora"] is not None else None
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        if lora_t is not None:
            y = F.linear_w8a8_lora(q, xs, s["wq"], s["ws"], s["bias"], lora_t, s["lora"][1], out_dtype)
        else:
            y = F.linear_w8a8(q, xs, s["wq"], s["ws"], s["bias"], out_dtype)
        if timed:
            e1.record()
            gemm_events.append((e0, e1))
        return y


    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i, False)
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
        step(i, True)
    t_end.record()
    launches_timed = nat.load().i8f_launch_count() - launches_before   # counted by the library itself
    sync_all()
    host_t1 = time.perf_counter()
    elapsed_ms = t_start.elapsed_time(t_end)
    clocks = sampler.stop(host_t0, host_t1) if sampler else None
    gemm_ms = sorted(a.elapsed_time(b) for a, b in gemm_events)
    gemm_avg_ms = sum(gemm_ms) / len(gemm_ms)

    # end-to-end: host buffers through the public forward call, copies inside the timed region.  The three phases of
    # consecutive steps overlap as a serving loop would run them: host->device copy on one stream, the forward on the
    # current stream, device->host copy of the result on a third (PCIe is full duplex); every step still moves its own
    # input and its own output.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    cur = torch.cuda.current_stream(dev)
    x_dev = [torch.empty_like(s["x"]) for s in sets]
    keep = [None] * N_BUFFER_SETS            # outputs stay referenced until their copy-out has been enqueued again
    fwd_done = [torch.cuda.Event() for _ in range(N_BUFFER_SETS)]
    in_done = [torch.cuda.Event() for _ in range(N_BUFFER_SETS)]
    for ev in fwd_done:
        ev.record(cur)

    def e2e_step(i: int):
        k = i % N_BUFFER_SETS
        s = sets[k]
        with torch.cuda.stream(s_in):
            s_in.wait_event(fwd_done[k])     # x_dev[k] was last read by the forward of step i - N_BUFFER_SETS
            x_dev[k].copy_(s["x_host"], non_blocking=True)
            in_done[k].record(s_in)
        cur.wait_event(in_done[k])
        xd = x_dev[k]
        if s["lora"] is not None:
            q, xs = F.quantize_rowwise(xd, hadamard=shape.hadamard)
            y = F.linear_w8a8_lora(q, xs, s["wq"], s["ws"], s["bias"], F.lora_down(xd, s["lora"][0]), s["lora"][1], out_dtype)
        else:
            y = F.linear_forward(xd, s["wq"], s["ws"], s["bias"], out_dtype, hadamard=shape.hadamard)
        fwd_done[k].record(cur)
        keep[k] = y
        y.record_stream(s_out)
        with torch.cuda.stream(s_out):
            s_out.wait_event(fwd_done[k])
            s["y_host"].copy_(y, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 40))
    for i in range(3):
        e2e_step(i)
    cur.wait_stream(s_out)
    sync_all()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for i in range(e2e_steps):
        e2e_step(i)
    cur.wait_stream(s_out)
    cur.wait_stream(s_in)
    e_end.record()
    sync_all()
    e2e_ms = e_start.elapsed_time(e_end)
    status = nat.device_status()

    if dist is not None:
        t = torch.tensor([elapsed_ms, e2e_ms, gemm_avg_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, gemm_avg_ms = (float(v) for v in t.tolist())
        dist.destroy_process_group()
    if rank != 0:
        return

    ops_step = 2.0 * M * N * K                       # int8 GEMM ops of one rank's step
    value = world * ops_step * args.steps / (elapsed_ms * 1e-3) / 1e12
    e2e_value = world * ops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
    peaks, peak_kind = measured_peaks()
    # int8 tensor throughput is twice the bf16 rate of the same tensor cores; the steps run back to
    # back for a short burst, so the burst figure is the denominator
    peak_tops = 2.0 * peaks["bf16_tflops"]
    achieved = ops_step / (gemm_avg_ms * 1e-3) / 1e12
    cpu_base, _ = cpu_reference_rate(shape, steps=20, warmup=2, budget_s=12.0)
    line = {
        "metric": "w8a8_linear_int8_throughput", "value": value, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config_dict(shape, world),
        "frac_of_nominal_int8_peak": value / (world * NOMINAL_INT8_TOPS),
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel<i8, pair" + (", fused LoRA>" if shape.lora_rank else ">"), "achieved": achieved, "peak": peak_tops,
                     "unit": "TFLOP/s", "frac": achieved / peak_tops, "traffic": NCU_GEMM_TRAFFIC_BYTES.get(shape.name),
                     "peak_source": f"2 x bf16_tflops (burst) of {peak_kind} MEASURED_PEAKS.json; int8 ops counted as 2*M*N*K",
                     "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS, "kernel_ms_avg": gemm_avg_ms,
                     "kernel_ms_best": gemm_ms[0], "kernel_launches_timed": len(gemm_ms)},
        "cpu_baseline": cpu_base,
        "e2e": {"value": e2e_value, "unit": "TOPS", "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": int(launches_timed) * world,
        "clocks": clocks,
        "device_status": status,
    }
    print(json.dumps(line))


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


def run_dit(args):
    import importlib
    import torch
    import __graft_entry__ as g
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    pkg = g.load_package()
    dit = importlib.import_module(pkg.__name__ + ".dit")
    cfg = dit.DiTConfig()
    if args.impl == "reference":
        if rank != 0:
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
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    model = dit.SyntheticDiT(cfg, seed=0, device=dev)
    gen = torch.Generator().manual_seed(1000 + rank)
    img_h = torch.randn(1, cfg.img_tokens, cfg.in_channels, generator=gen).bfloat16().pin_memory()
    txt_h = torch.randn(1, cfg.txt_tokens, cfg.txt_dim, generator=gen).bfloat16().pin_memory()
    out_h = torch.empty(1, cfg.img_tokens, cfg.in_channels, dtype=torch.bfloat16).pin_memory()
    img, txt = img_h.to(dev), txt_h.to(dev)
    t = torch.full((1,), 0.5, device=dev)
    steps = min(args.steps, 20)

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(3, min(args.warmup, 5))):
        out = model(img, txt, t)
    sync_all()
    graph = None
    if not args.no_graph:
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
    sampler = ClockSampler(local_rank) if rank == 0 else None
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
    status = pkg._native.device_status()
    finite = bool(torch.isfinite(out.float()).all())
    if dist is not None:
        tt = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_ms = (float(v) for v in tt.tolist())
        dist.destroy_process_group()
    if rank != 0:
        return
    n_int8 = cfg.double_blocks * 8 + cfg.single_blocks * 2
    peaks, peak_kind = measured_peaks()
    peak_tops = 2.0 * peaks["bf16_tflops_sustained"]
    achieved = cfg.int8_ops() / (ms * 1e-3) / 1e12
    cpu_sec, cpu_base = dit_cpu_seconds(cfg, budget_s=12.0)
    cpu_base = dict(cpu_base, value=cpu_sec, unit="s/it", sample=cpu_base["sample"] + "; step time = int8 ops / that rate")
    print(json.dumps({
        "metric": "dit_step_time", "value": ms * 1e-3, "unit": "s/it", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic", "config": dit_config_dict(cfg, world, graph is not None),
        "samples_per_s_all_gpus": world / (ms * 1e-3),
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel<i8,256> (whole step)", "achieved": achieved,
                     "peak": peak_tops, "unit": "TFLOP/s", "frac": achieved / peak_tops, "traffic": None,
                     "peak_source": f"2 x bf16_tflops_sustained of {peak_kind} MEASURED_PEAKS.json; achieved = int8 linear ops "
                                    "/ WHOLE step time (attention, norms and element-wise work included in the time)",
                     "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS},
        "cpu_baseline": cpu_base,
        "e2e": {"value": e2e_ms * 1e-3, "unit": "s/it", "h2d_bytes_per_step": img_h.numel() * 2 + txt_h.numel() * 2,
                "d2h_bytes_per_step": out_h.numel() * 2, "steps": steps},
        "gpu_launches": 2 * n_int8 * steps * world, "clocks": clocks, "device_status": status, "output_finite": finite}))


# ------------------------------------------- column-parallel sweep (config 4)
NVLINK_PEER_GBS = 770.0   # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)


def run_column_parallel(args):
    """W8A8 linear K=4096, N=16384 split over the ranks by output channel; every rank quantises the full x, runs
    its slice and the bf16 [M, N/P] blocks are all-gathered (NCCL).  One line with a result per M."""
    import torch
    import __graft_entry__ as g
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    K, N = 4096, 16384
    m_sweep = [1024, 4096, 16384, 32768]
    if args.impl == "reference":
        if rank != 0:
            return
        import __graft_entry__ as g2
        wl = g2.load_package().workloads
        base, dt = cpu_reference_rate(wl.LinearShape("c4_column_parallel", 4096, K, N, False, True, False), args.steps,
                                      args.warmup, budget_s=40.0)
        print(json.dumps({"impl": "reference", "metric": "w8a8_linear_int8_throughput", "value": base["value"], "unit": "TOPS",
                          "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
                          "data": "synthetic", "config": {"workload": "c4_column_parallel", "K": K, "N": N, "M": 4096},
                          "cpu_baseline": base, "gpu_launches": 0,
                          "e2e": {"value": base["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = g.load_package()
    F, par, wl = pkg.functional, pkg.parallel, pkg.workloads
    w = wl.weight_fp32(N, K, seed=4)
    b0, e0_ = par.shard_bounds(N, world, rank)
    wq, ws = F.quantize_weight_rows(w[b0:e0_].to(dev))
    n_local = e0_ - b0
    steps = min(args.steps, 50)
    results = []
    for M in m_sweep:
        x = wl.activation(M, K, seed=40).to(dev)          # same bits on every rank
        gathered = torch.empty((world * M, n_local), dtype=torch.bfloat16, device=dev)   # [P, M, N/P] blocks
        full = torch.empty((M, N), dtype=torch.bfloat16, device=dev)

        def step(relayout: bool):
            q, xs = F.quantize_rowwise(x)
            y = F.linear_w8a8(q, xs, wq, ws, None, torch.bfloat16)
            if world > 1:
                dist.all_gather_into_tensor(gathered, y)
                if relayout:
                    full.view(M, world, n_local).copy_(gathered.view(world, M, n_local).transpose(0, 1))
            return y

        def timed(relayout: bool):
            for _ in range(3):
                step(relayout)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                step(relayout)
            b.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        ms_blocks = timed(False)
        ms_full = timed(True) if world > 1 else ms_blocks
        ms_fused, fused_equal = None, None
        if world > 1 and n_local % 32 == 0:
            try:
                shard = par.ColumnShard(wq, ws, None, b0, e0_, N)
                fused = par.FusedColumnParallelOutput(M, N, torch.bfloat16, dev)
                step_nccl = step

                def step(relayout: bool):       # noqa: F811 - same timing harness, fused kernel
                    return fused.forward(x, shard)

                ms_fused = timed(False)
                y_all = fused.forward(x, shard)
                torch.cuda.synchronize()
                step = step_nccl
                step(True)
                torch.cuda.synchronize()
                fused_equal = bool(torch.equal(y_all, full))
                del fused
            except Exception as e:  # noqa: BLE001
                ms_fused, fused_equal = None, f"unavailable: {e!r}"
        # parity of the gathered result with the unsharded computation on rank 0's slice of columns
        ops = 2.0 * M * N * K
        comm_bytes = 2.0 * M * N * (world - 1) / world
        nvlink_ms = comm_bytes / (NVLINK_PEER_GBS * 1e9) * 1e3
        results.append({"M": M, "ms_fused_epilogue_scatter": ms_fused, "fused_equals_nccl_result": fused_equal,
                        "frac_of_nvlink_roofline_fused": (nvlink_ms / ms_fused) if ms_fused else None,
                        "ms_blocks_layout": ms_blocks, "ms_row_major_layout": ms_full,
                        "tops": ops / (ms_blocks * 1e-3) / 1e12, "allgather_bytes_in_per_gpu": comm_bytes,
                        "nvlink_roofline_ms": nvlink_ms, "frac_of_nvlink_roofline": (nvlink_ms / ms_blocks) if world > 1 else None})
        del x, gathered, full
    status = pkg._native.device_status()
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    ref = next(r for r in results if r["M"] == 4096)
    print(json.dumps({"metric": "w8a8_linear_int8_throughput", "value": ref["tops"], "unit": "TOPS", "n_gpus": world,
                      "steps": steps, "warmup": 3, "ms_per_step": ref["ms_blocks_layout"], "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                      "config": {"workload": "c4_column_parallel", "K": K, "N": N, "M": 4096, "weight_scale": "per_channel",
                                 "parallelism": f"column-parallel x{world}, NCCL all-gather of bf16 [M, N/P] blocks",
                                 "l2": "weights 64 MB / P per rank stay L2-resident across steps (real layers would not)"},
                      "sweep": results, "gpu_launches": 2 * steps * world * len(m_sweep) * 2, "device_status": status,
                      "note": "communication-bound by construction: bytes/op ratio is fixed by K; roofline is NVLink, "
                              f"{NVLINK_PEER_GBS} GB/s per direction per GPU (measured peer copy)"}))


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", choices=["c0", "c1", "c2", "c2merge", "c4", "dit", "smallm"], default="c1")
    ap.add_argument("--no-graph", action="store_true", help="dit: run eagerly instead of replaying a CUDA graph")
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
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
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
