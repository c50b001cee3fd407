"""Host side of the W8A8 linear: the functional API, the ops class ComfyUI
instantiates layers from, the INT8-space LoRA patch adapters and the
dynamic-LoRA hook.  Names, arguments and attribute surface follow the
ComfyUI-INT8-Fast node pack (its int8_quant.py) so existing workflows and
callers keep working; every quantised code path runs on the sm_100a kernels
of libi8f.so and raises if they are unavailable.
"""
from __future__ import annotations

import logging

import torch
import torch.nn.functional as TF
from torch import Tensor, nn

from . import _native as nat
from . import custom_ops
from . import functional as F
from . import quarot

SMALL_BATCH_ROWS = 16  # at or below this many tokens the weights are dequantised instead (int8_quant.py:751-760)


# =============================================================================
# Functional API                                             int8_quant.py:20-119
# =============================================================================
def quantize_int8(x: Tensor, scale) -> Tensor:
    """clamp(round(x * (1/scale)), -128, 127) as int8.   int8_quant.py:20-21"""
    nat.require_device(x.device)
    return x.float().mul(1.0 / scale).round_().clamp_(-128.0, 127.0).to(torch.int8)


def quantize_int8_tensorwise(x: Tensor) -> tuple[Tensor, Tensor]:
    """One absmax scale for the whole tensor.   int8_quant.py:23-26"""
    q, scale = F.quantize_tensorwise(x.reshape(-1, x.shape[-1]))
    return q.reshape(x.shape), scale


def quantize_int8_axiswise(x: Tensor, dim: int) -> tuple[Tensor, Tensor]:
    """Absmax scale per slice along `dim` (the last axis).   int8_quant.py:28-31

    Activations (bf16 / fp16) and weights (any float dtype, converted to fp32) share the arithmetic.
    """
    if dim not in (-1, x.dim() - 1):
        raise NotImplementedError("quantize_int8_axiswise supports the last axis only")
    x2 = x.reshape(-1, x.shape[-1])
    q, scale = F.quantize_rowwise(x2)
    return q.reshape(x.shape), scale.reshape(*x.shape[:-1], 1)


def dequantize(q: Tensor, scale) -> Tensor:
    """int8_quant.py:33-34"""
    return q.float() * scale


def stochastic_round_int8_delta(x: Tensor, scale, seed: int = 0) -> Tensor:
    """Stochastically rounded int8 of x/scale.   int8_quant.py:36-62

    The uniforms come from the kernel's Philox4x32-10 stream keyed by `seed` (the reference draws
    them from torch's generator, whose stream already differs between its CPU and CUDA runs).
    """
    dev = x.device
    if dev.type != "cuda":
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else dev
    x2 = x.to(dev).float()
    shape = x2.shape
    x2 = x2.reshape(-1, shape[-1]) if x2.dim() != 2 else x2
    if isinstance(scale, Tensor) and scale.numel() > 1 and scale.numel() != x2.shape[0]:
        raise ValueError("per-row scale does not match the rows of the delta")
    out = F.stochastic_round(x2, scale, seed=seed)
    return out.reshape(shape).to(x.device)


@torch.no_grad()
def int8_forward_dynamic(x: Tensor, weight: Tensor, weight_scale, bias: Tensor | None,
                         compute_dtype: torch.dtype) -> Tensor:
    """Dynamic per-token quantised linear with one weight scale.   int8_quant.py:67-88"""
    return F.linear_forward(x.reshape(-1, x.shape[-1]), weight, weight_scale, bias, compute_dtype)


@torch.no_grad()
def int8_forward_dynamic_per_row(x: Tensor, weight: Tensor, weight_scale: Tensor, bias: Tensor | None,
                                 compute_dtype: torch.dtype) -> Tensor:
    """Same with per-output-channel weight scales [N,1].   int8_quant.py:91-119"""
    return F.linear_forward(x.reshape(-1, x.shape[-1]), weight, weight_scale, bias, compute_dtype)


# =============================================================================
# LoRA delta reconstruction                                  int8_quant.py:128-208
# =============================================================================
def _cast(t, device, dtype):
    try:
        import comfy.model_management as mm
        return mm.cast_to_device(t, device, dtype)
    except ImportError:
        return t.to(device=device, dtype=dtype)


def lora_scale_of(alpha, rank, strength):
    return (alpha / rank) * strength if alpha is not None else strength


def reconstruct_lora_diff(weights, target_shape, device, dtype, strength):
    """High-precision delta of a LoRA (6-tuple), LoHa (8-tuple) or LoKr (9-tuple) patch and its scale."""
    v = weights
    kind = len(v)
    if kind == 6:
        up, down, alpha, mid = v[0], v[1], v[2], v[3]
        scale = lora_scale_of(alpha, down.shape[0], strength)
        inner = _cast(down, device, dtype).flatten(1)
        if mid is not None:
            inner = torch.mm(_cast(mid, device, dtype).flatten(1), inner)
        return torch.mm(_cast(up, device, dtype).flatten(1), inner).reshape(target_shape), scale
    if kind == 8:
        w1a, w1b, alpha, w2a, w2b, t1, t2 = v[:7]
        scale = lora_scale_of(alpha, w1b.shape[0], strength)
        if t1 is not None:
            tucker = "i j k l, j r, i p -> p r k l"
            m1 = torch.einsum(tucker, _cast(t1, device, dtype), _cast(w1b, device, dtype), _cast(w1a, device, dtype))
            m2 = torch.einsum(tucker, _cast(t2, device, dtype), _cast(w2b, device, dtype), _cast(w2a, device, dtype))
        else:
            m1 = torch.mm(_cast(w1a, device, dtype), _cast(w1b, device, dtype))
            m2 = torch.mm(_cast(w2a, device, dtype), _cast(w2b, device, dtype))
        return (m1 * m2).reshape(target_shape), scale
    if kind == 9:
        w1, w2, alpha, w1a, w1b, w2a, w2b, t2 = v[:8]
        dim = None
        if w1 is None:
            dim = w1b.shape[0]
            f1 = torch.mm(_cast(w1a, device, dtype), _cast(w1b, device, dtype))
        else:
            f1 = _cast(w1, device, dtype)
        if w2 is None:
            dim = w2b.shape[0]
            if t2 is None:
                f2 = torch.mm(_cast(w2a, device, dtype), _cast(w2b, device, dtype))
            else:
                f2 = torch.einsum("i j k l, j r, i p -> p r k l", _cast(t2, device, dtype), _cast(w2b, device, dtype),
                                  _cast(w2a, device, dtype))
        else:
            f2 = _cast(w2, device, dtype)
        if f2.dim() == 4:
            f1 = f1.unsqueeze(2).unsqueeze(2)
        scale = (alpha / dim) * strength if (alpha is not None and dim is not None) else strength
        return torch.kron(f1, f2).reshape(target_shape), scale
    return None, 1.0


def _compute_device(fallback: torch.device) -> torch.device:
    try:
        import comfy.model_management as mm
        return mm.get_torch_device()
    except ImportError:
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else fallback


def _slice_scale(ws, rows: int, offset):
    """Weight scale restricted to the rows ComfyUI handed over (fused-QKV slices).   int8_quant.py:249-272"""
    if not isinstance(ws, Tensor) or ws.numel() == 1:
        return ws
    if offset is not None:
        dim, start, size = offset
        if dim < ws.dim() and ws.shape[dim] > start:
            return ws.narrow(dim, start, min(size, ws.shape[dim] - start))
    if ws.shape[0] != rows and ws.shape[0] % rows == 0:
        return ws[:rows]
    return ws


def _slice_scale_strict(ws, rows: int, offset):
    """Variant used by the stacked adapter.   int8_quant.py:341-352"""
    if not isinstance(ws, Tensor) or ws.numel() == 1:
        return ws
    if offset is not None and ws.shape[0] != rows:
        dim, start, size = offset
        if dim == 0:
            return ws.narrow(0, start, size)
    if ws.shape[0] != rows and ws.shape[0] % rows == 0:
        return ws[:rows]
    return ws


def _quarot_enabled() -> bool:
    return bool(getattr(Int8TensorwiseOps, "enable_quarot", False)) if Int8TensorwiseOps is not None else False


def _merge_int8(weight: Tensor, factors, delta, eff_scale, seed: int, comp_device: torch.device) -> Tensor:
    """Common tail of both adapters: rotate (if QuaRot), round stochastically, add, clamp.

    `factors` = (up, down, scale) for a plain low-rank update (single fused kernel), else None and
    `delta` holds the reconstructed fp32 update.
    """
    origin = weight.device
    w = weight.to(comp_device).contiguous()
    if w.data_ptr() == weight.data_ptr():
        w = w.clone()
    rotate = _quarot_enabled() and weight.shape[1] % quarot.GROUP_SIZE == 0
    if factors is not None:
        up, down, scale = factors
        up, down = up.to(comp_device), down.to(comp_device)
        if up.shape[1] > F.lora_merge_max_rank(up.dtype):
            # the fused kernel keeps a whole [rank x 128] slice of `down` in shared memory; a stack (or a single file)
            # whose rank exceeds that takes the delta path below: the product in fp32, then ONE rounding, which is
            # what the reference does for any number of LoRAs at any rank (int8_quant.py:355-404)
            delta = torch.mm(up.float().flatten(1), down.float().flatten(1)) * scale
            factors = None
    if factors is not None:
        F.lora_merge_sr_(w, eff_scale, up, down, scale, hadamard=rotate, seed=seed)
    else:
        d = delta.to(comp_device, torch.float32)
        if rotate:
            d = quarot.rotate_weight(d, None, quarot.GROUP_SIZE)
        d8 = F.stochastic_round(d, eff_scale, seed=seed)
        w = torch.clamp(w.to(torch.int32) + d8.to(torch.int32), -128, 127).to(torch.int8)
    return w.to(origin)


try:
    from comfy.weight_adapter.lora import LoRAAdapter
    _LORA_ADAPTER_AVAILABLE = True
except ImportError:
    _LORA_ADAPTER_AVAILABLE = False

if _LORA_ADAPTER_AVAILABLE:

    class INT8LoRAPatchAdapter(LoRAAdapter):
        """Patches int8 weights in int8 space: delta -> stochastic rounding -> saturating add."""

        def __init__(self, loaded_keys, weights, weight_scale, seed=0):
            super().__init__(loaded_keys, weights)
            self.weight_scale = weight_scale
            self.seed = seed

        def _get_effective_scale(self, delta_f, offset):
            return _slice_scale(self.weight_scale, delta_f.shape[0], offset)

        def calculate_weight(self, weight, key, strength, strength_model, offset, function,
                             intermediate_dtype=torch.float32, original_weight=None):
            if intermediate_dtype == torch.int8:
                intermediate_dtype = torch.float32
            comp_device = _compute_device(weight.device)
            v = self.weights
            plain = len(v) == 6 and v[3] is None and weight.dtype == torch.int8 and weight.dim() == 2
            if plain:
                up, down = v[0].flatten(1), v[1].flatten(1)
                scale = lora_scale_of(v[2], v[1].shape[0], strength)
                eff = _slice_scale(self.weight_scale, weight.shape[0], offset)
                return _merge_int8(weight, (up, down, float(scale)), None, eff, self.seed, comp_device)
            diff, scale = reconstruct_lora_diff(v, weight.shape, comp_device, intermediate_dtype, strength)
            if diff is None:
                return weight
            if weight.dtype == torch.int8:
                delta = diff * scale
                return _merge_int8(weight, None, delta, self._get_effective_scale(delta, offset), self.seed, comp_device)
            return weight + (diff * scale).to(weight.device, weight.dtype)

    class INT8MergedLoRAPatchAdapter(LoRAAdapter):
        """Sums a stack of LoRAs in high precision and rounds once."""

        def __init__(self, patches, weight_scale, seed=0):
            first = patches[0][0]
            super().__init__(first.loaded_keys, first.weights)
            self.patches = patches  # list of (adapter, strength)
            self.weight_scale = weight_scale
            self.seed = seed

        def _get_effective_scale(self, delta_f, offset):
            return _slice_scale_strict(self.weight_scale, delta_f.shape[0], offset)

        def calculate_weight(self, weight, key, strength, strength_model, offset, function,
                             intermediate_dtype=torch.float32, original_weight=None):
            if intermediate_dtype == torch.int8:
                intermediate_dtype = torch.float32
            comp_device = _compute_device(weight.device)
            all_plain = weight.dtype == torch.int8 and weight.dim() == 2 and all(
                len(a.weights) == 6 and a.weights[3] is None for a, _ in self.patches)
            if all_plain:
                # sum_i s_i * up_i @ down_i == [s_1 up_1 | s_2 up_2 | ...] @ [down_1; down_2; ...]
                ups, downs = [], []
                for adapter, lora_strength in self.patches:
                    up, down, alpha = adapter.weights[0], adapter.weights[1], adapter.weights[2]
                    s = float(lora_scale_of(alpha, down.shape[0], lora_strength))
                    ups.append(up.flatten(1).to(comp_device, torch.float32) * s)
                    downs.append(down.flatten(1).to(comp_device, torch.float32))
                eff = _slice_scale_strict(self.weight_scale, weight.shape[0], offset)
                return _merge_int8(weight, (torch.cat(ups, dim=1), torch.cat(downs, dim=0), 1.0), None, eff, self.seed,
                                   comp_device)
            total = None
            for adapter, lora_strength in self.patches:
                d, scale = reconstruct_lora_diff(adapter.weights, weight.shape, comp_device, intermediate_dtype,
                                                 lora_strength)
                if d is None:
                    continue
                total = d * scale if total is None else total.add_(d * scale)
            if total is None:
                return weight
            if weight.dtype == torch.int8:
                return _merge_int8(weight, None, total, self._get_effective_scale(total, offset), self.seed, comp_device)
            return weight + total.to(weight.device, weight.dtype)


# =============================================================================
# Dynamic LoRA hook                                          int8_quant.py:415-507
# =============================================================================
class DynamicLoRAHook:
    """Forward-pre-hook on the diffusion model: keeps every quantised layer's lora_A / lora_B in
    sync with the `dynamic_loras` list carried in transformer_options."""

    def __init__(self):
        self.current_lora_id = None

    def pre_forward(self, module, input_args, input_kwargs):
        opts = input_kwargs.get("transformer_options", {})
        if not opts and len(input_args) > 2 and isinstance(input_args[2], dict):
            opts = input_args[2].get("transformer_options", {})
        loras = opts.get("dynamic_loras", [])
        lora_id = hash(tuple((id(d["patches"]), d["strength"]) for d in loras)) if loras else None
        if lora_id != self.current_lora_id:
            self.apply_composition(module, loras)
            self.current_lora_id = lora_id
        return None

    def apply_composition(self, diffusion_model, dynamic_loras):
        per_layer: dict = {}
        for entry in dynamic_loras or []:
            for key, adapter in entry["patches"].items():
                per_layer.setdefault(key, []).append((adapter, entry["strength"]))
        for name, module in diffusion_model.named_modules():
            if not hasattr(module, "lora_A"):
                continue
            patches = per_layer.get(f"diffusion_model.{name}.weight") or per_layer.get(f"{name}.weight")
            module.lora_alpha = None
            module._lora_cache = None      # converted copies of the factors belong to the tensors replaced below
            if not patches:
                module.lora_A = module.lora_B = None
                continue
            downs, ups = [], []
            for adapter, strength in patches:
                up, down, alpha, mid = adapter.weights[:4]
                rank = down.shape[0] if down.ndim >= 2 else 1
                if mid is not None:
                    down = torch.mm(mid.flatten(1), down.flatten(1)).reshape(down.shape)
                downs.append(down * lora_scale_of(alpha, rank, strength))
                ups.append(up)
            device = getattr(module, "weight", torch.tensor(0)).device
            module.lora_A = torch.cat(downs, dim=0).to(device)   # [sum r, K]
            module.lora_B = torch.cat(ups, dim=1).to(device)     # [N, sum r]

    @classmethod
    def register(cls, diffusion_model):
        if not hasattr(diffusion_model, "_dynamic_lora_hook"):
            hook = cls()
            diffusion_model._dynamic_lora_hook = hook
            diffusion_model.register_forward_pre_hook(hook.pre_forward, with_kwargs=True)
        return diffusion_model._dynamic_lora_hook


# =============================================================================
# Int8TensorwiseOps                                          int8_quant.py:522-792
# =============================================================================
def _convert_lora(module, device: torch.device, dtype: torch.dtype):
    """lora_A / lora_B in the compute dtype on `device`, rank padded to a multiple of 8 (16-byte rows for the TMA
    loads); plain tensor operations, so it also traces under torch.compile."""
    a = module.lora_A.to(device=device, dtype=dtype).flatten(1)
    b = module.lora_B.to(device=device, dtype=dtype).flatten(1)
    if module.lora_alpha is not None:
        b = (b.float() * module.lora_alpha).to(dtype)
    pad = (-a.shape[0]) % 8
    if pad:
        a = torch.cat([a, a.new_zeros(pad, a.shape[1])], dim=0)
        b = torch.cat([b, b.new_zeros(b.shape[0], pad)], dim=1)
    return a.contiguous(), b.contiguous()


def _prepare_lora(module, device: torch.device, dtype: torch.dtype):
    """The converted factors, cached on the module until the source tensors are replaced.  While a compiler traces
    the forward the conversion is simply part of the graph (no cache: attribute writes would break the trace)."""
    if torch.compiler.is_compiling():
        return _convert_lora(module, device, dtype)
    # The entry keeps the SOURCE tensors and is matched by identity: a key made of id() values alone could match a
    # new pair of tensors that was allocated at the addresses of a freed pair (LoRA X -> none -> LoRA Y), and the
    # layer would silently keep running X's converted factors.
    key = (device, dtype, module.lora_alpha)
    cache = getattr(module, "_lora_cache", None)
    if cache is not None and cache[0] == key and cache[3] is module.lora_A and cache[4] is module.lora_B:
        return cache[1], cache[2]
    a, b = _convert_lora(module, device, dtype)
    module._lora_cache = (key, a, b, module.lora_A, module.lora_B)
    return a, b


def _define_ops(manual_cast, cast_bias_weight, uncast_bias_weight):
    class Int8TensorwiseOps(manual_cast):
        """ComfyUI custom operations: Linear layers hold int8 weights and run the sm_100a W8A8 kernels."""
        excluded_names: list = []
        dynamic_quantize = False      # quantise float checkpoints while loading
        enable_quarot = False         # rotate weights (load) and activations (forward) by blocks of 128
        use_triton = True             # accepted for compatibility; there is only the CUDA path
        _is_prequantized = False
        lora_uses_rotated_input = True  # the reference feeds the rotated activations to the dynamic LoRA

        class Linear(manual_cast.Linear):
            def __init__(self, *args, **kwargs):
                super().__init__(*args, **kwargs)
                self.register_buffer("weight_scale", None)
                self._is_quantized = False
                self._is_per_row = False
                self._use_quarot = False
                self._weight_scale_scalar = None
                self.compute_dtype = torch.bfloat16
                self.lora_A = None
                self.lora_B = None
                self.lora_alpha = None
                self._scalar_scale_dev = None

            def reset_parameters(self):
                return None

            # ----------------------------------------------------------- loading
            def _adopt_scale(self, weight_scale):
                if isinstance(weight_scale, Tensor) and weight_scale.numel() > 1:
                    self.register_buffer("weight_scale", weight_scale.float())
                    self._weight_scale_scalar = None
                    self._is_per_row = weight_scale.dim() == 2 and weight_scale.shape[1] == 1
                else:
                    value = weight_scale.float().item() if isinstance(weight_scale, Tensor) else float(weight_scale)
                    self._weight_scale_scalar = value
                    self.weight_scale = None
                    self._is_per_row = False
                self._scalar_scale_dev = None

            def _quantize_on_load(self, weight_tensor):
                if not torch.cuda.is_available():
                    raise nat.NativeLibraryError("on-the-fly quantisation needs a CUDA device (no CPU fallback)")
                w_gpu = weight_tensor.to("cuda", non_blocking=True).float()
                self._use_quarot = bool(getattr(Int8TensorwiseOps, "enable_quarot", False)) and \
                    self.in_features % quarot.GROUP_SIZE == 0
                q, scale = F.quantize_weight_rows(w_gpu, hadamard=self._use_quarot)
                self.weight = nn.Parameter(q.cpu(), requires_grad=False)
                self.register_buffer("weight_scale", scale.cpu())
                self._weight_scale_scalar = None
                self._is_quantized = True
                self._is_per_row = True

            def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs):
                weight_scale = state_dict.pop(prefix + "weight_scale", None)
                state_dict.pop(prefix + "comfy_quant", None)
                state_dict.pop(prefix + "input_scale", None)   # present in some checkpoints, unused
                weight = state_dict.pop(prefix + "weight", None)
                bias = state_dict.pop(prefix + "bias", None)

                if weight is None:
                    missing_keys.append(prefix + "weight")
                elif weight.dtype == torch.int8 and weight_scale is not None:
                    self._is_quantized = True
                    self.weight = nn.Parameter(weight, requires_grad=False)
                    Int8TensorwiseOps._is_prequantized = True
                    self._adopt_scale(weight_scale)
                elif weight.dtype in (torch.float16, torch.bfloat16, torch.float32):
                    skip = (any(ex in prefix for ex in Int8TensorwiseOps.excluded_names)
                            or self.in_features == 1 or self.out_features == 1 or weight.ndim == 1
                            or not Int8TensorwiseOps.dynamic_quantize)
                    if not skip and self.in_features % 16 != 0:
                        logging.info("INT8 Fast: %sweight kept in %s (in_features %d is not a multiple of 16)", prefix,
                                     weight.dtype, self.in_features)
                        skip = True
                    if skip:
                        self._is_quantized = False
                        self.weight = nn.Parameter(weight, requires_grad=False)
                    else:
                        self._quantize_on_load(weight)
                else:
                    self._is_quantized = False
                    self.weight = nn.Parameter(weight, requires_grad=False)

                self.bias = nn.Parameter(bias, requires_grad=False) if bias is not None else None
                # ComfyUI archived the dtypes before loading; tell its memory accounting what is stored now
                if self.weight is not None:
                    self.weight_comfy_model_dtype = self.weight.dtype
                if self.weight_scale is not None:
                    self.weight_scale_comfy_model_dtype = self.weight_scale.dtype
                if self.bias is not None:
                    self.bias_comfy_model_dtype = self.bias.dtype

            # ------------------------------------------------------ patcher hooks
            def _get_weight_scale(self):
                return self._weight_scale_scalar if self._weight_scale_scalar is not None else self.weight_scale

            def convert_weight(self, _weight, inplace=False):
                return self.weight if self._is_quantized else _weight

            def _store(self, name, value, inplace_update):
                if inplace_update and getattr(self, name) is not None:
                    getattr(self, name).data.copy_(value)
                elif not inplace_update:
                    setattr(self, name, nn.Parameter(value, requires_grad=False))

            def set_weight(self, out_weight, inplace_update=False, seed=0, return_weight=False, **kwargs):
                if not self._is_quantized:
                    new_weight = out_weight.to(self.weight.dtype)
                elif out_weight.dtype == torch.int8:
                    new_weight = out_weight
                else:  # a float result reached a quantised layer: re-quantise with the layer's scale
                    new_weight = stochastic_round_int8_delta(out_weight, self._get_weight_scale(), seed)
                if return_weight:
                    return new_weight
                self._store("weight", new_weight, inplace_update)

            def set_bias(self, out_bias, inplace_update=False, seed=0, return_weight=False, **kwargs):
                if out_bias is None:
                    return None
                if return_weight:
                    return out_bias
                self._store("bias", out_bias, inplace_update)

            # ------------------------------------------------------------ forward
            def _scale_on(self, device):
                if self._weight_scale_scalar is not None:
                    if torch.compiler.is_compiling():   # a constant of the traced graph; no attribute is written
                        return torch.full((1,), self._weight_scale_scalar, dtype=torch.float32, device=device)
                    cached = self._scalar_scale_dev   # (value, device, 1-element fp32 tensor)
                    if cached is None or cached[0] != self._weight_scale_scalar or cached[1] != device:
                        t = torch.tensor([self._weight_scale_scalar], dtype=torch.float32, device=device)
                        cached = self._scalar_scale_dev = (self._weight_scale_scalar, device, t)
                    return cached[2]
                ws = self.weight_scale
                return ws if ws.device == device else ws.to(device, non_blocking=True)

            def forward(self, x: Tensor) -> Tensor:
                need_cast = self.comfy_cast_weights or len(self.weight_function) > 0 or len(self.bias_function) > 0
                if not self._is_quantized:
                    if not need_cast:
                        return TF.linear(x, self.weight, self.bias)
                    weight, bias, stream = cast_bias_weight(self, x, offloadable=True)
                    out = TF.linear(x, weight, bias)
                    uncast_bias_weight(self, weight, bias, stream)
                    return out

                if not torch.compiler.is_compiling():   # the operators below check the device themselves when they run
                    nat.require_device(x.device)
                if need_cast:
                    weight, bias, stream = cast_bias_weight(self, input=None, dtype=torch.int8, device=x.device,
                                                            bias_dtype=x.dtype, offloadable=True)
                else:
                    weight, bias, stream = self.weight, self.bias, None
                w_scale = self._scale_on(x.device)
                compute_dtype = x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16
                x2 = x.reshape(-1, x.shape[-1])
                if x2.dtype != compute_dtype:
                    x2 = x2.to(compute_dtype)
                rows = x2.shape[0]
                has_lora = self.lora_A is not None and self.lora_B is not None

                if rows > SMALL_BATCH_ROWS and has_lora:
                    # t = x @ A^T first; t @ B^T is accumulated inside the int8 GEMM kernel and added in its
                    # epilogue with the reference's roundings: y = round(round(dequant + bias) + round(lora_y))
                    lora_a, lora_b = _prepare_lora(self, x.device, compute_dtype)
                    y = custom_ops.linear_lora_forward(x2, weight, w_scale, bias, lora_a, lora_b, compute_dtype,
                                                       self._use_quarot, Int8TensorwiseOps.lora_uses_rotated_input,
                                                       nat.EPI_PYTORCH)
                elif rows > SMALL_BATCH_ROWS:
                    if torch.compiler.is_compiling():    # one opaque node for the tracer
                        y = custom_ops.linear_forward(x2, weight, w_scale, bias, compute_dtype, self._use_quarot,
                                                      nat.EPI_PYTORCH)
                    else:                                # eager: straight to the library, without the operator dispatch
                        y = F.linear_forward(x2, weight, w_scale, bias, compute_dtype, hadamard=self._use_quarot)
                else:
                    lora_a, lora_b = _prepare_lora(self, x.device, compute_dtype) if has_lora else (None, None)
                    y = custom_ops.small_batch_forward(x2, weight, w_scale, bias, lora_a, lora_b, self._use_quarot)

                if need_cast:
                    uncast_bias_weight(self, weight, bias, stream)
                return y.reshape(*x.shape[:-1], y.shape[-1])

        class GroupNorm(manual_cast.GroupNorm):
            pass

        class LayerNorm(manual_cast.LayerNorm):
            pass

        class Conv2d(manual_cast.Conv2d):
            pass

        class Conv3d(manual_cast.Conv3d):
            pass

        class ConvTranspose2d(manual_cast.ConvTranspose2d):
            pass

        class Embedding(manual_cast.Embedding):
            pass

        @classmethod
        def conv_nd(cls, dims, *args, **kwargs):
            if dims == 2:
                return cls.Conv2d(*args, **kwargs)
            if dims == 3:
                return cls.Conv3d(*args, **kwargs)
            raise ValueError(f"unsupported dimensions: {dims}")

    return Int8TensorwiseOps


try:
    from comfy.ops import cast_bias_weight, manual_cast, uncast_bias_weight
    _COMFY_OPS_AVAILABLE = True
except ImportError:
    _COMFY_OPS_AVAILABLE = False

Int8TensorwiseOps = _define_ops(manual_cast, cast_bias_weight, uncast_bias_weight) if _COMFY_OPS_AVAILABLE else None


# -----------------------------------------------------------------------------
# The same ops class without ComfyUI (benchmarks, stand-alone use): plain torch layers as the base and
# no weight-offloading handshake (weights live on the device).
# -----------------------------------------------------------------------------
class _PlainBase:
    class Linear(nn.Linear):
        comfy_cast_weights = False

        def __init__(self, in_features, out_features, bias=True, device=None, dtype=None):
            super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
            self.weight_function = []
            self.bias_function = []

    GroupNorm, LayerNorm, Conv2d, Conv3d = nn.GroupNorm, nn.LayerNorm, nn.Conv2d, nn.Conv3d
    ConvTranspose2d, Embedding = nn.ConvTranspose2d, nn.Embedding


def _plain_cast(module, input=None, dtype=None, device=None, bias_dtype=None, offloadable=False):
    if input is not None:
        dtype, device = input.dtype, input.device
    bias = None if module.bias is None else module.bias.to(device=device, dtype=bias_dtype or dtype)
    return module.weight.to(device=device, dtype=dtype), bias, None


def _plain_uncast(module, weight, bias, offload_stream):
    return None


StandaloneInt8Ops = _define_ops(_PlainBase, _plain_cast, _plain_uncast)
