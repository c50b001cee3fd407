"""The five ComfyUI nodes of the INT8 node pack (loader, stochastic LoRA x2,
dynamic LoRA x2).  Node ids, widget names, orders, ranges and defaults are the
ones saved workflows refer to; the work behind them runs on the sm_100a
kernels via ops.py.
"""
from __future__ import annotations

import logging

import comfy.lora
import comfy.sd
import comfy.utils
import folder_paths
import torch

from .ops import DynamicLoRAHook, Int8TensorwiseOps

# Name fragments of layers that stay in high precision, per model family   (int8_unet_loader.py:54-93)
EXCLUDED_LAYERS = {
    "flux2": ["img_in", "time_in", "guidance_in", "txt_in", "final_layer", "double_stream_modulation_img",
              "double_stream_modulation_txt", "single_stream_modulation"],
    "z-image": ["cap_embedder", "t_embedder", "x_embedder", "cap_pad_token", "context_refiner", "final_layer",
                "noise_refiner", "adaLN", "x_pad_token", "layers.0."],
    "chroma": ["distilled_guidance_layer", "final_layer", "img_in", "txt_in", "nerf_image_embedder", "nerf_blocks",
               "nerf_final_layer_conv", "__x0__", "nerf_final_layer_conv"],
    "wan": ["patch_embedding", "text_embedding", "time_embedding", "time_projection", "head", "img_emb"],
    "ltx2": ["adaln_single", "audio_adaln_single", "audio_caption_projection", "audio_patchify_proj", "audio_proj_out",
             "audio_scale_shift_table", "av_ca_a2v_gate_adaln_single", "av_ca_audio_scale_shift_adaln_single",
             "av_ca_v2a_gate_adaln_single", "av_ca_video_scale_shift_adaln_single", "caption_projection",
             "patchify_proj", "proj_out", "scale_shift_table"],
    "qwen": ["time_text_embed", "img_in", "norm_out", "proj_out", "txt_in"],
    "ernie": ["time", "x_embedder", "adaLN", "final", "text_proj", "norm", "layers.0.", "layers.35"],
    "anima": ["embed", "llm", "blocks.0.", "blocks.1.", "blocks.2."],
}
MODEL_TYPES = ["flux2", "z-image", "chroma", "wan", "ltx2", "qwen", "ernie", "anima"]
STOCHASTIC_SEED = 318008
STACK_SLOTS = 10


class UNetLoaderINTW8A8:
    """Loads a diffusion model with Int8TensorwiseOps: pre-quantised int8 checkpoints directly, float
    checkpoints quantised while loading when on_the_fly_quantization is set."""

    @classmethod
    def INPUT_TYPES(s):
        return {"required": {
            "unet_name": (folder_paths.get_filename_list("diffusion_models"),),
            "weight_dtype": (["default", "fp8_e4m3fn", "fp16", "bf16"],),
            "model_type": (list(MODEL_TYPES),),
            "on_the_fly_quantization": ("BOOLEAN", {"default": False}),
            "enable_quarot": ("BOOLEAN", {"default": False,
                                          "tooltip": "Enable QuaRot (Hadamard rotation) for better quantization."}),
        }}

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "load_unet"
    CATEGORY = "loaders"
    DESCRIPTION = "Load INT8 quantized diffusion models; W8A8 linears run on B200 tensor cores."

    def load_unet(self, unet_name, weight_dtype, model_type, on_the_fly_quantization, enable_quarot=False):
        path = folder_paths.get_full_path("diffusion_models", unet_name)
        Int8TensorwiseOps.excluded_names = list(EXCLUDED_LAYERS.get(model_type, []))
        Int8TensorwiseOps.dynamic_quantize = on_the_fly_quantization
        Int8TensorwiseOps.enable_quarot = enable_quarot
        Int8TensorwiseOps.use_triton = True
        Int8TensorwiseOps._is_prequantized = False
        model = comfy.sd.load_diffusion_model(path, model_options={"custom_operations": Int8TensorwiseOps})
        return (model,)


# --------------------------------------------------------------------- helpers
def _lora_patches(model_patcher, lora_state):
    """ComfyUI's key map + patch dict for one LoRA state dict."""
    key_map = {}
    if model_patcher.model.model_type.name != "ModelType.CLIP":
        key_map = comfy.lora.model_lora_keys_unet(model_patcher.model, key_map)
    return comfy.lora.load_lora(lora_state, key_map, log_missing=True)


def _target_module(model_patcher, key):
    """Module a patch key points at: 'diffusion_model.a.0.b.weight' or ('...', (dim, start, size))."""
    name = key[0] if isinstance(key, tuple) else key
    if name.endswith(".weight"):
        name = name[: -len(".weight")]
    parts = name.split(".")
    if parts[0] == "diffusion_model":
        parts = parts[1:]
    module = model_patcher.model.diffusion_model
    for part in parts:
        module = module[int(part)] if part.isdigit() else getattr(module, part)
    return module


def _scale_of(module):
    ws = module._get_weight_scale()
    if isinstance(ws, torch.Tensor) and ws.numel() == 1:
        ws = ws.item()
    return ws


def _stack_entries(kwargs):
    for i in range(1, STACK_SLOTS + 1):
        name, strength = kwargs.get(f"lora_{i}"), kwargs.get(f"strength_{i}", 0)
        if name and name != "None" and strength != 0:
            yield name, strength


def _stack_inputs(limit):
    inputs = {"required": {"model": ("MODEL",)}, "optional": {}}
    names = ["None"] + folder_paths.get_filename_list("loras")
    for i in range(1, STACK_SLOTS + 1):
        inputs["optional"][f"lora_{i}"] = (names,)
        inputs["optional"][f"strength_{i}"] = ("FLOAT", {"default": 1.0, "min": -limit, "max": limit, "step": 0.01})
    return inputs


# ------------------------------------------------------------ stochastic LoRA
class INT8LoraLoader:
    """Registers a LoRA as INT8-space patches: ComfyUI's patcher hands each quantised layer's raw
    int8 weight to the adapter, which merges the update with stochastic rounding."""

    @classmethod
    def INPUT_TYPES(s):
        return {"required": {
            "model": ("MODEL",),
            "lora_name": (folder_paths.get_filename_list("loras"),),
            "strength": ("FLOAT", {"default": 1.0, "min": -10.0, "max": 10.0, "step": 0.01}),
        }}

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "load_lora"
    CATEGORY = "loaders"
    DESCRIPTION = "Loads LoRA for INT8 models with INT8-space patching (stochastic rounding)."

    def load_lora(self, model, lora_name, strength, seed=STOCHASTIC_SEED):
        if strength == 0:
            return (model,)
        from .ops import INT8LoRAPatchAdapter
        state = comfy.utils.load_torch_file(folder_paths.get_full_path("loras", lora_name), safe_load=True)
        patcher = model.clone()
        patches = _lora_patches(patcher, state)
        del state
        upgraded, out = 0, {}
        for key, adapter in patches.items():
            out[key] = adapter
            try:
                module = _target_module(patcher, key)
                if getattr(module, "_is_quantized", False):
                    out[key] = INT8LoRAPatchAdapter(adapter.loaded_keys, adapter.weights, _scale_of(module), seed=seed)
                    upgraded += 1
            except (AttributeError, KeyError, IndexError, TypeError):
                pass  # not resolvable: keep ComfyUI's stock adapter
        patcher.add_patches(out, strength)
        logging.info(f"INT8 LoRA: Registered '{lora_name}' with strength {strength:.2f} for {upgraded} quantized layers.")
        print(f"[INT8 LoRA] Patched {upgraded} layers, skipped {len(patches) - upgraded}.")
        return (patcher,)


class INT8LoraLoaderStack:
    """Up to ten stochastic LoRAs: deltas are summed in high precision and rounded once per layer."""

    @classmethod
    def INPUT_TYPES(s):
        return _stack_inputs(10.0)

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "apply_stack"
    CATEGORY = "loaders"
    DESCRIPTION = "Applies a stack of LoRAs using stochastic rounding for INT8 models."

    def apply_stack(self, model, seed=STOCHASTIC_SEED, **kwargs):
        from .ops import INT8MergedLoRAPatchAdapter
        loaded = [(comfy.utils.load_torch_file(folder_paths.get_full_path("loras", name), safe_load=True), strength)
                  for name, strength in _stack_entries(kwargs)]
        if not loaded:
            return (model,)
        patcher = model.clone()
        per_key: dict = {}
        for state, strength in loaded:
            for key, adapter in _lora_patches(patcher, state).items():
                per_key.setdefault(key, []).append((adapter, strength))
        merged, quantized = {}, 0
        for key, stack in per_key.items():
            try:
                module = _target_module(patcher, key)
                scale = 1.0
                if getattr(module, "_is_quantized", False):
                    scale = _scale_of(module)
                    quantized += 1
                merged[key] = INT8MergedLoRAPatchAdapter(stack, scale, seed=seed)
            except Exception:  # noqa: BLE001 - unresolvable target: apply the stack one by one
                for adapter, strength in stack:
                    patcher.add_patches({key: adapter}, strength)
        patcher.add_patches(merged, 1.0)   # strengths are applied inside the merged adapter
        logging.info(f"INT8 LoRA Stack: Merged {len(loaded)} LoRAs for {quantized} quantized layers.")
        print(f"[INT8 LoRA Stack] Applied {len(loaded)} LoRAs, merged {quantized} quantized layers.")
        return (patcher,)


# --------------------------------------------------------------- dynamic LoRA
class INT8DynamicLoraLoader:
    """Keeps the weights untouched and adds the low-rank path at run time (hook + transformer_options)."""

    @classmethod
    def INPUT_TYPES(s):
        return {"required": {
            "model": ("MODEL",),
            "lora_name": (folder_paths.get_filename_list("loras"),),
            "strength": ("FLOAT", {"default": 1.0, "min": -20.0, "max": 20.0, "step": 0.01}),
        }}

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "load_lora"
    CATEGORY = "loaders"

    def load_lora(self, model, lora_name, strength):
        if strength == 0:
            return (model,)
        state = comfy.utils.load_torch_file(folder_paths.get_full_path("loras", lora_name), safe_load=True)
        patcher = model.clone()
        patches = _lora_patches(patcher, state)
        DynamicLoRAHook.register(patcher.model.diffusion_model)
        opts = patcher.model_options.setdefault("transformer_options", {})
        # copy so that the parent patcher's list is not extended
        opts["dynamic_loras"] = list(opts.get("dynamic_loras", []))
        opts["dynamic_loras"].append({"name": lora_name, "strength": strength, "patches": patches})
        return (patcher,)


class INT8DynamicLoraStack:
    """Up to ten dynamic LoRAs in one node."""

    @classmethod
    def INPUT_TYPES(s):
        return _stack_inputs(20.0)

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "apply_stack"
    CATEGORY = "loaders"

    def apply_stack(self, model, **kwargs):
        loader = INT8DynamicLoraLoader()
        for name, strength in _stack_entries(kwargs):
            (model,) = loader.load_lora(model, name, strength)
        return (model,)


NODE_CLASS_MAPPINGS = {
    "OTUNetLoaderW8A8": UNetLoaderINTW8A8,
    "INT8LoraLoader": INT8LoraLoader,
    "INT8LoraLoaderStack": INT8LoraLoaderStack,
    "INT8DynamicLoraLoader": INT8DynamicLoraLoader,
    "INT8DynamicLoraStack": INT8DynamicLoraStack,
}

NODE_DISPLAY_NAME_MAPPINGS = {
    "OTUNetLoaderW8A8": "Load Diffusion Model INT8 (W8A8)",
    "INT8LoraLoader": "Load LoRA INT8 (Stochastic)",
    "INT8LoraLoaderStack": "INT8 LoRA Stack (Stochastic)",
    "INT8DynamicLoraLoader": "Load LoRA INT8 (Dynamic)",
    "INT8DynamicLoraStack": "INT8 LoRA Stack (Dynamic)",
}
