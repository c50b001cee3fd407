"""Stand-in for comfy.lora: key map + LoRA state-dict -> adapter patches."""
from comfy.weight_adapter.lora import LoRAAdapter


def model_lora_keys_unet(model, key_map=None):
    key_map = {} if key_map is None else key_map
    for name, _ in model.diffusion_model.named_parameters():
        if name.endswith(".weight"):
            key_map[f"diffusion_model.{name[:-7]}"] = f"diffusion_model.{name}"
    return key_map


def load_lora(lora, to_load, log_missing=True):
    """`lora` maps '<prefix>.lora_up.weight', '<prefix>.lora_down.weight', optional '<prefix>.alpha'."""
    patches = {}
    for prefix, target in to_load.items():
        up, down = lora.get(f"{prefix}.lora_up.weight"), lora.get(f"{prefix}.lora_down.weight")
        if up is None or down is None:
            continue
        alpha = lora.get(f"{prefix}.alpha")
        alpha = float(alpha) if alpha is not None else None
        keys = {f"{prefix}.lora_up.weight", f"{prefix}.lora_down.weight"}
        patches[target] = LoRAAdapter(keys, (up, down, alpha, None, None, None))
    return patches
