"""Stand-in for comfy.model_management."""
import torch

_FORCED_DEVICE = None


def get_torch_device():
    if _FORCED_DEVICE is not None:
        return _FORCED_DEVICE
    return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")


def cast_to_device(tensor, device, dtype, copy=False):
    return tensor.to(device=device, dtype=dtype, copy=copy)
