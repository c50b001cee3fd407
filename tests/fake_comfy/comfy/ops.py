"""Stand-in for comfy.ops: an ops namespace whose layers skip weight init and
can cast weights on demand."""
import torch
from torch import nn


def cast_bias_weight(module, input=None, dtype=None, device=None, bias_dtype=None, offloadable=False):
    """Return (weight, bias, offload_stream) moved to the input's device/dtype."""
    if input is not None:
        dtype = dtype if dtype is not None else input.dtype
        device = device if device is not None else input.device
        bias_dtype = bias_dtype if bias_dtype is not None else dtype
    w = module.weight.to(device=device, dtype=dtype)
    for fn in getattr(module, "weight_function", []):
        w = fn(w)
    b = None
    if module.bias is not None:
        b = module.bias.to(device=device, dtype=bias_dtype if bias_dtype is not None else module.bias.dtype)
        for fn in getattr(module, "bias_function", []):
            b = fn(b)
    module._cast_calls = getattr(module, "_cast_calls", 0) + 1
    return w, b, None


def uncast_bias_weight(module, weight, bias, offload_stream):
    module._uncast_calls = getattr(module, "_uncast_calls", 0) + 1


class _CastMixin:
    comfy_cast_weights = False

    def _init_cast_state(self):
        self.weight_function = []
        self.bias_function = []

    def reset_parameters(self):
        return None


class disable_weight_init:
    class Linear(nn.Linear, _CastMixin):
        def __init__(self, in_features, out_features, bias=True, device=None, dtype=None):
            super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
            self._init_cast_state()

    class GroupNorm(nn.GroupNorm, _CastMixin):
        pass

    class LayerNorm(nn.LayerNorm, _CastMixin):
        pass

    class Conv2d(nn.Conv2d, _CastMixin):
        pass

    class Conv3d(nn.Conv3d, _CastMixin):
        pass

    class ConvTranspose2d(nn.ConvTranspose2d, _CastMixin):
        pass

    class Embedding(nn.Embedding, _CastMixin):
        pass

    @classmethod
    def conv_nd(cls, dims, *args, **kwargs):
        if dims == 2:
            return cls.Conv2d(*args, **kwargs)
        if dims == 3:
            return cls.Conv3d(*args, **kwargs)
        raise ValueError(f"unsupported dimensions: {dims}")


class manual_cast(disable_weight_init):
    class Linear(disable_weight_init.Linear):
        comfy_cast_weights = False

    class GroupNorm(disable_weight_init.GroupNorm):
        pass

    class LayerNorm(disable_weight_init.LayerNorm):
        pass

    class Conv2d(disable_weight_init.Conv2d):
        pass

    class Conv3d(disable_weight_init.Conv3d):
        pass

    class ConvTranspose2d(disable_weight_init.ConvTranspose2d):
        pass

    class Embedding(disable_weight_init.Embedding):
        pass
