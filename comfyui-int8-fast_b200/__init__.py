"""INT8 Fast for B200: the W8A8 linear hot path of the ComfyUI-INT8-Fast node pack on hand-written
sm_100a kernels.

The directory is a ComfyUI custom-node package (drop it under ``custom_nodes/``): it registers the
``int8_tensorwise`` quantised layout, exports ``Int8TensorwiseOps`` and the five nodes.  Outside
ComfyUI it can be loaded with importlib under any module name; the ComfyUI-dependent parts then
degrade to empty mappings.  The kernels live in ``libi8f.so`` (see ``build_native.py``); there is
no Triton, CPU or other fallback for them.
"""
import logging

import torch

from . import _native, custom_ops, functional, parallel, quarot, workloads  # noqa: F401


def _register_layouts():
    """Registers the Int8Tensorwise layout and the int8_tensorwise algorithm with ComfyUI's quantisation
    registry (checkpoint keys: '<prefix>weight' int8, '<prefix>weight_scale', optional 'input_scale')."""
    try:
        from comfy.quant_ops import QUANT_ALGOS, QuantizedLayout, register_layout_class
    except ImportError:
        try:
            import comfy  # noqa: F401
            logging.warning("INT8 Fast: ComfyUI Quantization system not found (Update ComfyUI?)")
        except ImportError:
            logging.info("INT8 Fast: running outside ComfyUI, no layout registered")
        return None
    try:
        class Int8TensorwiseLayout(QuantizedLayout):
            class Params:
                def __init__(self, scale=None, orig_dtype=None, orig_shape=None, **kwargs):
                    self.scale, self.orig_dtype, self.orig_shape = scale, orig_dtype, orig_shape

                def clone(self):
                    scale = self.scale.clone() if isinstance(self.scale, torch.Tensor) else self.scale
                    return Int8TensorwiseLayout.Params(scale=scale, orig_dtype=self.orig_dtype, orig_shape=self.orig_shape)

            @classmethod
            def state_dict_tensors(cls, qdata, params):
                return {"": qdata, "weight_scale": params.scale}

            @classmethod
            def dequantize(cls, qdata, params):
                return qdata.float() * params.scale

        register_layout_class("Int8TensorwiseLayout", Int8TensorwiseLayout)
        QUANT_ALGOS.setdefault("int8_tensorwise", {
            "storage_t": torch.int8,
            # input_scale is listed so ComfyUI extracts it from checkpoints that carry one; the linear ignores it
            "parameters": {"weight_scale", "input_scale"},
            "comfy_tensor_layout": "Int8TensorwiseLayout",
        })
        return Int8TensorwiseLayout
    except Exception as e:  # noqa: BLE001
        logging.error(f"INT8 Fast: Failed to register layouts: {e}")
        return None


Int8TensorwiseLayout = _register_layouts()

from . import ops  # noqa: E402
from .ops import Int8TensorwiseOps  # noqa: E402,F401

try:
    from .nodes import NODE_CLASS_MAPPINGS, NODE_DISPLAY_NAME_MAPPINGS
except ImportError as e:
    # outside ComfyUI (benchmarks, tests of the kernels) there is nothing to register; inside it this is an error
    _outside_comfy = getattr(e, "name", None) in ("comfy", "folder_paths")
    logging.log(logging.INFO if _outside_comfy else logging.ERROR, f"INT8 Fast: Failed to import nodes: {e}")
    NODE_CLASS_MAPPINGS = {}
    NODE_DISPLAY_NAME_MAPPINGS = {}

__all__ = ["NODE_CLASS_MAPPINGS", "NODE_DISPLAY_NAME_MAPPINGS", "Int8TensorwiseOps"]
