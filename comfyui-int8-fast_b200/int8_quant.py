"""Import-path compatibility: the node pack's public names under its original module name."""
from .ops import *  # noqa: F401,F403
from .ops import (DynamicLoRAHook, Int8TensorwiseOps, dequantize, int8_forward_dynamic,  # noqa: F401
                  int8_forward_dynamic_per_row, quantize_int8, quantize_int8_axiswise, quantize_int8_tensorwise,
                  reconstruct_lora_diff, stochastic_round_int8_delta)

try:
    from .ops import INT8LoRAPatchAdapter, INT8MergedLoRAPatchAdapter  # noqa: F401
except ImportError:
    pass
