"""Stand-in for comfy.weight_adapter.lora."""


class LoRAAdapter:
    name = "lora"

    def __init__(self, loaded_keys, weights):
        self.loaded_keys = loaded_keys
        self.weights = weights

    def calculate_weight(self, weight, key, strength, strength_model, offset, function, intermediate_dtype=None,
                         original_weight=None):
        raise NotImplementedError
