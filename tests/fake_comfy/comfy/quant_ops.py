"""Stand-in for comfy.quant_ops: layout registry."""
QUANT_ALGOS = {}
LAYOUTS = {}


class QuantizedLayout:
    pass


def register_layout_class(name, cls):
    LAYOUTS[name] = cls
