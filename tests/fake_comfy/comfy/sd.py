"""Stand-in for comfy.sd: tests register a loader callable."""
LOADER = None


def load_diffusion_model(path, model_options=None):
    if LOADER is None:
        raise RuntimeError("tests must set comfy.sd.LOADER")
    return LOADER(path, model_options or {})
