"""Stand-in for ComfyUI's folder_paths."""
FILES = {"diffusion_models": [], "loras": []}


def get_filename_list(kind):
    return list(FILES.get(kind, []))


def get_full_path(kind, name):
    return f"/{kind}/{name}"
