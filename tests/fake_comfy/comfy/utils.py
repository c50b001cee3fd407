"""Stand-in for comfy.utils: files are an in-memory table filled by tests."""
FILES = {}


def load_torch_file(path, safe_load=True):
    return dict(FILES[path])
