"""INT8 Fast for B200: the W8A8 linear hot path of ComfyUI-INT8-Fast on hand-written sm_100a kernels.

The directory is a ComfyUI custom-node package (drop it under ``custom_nodes/``);
outside ComfyUI it can be loaded with importlib under any module name.  The
kernels live in ``libi8f.so`` (see ``build_native.py``); there is no Triton,
CPU or other fallback.
"""
from . import _native, functional, workloads  # noqa: F401

__all__ = ["_native", "functional", "workloads"]
