"""Minimal stand-in for the ComfyUI `comfy` package (tests only)."""
