"""Editable associative memory: facts that can be written, read, listed, deleted and undone while
the server runs (python/minisgl/cam/memory.py, python/minisgl/server/cam_api.py)."""
from .client import CamClient, CamError
from .memory import CamMemory, Fact

__all__ = ["CamClient", "CamError", "CamMemory", "Fact"]
