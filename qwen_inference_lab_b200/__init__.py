"""A single-GPU inference engine for dense Qwen3 on NVIDIA B200 (sm_100a).

``Engine`` and ``Qwen3`` are loaded on first use, as the reference's package does
(qil/__init__.py:5-15), so that importing the package needs neither a GPU nor the
compiled kernels.
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "Qwen3":
        from .loading import Qwen3
        return Qwen3
    if name == "load_model":
        from .loading import load_model
        return load_model
    raise AttributeError(name)


__all__ = ["Engine", "Qwen3", "load_model"]
