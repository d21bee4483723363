"""Import name of the library whose sources live in ``pico-engine_b200/``.

That folder's name is no Python identifier, so this package adds it to its search path:
``import pico_engine.config`` loads ``pico-engine_b200/config/``, and ``python -m pico_engine``
runs ``pico-engine_b200/__main__.py``.  The import name is the one pico-engine itself uses
(src/pico_engine/__init__.py), and like there the heavy names are loaded on first use.
"""
import os as _os

__path__.append(_os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "pico-engine_b200"))

__all__ = ["Engine", "read_config", "Qwen2Config"]


def __getattr__(name: str):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name in ("read_config", "Qwen2Config"):
        from . import config
        return getattr(config, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
