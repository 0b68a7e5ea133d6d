"""Typed configurations, read from each architecture's own config.json keys."""
from .llama import ConfigError, LlamaConfig, RopeScaling  # noqa: F401

from pathlib import Path as _Path

PRESET_DIR = _Path(__file__).resolve().parent / "presets"
_registered = {}


def register_preset(name: str, path) -> None:
    """Adds a named configuration (a config.json of any registered architecture) to the ones
    shipped with the library; ``--model NAME --random-weights`` and ``preset_path`` then find it."""
    path = _Path(path)
    if not path.exists():
        raise FileNotFoundError(f"no config.json at {path}")
    _registered[name] = path


def preset_names():
    return sorted({q.stem for q in PRESET_DIR.glob("*.json")} | set(_registered))


def preset_path(name: str) -> _Path:
    """Path of a named config.json: one shipped with the library (sizes live in these files, not
    in code) or one added with ``register_preset``."""
    if name in _registered:
        return _registered[name]
    p = PRESET_DIR / f"{name}.json"
    if not p.exists():
        raise FileNotFoundError(f"no preset {name!r}; have: {', '.join(preset_names())}")
    return p
