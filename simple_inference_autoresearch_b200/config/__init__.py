"""Typed configurations, read from each architecture's own config.json keys."""
from .llama import ConfigError, LlamaConfig, RopeScaling  # noqa: F401

from pathlib import Path as _Path

PRESET_DIR = _Path(__file__).resolve().parent / "presets"


def preset_path(name: str) -> _Path:
    """Path of a config.json shipped with the library (sizes live in these files, not in code)."""
    p = PRESET_DIR / f"{name}.json"
    if not p.exists():
        raise FileNotFoundError(f"no preset {name!r}; have: {', '.join(sorted(q.stem for q in PRESET_DIR.glob('*.json')))}")
    return p
