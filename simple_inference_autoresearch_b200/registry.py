"""One registry from an architecture's name to its configuration class and model.

The reference keys its plugins by the checkpoint's ``model_type`` and prefers a
nested ``text_config.model_type`` (model/registry.py:45-93); a duplicate
registration and an unknown type are ``ValueError``s there and here.  Here the
first name in ``architectures`` is looked up first (it is the more specific key),
then the model type.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, Mapping, Tuple


@dataclass(frozen=True)
class Architecture:
    name: str
    model_types: Tuple[str, ...]
    config_cls: Any                      # has from_dict(dict) and to_dict()
    spec_builder: Callable[..., Any]     # config -> ModelSpec


_BY_NAME: Dict[str, Architecture] = {}
_BY_TYPE: Dict[str, Architecture] = {}
_builtins_loaded = False


def register_architecture(name: str, model_types=(), config_cls=None, spec_builder=None) -> Architecture:
    arch = Architecture(name, tuple(model_types), config_cls, spec_builder)
    old = _BY_NAME.get(name)
    if old is not None and (old.config_cls is not config_cls or old.spec_builder is not spec_builder):
        raise ValueError(f"architecture {name!r} is already registered")
    for mt in arch.model_types:
        o = _BY_TYPE.get(mt)
        if o is not None and o.name != name:
            raise ValueError(f"model type {mt!r} is already registered by {o.name!r}")
    _BY_NAME[name] = arch
    for mt in arch.model_types:
        _BY_TYPE[mt] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _BY_NAME.pop(name, None)
    if arch:
        for mt in arch.model_types:
            if _BY_TYPE.get(mt) is arch:
                del _BY_TYPE[mt]


def _load_builtins() -> None:
    global _builtins_loaded
    if not _builtins_loaded:
        _builtins_loaded = True
        from . import architectures  # noqa: F401


def registered() -> Tuple[str, ...]:
    _load_builtins()
    return tuple(sorted(_BY_NAME))


def checkpoint_keys(raw: Mapping[str, Any]) -> Tuple[Tuple[str, ...], str]:
    archs = tuple(str(a) for a in (raw.get("architectures") or ()))
    text = raw.get("text_config")
    if isinstance(text, Mapping) and text.get("model_type"):
        return archs, str(text["model_type"])
    return archs, str(raw.get("model_type") or "")


def resolve(raw: Mapping[str, Any]) -> Architecture:
    """The architecture a config.json (as a dict) asks for."""
    _load_builtins()
    archs, model_type = checkpoint_keys(raw)
    for a in archs:
        if a in _BY_NAME:
            return _BY_NAME[a]
    if model_type in _BY_TYPE:
        return _BY_TYPE[model_type]
    if not archs and not model_type:
        raise ValueError("config.json names neither 'architectures' nor 'model_type'")
    raise ValueError(f"unsupported architecture {list(archs) or model_type!r} (model_type {model_type!r}); "
                     f"registered: {', '.join(sorted(_BY_NAME))}; model types: {', '.join(sorted(_BY_TYPE))}")


def resolve_path(path) -> Tuple[Architecture, Any]:
    """(architecture, typed config) of a model folder or config.json path."""
    path = Path(path)
    if path.is_dir():
        path = path / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"no config.json at {path}")
    with open(path) as f:
        raw = json.load(f)
    arch = resolve(raw)
    return arch, arch.config_cls.from_dict(raw)
