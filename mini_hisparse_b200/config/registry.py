"""One registry from the architecture's name (config.json "architectures"[0]) to its model.

The reference accepts exactly one model type and raises for anything else
(mini_hisparse/model.py:107-111).  Here an architecture is an entry of a table: a typed
configuration class and a function from that configuration to a ModelSpec.  Adding an
architecture is adding an entry; nothing else in the framework names one.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                    # has from_dict(mapping) -> typed config
    make_spec: Callable[[Any], Any]      # typed config -> ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, make_spec, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, make_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(config: Mapping[str, Any]) -> Architecture:
    names = config.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    if not names:
        raise KeyError(
            'config.json has no "architectures" entry; known architectures: '
            + ", ".join(known_architectures())
        )
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise KeyError(
        f"architecture {names[0]!r} is not registered; known architectures: "
        + ", ".join(known_architectures())
    )


def read_config(source) -> dict:
    """A config.json as a dict, from a folder, a file or a mapping."""
    if isinstance(source, Mapping):
        return dict(source)
    path = Path(source)
    if path.is_dir():
        path = path / "config.json"
    return json.loads(path.read_text())


def resolve(source):
    """(typed config, ModelSpec) of a folder, a config file or a config mapping."""
    raw = read_config(source)
    arch = architecture_of(raw)
    cfg = arch.config_class.from_dict(raw)
    return cfg, arch.make_spec(cfg)
