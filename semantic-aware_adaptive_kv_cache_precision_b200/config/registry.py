"""One registry from an architecture's name (config.json `architectures[0]`) to
the class that reads its configuration. The model itself is always built by
`engine.model.DecoderModel` from the `ModelSpec` that class produces."""

from __future__ import annotations

import json
from pathlib import Path

from .specs import ConfigError

_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_class: type) -> None:
    """Make `name` loadable. `config_class` needs `from_dict(raw) -> config`,
    and the config needs `model_spec() -> ModelSpec` and `to_dict()`."""
    _ARCHITECTURES[name] = config_class


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_name(raw: dict) -> str:
    names = raw.get("architectures")
    if not isinstance(names, (list, tuple)) or not names or not isinstance(names[0], str):
        raise ConfigError("config.json has no `architectures` list naming the model class; "
                          f"known architectures: {', '.join(known_architectures())}")
    return names[0]


def config_from_dict(raw: dict):
    name = architecture_name(raw)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; known architectures: "
                          f"{', '.join(known_architectures())}")
    return _ARCHITECTURES[name].from_dict(raw)


def config_from_folder(folder):
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist: a model folder holds config.json and "
                          "model.safetensors")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not JSON: {exc}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return config_from_dict(raw)
