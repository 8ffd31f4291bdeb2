"""One table from an architecture's name, as ``config.json`` spells it, to its model.

An architecture is registered with the class that types its ``config.json`` and a function
that turns such a configuration into a :class:`~miniserve_b200.parts.spec.ModelSpec`: the
list of layers with their parts, the order in which they run, and the tensor names.  Nothing
else in the package names an architecture; adding one is one ``register_architecture`` call.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping


class UnsupportedModelError(ValueError):
    """The configuration names no registered architecture, or asks for what is not implemented."""


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_spec: Callable[[Any], Any]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable[[Any], Any]) -> Architecture:
    """Registers (or replaces) the architecture ``name``.

    ``config_class.from_dict(mapping)`` must return the typed configuration and
    ``build_spec(configuration)`` the model description.
    """
    entry = Architecture(name, config_class, build_spec)
    _ARCHITECTURES[name] = entry
    return entry


def registered_architectures() -> tuple[str, ...]:
    _load_builtin()
    return tuple(sorted(_ARCHITECTURES))


def _load_builtin() -> None:
    from .. import architectures  # noqa: F401  (registers on import)


def resolve_architecture(config: Mapping[str, Any]) -> Architecture:
    """The registered architecture that ``config['architectures']`` names (exactly one name)."""
    _load_builtin()
    names = config.get("architectures") or ()
    if not isinstance(names, (list, tuple)) or len(names) != 1 or not isinstance(names[0], str):
        raise UnsupportedModelError(
            f"UNSUPPORTED_MODEL_CONFIGURATION: config.json must name exactly one architecture, got {names!r}; "
            f"registered: {', '.join(sorted(_ARCHITECTURES))}")
    try:
        return _ARCHITECTURES[names[0]]
    except KeyError:
        raise UnsupportedModelError(
            f"UNSUPPORTED_MODEL_CONFIGURATION: architecture {names[0]!r} is not registered; "
            f"registered: {', '.join(sorted(_ARCHITECTURES))}") from None


def read_config_json(folder: str | Path) -> dict[str, Any]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and *.safetensors")
    data = json.loads(path.read_text(encoding="utf-8"))
    if not isinstance(data, dict):
        raise UnsupportedModelError(f"{path} does not hold a JSON object")
    return data


def load_model_config(folder: str | Path):
    """``(architecture, typed configuration)`` of a model folder."""
    data = read_config_json(folder)
    architecture = resolve_architecture(data)
    return architecture, architecture.config_class.from_dict(data)
