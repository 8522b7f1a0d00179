"""One registry from an architecture's name to its configuration class and model builder.

The reference resolves a file's architecture string against an ordered list of
classes and fails closed when none matches (app/architectures/registry.py:25-53).
Here the key is ``architectures[0]`` or ``model_type`` from config.json; an
unknown name is an error, never an approximate run.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from matricxon_b200.config.base import ConfigError, read_config_json


class UnsupportedArchitectureError(ConfigError):
    """config.json names an architecture that no entry of the registry covers."""


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    aliases: tuple[str, ...]
    config_class: type
    # (config, runtime) -> model; imported lazily so that reading a config needs no GPU code
    build_model: Callable[[Any, Any], Any]


_REGISTRY: dict[str, ArchitectureEntry] = {}


def register_architecture(entry: ArchitectureEntry) -> None:
    for key in (entry.name, *entry.aliases):
        existing = _REGISTRY.get(key)
        if existing is not None and existing is not entry:
            raise ValueError(f"architecture name {key!r} is already registered for {existing.name}")
        _REGISTRY[key] = entry


def supported_names() -> list[str]:
    return sorted(_REGISTRY)


def resolve_architecture(raw: dict[str, Any]) -> ArchitectureEntry:
    names: list[str] = []
    architectures = raw.get("architectures")
    if isinstance(architectures, list):
        names.extend(str(a) for a in architectures)
    if isinstance(raw.get("model_type"), str):
        names.append(raw["model_type"])
    if not names:
        raise UnsupportedArchitectureError(
            "config.json has neither 'architectures' nor 'model_type'; cannot choose a model")
    for name in names:
        if name in _REGISTRY:
            return _REGISTRY[name]
    raise UnsupportedArchitectureError(
        f"unsupported architecture {names!r}; this engine runs {supported_names()}")


def config_from_dict(raw: dict[str, Any], where: str = "config.json"):
    return resolve_architecture(raw).config_class.from_dict(raw, where)


def load_config(model_dir: str | Path):
    """Reads ``model_dir/config.json`` into the typed config of the architecture it names."""
    raw = read_config_json(model_dir)
    return config_from_dict(raw, str(Path(model_dir) / "config.json"))


def entry_for_config(config: Any) -> ArchitectureEntry:
    for entry in set(_REGISTRY.values()):
        if isinstance(config, entry.config_class):
            return entry
    raise UnsupportedArchitectureError(f"no registered architecture uses {type(config).__name__}")


def _build_decoder(config: Any, runtime: Any) -> Any:
    from matricxon_b200.models.decoder import DecoderModel

    return DecoderModel(config.model_spec(), runtime)


def _register_builtin() -> None:
    from matricxon_b200.config.starcoder2 import Starcoder2Config

    register_architecture(ArchitectureEntry(
        name="starcoder2",
        aliases=("Starcoder2ForCausalLM",),
        config_class=Starcoder2Config,
        build_model=_build_decoder,
    ))


_register_builtin()
