"""One registry from an architecture's name to its model.

An entry knows how to read the architecture's config.json into a typed configuration and how to turn that
into a ``ModelSpec`` (parts, run order, checkpoint names). The model class is chosen by config.json everywhere
in the package: ``architectures[0]`` first, ``model_type`` second. The reference binds a model id to a model in
its worker (src/Starlings.Roost.Worker.Runtime/Program.cs:28-33) and names the served ids when the id is
unknown; an unknown architecture here lists the registered ones.

Adding an architecture: write a module that builds a ``ModelSpec`` from its configuration and call
``register_architecture`` (the engine, cache manager, scheduler and step function do not change).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .config.reader import ConfigError, ConfigReader


@dataclass(frozen=True)
class Architecture:
    name: str
    model_types: tuple
    read_config: Callable          # ConfigReader -> typed configuration
    to_spec: Callable              # (configuration, tied: bool | None) -> ModelSpec
    # configuration -> [(slot name, shape, checkpoint tensors)]: the weight slots as the reference's model definition of
    # this architecture names them, for its seeded weight generator; None when the reference defines no such model
    reference_slots: Callable | None = None


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, *, model_types=(), read_config, to_spec, reference_slots=None) -> None:
    _ARCHITECTURES[name] = Architecture(name, tuple(model_types), read_config, to_spec, reference_slots)


def registered() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve(reader: ConfigReader) -> Architecture:
    names = reader.opt_strs("architectures") or []
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    model_type = reader.opt_str("model_type")
    if model_type is not None:
        for a in _ARCHITECTURES.values():
            if model_type in a.model_types:
                return a
    asked = ", ".join(names) or (f"model_type '{model_type}'" if model_type else "nothing (neither 'architectures' nor 'model_type' is set)")
    raise ConfigError(f"{reader.source}: no model is registered for {asked}; registered architectures: {', '.join(registered()) or 'none'}")


def _register_builtin() -> None:
    from .config import qwen3
    register_architecture(qwen3.ARCHITECTURE, model_types=(qwen3.MODEL_TYPE,), read_config=qwen3.Qwen3Config.from_reader,
                          to_spec=lambda cfg, tied=None: cfg.to_spec(tied), reference_slots=lambda cfg: cfg.reference_slots())


_register_builtin()
