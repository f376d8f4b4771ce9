"""The one registry from an architecture's name (``config.json``'s ``architectures[0]``) to
its typed configuration and model.

The reference has no registry (its model is constructed directly from ``ModelConfig``,
src/scratch_llm/train.py:164-183); a model folder here names its architecture, and everything
that opens a folder goes through :func:`load_config`.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping, Protocol


class ArchConfig(Protocol):
    """What a configuration class must offer to be registered."""

    architecture: str

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ArchConfig": ...

    def to_dict(self) -> dict[str, Any]: ...

    def model_spec(self): ...  # -> config.spec.ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    # model factory: (ModelSpec, dtype, device) -> model; None means the generic decoder of
    # scratch_llm_b200.engine.model, which every spec made of registered parts can use
    model_factory: Callable[..., Any] | None = None


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type,
                          model_factory: Callable[..., Any] | None = None) -> None:
    if name in ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = Architecture(name, config_cls, model_factory)


def get_architecture(name: str) -> Architecture:
    try:
        return ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(ARCHITECTURES)) or "(none)"
        raise ValueError(f"unknown architecture {name!r}; registered: {known}") from None


def config_from_dict(raw: Mapping[str, Any]):
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ValueError("config.json must name exactly one architecture in 'architectures', "
                         f"got {archs!r}")
    return get_architecture(archs[0]).config_cls.from_dict(raw)


def load_config(model_dir: str | Path):
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and "
                                "model.safetensors")
    return config_from_dict(json.loads(path.read_text(encoding="utf-8")))


def save_config(config, model_dir: str | Path) -> Path:
    path = Path(model_dir) / "config.json"
    path.write_text(json.dumps(config.to_dict(), indent=2) + "\n", encoding="utf-8")
    return path
