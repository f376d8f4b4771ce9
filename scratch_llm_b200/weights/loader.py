"""Loading a model folder's tensors by name.

A model states which tensors it wants (:class:`ParamSpec` by name); the loader opens
``model.safetensors`` (or the shards of ``model.safetensors.index.json``), checks the whole
set once and raises ONE :class:`WeightError` that lists every missing tensor, every unexpected
tensor and every wrong shape.  The reference gets the same strictness from
``load_state_dict(strict=True)`` (src/scratch_llm/train.py:164-183).

Dtype rule: tensors come back as the file stores them (bfloat16 stays bfloat16, a tensor
stored in 32-bit stays 32-bit, float16 is widened to bfloat16's range by a cast to bfloat16,
integer tables become int32).  Casting to what a kernel computes in is the part's decision
(:meth:`scratch_llm_b200.parts.base.Part.load`), never the loader's.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Mapping

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile

FLOAT_KINDS = ("matrix", "gain")


@dataclass(frozen=True)
class ParamSpec:
    """``kind``: ``"matrix"`` (an operand of a matrix product: cast to the compute dtype by its
    part), ``"gain"`` (a norm weight or other small vector: kept or widened to 32-bit),
    ``"int"`` (an integer table: int32)."""

    shape: tuple[int, ...]
    kind: str = "matrix"


class WeightError(ValueError):
    """The folder's tensors do not match what the model expects."""

    def __init__(self, where: str, missing: list[str], unexpected: list[str],
                 wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]],
                 wrong_dtype: list[tuple[str, str]] | None = None) -> None:
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        self.wrong_dtype = wrong_dtype or []
        lines = [f"weights in {where} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in self.wrong_dtype))
        super().__init__("\n".join(lines))


def _open_files(model_dir: Path) -> list[SafetensorsFile]:
    index = model_dir / "model.safetensors.index.json"
    single = model_dir / "model.safetensors"
    if single.is_file():
        return [SafetensorsFile(single)]
    if index.is_file():
        weight_map = json.loads(index.read_text(encoding="utf-8"))["weight_map"]
        return [SafetensorsFile(model_dir / name) for name in sorted(set(weight_map.values()))]
    raise FileNotFoundError(f"{model_dir} holds neither model.safetensors nor "
                            "model.safetensors.index.json")


def _as_stored(t: torch.Tensor, kind: str) -> torch.Tensor:
    if kind == "int":
        return t.to(torch.int32)
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    return t


def load_tensors(model_dir: str | Path, specs: Mapping[str, ParamSpec],
                 aliases: Mapping[str, str] | None = None,
                 optional: Mapping[str, str] | None = None) -> dict[str, torch.Tensor]:
    """Return ``{name: CPU tensor}`` for exactly the names of ``specs``.

    ``aliases`` maps other spellings of a tensor name onto the expected one.  ``optional``
    maps a name that the file may carry although the model does not want it onto the wanted
    tensor it must then equal (a tied output matrix stored beside the embedding)."""
    model_dir = Path(model_dir)
    files = _open_files(model_dir)
    found: dict[str, tuple[SafetensorsFile, str]] = {}
    unexpected: list[str] = []
    aliases = aliases or {}
    optional = optional or {}
    for f in files:
        for stored in f:
            name = stored if stored in specs or stored in optional else aliases.get(stored, stored)
            if name in found:
                unexpected.append(f"{stored} (a second tensor for {name})")
            elif name in specs or name in optional:
                found[name] = (f, stored)
            else:
                unexpected.append(stored)
    missing = [n for n in specs if n not in found]
    wrong_shape = []
    wrong_dtype = []
    for name, (f, stored) in found.items():
        e = f.entries[stored]
        spec = specs[name] if name in specs else specs.get(optional[name])
        if spec is None:
            continue
        if e.shape != tuple(spec.shape):
            wrong_shape.append((stored, e.shape, tuple(spec.shape)))
        is_float = e.dtype in (torch.float32, torch.bfloat16, torch.float16, torch.float64)
        if (spec.kind in FLOAT_KINDS) != is_float:
            wrong_dtype.append((stored, str(e.dtype).replace("torch.", "")))
    if not (missing or wrong_shape or wrong_dtype):
        for name, target in optional.items():
            if name in found and target in found:
                f, stored = found[name]
                g, other = found[target]
                if not torch.equal(f.tensor(stored), g.tensor(other)):
                    unexpected.append(f"{stored} (the model ties it to {other}, but the "
                                      "file's two tensors differ)")
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(str(model_dir), sorted(missing), sorted(unexpected), wrong_shape,
                          wrong_dtype)
    out = {}
    for name, spec in specs.items():
        f, stored = found[name]
        out[name] = _as_stored(f.tensor(stored), spec.kind)
    return out


__all__ = ["ParamSpec", "SafetensorsError", "WeightError", "load_tensors"]
