"""Seeded random weights: every matrix ~ N(0, std^2), every gain 1, each tensor drawn from a
generator keyed by (seed, tensor name) so that the values do not depend on the order in which
tensors are made.

The reference's tests build a fresh ``TransformerLM`` under ``torch.manual_seed``
(tests/test_continuous.py:25-30), whose init scheme is src/scratch_llm/model.py:117-146; the
engine's random mode instead writes a model folder (config.json, model.safetensors) that every
other entry point can open.
"""

from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Mapping

import torch

from .loader import ParamSpec
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensors(specs: Mapping[str, ParamSpec], seed: int, dtype: torch.dtype,
                   std: float = 0.02, device: str | torch.device = "cpu"
                   ) -> dict[str, torch.Tensor]:
    """Draw every tensor of ``specs``.  On the CPU the values are a function of (seed, name)
    alone; on a CUDA device they come from that device's generator, seeded the same way."""
    device = torch.device(device)
    out: dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        if spec.kind == "gain":
            out[name] = torch.ones(spec.shape, dtype=torch.float32 if dtype == torch.float32
                                   else dtype, device=device)
        elif spec.kind == "int":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        else:
            gen = torch.Generator(device=device)
            gen.manual_seed(_tensor_seed(seed, name))
            t = torch.empty(spec.shape, dtype=torch.float32, device=device)
            t.normal_(0.0, std, generator=gen)
            out[name] = t.to(dtype)
    return out


def write_random_model(config, model_dir: str | Path, seed: int, std: float = 0.02,
                       dtype: str | None = None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded weights.
    ``dtype`` ("bfloat16" or "float32") defaults to the configuration's ``torch_dtype``."""
    from ..config import get_architecture, save_config
    from ..engine.model import build_model

    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    get_architecture(config.architecture)  # an unregistered architecture fails here
    store = _STORE[dtype or getattr(config, "torch_dtype", "bfloat16")]
    model = build_model(config)
    tensors = random_tensors(model.param_specs(), seed, store, std)
    save_config(config, model_dir)
    write_safetensors(model_dir / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed), "std": repr(std)})
    return model_dir
