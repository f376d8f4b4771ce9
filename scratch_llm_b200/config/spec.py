"""Architecture-neutral description of a decoder: what each layer is made of and in which
order layers run.

An architecture's typed configuration (for instance :class:`LlamaConfig`) translates its
``config.json`` keys into a :class:`ModelSpec`.  The engine builds parts from the spec alone:
no part and no engine file reads an architecture's configuration object, so another
architecture is added by writing a configuration class that emits a ``ModelSpec`` and
registering it.

The reference builds its model from a ``ModelConfig`` dataclass in code
(src/scratch_llm/model.py:56-114) with one repeated block (src/scratch_llm/model.py:449-469);
here the layer list and the run order are data.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` is a key of the matching registry in
    :mod:`scratch_llm_b200.parts.registry`; ``args`` are the part's sizes and constants."""

    kind: str
    args: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """What one layer is made of: ``block`` names the arrangement (a key of BLOCKS), ``parts``
    gives a :class:`PartSpec` for every role that arrangement has.  Which roles there are, and
    which registry each role's part comes from, is the block class's statement (its ``ROLES``):
    a layer with other roles (no feed-forward, four norms) needs another block class and
    nothing else.  ``prefix`` is the tensor-name prefix of the layer's weights; ``names`` gives
    the sub-prefix of each role below it (default: the role's name)."""

    prefix: str
    block: str
    parts: Mapping[str, PartSpec]
    names: Mapping[str, str] = field(default_factory=dict)


def standard_layer(prefix: str, block: str, mixer: PartSpec, feed_forward: PartSpec,
                   mixer_norm: PartSpec, feed_forward_norm: PartSpec, position: PartSpec,
                   names: Mapping[str, str] | None = None) -> LayerSpec:
    """A layer of the five roles that ``pre_norm`` (and any block of the same roles) arranges:
    mixer, feed-forward, a norm before each, and the mixer's position encoding."""
    return LayerSpec(prefix, block, {"mixer": mixer, "feed_forward": feed_forward,
                                     "mixer_norm": mixer_norm,
                                     "feed_forward_norm": feed_forward_norm,
                                     "position": position}, dict(names or {}))


@dataclass(frozen=True)
class Run:
    """One entry of the run order: run ``layer`` against cache entry ``cache``.

    ``write`` False means the mixer reads the cache entry another run filled earlier in the
    same step and stores nothing itself."""

    layer: int
    cache: int
    write: bool = True


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: tuple[LayerSpec, ...]
    order: tuple[Run, ...]
    final_norm: PartSpec
    embed_name: str
    final_norm_name: str
    lm_head_name: str
    tie_embeddings: bool
    #: the embedded tokens are multiplied by this before the first layer
    embedding_multiplier: float = 1.0
    #: the logits are multiplied by this, and then, if ``logit_softcap`` > 0, squashed to
    #: ``logit_softcap * tanh(logits / logit_softcap)``
    logit_scale: float = 1.0
    logit_softcap: float = 0.0

    def __post_init__(self) -> None:
        if self.logit_softcap < 0:
            raise ValueError(f"logit_softcap must not be negative, got {self.logit_softcap}")
        seen_write: set[int] = set()
        for run in self.order:
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run order names layer {run.layer}, but there are "
                                 f"{len(self.layers)} layers")
            if run.write:
                if run.cache in seen_write:
                    raise ValueError(f"cache entry {run.cache} is written by two runs")
                seen_write.add(run.cache)
            elif run.cache not in seen_write:
                raise ValueError(f"a run reads cache entry {run.cache} before any run wrote it")

    @property
    def n_cache_entries(self) -> int:
        return len({r.cache for r in self.order})


def sequential_order(n_layers: int) -> tuple[Run, ...]:
    """Every layer once, in index order, each with a cache entry of its own."""
    return tuple(Run(layer=i, cache=i) for i in range(n_layers))
