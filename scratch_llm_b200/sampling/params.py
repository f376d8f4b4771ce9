"""Decode configuration, with the reference's names and meanings
(src/scratch_llm/sampling.py:49-57): ``temperature`` 0 is greedy argmax, otherwise logits are
divided by it; ``top_p`` >= 1 switches the nucleus filter off; ``max_tokens`` is the budget of
generated tokens; generation stops as soon as a token of ``stop_ids`` is produced (that token is
kept in the output); ``seed`` seeds the request's own generator (None: a seed derived from the
request's id)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    max_tokens: int = 256
    stop_ids: tuple[int, ...] = ()
    seed: int | None = None

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0 < self.top_p:
            raise ValueError(f"top_p must be positive, got {self.top_p}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be at least 1, got {self.max_tokens}")
        object.__setattr__(self, "stop_ids", tuple(int(t) for t in self.stop_ids))
