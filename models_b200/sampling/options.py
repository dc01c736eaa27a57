"""Sampling options with integrallis/models' names, meanings, defaults and checks
(models-api/.../SamplingOptions.java:28-61 validation, :121-130 builder defaults):
temperature >= 0 (0 is greedy), top_p in (0, 1], top_k > 0, max_tokens > 0, a nullable seed,
repetition_penalty >= 1.  Text stop sequences need a tokenizer, which this library does not have;
their place is taken by `stop_token_ids`, checked on token ids.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class SamplingOptions:
    temperature: float = 1.0
    top_p: float = 0.9
    top_k: int = 40
    max_tokens: int = 256
    seed: Optional[int] = None
    repetition_penalty: float = 1.0
    stop_token_ids: Tuple[int, ...] = ()

    def __post_init__(self):
        if not _finite(self.temperature) or self.temperature < 0:
            raise ValueError(f"temperature must be finite and >= 0, got: {self.temperature}")
        if not _finite(self.top_p) or self.top_p <= 0 or self.top_p > 1.0:
            raise ValueError(f"topP must be finite and in (0, 1], got: {self.top_p}")
        if isinstance(self.top_k, bool) or not isinstance(self.top_k, int) or self.top_k <= 0:
            raise ValueError(f"topK must be > 0, got: {self.top_k}")
        if isinstance(self.max_tokens, bool) or not isinstance(self.max_tokens, int) or self.max_tokens <= 0:
            raise ValueError(f"maxTokens must be > 0, got: {self.max_tokens}")
        if not _finite(self.repetition_penalty) or self.repetition_penalty < 1.0:
            raise ValueError(f"repetitionPenalty must be finite and >= 1.0, got: {self.repetition_penalty}")
        if self.seed is not None and (isinstance(self.seed, bool) or not isinstance(self.seed, int)):
            raise ValueError(f"seed must be an integer or None, got: {self.seed!r}")
        stops = tuple(self.stop_token_ids)
        for s in stops:
            if isinstance(s, bool) or not isinstance(s, int) or s < 0:
                raise ValueError(f"stop token ids must be non-negative integers, got: {s!r}")
        object.__setattr__(self, "stop_token_ids", stops)

    @property
    def greedy(self) -> bool:
        """The reference's fast path: argmax with no copy of the logits
        (models-runtime/.../Sampler.java:37-44)."""
        return self.temperature == 0.0 and self.repetition_penalty == 1.0

    @staticmethod
    def builder() -> "SamplingOptionsBuilder":
        return SamplingOptionsBuilder()


class SamplingOptionsBuilder:
    """Fluent form, as the reference's SamplingOptions.builder()."""

    def __init__(self):
        self._values = {}
        self._stops = []

    def temperature(self, value: float):
        self._values["temperature"] = float(value)
        return self

    def top_p(self, value: float):
        self._values["top_p"] = float(value)
        return self

    def top_k(self, value: int):
        self._values["top_k"] = value
        return self

    def max_tokens(self, value: int):
        self._values["max_tokens"] = value
        return self

    def seed(self, value: int):
        self._values["seed"] = value
        return self

    def repetition_penalty(self, value: float):
        self._values["repetition_penalty"] = float(value)
        return self

    def stop_token_id(self, value: int):
        self._stops.append(value)
        return self

    def build(self) -> SamplingOptions:
        return SamplingOptions(stop_token_ids=tuple(self._stops), **self._values)


def _finite(value) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)
