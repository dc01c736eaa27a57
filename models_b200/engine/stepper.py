"""The generation loop's view of a real engine: prompts in one prefill step, then one token per
live sequence per step (from a CUDA graph when enabled), and sampling on the device."""

from __future__ import annotations

from typing import List, Sequence

import torch

from ..sampling.options import SamplingOptions
from ..sampling.sampler import BatchSampler, RequestSampling
from .engine import Engine, StepEntry


class EngineStepper:
    def __init__(self, engine: Engine):
        self.engine = engine
        self.sampler = BatchSampler(engine.spec.vocab_size, engine.device)
        self.page_size = engine.cache.page_size
        self.capacity_tokens = engine.cache.num_pages * engine.cache.page_size
        self.max_positions = engine.runtime.max_positions

    def open_slot(self) -> int:
        return self.engine.open_slot()

    def release_slot(self, slot: int) -> None:
        self.engine.release_slot(slot)

    def check_options(self, options: SamplingOptions) -> None:
        self.sampler.check(options)

    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> torch.Tensor:
        return self.engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])

    def decode(self, slots: Sequence[int], tokens: Sequence[int]) -> torch.Tensor:
        return self.engine.decode(slots, tokens)

    def sample(self, logits: torch.Tensor, requests: Sequence[RequestSampling]) -> List[int]:
        return self.sampler.sample(logits, requests, self.engine.greedy_tokens).tolist()
