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
        self._pinned = [(torch.empty((256,), dtype=torch.int32).pin_memory(), torch.cuda.Event()) for _ in range(4)]
        self._pinned_next = 0

    def open_slot(self) -> int:
        return self.engine.open_slot()

    def release_slot(self, slot: int) -> None:
        self.engine.release_slot(slot)

    def rewind(self, slot: int, length: int) -> None:
        """Cuts the sequence back to its first `length` positions (raises where the cache cannot)."""
        self.engine.rewind(slot, length)

    def concat(self, first: torch.Tensor, second: torch.Tensor) -> torch.Tensor:
        """The rows of two steps' logits as one tensor (a copy: a replayed step's logits are its graph's own buffer)."""
        return torch.cat([first, second], dim=0)

    def check_options(self, options: SamplingOptions) -> None:
        self.sampler.check(options)

    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> torch.Tensor:
        return self.engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])

    def decode(self, slots: Sequence[int], tokens: Sequence[int]) -> torch.Tensor:
        return self.engine.decode(slots, tokens)

    def sample(self, logits: torch.Tensor, requests: Sequence[RequestSampling]) -> List[int]:
        return self.sampler.sample(logits, requests, self.engine.greedy_tokens).tolist()

    # -- the same in two halves, so that the next step can be queued before the ids reach the host

    def sample_start(self, logits: torch.Tensor, requests: Sequence[RequestSampling]) -> "PendingTokens":
        """Launches the sampling and the copy of the ids to the host; returns at once."""
        tokens = self.sampler.sample(logits, requests, self.engine.greedy_tokens)
        host, event = self._pinned[self._pinned_next]
        self._pinned_next = (self._pinned_next + 1) % len(self._pinned)
        if host.numel() < tokens.numel():
            host = torch.empty((max(256, tokens.numel()),), dtype=torch.int32).pin_memory()
            self._pinned[(self._pinned_next - 1) % len(self._pinned)] = (host, event)
        event.synchronize()  # the copy that last used this buffer (several steps ago) is done
        host[: tokens.numel()].copy_(tokens, non_blocking=True)
        event.record()
        return PendingTokens(tokens, host, event, tokens.numel())

    def decode_pending(self, slots: Sequence[int], pending: "PendingTokens", rows: Sequence[int]) -> torch.Tensor:
        """One more token for each slot, the token being row rows[i] of `pending` -- taken on the device."""
        tokens = pending.device
        if list(rows) != list(range(pending.count)):
            tokens = tokens[torch.tensor(list(rows), dtype=torch.long, device=tokens.device)]
        return self.engine.decode_device_tokens(slots, tokens)


class PendingTokens:
    """Sampled ids that are on the device and on their way to the host."""

    def __init__(self, device: torch.Tensor, host: torch.Tensor, event, count: int):
        self.device, self._host, self._event, self.count = device, host, event, count
        self._values = None

    def result(self) -> List[int]:
        if self._values is None:
            self._event.synchronize()
            self._values = self._host[: self.count].tolist()
        return self._values
