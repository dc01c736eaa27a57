"""Picks the next token of every row of a batch of logits on the device.

Rows whose options are plain greedy take the argmax kernel; the others take the sampling kernel,
which follows integrallis/models' Sampler step by step (models-runtime/.../Sampler.java:78-151).
Each request draws from its own stream: Philox keyed by its seed, counted by its draws.
"""

from __future__ import annotations

import secrets
from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from .options import SamplingOptions


class RequestSampling:
    """Sampling state of one request: its options, its seed, how many draws it has made."""

    def __init__(self, options: SamplingOptions, prompt: Sequence[int]):
        self.options = options
        self.seed = options.seed if options.seed is not None else secrets.randbits(62)
        self.draws = 0
        # the reference penalises every earlier token, prompt included (GenerationLoop.java:165-169)
        self.history: Optional[List[int]] = list(prompt) if options.repetition_penalty > 1.0 else None


class BatchSampler:
    def __init__(self, vocab_size: int, device):
        self.vocab = vocab_size
        self.device = torch.device(device)
        self._max_sorted = None

    def check(self, options: SamplingOptions) -> None:
        """Refuses what the kernel cannot do exactly, before any step runs."""
        if options.temperature == 0.0:
            return
        if self._max_sorted is None:
            self._max_sorted = ops.sample_max_sorted()
        if min(options.top_k, self.vocab) > self._max_sorted and options.top_p < 1.0:
            raise ValueError(
                f"top_p < 1 needs the candidates sorted, which the sampling kernel does for at most "
                f"{self._max_sorted} of them: use top_k <= {self._max_sorted}, or top_p = 1 (got top_k "
                f"{options.top_k}, top_p {options.top_p})")

    def sample(self, logits: torch.Tensor, requests: Sequence[RequestSampling], greedy=None) -> torch.Tensor:
        """logits: float32 [len(requests), vocab] on the device.  Returns int32 token ids on the
        device, one per request, and advances the draw counters.  `greedy(logits)`, if given,
        supplies the argmax of every row (the decode graph computes it along with the logits)."""
        rows = len(requests)
        if logits.shape[0] < rows or logits.shape[1] != self.vocab:
            raise ValueError(f"logits {tuple(logits.shape)} do not fit {rows} requests of vocabulary {self.vocab}")
        if all(r.options.greedy for r in requests):
            return greedy(logits)[:rows] if greedy is not None else ops.argmax_rows(logits[:rows])
        logits = logits[:rows]
        temperature = torch.tensor([r.options.temperature for r in requests], dtype=torch.float32)
        top_k = torch.tensor([min(r.options.top_k, self.vocab) for r in requests], dtype=torch.int32)
        top_p = torch.tensor([r.options.top_p for r in requests], dtype=torch.float32)
        penalty = torch.tensor([r.options.repetition_penalty for r in requests], dtype=torch.float32)
        seeds = torch.tensor([r.seed for r in requests], dtype=torch.int64)
        counters = torch.tensor([r.draws for r in requests], dtype=torch.int64)
        history = history_len = counts = None
        if any(r.history is not None for r in requests):
            longest = max(len(r.history) if r.history is not None else 0 for r in requests)
            host = torch.zeros((rows, max(1, longest)), dtype=torch.int32)
            lens = torch.zeros((rows,), dtype=torch.int32)
            for i, r in enumerate(requests):
                if r.history is not None:
                    host[i, :len(r.history)] = torch.tensor(r.history, dtype=torch.int32)
                    lens[i] = len(r.history)
            history, history_len = host.to(self.device), lens.to(self.device)
            counts = torch.empty((rows, self.vocab), dtype=torch.int32, device=self.device)
        work = torch.empty((rows, self.vocab), dtype=torch.float32, device=self.device)
        d = self.device
        out = ops.sample_rows(logits, work, counts, temperature.to(d), top_k.to(d), top_p.to(d), penalty.to(d), history,
                              history_len, seeds.to(d), counters.to(d))
        for r in requests:
            if r.options.temperature > 0.0:
                r.draws += 1
        return out

    @staticmethod
    def record(requests: Sequence[RequestSampling], tokens: Sequence[int]) -> None:
        for r, t in zip(requests, tokens):
            if r.history is not None:
                r.history.append(int(t))
