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
        # the same tokens on the device (int32, room for every token the request may still get): the
        # sampling kernel reads them there and stores each new id behind them, so a step sends no history
        self.history_device: Optional[torch.Tensor] = None
        self.history_sent = 0  # tokens of the history that the device array holds


class BatchSampler:
    def __init__(self, vocab_size: int, device):
        self.vocab = vocab_size
        self.device = torch.device(device)
        self._max_sorted = None
        self._staging = None
        self._staging_next = 0

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
        penalised = any(r.history is not None for r in requests)
        if penalised:
            for r in requests:
                if r.history is not None:
                    self._history_on_device(r)
        temperature, top_k, top_p, penalty, seeds, counters, history_rows, history_len = self._parameters(requests)
        counts = torch.empty((rows, self.vocab), dtype=torch.int32, device=self.device) if penalised else None
        if not penalised:
            history_rows = history_len = None
        work = torch.empty((rows, self.vocab), dtype=torch.float32, device=self.device)
        # the largest candidate set among the rows that cut anything (1 if none does): it picks the kernel
        most = max([min(r.options.top_k, self.vocab) for r in requests
                    if r.options.top_k < self.vocab or r.options.top_p < 1.0] or [1])
        out = ops.sample_rows(logits, work, counts, temperature, top_k, top_p, penalty, None, history_len, seeds, counters,
                              max_candidates=most, history_rows=history_rows, append=history_rows is not None)
        for r in requests:
            if r.options.temperature > 0.0:
                r.draws += 1
            if r.history_device is not None:
                r.history_sent += 1  # the kernel has stored this step's id behind the others
        return out

    def _history_on_device(self, r: RequestSampling) -> None:
        """The request's earlier tokens as a device array that the kernel extends by itself.  Sent once
        (the prompt); sent again only if the host's list and the device's count ever disagree, which
        happens when ids were recorded that this sampler did not draw."""
        room = len(r.history) + max(1, int(r.options.max_tokens)) + 4  # a finished request may be sampled once more
        if r.history_device is None or r.history_sent != len(r.history) or r.history_device.numel() < len(r.history) + 1:
            host = torch.zeros((room,), dtype=torch.int32)
            host[: len(r.history)] = torch.tensor(r.history, dtype=torch.int32)
            r.history_device = host.to(self.device)
            r.history_sent = len(r.history)

    def _parameters(self, requests: Sequence[RequestSampling]):
        """The per-row options on the device, sent as one asynchronous copy from pinned memory (a
        copy from ordinary memory would wait for every step that is still queued)."""
        rows = len(requests)
        if self._staging is None or self._staging[0][0].numel() < 48 * rows:
            size = 48 * max(64, rows)
            self._staging = [(torch.empty((size,), dtype=torch.uint8).pin_memory(), torch.cuda.Event()) for _ in range(4)]
        host, event = self._staging[self._staging_next]
        self._staging_next = (self._staging_next + 1) % len(self._staging)
        event.synchronize()  # the copy that last read this buffer, four calls ago
        device = torch.empty((48 * rows,), dtype=torch.uint8, device=self.device)

        def views(buffer):
            floats = buffer[: 12 * rows].view(torch.float32).view(3, rows)
            ints = buffer[12 * rows: 16 * rows].view(torch.int32)
            longs = buffer[16 * rows: 40 * rows].view(torch.int64).view(3, rows)
            lens = buffer[40 * rows: 44 * rows].view(torch.int32)
            return floats, ints, longs, lens

        floats, ints, longs, lens = views(host)
        floats.copy_(torch.tensor([[r.options.temperature for r in requests], [r.options.top_p for r in requests],
                                   [r.options.repetition_penalty for r in requests]], dtype=torch.float32))
        ints.copy_(torch.tensor([min(r.options.top_k, self.vocab) for r in requests], dtype=torch.int32))
        longs.copy_(torch.tensor([[r.seed for r in requests], [r.draws for r in requests],
                                  [r.history_device.data_ptr() if r.history_device is not None else 0 for r in requests]],
                                 dtype=torch.int64))
        lens.copy_(torch.tensor([r.history_sent if r.history_device is not None else 0 for r in requests], dtype=torch.int32))
        device.copy_(host[: 48 * rows], non_blocking=True)
        event.record()
        floats, ints, longs, lens = views(device)
        return floats[0], ints, floats[1], floats[2], longs[0], longs[1], longs[2], lens

    @staticmethod
    def record(requests: Sequence[RequestSampling], tokens: Sequence[int]) -> None:
        for r, t in zip(requests, tokens):
            if r.history is not None:
                r.history.append(int(t))
