"""Decode steps as CUDA graphs: one token per live sequence, the whole model in one launch.

A decode step at small batch is a few hundred short kernels, so launching them costs more than
running them.  For each batch size out of a short ladder the step is captured once over fixed
device buffers; a step then copies its indices (tokens, positions, page tables) into those
buffers and replays.  A batch smaller than its rung is padded with sequences of one token that
point at the cache's spare page and store nothing, so padding changes no result.
"""

from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

from ..kernels import ops
from .batch import StepLayout, batch_from_buffer, pack_step


def ladder(max_batch: int) -> List[int]:
    sizes, b = [], 1
    while b < max_batch:
        sizes.append(b)
        b *= 2
    sizes.append(max_batch)
    return sizes


class _Captured:
    def __init__(self, engine, size: int, blocks: int, pool):
        self.size = size
        cache = engine.cache
        self.layout = StepLayout(size, size, size, blocks, len(cache.groups))
        self.host = torch.zeros(self.layout.total, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.layout.total, dtype=torch.int32, device=engine.device)
        # a first layout that is valid to run: every row is padding
        pack_step(cache, [], self.layout, self.host_np, cache.max_slots)
        self.dev.copy_(self.host)
        self.batch = batch_from_buffer(self.dev, self.layout, [1] * size, 1, [])
        stream = torch.cuda.Stream(device=engine.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up outside the capture: libraries load, attributes are set
                engine.model.forward(self.batch, engine.runs)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(engine.device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(self.graph, pool=pool, stream=stream):
            self.logits = engine.model.forward(self.batch, engine.runs)
        self.kernels = ops.launch_count() - before  # this package's kernels inside one replay
        ops.add_launches(-self.kernels)  # a capture launches nothing


class DecodeGraphs:
    def __init__(self, engine, max_batch: int, blocks: int):
        self.engine = engine
        self.max_batch = max_batch
        self.blocks = blocks
        self.sizes = ladder(max_batch)
        self.captured: Dict[int, _Captured] = {}
        self.pool = torch.cuda.graph_pool_handle()

    def rung(self, n: int) -> int:
        for size in self.sizes:
            if size >= n:
                return size
        raise ValueError(f"a decode batch of {n} exceeds the largest captured size {self.max_batch}")

    def step(self, entries: Sequence) -> torch.Tensor:
        """entries: (slot, [token], [0]) each; the cache already has room.  Returns logits
        [len(entries), vocab]; they live in the graph's output buffer until the next replay."""
        engine = self.engine
        size = self.rung(len(entries))
        captured = self.captured.get(size)
        if captured is None:
            captured = self.captured[size] = _Captured(engine, size, self.blocks, self.pool)
        pack_step(engine.cache, entries, captured.layout, captured.host_np, engine.cache.max_slots)
        captured.dev.copy_(captured.host, non_blocking=True)
        captured.graph.replay()
        ops.add_launches(captured.kernels)
        return captured.logits[: len(entries)]
