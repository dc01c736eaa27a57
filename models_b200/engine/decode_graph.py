"""Steps as CUDA graphs: the whole model in one launch.

A decode step at small batch is a few hundred short kernels, so launching them costs more than
running them.  For each batch size out of a short ladder the step is captured once over fixed
device buffers; a step then copies its indices (tokens, positions, page tables) into those
buffers and replays.  A batch smaller than its rung is padded with sequences of one token that
point at the cache's spare page and store nothing, so padding changes no result.

Prompts are in the same position: a step of a few hundred tokens runs for a fraction of a
millisecond and takes two to launch (a thousand tokens: 2.3 ms of kernels, 1.9 ms of launching).  Steps of up to PROMPT_TOKENS[-1] tokens are captured by
(batch size, token count) class, the token count rounded up to one of PROMPT_TOKENS; sequences
that are missing are empty, and the rows left over belong to no sequence.
"""

from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .batch import StepLayout, batch_from_buffer, pack_step


def ladder(max_batch: int) -> List[int]:
    """Powers of two up to max_batch (and max_batch itself): the batch sizes that are captured."""
    sizes, b = [], 1
    while b < max_batch:
        sizes.append(b)
        b *= 2
    sizes.append(max_batch)
    return sizes


class DecodeRows:
    """The indices of a captured decode step on the host, kept up to date in place from one step to the
    next (host arithmetic only: it runs without a GPU).  `buffer` is the step's int32 buffer in the
    order of `layout`; it must hold a valid all-padding step when this is made."""

    def __init__(self, layout: StepLayout, buffer: np.ndarray):
        off = [int(o) for o in layout.offsets]
        size, blocks, n = layout.sequences, layout.blocks, buffer
        self.tokens_h, self.positions_h = n[off[0]:off[1]], n[off[1]:off[2]]
        self.kv_lens_h, self.slots_h = n[off[3]:off[4]], n[off[4]:off[5]]
        self.tables_h = [n[off[6 + 2 * g]:off[7 + 2 * g]].reshape(size, blocks) for g in range(layout.groups)]
        self.mappings_h = [n[off[7 + 2 * g]:off[8 + 2 * g]] for g in range(layout.groups)]
        self.row_stamps = [0] * size  # the cache's table stamp of what each row of the page tables holds (0: nothing)
        self.live = 0

    def update(self, cache, slots: Sequence[int], tokens: Optional[Sequence[int]]) -> None:
        """The indices of one decode step, written in place: one token per slot, appended at each
        slot's length.  A row of the page tables is rewritten only when the cache's stamp of the slot's
        tables differs from the one the row was written with (another sequence, a new page, a rewind).
        `tokens` None: the token ids are already on the device."""
        live, page = len(slots), cache.page_size
        pad_row = cache.max_slots
        lengths = [cache.lengths[s] for s in slots]
        if tokens is not None:
            self.tokens_h[:live] = tokens
        self.positions_h[:live] = lengths
        self.kv_lens_h[:live] = lengths
        self.kv_lens_h[:live] += 1
        self.slots_h[:live] = slots
        if live < self.live:  # rows that fell out of the batch become padding
            self.tokens_h[live:self.live] = 0
            self.positions_h[live:self.live] = 0
            self.kv_lens_h[live:self.live] = 1
            self.slots_h[live:self.live] = pad_row
            for g in range(len(self.tables_h)):
                self.tables_h[g][live:self.live] = 0
                self.mappings_h[g][live:self.live] = -1
            for b in range(live, self.live):
                self.row_stamps[b] = 0
        self.live = live
        for b, slot in enumerate(slots):
            length = lengths[b]
            block, offset = length // page, length % page
            # a slot id is handed out again and so are pages, in any order: only the stamp says whether
            # the row still holds this sequence's tables as they are now
            stamp = cache.table_stamps[slot]
            refresh = self.row_stamps[b] != stamp
            self.row_stamps[b] = stamp
            for g, group in enumerate(cache.groups):
                table = group.tables[slot]
                self.mappings_h[g][b] = table[block] * page + offset
                if refresh:  # pages a window group gave back are never read: their stale ids may stay
                    row = self.tables_h[g][b]
                    row[:len(table)] = [p if p >= 0 else 0 for p in table]
                    row[len(table):] = 0


class _Captured:
    """One captured step: `size` sequences of one token each, or with `tokens` a step of so many
    rows shared by up to `size` sequences in any way."""

    def __init__(self, engine, size: int, blocks: int, pool, span: int = 0, tokens: Optional[int] = None):
        self.size = size
        self.span = span  # the class of context lengths the capture is for (ops.decode_span)
        cache = engine.cache
        prompts = tokens is not None
        self.layout = StepLayout(size, tokens if prompts else size, size, blocks, len(cache.groups))
        self.host = torch.zeros(self.layout.total, dtype=torch.int32)  # the step's indices, kept up to date in place
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.layout.total, dtype=torch.int32, device=engine.device)
        # a first layout that is valid to run: every row is padding
        pack_step(cache, [], self.layout, self.host_np, cache.max_slots, empty_padding=prompts)
        offsets = [int(o) for o in self.layout.offsets]
        if not prompts:
            self.host_np[offsets[5]:offsets[6]] = np.arange(size, dtype=np.int32)  # every row's logits, row by row
        self.dev.copy_(self.host)
        # the sizes kernels are launched with: one token each, or as if one sequence held every row
        q_lens = [tokens] + [0] * (size - 1) if prompts else [1] * size
        self.batch = batch_from_buffer(self.dev, self.layout, q_lens, max(1, span), [])
        stream = torch.cuda.Stream(device=engine.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up outside the capture: libraries load, attributes are set
                ops.argmax_rows(engine.model.forward(self.batch, engine.runs))
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(engine.device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        # No garbage collection inside the capture: a finaliser that frees device or pinned memory (an
        # older model's, say) is a call that a capture forbids, and it would invalidate this one.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, pool=pool, stream=stream), ops.recording() as names:
                self.logits = engine.model.forward(self.batch, engine.runs)
                self.argmax = ops.argmax_rows(self.logits)  # greedy choice of every row, for callers that want only that
            self.kernel_names = names  # which launcher ran each kernel of the step, in order
        finally:
            if collecting:
                gc.enable()
        self.kernels = ops.launch_count() - before  # this package's kernels inside one replay
        ops.add_launches(-self.kernels)  # a capture launches nothing
        self.rows = DecodeRows(self.layout, self.host_np)  # the quick per-step update of the indices
        self.staging = [(torch.zeros_like(self.host).pin_memory(), torch.cuda.Event()) for _ in range(4)]
        self.staging_next = 0

    def upload(self, skip_tokens: bool = False) -> None:
        """Copies the indices to the device through a small ring of pinned buffers: the copy is
        asynchronous, so the buffer it reads must not be rewritten before it has run.  With
        `skip_tokens` the token ids (the first part of the buffer) are left as they are on the device:
        the sampler has written them there."""
        staging, event = self.staging[self.staging_next]
        self.staging_next = (self.staging_next + 1) % len(self.staging)
        event.synchronize()  # returns at once unless the host is several steps ahead of the GPU
        staging.copy_(self.host)
        first = self.layout.tokens if skip_tokens else 0
        self.dev[first:].copy_(staging[first:], non_blocking=True)
        event.record()

    def fill(self, cache, entries) -> int:
        """The indices of a step of any shape that fits (prompts of unequal lengths), packed anew;
        returns how many rows of logits the step wants."""
        pack_step(cache, entries, self.layout, self.host_np, cache.max_slots, empty_padding=True)
        return sum(len(want) for _, _, want in entries)

    def update(self, cache, slots: Sequence[int], tokens: Optional[Sequence[int]]) -> None:
        self.rows.update(cache, slots, tokens)


class DecodeGraphs:
    def __init__(self, engine, max_batch: int, blocks: int):
        self.engine = engine
        self.max_batch = max_batch
        self.blocks = blocks
        self.sizes = ladder(max_batch)
        self.captured: Dict[tuple, _Captured] = {}  # (batch size, launch class: page-table width and the mixers' classes)
        self.last_argmax = None  # first maximum of every row of the last step's logits (device, int32)
        self.pool = torch.cuda.graph_pool_handle()

    def rung(self, n: int) -> int:
        for size in self.sizes:
            if size >= n:
                return size
        raise ValueError(f"a decode batch of {n} exceeds the largest captured size {self.max_batch}")

    def table_width(self, max_kv_len: int) -> int:
        """Pages per sequence in the page tables of the capture for this length: the next of 4, 8, 16, ...
        that holds it, at most the engine's longest sequence.  The width is part of the captured launches
        (the kernels stride the tables by it) and of what every step copies to the device, so short
        sequences do not carry the longest one's tables."""
        need = -(-max_kv_len // self.engine.cache.page_size)
        width = 4
        while width < need:
            width *= 2
        return min(width, self.blocks)

    def launch_class(self, size: int, max_kv_len: int) -> tuple:
        """What the launches of a decode step of `size` sequences depend on besides the batch size: the
        width of the page tables, and every mixer's answer for the class of context lengths (long
        contexts split their keys over more blocks, and the split is part of the captured launches).
        Most steps share one class."""
        span = ops.decode_span(max_kv_len)
        mixers = [block.mixer for block in self.engine.model.blocks]
        return (self.table_width(max_kv_len),) + tuple(
            m.decode_class(size, span) if hasattr(m, "decode_class") else 0 for m in mixers)

    def prepare(self, size: int, max_kv_len: int) -> _Captured:
        """The capture for `size` sequences (a rung) of up to `max_kv_len` positions, made if it is not
        there yet: a capture costs tens of steps, so a caller that knows what is coming can have it made
        before it counts."""
        key = (size, self.launch_class(size, max_kv_len))
        captured = self.captured.get(key)
        if captured is None:
            captured = self.captured[key] = _Captured(self.engine, size, key[1][0], self.pool, ops.decode_span(max_kv_len))
        return captured

    def step(self, entries: Sequence, device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """entries: (slot, [token], [0]) each; the cache already has room.  Returns logits
        [len(entries), vocab]; they live in the graph's output buffer until the next replay.
        `device_tokens` (int32 [len(entries)], on the device) replaces the entries' token ids: the
        step then needs nothing from the host that depends on the step before it."""
        engine = self.engine
        size = self.rung(len(entries))
        captured = self.prepare(size, 1 + max((engine.cache.lengths[e[0]] for e in entries), default=0))
        if device_tokens is None:
            captured.update(engine.cache, [e[0] for e in entries], [e[1][0] for e in entries])
            captured.upload()
        else:
            captured.update(engine.cache, [e[0] for e in entries], None)
            captured.upload(skip_tokens=True)
            captured.batch.tokens[: len(entries)].copy_(device_tokens)
        captured.graph.replay()
        ops.add_launches(captured.kernels)
        self.last_argmax = captured.argmax[: len(entries)]
        return captured.logits[: len(entries)]


# Token counts at which prompt steps are captured.  Rows added to reach the next count are computed for nothing, so the
# counts lie closer together (in proportion) as they grow; past the last one the kernels of a step run longer than the
# host needs to launch them one by one.
PROMPT_TOKENS = (16, 32, 64, 128, 256, 384, 512, 640, 768, 896, 1024, 1280, 1536, 1792, 2048)
EAGER_USES = 2  # a class of steps is captured when it comes up for the third time: a capture costs tens of steps
MAX_PROMPT_CAPTURES = 64  # classes beyond so many run launch by launch: every capture keeps its graph and its outputs


class PromptGraphs:
    """Steps that bring several tokens to their sequences, replayed from captures by class."""

    def __init__(self, decode_graphs: DecodeGraphs):
        self.decode_graphs = decode_graphs
        self.engine = decode_graphs.engine
        self.captured: Dict[tuple, _Captured] = {}  # (batch size, token count, page-table width)
        self.uses: Dict[tuple, int] = {}

    def bucket(self, entries: Sequence) -> Optional[tuple]:
        """The class of the step, or None for one that runs launch by launch: too many tokens or
        sequences, more logits wanted than sequences (or none), a page table wider than the captures'."""
        graphs, cache = self.decode_graphs, self.engine.cache
        total = sum(len(tokens) for _, tokens, _ in entries)
        wanted = sum(len(want) for _, _, want in entries)
        if len(entries) > graphs.max_batch or total > PROMPT_TOKENS[-1] or wanted == 0:
            return None
        size = graphs.rung(len(entries))
        if wanted > size:
            return None
        longest = max(cache.lengths[slot] + len(tokens) for slot, tokens, _ in entries)
        if -(-longest // cache.page_size) > graphs.blocks:
            return None
        return size, next(t for t in PROMPT_TOKENS if t >= total), graphs.table_width(longest)

    def step(self, entries: Sequence) -> Optional[torch.Tensor]:
        """entries: (slot, tokens, wanted places); the cache already has room.  Returns the logits of
        the wanted places (a copy: the capture's buffer is rewritten by its next replay), or None
        when the step is not one for a capture -- the caller then runs it launch by launch."""
        key = self.bucket(entries)
        if key is None:
            return None
        captured = self.captured.get(key)
        if captured is None:
            self.uses[key] = self.uses.get(key, 0) + 1
            if self.uses[key] <= EAGER_USES or len(self.captured) >= MAX_PROMPT_CAPTURES:
                return None
            graphs = self.decode_graphs
            captured = self.captured[key] = _Captured(self.engine, key[0], key[2], graphs.pool, tokens=key[1])
        wanted = captured.fill(self.engine.cache, entries)
        captured.upload()
        captured.graph.replay()
        ops.add_launches(captured.kernels)
        return captured.logits[:wanted].clone()
