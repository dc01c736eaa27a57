"""The engine: a model on one GPU, its cache, and the one step function everything drives.

`step(entries)` runs exactly the tokens it is given, as one batch, on top of what earlier steps
left in the cache, and returns the logits at the wanted places.  The requests of a step either all
start (their prompts, of unequal lengths, in one step) or all go on by one token; nothing in the
code needs that distinction -- a step may also bring several tokens to a sequence that already
holds some -- it only decides which attention kernel is the fast one.

integrallis/models has the pieces separately: whole-prompt prefill of one sequence
(backend-java/.../llama/LlamaForwardPass.java:351-370), one token for each of several sessions
(:471-481,709-723), logits for chosen rows only (Head.LOGITS/NONE, :984-991), and checks before any
state changes (:933-960, :1008-1014).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence

import torch

from ..cache import KvCache, StateArea
from ..cache.kv_cache import PAGE_SIZE
from ..config.specs import ModelSpec
from ..parts import RunContext, Runtime
from .batch import build_step_batch
from .model import DecoderModel


class StepError(ValueError):
    """A step that was refused; nothing changed."""


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError(
            "models_b200 runs its own CUDA kernels and has no CPU path: a CUDA device is required "
            f"(asked for {device}, torch.cuda.is_available() is {torch.cuda.is_available()})")
    return device


class Engine:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], dtype: str = "bfloat16",
                 max_tokens: int = 4096, max_slots: Optional[int] = None, device="cuda:0",
                 max_sequence: Optional[int] = None, max_step_tokens: Optional[int] = None,
                 page_size: int = PAGE_SIZE):
        """`max_tokens`: the most positions live sequences hold at any time, each rounded up to whole
        pages.  `max_sequence`: a cap on one sequence's positions below the model's.  `max_step_tokens`:
        the most tokens a step may bring to one sequence (None: no limit); stating it lets cache groups
        that keep only a window of positions be made with the pages a window needs instead of
        `max_tokens`.  `page_size`: positions per cache page; the tensor-core attention kernels tile the
        cache in pages of 64, so the bfloat16 mode takes no other size."""
        self.device = require_cuda(device)
        torch.cuda.set_device(self.device)
        self.spec = spec
        if dtype == "bfloat16" and page_size != PAGE_SIZE:
            raise ValueError(f"the bfloat16 attention kernels read cache pages of {PAGE_SIZE} positions; page_size "
                             f"{page_size} runs in the float32 mode only")
        if max_step_tokens is not None and max_step_tokens <= 0:
            raise ValueError(f"max_step_tokens must be positive, got {max_step_tokens}")
        self.max_step_tokens = max_step_tokens
        page_tokens = -(-max_tokens // page_size) * page_size
        longest = min(spec.max_positions, page_tokens)
        if max_sequence is not None:
            longest = min(longest, max(1, max_sequence))
        self.runtime = Runtime(self.device, dtype, max_positions=longest)
        self.model = DecoderModel(spec, self.runtime)
        self.model.load(tensors)
        cache_from = [entry.cache_from for entry in spec.schedule]
        self.cache = KvCache(self.model.kv_requests(), cache_from, max_tokens, max_slots, page_size, max_step_tokens)
        dtype_t = self.runtime.compute_dtype
        self.cache_elements = self.cache.allocate_storage(
            lambda shape: torch.zeros(shape, dtype=dtype_t, device=self.device))
        self.state = StateArea(
            self.model.state_requests(), self.cache.max_slots,
            lambda shape, dt: torch.zeros(shape, dtype=dt, device=self.device))
        self.runs: List[RunContext] = []
        for run, entry in enumerate(spec.schedule):
            ctx = RunContext(run=run, writes_cache=entry.cache_from is None, state=self.state.of_run(run))
            if run in self.cache.run_location:
                ctx.group, ctx.k_pool, ctx.v_pool = self.cache.pools(run)
            self.runs.append(ctx)
        self.steps = 0
        self.decode_graphs = None
        self.prompt_graphs = None
        self.last_argmax = None
        self._last_logits = None

    def enable_decode_graphs(self, max_batch: int, max_sequence: Optional[int] = None) -> None:
        """Captures decode steps of up to `max_batch` sequences of up to `max_sequence` positions
        as CUDA graphs (lazily, one per batch size of a ladder)."""
        from .decode_graph import DecodeGraphs, PromptGraphs

        longest = min(max_sequence or self.runtime.max_positions, self.runtime.max_positions)
        self.decode_graphs = DecodeGraphs(self, max_batch, -(-longest // self.cache.page_size))
        # short prompt steps too, unless a part keeps state of its own per sequence: such a part may
        # walk the sequences on the host, which a capture would freeze
        self.prompt_graphs = None if self.state.tensors else PromptGraphs(self.decode_graphs)

    # ------------------------------------------------------------------ slots

    def open_slot(self) -> int:
        slot = self.cache.open_slot()
        self.state.reset(slot)
        return slot

    def release_slot(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def rewind(self, slot: int, length: int) -> None:
        if self.state.tensors:
            raise StepError("a model with per-sequence state cannot rewind: state is not a length that can be cut")
        self.cache.rewind(slot, length)

    # ------------------------------------------------------------------ the step

    def validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        vocab = self.spec.vocab_size
        limit = self.runtime.max_positions
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if e.slot not in self.cache.lengths:
                raise StepError(f"slot {e.slot} is not open")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"slot {e.slot}: a step must bring at least one token")
            if self.max_step_tokens is not None and n > self.max_step_tokens:
                raise StepError(f"slot {e.slot}: {n} tokens in one step exceed the engine's max_step_tokens of "
                                f"{self.max_step_tokens}; bring them in several steps")
            for t in e.tokens:
                if not 0 <= int(t) < vocab:
                    raise StepError(f"slot {e.slot}: token id {t} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside the {n} tokens of this step")
            if self.cache.lengths[e.slot] + n > limit:
                raise StepError(
                    f"slot {e.slot}: {self.cache.lengths[e.slot]} + {n} positions exceed the limit of {limit} "
                    "(the model's max positions, or the size the cache was made for)")

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Appends each entry's tokens to its slot and returns float32 logits [wanted, vocab] in the
        order of the entries and of their `want` lists (None if nothing is wanted).  A refused step
        (StepError, CacheFull) leaves every slot as it was.  With graphs enabled a step of one token
        per sequence that wants each token's logits is the captured decode step (the result is a copy)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self.validate(entries)
        if self._fits_decode_graphs(entries) and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return self._decode_from_graph(entries).clone()
        return self._step(entries)

    def _step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        appends = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.append(appends)
        packed = [(e.slot, e.tokens, e.want) for e in entries]
        logits = self.prompt_graphs.step(packed) if self.prompt_graphs is not None else None
        if logits is None:
            batch = build_step_batch(self.cache, packed, self.device, state_pad_row=self.cache.max_slots)
            logits = self.model.forward(batch, self.runs)
        self.cache.commit(appends)
        self.steps += 1
        self.last_argmax = None
        return logits

    def _fits_decode_graphs(self, entries: Sequence[StepEntry]) -> bool:
        """Whether the captured decode steps take this batch: graphs enabled, no more sequences than the
        largest capture, no sequence longer than the captures' page tables."""
        graphs = self.decode_graphs
        if graphs is None or len(entries) > graphs.max_batch:
            return False
        page = self.cache.page_size
        return all(-(-(self.cache.lengths[e.slot] + 1) // page) <= graphs.blocks for e in entries)

    def _decode_from_graph(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        graphs = self.decode_graphs
        appends = [(e.slot, 1) for e in entries]
        self.cache.append(appends)
        logits = graphs.step([(e.slot, e.tokens, e.want) for e in entries], device_tokens=device_tokens)
        self.last_argmax = graphs.last_argmax  # the graph holds the greedy choice too
        self._last_logits = logits
        self.cache.commit(appends)
        self.steps += 1
        return logits

    def decode(self, slots: Sequence[int], tokens: Sequence[int]) -> torch.Tensor:
        """One more token for each slot; logits [len(slots), vocab] for these tokens.  The same as
        `step` with single-token entries that each want place 0, replayed from a CUDA graph when
        graphs are enabled and the batch fits them; the result is then the graph's own buffer, which
        the next decode overwrites."""
        entries = [StepEntry(s, [int(t)], [0]) for s, t in zip(slots, tokens)]
        self.validate(entries)
        if not self._fits_decode_graphs(entries):
            return self._step(entries)
        return self._decode_from_graph(entries)

    def decode_device_tokens(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """`decode` with the token ids still on the device (int32 [len(slots)], what a sampler just
        wrote): the step is queued without waiting for them, so the host can prepare it while the
        step before it runs.  Without decode graphs (or beyond their sizes) the ids are fetched and
        the step runs as `decode` does."""
        entries = [StepEntry(s, [0], [0]) for s in slots]  # ids come from the device; a sampler's ids are in range
        self.validate(entries)
        if not self._fits_decode_graphs(entries):
            return self.decode(slots, tokens.tolist())
        return self._decode_from_graph(entries, device_tokens=tokens)

    def greedy_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        """First maximum of every row of `logits` (device, int32): taken from the decode graph when
        `logits` is what the last `decode` returned, else computed."""
        from ..kernels import ops

        if self.last_argmax is not None and logits is self._last_logits:
            return self.last_argmax
        return ops.argmax_rows(logits)

    # ------------------------------------------------------------------ facts

    def diagnostics(self) -> Dict[str, object]:
        props = torch.cuda.get_device_properties(self.device)
        element = 2 if self.runtime.mode == "bfloat16" else 4
        from ..kernels.build import loaded_libraries

        return {
            "device": props.name,
            "multiprocessors": props.multi_processor_count,
            "dtype": self.runtime.mode,
            "architecture": self.spec.architecture,
            "cache_groups": len(self.cache.groups),
            "cache_pages": [group.num_pages for group in self.cache.groups],
            "page_size": self.cache.page_size,
            "cache_bytes": self.cache_elements * element,
            "state_bytes": self.state.bytes,
            "max_positions": self.runtime.max_positions,
            "kernel_libraries": loaded_libraries(),
        }
