"""The generation loop above the step function: batches of unequal prompts, stop tokens, sequences
that end earlier, and as many batches one after another as there are requests.

Per request it follows integrallis/models' loop (models-runtime/.../GenerationLoop.java:250-279):
sample from the last logits; an end-of-generation token ends the request and is neither emitted
nor counted (:263-265); otherwise the token is emitted; when it was the last one allowed, the
request ends without running the model again (:273-275); else the token goes through the model.
An empty prompt is refused (:148-151).  Usage counts prompt and emitted tokens (:198-199).

The reference serves one request at a time; batching is this library's own: requests that fit
start together in one prefill step and decode together, a finished request gives its slot back at
once, and no request joins a batch that has started.  The loop only decides; it talks to the model
through a small `Stepper`, so its decisions can be tested with a scripted one.

Prompt-prefix reuse between requests (models-runtime/.../GenerationLoop.java:217-248), when asked
for: a request that comes alone keeps its sequence in the cache when it ends; if the next request
that comes alone begins with tokens that sequence holds, the sequence is cut back to the shared
prefix (at most the prompt less one token, so that a step always runs) and only the rest of the
prompt goes through the model.  Anything else that runs in between gives the kept sequence back first.

Continuous batching, when asked for: a request that waits takes the place of one that has ended
while the others of the batch still run.  Its prompt runs as a step of its own between two of their
decode steps, and from then on it decodes with them; requests are admitted in their order, none
overtakes another, and never more than fit the cache at their longest.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional, Protocol, Sequence

from ..sampling.options import SamplingOptions
from ..sampling.sampler import RequestSampling


@dataclass(frozen=True)
class GenerationUsage:
    """Exact token counts of one request (models-api/.../GenerationUsage.java:19-34)."""

    prompt_tokens: int
    completion_tokens: int


@dataclass(frozen=True)
class PromptCacheMetrics:
    """What the last request took from the sequence kept before it, in tokens
    (models-runtime/.../PromptCacheMetrics.java:19-38): `supported` is whether reuse was possible for
    that request at all; without it no activity is reported."""

    supported: bool
    input_tokens: int
    cache_read_input_tokens: int  # found in the kept sequence
    cache_write_input_tokens: int  # run through the model

    def __post_init__(self):
        read, written = self.cache_read_input_tokens, self.cache_write_input_tokens
        if self.input_tokens < 0 or read < 0 or written < 0 or read + written > self.input_tokens:
            raise ValueError("cache token counts must be non-negative and not exceed input_tokens")
        if not self.supported and (read or written):
            raise ValueError("an unsupported prompt cache cannot report cache activity")

    @property
    def hit_rate(self) -> float:
        return self.cache_read_input_tokens / self.input_tokens if self.input_tokens else 0.0


@dataclass
class GenerationResult:
    tokens: List[int]
    usage: GenerationUsage
    finish_reason: str  # "stop": an end-of-generation token was sampled; "length": max_tokens or the context ran out


class Stepper(Protocol):
    """What the loop needs of a model."""

    page_size: int
    capacity_tokens: int  # positions the cache holds, in whole pages
    max_positions: int  # longest sequence

    def open_slot(self) -> int: ...

    def release_slot(self, slot: int) -> None: ...

    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]): ...

    def decode(self, slots: Sequence[int], tokens: Sequence[int]): ...

    def sample(self, logits, requests: Sequence[RequestSampling]) -> List[int]: ...

    def check_options(self, options: SamplingOptions) -> None: ...


@dataclass
class _Live:
    index: int
    prompt: List[int]
    sampling: RequestSampling
    limit: int  # most tokens this request may emit
    slot: int = -1
    tokens: List[int] = field(default_factory=list)
    last: int = -1
    start: int = 0  # tokens of the prompt that the slot already holds
    keep: bool = False  # the sequence stays in the cache when the request ends
    pages: int = 0  # cache pages the request needs at its longest


class GenerationLoop:
    def __init__(self, stepper: Stepper, max_batch: int, stop_token_ids: Iterable[int] = (), reuse_prefix: bool = False,
                 continuous: bool = False):
        if max_batch <= 0:
            raise ValueError(f"max_batch must be positive, got {max_batch}")
        self.stepper = stepper
        self.max_batch = max_batch
        self.stop_token_ids = frozenset(int(t) for t in stop_token_ids)
        # a sequence can only be cut back by a stepper that says how
        self.reuse_prefix = bool(reuse_prefix) and hasattr(stepper, "rewind")
        # rows of logits from two steps have to be put together, which only the stepper can do
        self.continuous = bool(continuous) and hasattr(stepper, "concat")
        self._kept: Optional[tuple] = None  # (slot, the tokens it holds) of the last request that came alone
        self.last_prompt_cache = PromptCacheMetrics(False, 0, 0, 0)

    # ------------------------------------------------------------------ the kept sequence

    def drop_kept(self) -> None:
        """Gives the kept sequence's slot back (the next request starts from nothing)."""
        if self._kept is not None:
            slot = self._kept[0]
            self._kept = None
            self.stepper.release_slot(slot)

    @staticmethod
    def shared_prefix(held: Sequence[int], prompt: Sequence[int]) -> int:
        """Tokens of `prompt` that a sequence holding `held` need not run again: the common prefix, but
        at most the prompt less one token (models-runtime/.../GenerationLoop.java:240-248)."""
        shared = 0
        limit = min(len(held), len(prompt))
        while shared < limit and held[shared] == prompt[shared]:
            shared += 1
        return min(shared, len(prompt) - 1)

    def _resume(self, request: _Live) -> None:
        """Lets a request that comes alone go on from the kept sequence where their tokens agree."""
        request.keep = True
        reused = 0
        if self._kept is not None:
            slot, held = self._kept
            shared = self.shared_prefix(held, request.prompt)
            if shared > 0:
                try:
                    self.stepper.rewind(slot, shared)
                    self._kept = None
                    request.slot, request.start, reused = slot, shared, shared
                except Exception:  # a window that has let go of what the shorter sequence needs, a model with state
                    pass
            self.drop_kept()
        self.last_prompt_cache = PromptCacheMetrics(True, len(request.prompt), reused, len(request.prompt) - reused)

    # ------------------------------------------------------------------ planning

    def _pages(self, tokens: int) -> int:
        page = self.stepper.page_size
        return -(-tokens // page)

    def plan_batches(self, prompts: Sequence[Sequence[int]], limits: Sequence[int]) -> List[List[int]]:
        """Request indices batch by batch, in order: a batch takes requests while there are at most
        max_batch of them and the cache can hold every one of them at its longest."""
        budget = self.stepper.capacity_tokens // self.stepper.page_size
        batches: List[List[int]] = []
        current: List[int] = []
        used = 0
        for i, (prompt, limit) in enumerate(zip(prompts, limits)):
            need = self._pages(len(prompt) + limit - 1)
            if need > budget:
                raise ValueError(
                    f"request {i}: {len(prompt)} prompt tokens plus {limit} generated need {need} cache pages, "
                    f"the cache has {budget}")
            if current and (len(current) == self.max_batch or used + need > budget):
                batches.append(current)
                current, used = [], 0
            current.append(i)
            used += need
        if current:
            batches.append(current)
        return batches

    # ------------------------------------------------------------------ running

    def run(self, prompts: Sequence[Sequence[int]], options: Sequence[SamplingOptions] | SamplingOptions,
            on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        """Generates for every prompt; results keep the order of the prompts.
        `on_token(request index, token)` is called for each emitted token, in order per request."""
        if isinstance(options, SamplingOptions):
            options = [options] * len(prompts)
        if len(options) != len(prompts):
            raise ValueError(f"{len(prompts)} prompts but {len(options)} sampling options")
        prompts = [[int(t) for t in p] for p in prompts]
        limits = []
        for i, (p, o) in enumerate(zip(prompts, options)):
            if len(p) == 0:
                raise ValueError("prompt must not be empty" if len(prompts) == 1 else f"prompt {i} must not be empty")
            if len(p) > self.stepper.max_positions:
                raise ValueError(f"prompt {i} has {len(p)} tokens, the context holds {self.stepper.max_positions}")
            self.stepper.check_options(o)
            # the last emitted token is never fed back, so a sequence needs prompt + limit - 1 positions
            limits.append(min(o.max_tokens, self.stepper.max_positions - len(p) + 1))
        results: List[Optional[GenerationResult]] = [None] * len(prompts)
        batches = self.plan_batches(prompts, limits)
        alone = self.reuse_prefix and len(prompts) == 1
        if not alone:
            self.drop_kept()
            self.last_prompt_cache = PromptCacheMetrics(False, sum(len(p) for p in prompts), 0, 0)
        if self.continuous and len(batches) > 1:
            waiting = [_Live(i, prompts[i], RequestSampling(options[i], prompts[i]), limits[i],
                             pages=self._pages(len(prompts[i]) + limits[i] - 1)) for i in range(len(prompts))]
            while waiting:  # (one pass: whoever waits is admitted as soon as the running ones leave room)
                self._run_batch(self._admit(waiting, []), results, on_token, waiting)
            return results  # type: ignore[return-value]
        for batch in batches:
            live = [_Live(i, prompts[i], RequestSampling(options[i], prompts[i]), limits[i]) for i in batch]
            if alone:
                self._resume(live[0])
            self._run_batch(live, results, on_token)
        return results  # type: ignore[return-value]

    def _admit(self, waiting: List[_Live], running: Sequence[_Live]) -> List[_Live]:
        """Takes from the head of the queue the requests that fit beside the running ones: at most max_batch
        together, and no more pages than the cache has when every one of them is at its longest.  In order: a
        request that does not fit yet holds back those behind it."""
        budget = self.stepper.capacity_tokens // self.stepper.page_size
        used = sum(r.pages for r in running)
        admitted: List[_Live] = []
        while waiting and len(running) + len(admitted) < self.max_batch and used + waiting[0].pages <= budget:
            used += waiting[0].pages
            admitted.append(waiting.pop(0))
        return admitted

    def _finish(self, request: _Live, reason: str, results) -> None:
        if request.keep:
            # what went through the model: the prompt and every emitted token that another one followed; after a stop
            # token all of them (the stop token was sampled from the last one's logits)
            fed = request.tokens if reason == "stop" else request.tokens[:-1]
            self._kept = (request.slot, request.prompt + fed)
        else:
            self.stepper.release_slot(request.slot)
        request.slot = -1
        results[request.index] = GenerationResult(
            request.tokens, GenerationUsage(len(request.prompt), len(request.tokens)), reason)

    def _take(self, r: _Live, token: int, results, on_token) -> bool:
        """What the reference's loop does with one sampled token; True if the request goes on."""
        stops = self.stop_token_ids | set(r.sampling.options.stop_token_ids)
        if token in stops:
            self._finish(r, "stop", results)
            return False
        r.tokens.append(token)
        if r.sampling.history is not None:
            r.sampling.history.append(token)
        if on_token is not None:
            on_token(r.index, token)
        if len(r.tokens) >= r.limit:
            self._finish(r, "length", results)
            return False
        r.last = token
        return True

    def _run_batch_pipelined(self, live: List[_Live], results, on_token, waiting: Optional[List[_Live]] = None) -> None:
        """The same decisions, one step ahead of the ids: the next decode step is queued for every
        request that has room for another token before the last ids have reached the host, with
        the ids taken on the device.  A request whose pending token turns out to be a stop token
        has then been stepped once more than needed; that step's row is dropped, nothing of it is
        emitted, and the slot goes back as always.  The rows of such a step are sampled with the
        others (their ids are never read).  Tokens, order and counts are those of the unpipelined loop.
        `waiting`: requests that join as others end (continuous batching)."""
        stepper = self.stepper
        rows: List[Optional[_Live]] = list(live)  # aligned with the rows of `pending`; None: finished
        live = list(live)  # everyone who may hold a slot, for the failure path
        try:
            for r in live:
                if r.slot < 0:
                    r.slot = stepper.open_slot()
            logits = stepper.prefill([r.slot for r in live], [r.prompt[r.start:] for r in live])
            pending = stepper.sample_start(logits, [r.sampling for r in live])
            samplings = [r.sampling for r in live]
            while any(r is not None for r in rows):
                ahead = [i for i, r in enumerate(rows) if r is not None and len(r.tokens) + 1 < r.limit]
                next_logits = None
                if ahead:
                    next_logits = stepper.decode_pending([rows[i].slot for i in ahead], pending, ahead)
                tokens = pending.result()
                for i, r in enumerate(rows):
                    if r is not None and not self._take(r, int(tokens[i]), results, on_token):
                        rows[i] = None
                samplings = [samplings[i] for i in ahead]
                rows = [rows[i] for i in ahead]
                joiners = self._admit(waiting, [r for r in rows if r is not None]) if waiting else []
                if joiners:
                    # their prompts run as a step of its own, behind the step that is already queued for the others
                    live.extend(joiners)
                    for r in joiners:
                        r.slot = stepper.open_slot()
                    joined = stepper.prefill([r.slot for r in joiners], [r.prompt for r in joiners])
                    next_logits = joined if next_logits is None else stepper.concat(next_logits, joined)
                    rows.extend(joiners)
                    samplings.extend(r.sampling for r in joiners)
                if any(r is not None for r in rows):
                    pending = stepper.sample_start(next_logits, samplings)
        except BaseException:
            for r in live:
                if r.slot >= 0:
                    try:
                        stepper.release_slot(r.slot)
                    except Exception:
                        pass
                    r.slot = -1
            raise

    def _run_batch(self, live: List[_Live], results, on_token, waiting: Optional[List[_Live]] = None) -> None:
        stepper = self.stepper
        if hasattr(stepper, "decode_pending") and hasattr(stepper, "sample_start"):
            return self._run_batch_pipelined(live, results, on_token, waiting)
        started = list(live)  # everyone who may hold a slot, for the failure path
        try:
            for r in live:
                if r.slot < 0:
                    r.slot = stepper.open_slot()
            logits = stepper.prefill([r.slot for r in live], [r.prompt[r.start:] for r in live])
            while live:
                sampled = stepper.sample(logits, [r.sampling for r in live])
                live = [r for r, token in zip(live, sampled) if self._take(r, int(token), results, on_token)]
                joiners = self._admit(waiting, live) if waiting else []
                if live:
                    logits = stepper.decode([r.slot for r in live], [r.last for r in live])
                if joiners:
                    started.extend(joiners)
                    for r in joiners:
                        r.slot = stepper.open_slot()
                    joined = stepper.prefill([r.slot for r in joiners], [r.prompt for r in joiners])
                    logits = stepper.concat(logits, joined) if live else joined
                    live = live + joiners
        except BaseException:
            for r in started:
                if r.slot >= 0:
                    try:
                        stepper.release_slot(r.slot)
                    except Exception:
                        pass
                    r.slot = -1
            raise
