"""The Python entry point, in integrallis/models' manner: load a model, generate (blocking or
streamed through callbacks), and the lower-level pipeline calls.

Counterparts: `PureJavaBackend.load(path)` (backend-java/.../PureJavaBackend.java:128),
`TextGenerationModel.generate(prompt, options[, stream])` and `TokenStream`
(models-api/.../TextGenerationModel.java:31-112, models-api/.../TokenStream.java:27-48), and
`InferencePipeline`'s prefill / forward / resetContext / checkpoint / rewind / contextWindow /
metadata / diagnostics / close (models-runtime/.../InferencePipeline.java:43-220).  Prompts and
outputs are token ids: this library has no tokenizer.
"""

from __future__ import annotations

import queue
import threading
from dataclasses import dataclass
from typing import Callable, Dict, Iterator, List, Optional, Sequence

from .engine.generation import GenerationLoop, GenerationResult, GenerationUsage
from .sampling.options import SamplingOptions


class TokenStream:
    """Callbacks of a streamed generation.  They are called serially and in token order; exactly
    one of on_complete / on_error is called, last (models-api/.../TokenStream.java:21-25)."""

    def on_token(self, token: int) -> None:
        pass

    def on_complete(self, usage: GenerationUsage) -> None:
        pass

    def on_error(self, failure: BaseException) -> None:
        pass


class CallbackStream(TokenStream):
    def __init__(self, on_token=None, on_complete=None, on_error=None):
        self._token, self._complete, self._error = on_token, on_complete, on_error

    def on_token(self, token):
        if self._token:
            self._token(token)

    def on_complete(self, usage):
        if self._complete:
            self._complete(usage)

    def on_error(self, failure):
        if self._error:
            self._error(failure)


@dataclass(frozen=True)
class ModelMetadata:
    """models-api/.../ModelMetadata.java:26-49."""

    family: str
    name: str
    context_length: int
    vocab_size: int
    embedding_dim: int
    layers: int
    heads: int
    kv_heads: int


class _StreamAbandoned(Exception):
    """Raised inside the generation of a stream nobody reads any more."""


class TextGenerationModel:
    def __init__(self, engine, max_batch: int, name: str, cuda_graphs: bool = True, context: Optional[int] = None,
                 reuse_prefix: bool = False, continuous: bool = False):
        from .engine.stepper import EngineStepper

        self.engine = engine
        self.name = name
        self.max_batch = max_batch
        if cuda_graphs:
            engine.enable_decode_graphs(max_batch, context)
        self._stepper = EngineStepper(engine)
        self._loop = GenerationLoop(self._stepper, max_batch, engine.spec.stop_token_ids, reuse_prefix=reuse_prefix,
                                    continuous=continuous)
        self._lock = threading.Lock()  # one generation at a time, as the reference serialises on its backend
        self._session: Optional[int] = None
        self._closed = False

    # ------------------------------------------------------------------ facts

    def model_name(self) -> str:
        return self.name

    @property
    def metadata(self) -> ModelMetadata:
        spec = self.engine.spec
        mixer = spec.layers[0].mixer
        return ModelMetadata(
            family=spec.architecture, name=self.name, context_length=spec.max_positions, vocab_size=spec.vocab_size,
            embedding_dim=spec.hidden_size, layers=len(spec.schedule), heads=getattr(mixer, "num_heads", 0),
            kv_heads=getattr(mixer, "num_kv_heads", 0))

    @property
    def context_window(self) -> int:
        """Positions one sequence may hold here: the model's, or less if the cache is smaller."""
        return self.engine.runtime.max_positions

    def diagnostics(self) -> Dict[str, object]:
        out = self.engine.diagnostics()
        out["max_batch"] = self.max_batch
        out["cuda_graphs"] = self.engine.decode_graphs is not None
        return out

    # ------------------------------------------------------------------ generation

    def _require_open(self):
        if self._closed:
            raise RuntimeError("the model is closed")

    def generate(self, prompt: Sequence[int], options: Optional[SamplingOptions] = None,
                 stream: Optional[TokenStream] = None):
        """Blocking form: returns the generated token ids.  With `stream`: calls its callbacks
        instead, reports a failure through on_error, and returns None."""
        options = options or SamplingOptions()
        if stream is None:
            return self.generate_batch([prompt], options)[0].tokens
        try:
            self._require_open()
            with self._lock:
                result = self._loop.run([prompt], options, on_token=lambda _, token: stream.on_token(token))[0]
        except Exception as failure:  # exactly one terminal callback
            stream.on_error(failure)
            return None
        stream.on_complete(result.usage)
        return None

    def generate_batch(self, prompts: Sequence[Sequence[int]], options=None,
                       on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        """Every prompt, batched as the cache allows; results in the order of the prompts.
        `options`: one SamplingOptions for all, or one per prompt."""
        self._require_open()
        options = options or SamplingOptions()
        with self._lock:
            return self._loop.run(prompts, options, on_token)

    @property
    def last_prompt_cache(self):
        """What the last request took from the sequence kept before it (PromptCacheMetrics)."""
        return self._loop.last_prompt_cache

    def stream(self, prompt: Sequence[int], options: Optional[SamplingOptions] = None) -> Iterator[int]:
        """Token ids as they are generated.  An iterator that is closed or dropped before its end
        stops the generation behind it at its next token; the sequence's slot goes back."""
        done = object()
        items: "queue.Queue" = queue.Queue()
        abandoned = threading.Event()

        def on_token(token: int) -> None:
            if abandoned.is_set():
                raise _StreamAbandoned()
            items.put(token)

        handler = CallbackStream(on_token, lambda usage: items.put(done), lambda failure: items.put(failure))
        worker = threading.Thread(target=self.generate, args=(prompt, options, handler), daemon=True)
        worker.start()
        try:
            while True:
                item = items.get()
                if item is done:
                    break
                if isinstance(item, BaseException):
                    raise item
                yield item
        finally:
            abandoned.set()
            worker.join()

    # ------------------------------------------------------------------ pipeline calls (one default sequence)

    def _default_session(self) -> int:
        if self._session is None:
            self._session = self.engine.open_slot()
        return self._session

    def prefill(self, tokens: Sequence[int]):
        """Appends `tokens` to the default sequence; float32 logits of the last one (a device tensor)."""
        from .engine import StepEntry

        self._require_open()
        if len(tokens) == 0:
            raise ValueError("prompt must not be empty")
        return self.engine.step([StepEntry(self._default_session(), list(tokens), [len(tokens) - 1])])[0]

    def forward(self, token: int):
        """One more token on the default sequence; its logits (the caller's own copy: a replayed step
        writes its logits into a buffer that the next step writes again)."""
        self._require_open()
        return self.engine.decode([self._default_session()], [token])[0].clone()

    def checkpoint(self) -> int:
        return 0 if self._session is None else self.engine.length(self._session)

    def rewind(self, checkpoint: int) -> None:
        if self._session is None:
            if checkpoint != 0:
                raise ValueError(f"cannot rewind to {checkpoint}: the context is empty")
            return
        self.engine.rewind(self._session, checkpoint)

    def reset_context(self) -> None:
        if self._session is not None:
            self.engine.release_slot(self._session)
            self._session = None

    def step(self, entries):
        """The engine's step function itself: entries of (slot, tokens, wanted places)."""
        self._require_open()
        return self.engine.step(entries)

    def open_slot(self) -> int:
        return self.engine.open_slot()

    def release_slot(self, slot: int) -> None:
        self.engine.release_slot(slot)

    def close(self) -> None:
        """Idempotent (models-runtime/.../InferencePipeline.java:197-205)."""
        if self._closed:
            return
        self.reset_context()
        self._loop.drop_kept()
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def load_model(path=None, *, config=None, seed: Optional[int] = None, dtype: str = "bfloat16", max_batch: int = 8,
               context: Optional[int] = None, device="cuda:0", cuda_graphs: bool = True,
               reuse_prefix: bool = False, continuous: bool = False) -> TextGenerationModel:
    """A model ready to generate.  `path`: a folder with config.json and model.safetensors; or
    `config` (a typed configuration or a config.json dict) with `seed` for random weights.
    `context`: most positions per sequence (default: the model's, at most 4096); the cache is sized
    for `max_batch` sequences of that length.  `reuse_prefix`: a request that comes alone keeps its
    sequence in the cache when it ends, and the next such request runs only what follows their common
    prefix (models-runtime/.../GenerationLoop.java:217-248).  `continuous`: when there are more requests than
    run together, one that waits joins the running ones as soon as another ends, instead of waiting for all of them."""
    from .config import config_from_dict, load_config
    from .engine.loading import engine_from_config, engine_from_folder

    if (path is None) == (config is None):
        raise ValueError("give either a model folder or a config with a seed")
    if path is not None:
        typed = load_config(path)
    else:
        typed = config_from_dict(config) if isinstance(config, dict) else config
        if seed is None:
            raise ValueError("random weights need a seed")
    longest = typed.model_spec().max_positions
    context = min(context or min(longest, 4096), longest)
    max_tokens = max_batch * (-(-context // 64) * 64)
    if path is not None:
        engine = engine_from_folder(path, dtype, max_tokens, device=device, max_sequence=context)
        name = str(path)
    else:
        engine = engine_from_config(typed, seed, dtype, max_tokens, device=device, max_sequence=context)
        name = f"{typed.architecture}-random-{seed}"
    return TextGenerationModel(engine, max_batch, name, cuda_graphs, context, reuse_prefix, continuous)
