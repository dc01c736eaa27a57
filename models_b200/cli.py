"""Command line of models_b200, in the manner of integrallis/models' benchmark CLI: a subcommand,
then strict `--name value` pairs; an unknown or repeated option is an error
(models-bench/.../BenchmarkCliArguments.java:12-31; subcommands
models-bench/.../InferenceBenchmarkCli.java:73-108; option names follow PrefillProfileCli,
DecodeProfileCli and SessionBatchProfileCli of the same package).

    python -m models_b200 generate --model DIR --prompt 1,2,3 --max-tokens 16 --temperature 0
    python -m models_b200 profile-prefill --model DIR --prompt-tokens 2048 --context 4096
    python -m models_b200 profile-decode --model DIR --prompt-tokens 512 --measure-tokens 64
    python -m models_b200 profile-sessions --model DIR --concurrency 8 --mode batched
    python -m models_b200 random-model --config config.json --seed 1 --output DIR
    python -m models_b200 replay --model DIR --dtype float32 --out DIR --max-tokens 4096 < trace.jsonl

Prompts are token ids (comma or space separated): there is no tokenizer here.
"""

from __future__ import annotations

import json
import sys
import time
from pathlib import Path
from typing import Dict, List, Optional, Set

MODEL_OPTIONS = {"model", "config", "random-seed", "dtype", "context"}
PROMPT_OPTIONS = {"prompt", "prompt-file", "prompt-tokens"}

OPTIONS: Dict[str, Set[str]] = {
    "generate": MODEL_OPTIONS | PROMPT_OPTIONS | {
        "max-tokens", "temperature", "top-k", "top-p", "seed", "repetition-penalty", "stop-ids", "concurrency",
        "output"},
    "profile-prefill": MODEL_OPTIONS | PROMPT_OPTIONS | {"warmups", "iterations", "output"},
    "profile-decode": MODEL_OPTIONS | PROMPT_OPTIONS | {"token-id", "warmup-tokens", "measure-tokens", "output"},
    "profile-sessions": MODEL_OPTIONS | PROMPT_OPTIONS | {
        "concurrency", "warmup-steps", "measure-steps", "mode", "output"},
    "random-model": {"config", "seed", "output", "dtype"},
    "replay": {"model", "dtype", "out", "max-tokens"},
}


class CliError(ValueError):
    pass


def parse_options(args: List[str], allowed: Set[str]) -> Dict[str, str]:
    if len(args) % 2:
        raise CliError("options must be provided as --name value pairs")
    values: Dict[str, str] = {}
    for i in range(0, len(args), 2):
        option = args[i]
        if not option.startswith("--"):
            raise CliError(f"expected option, got: {option}")
        name = option[2:]
        if name not in allowed:
            raise CliError(f"unknown option: {option}")
        if name in values:
            raise CliError(f"duplicate option: {option}")
        values[name] = args[i + 1]
    return values


def integer(values, name: str, default: Optional[int] = None) -> Optional[int]:
    if name not in values:
        return default
    try:
        return int(values[name])
    except ValueError:
        raise CliError(f"--{name} must be an integer: {values[name]}") from None


def number(values, name: str, default: float) -> float:
    if name not in values:
        return default
    try:
        return float(values[name])
    except ValueError:
        raise CliError(f"--{name} must be a number: {values[name]}") from None


def token_list(text: str, what: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise CliError(f"{what} must hold token ids separated by commas or spaces") from None


def read_prompts(values, vocab: int) -> List[List[int]]:
    """--prompt: ids; --prompt-file: one prompt of ids per line; --prompt-tokens N: N seeded random ids."""
    given = [n for n in ("prompt", "prompt-file", "prompt-tokens") if n in values]
    if len(given) != 1:
        raise CliError("give exactly one of --prompt, --prompt-file, --prompt-tokens")
    if "prompt" in values:
        return [token_list(values["prompt"], "--prompt")]
    if "prompt-file" in values:
        lines = [l for l in Path(values["prompt-file"]).read_text().splitlines() if l.strip()]
        return [token_list(l, "--prompt-file") for l in lines]
    import numpy as np

    n = integer(values, "prompt-tokens")
    if n <= 0:
        raise CliError("--prompt-tokens must be positive")
    return [[int(t) for t in np.random.default_rng(0).integers(0, vocab, size=n)]]


def open_model(values, max_batch: int, cuda_graphs: bool = True):
    import models_b200

    dtype = values.get("dtype", "bfloat16")
    if dtype not in ("bfloat16", "float32"):
        raise CliError(f"--dtype must be bfloat16 or float32: {dtype}")
    context = integer(values, "context")
    if ("model" in values) == ("config" in values):
        raise CliError("give either --model DIR, or --config FILE with --random-seed N")
    if "model" in values:
        return models_b200.load_model(values["model"], dtype=dtype, max_batch=max_batch, context=context,
                                      cuda_graphs=cuda_graphs)
    if "random-seed" not in values:
        raise CliError("--config needs --random-seed")
    raw = json.loads(Path(values["config"]).read_text())
    return models_b200.load_model(config=raw, seed=integer(values, "random-seed"), dtype=dtype, max_batch=max_batch,
                                  context=context, cuda_graphs=cuda_graphs)


def emit(values, report: dict) -> None:
    text = json.dumps(report, indent=2)
    if "output" in values:
        Path(values["output"]).write_text(text + "\n")
    print(text)


# ---------------------------------------------------------------------------------------- subcommands

def cmd_generate(values) -> int:
    from models_b200 import SamplingOptions

    concurrency = integer(values, "concurrency", 8)
    model = open_model(values, concurrency)
    prompts = read_prompts(values, model.metadata.vocab_size)
    seed = integer(values, "seed")
    options = SamplingOptions(
        temperature=number(values, "temperature", 1.0), top_p=number(values, "top-p", 0.9),
        top_k=integer(values, "top-k", 40), max_tokens=integer(values, "max-tokens", 256), seed=seed,
        repetition_penalty=number(values, "repetition-penalty", 1.0),
        stop_token_ids=tuple(token_list(values.get("stop-ids", ""), "--stop-ids")))
    started = time.perf_counter()
    results = model.generate_batch(prompts, options)
    elapsed = time.perf_counter() - started
    emit(values, {
        "model": model.model_name(),
        "results": [{"tokens": r.tokens, "finish_reason": r.finish_reason, "prompt_tokens": r.usage.prompt_tokens,
                     "completion_tokens": r.usage.completion_tokens} for r in results],
        "seconds": elapsed,
    })
    model.close()
    return 0


def _cuda_time(fn) -> float:
    import torch

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / 1e3


def cmd_profile_prefill(values) -> int:
    """Time to push a prompt through the model in one step (prefill rate = prompt tokens / time in
    prefill, models-bench/.../TimingBackend.java:77-82)."""
    model = open_model(values, 1)
    prompt = read_prompts(values, model.metadata.vocab_size)[0]
    times = []
    for i in range(integer(values, "warmups", 2) + integer(values, "iterations", 5)):
        model.reset_context()
        times.append(_cuda_time(lambda: model.prefill(prompt)))
    measured = sorted(times[integer(values, "warmups", 2):])
    p50 = measured[(len(measured) - 1) // 2]
    emit(values, {"prompt_tokens": len(prompt), "prefill_seconds_p50": p50, "prefill_tokens_per_second": len(prompt) / p50,
                  "diagnostics": model.diagnostics()})
    return 0


def cmd_profile_decode(values) -> int:
    """Warmed-up one-sequence decode at the position the prompt leaves
    (models-bench/.../DecodeProfileCli.java:92-165)."""
    import torch

    model = open_model(values, 1)
    prompt = read_prompts(values, model.metadata.vocab_size)[0]
    token = integer(values, "token-id", prompt[-1])
    model.prefill(prompt)
    for _ in range(integer(values, "warmup-tokens", 8)):
        model.forward(token)
    n = integer(values, "measure-tokens", 64)
    seconds = _cuda_time(lambda: [model.forward(token) for _ in range(n)])
    emit(values, {"prompt_tokens": len(prompt), "measured_tokens": n, "decode_seconds": seconds,
                  "decode_tokens_per_second": n / seconds, "diagnostics": model.diagnostics()})
    return 0


def cmd_profile_sessions(values) -> int:
    """Decode across several sessions, batched in one step or one after another
    (models-bench/.../SessionBatchProfileCli.java:119-272)."""
    concurrency = integer(values, "concurrency", 4)
    mode = values.get("mode", "batched")
    if mode not in ("sequential", "batched"):
        raise CliError(f"--mode must be sequential or batched: {mode}")
    model = open_model(values, concurrency)
    prompt = read_prompts(values, model.metadata.vocab_size)[0]
    engine = model.engine
    slots = [engine.open_slot() for _ in range(concurrency)]
    from models_b200.engine import StepEntry

    engine.step([StepEntry(s, prompt, []) for s in slots])
    tokens = [prompt[-1]] * concurrency

    def one_step():
        if mode == "batched":
            engine.decode(slots, tokens)
        else:
            for s, t in zip(slots, tokens):
                engine.decode([s], [t])

    for _ in range(integer(values, "warmup-steps", 4)):
        one_step()
    steps = integer(values, "measure-steps", 32)
    seconds = _cuda_time(lambda: [one_step() for _ in range(steps)])
    emit(values, {"mode": mode, "concurrency": concurrency, "measure_steps": steps, "seconds": seconds,
                  "aggregate_tokens_per_second": steps * concurrency / seconds, "diagnostics": model.diagnostics()})
    return 0


def cmd_random_model(values) -> int:
    import torch

    import models_b200
    from models_b200.config import config_from_dict

    for name in ("config", "seed", "output"):
        if name not in values:
            raise CliError(f"--{name} is required")
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(values.get("dtype", "bfloat16"))
    if dtype is None:
        raise CliError(f"--dtype must be bfloat16 or float32: {values['dtype']}")
    config = config_from_dict(json.loads(Path(values["config"]).read_text()))
    folder = models_b200.write_random_model(values["output"], config, integer(values, "seed"), dtype=dtype)
    print(folder)
    return 0


def cmd_replay(values) -> int:
    from .engine.trace import main as trace_main

    argv = []
    for name in ("model", "dtype", "out", "max-tokens"):
        if name not in values:
            raise CliError(f"--{name} is required")
        argv += [f"--{name}", values[name]]
    return trace_main(argv)


COMMANDS = {
    "generate": cmd_generate,
    "profile-prefill": cmd_profile_prefill,
    "profile-decode": cmd_profile_decode,
    "profile-sessions": cmd_profile_sessions,
    "random-model": cmd_random_model,
    "replay": cmd_replay,
}


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    command = argv[0]
    if command not in COMMANDS:
        print(f"unknown subcommand: {command} (known: {', '.join(COMMANDS)})", file=sys.stderr)
        return 2
    try:
        values = parse_options(argv[1:], OPTIONS[command])
        return COMMANDS[command](values)
    except CliError as error:
        print(f"error: {error}", file=sys.stderr)
        return 2
