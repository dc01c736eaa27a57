"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and owns no model code: every step goes through `Engine.step`, the function
generation uses, with the engine's cache and kernels -- and, as in generation, with steps replayed
from CUDA graphs where the engine captures them (one token per sequence; short prompt steps from
their third occurrence on).  `--graphs off` runs every step launch by launch instead.  The nearest pieces of integrallis/models are
`verify`, which returns the logits of every consumed token
(backend-java/.../llama/LlamaForwardPass.java:1199-1249), and its determinism audit
(models-bench/.../DeterminismAuditCli.java:115-140).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
A request gets a slot at its first appearance and gives it back when a step's `end` names it.
For a step that wants something, `<out>/<step>.f32` holds the logits at the wanted places, in the
order of the entries and of `want`, as little-endian float32 [wanted, vocab].  After every step a
line `done <step>` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Dict, IO

from .engine import Engine, StepEntry
from .loading import engine_from_folder


class TraceError(ValueError):
    pass


class TraceReplayer:
    def __init__(self, engine: Engine, out_dir):
        self.engine = engine
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.slots: Dict[str, int] = {}

    def run_step(self, record: dict) -> None:
        if "step" not in record or "entries" not in record:
            raise TraceError(f"a trace line needs 'step' and 'entries': {record!r}")
        step = record["step"]
        entries = []
        opened = []
        try:
            for item in record["entries"]:
                rid = str(item["id"])
                if rid not in self.slots:
                    self.slots[rid] = self.engine.open_slot()
                    opened.append(rid)
                entries.append(StepEntry(self.slots[rid], [int(t) for t in item["tokens"]],
                                         [int(w) for w in item.get("want", [])]))
            logits = self.engine.step(entries) if entries else None
        except Exception:
            for rid in opened:  # a refused step leaves no half-opened request behind
                self.engine.release_slot(self.slots.pop(rid))
            raise
        if logits is not None:
            data = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            tmp = self.out_dir / f".{step}.f32.tmp"
            data.tofile(tmp)
            tmp.replace(self.out_dir / f"{step}.f32")
        for rid in record.get("end", []) or []:
            rid = str(rid)
            if rid not in self.slots:
                raise TraceError(f"step {step}: 'end' names request {rid!r}, which is not live")
            self.engine.release_slot(self.slots.pop(rid))

    def replay(self, lines: IO[str], done: IO[str]) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            self.run_step(record)
            done.write(f"done {record['step']}\n")
            done.flush()


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", required=True, type=int,
                        help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    parser.add_argument("--graphs", default="on", choices=["on", "off"],
                        help="replay captured steps as generation does (default), or launch every kernel of every step")
    args = parser.parse_args(argv)
    if args.max_tokens <= 0:
        parser.error("--max-tokens must be positive")
    engine = engine_from_folder(args.model, args.dtype, args.max_tokens)
    if args.graphs == "on":
        # any number of live requests the cache has slots for, of any length it has pages for; captures
        # are made when a batch size and a class of lengths first come up
        engine.enable_decode_graphs(engine.cache.max_slots)
    TraceReplayer(engine, args.out).replay(sys.stdin, sys.stdout)
    return 0
