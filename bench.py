#!/usr/bin/env python3
"""Benchmark of models_b200 on one B200: decode tokens per second of Llama 3.2 1B (bfloat16, random
weights, synthetic token ids), with prefill and roofline figures on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

A "step" is one decode step of the whole batch.  `value` is device-timed (CUDA events around K
steps); `e2e` is the same rate through the Python entry point (`generate_batch`: host token ids in,
host token ids out, every step's indices copied to the device and its sampled ids copied back).
Each decode step reads about 2.5 GB of weights, far more than the 126 MB L2, so successive steps
do not find their inputs in the cache.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Llama 3.2 1B
LLAMA_3_2_1B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 16,
    "hidden_size": 2048,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 64,
    "intermediate_size": 8192,
    "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 131072,
    "hidden_act": "silu",
}
CONTEXT = 4096
PROMPT_TOKENS = 512
PREFILL_TOKENS = 2048

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None
        self.skip = 0

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None
            return
        # the tool takes a moment to come up; the timed region starts once it is sampling
        deadline = time.perf_counter() + 3.0
        while time.perf_counter() < deadline and os.path.getsize(self.file.name) == 0:
            time.sleep(0.02)
        self.skip = os.path.getsize(self.file.name)  # what it printed before the timed region

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        self.file.flush()
        self.file.seek(self.skip)
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def matmul_params(c, layers):
    q, kv = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    d, i = c["hidden_size"], c["intermediate_size"]
    per_layer = d * (q + 2 * kv) + q * d + 3 * d * i
    return layers * per_layer, c["vocab_size"] * d


def decode_bytes(c, layers, kv_tokens_total):
    """Bytes a decode step has to read: every weight once (layers, norms, output matrix), and the
    keys and values of the live requests."""
    layer_params, head_params = matmul_params(c, layers)
    norms = (2 * layers + 1) * c["hidden_size"]
    weights = 2 * (layer_params + head_params) + 4 * norms
    kv = kv_tokens_total * layers * 2 * c["num_key_value_heads"] * c["head_dim"] * 2
    return weights + kv


def prefill_flops(c, layers, tokens):
    layer_params, head_params = matmul_params(c, layers)
    gemm = 2 * tokens * layer_params + 2 * head_params  # the output matrix runs on one row
    attention = layers * 4 * c["num_attention_heads"] * c["head_dim"] * tokens * tokens / 2
    return gemm + attention


def make_model(config, max_batch):
    import models_b200

    return models_b200.load_model(config=config, seed=0, dtype="bfloat16", max_batch=max_batch, context=CONTEXT)


def random_prompts(n, length, vocab, seed):
    import numpy as np

    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(0, vocab, size=length)] for _ in range(n)]


def device_decode(model, batch, steps, warmup, sample_clocks=False):
    """K decode steps of `batch` sequences after 512-token prompts, greedy, timed on the device.
    As in generation, a step is queued with the ids of the step before it still on the device, and
    the host reads every step's ids while the next step runs."""
    import torch

    from models_b200 import SamplingOptions
    from models_b200.engine.stepper import EngineStepper
    from models_b200.kernels import ops
    from models_b200.sampling.sampler import RequestSampling

    engine = model.engine
    vocab = engine.spec.vocab_size
    prompts = random_prompts(batch, PROMPT_TOKENS, vocab, 1)
    stepper = EngineStepper(engine)
    greedy = [RequestSampling(SamplingOptions(temperature=0.0), p) for p in prompts]
    rows = list(range(batch))
    slots = [stepper.open_slot() for _ in range(batch)]
    pending = stepper.sample_start(stepper.prefill(slots, prompts), greedy)
    for _ in range(warmup):
        logits = stepper.decode_pending(slots, pending, rows)
        pending.result()
        pending = stepper.sample_start(logits, greedy)
    sampler = ClockSampler() if sample_clocks else None
    if sampler:
        sampler.start()
    kv_total = 0
    launches_before = ops.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        kv_total += sum(engine.length(s) + 1 for s in slots)
        logits = stepper.decode_pending(slots, pending, rows)
        pending.result()
        pending = stepper.sample_start(logits, greedy)
    end.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(end) / 1e3
    launches = ops.launch_count() - launches_before
    clocks = sampler.stop() if sampler else None
    for s in slots:
        engine.release_slot(s)
    return {"seconds": seconds, "tokens_per_second": batch * steps / seconds, "ms_per_step": 1e3 * seconds / steps,
            "kv_tokens_per_step": kv_total / steps, "launches": launches, "clocks": clocks}


def e2e_decode(model, batch, steps, warmup):
    """The same through generate_batch: host ids in, host ids out; rate over the decode steps
    (tokens after each request's first, as integrallis/models' TrialMeasurement counts them)."""
    from models_b200 import SamplingOptions

    vocab = model.metadata.vocab_size
    prompts = random_prompts(batch, PROMPT_TOKENS, vocab, 2)
    stamps = []

    def on_token(index, token):
        if index == 0:
            stamps.append(time.perf_counter())

    model.generate_batch(prompts, SamplingOptions(temperature=0.0, max_tokens=warmup + 1))  # warm-up
    model.generate_batch(prompts, SamplingOptions(temperature=0.0, max_tokens=steps + 1), on_token=on_token)
    seconds = stamps[-1] - stamps[0]
    graphs = model.engine.decode_graphs
    h2d = 0  # the step's indices; the ids themselves stay on the device
    if graphs and graphs.captured:
        layout = graphs.captured[graphs.rung(batch)].layout
        h2d = 4 * (layout.total - layout.tokens)
    return {"tokens_per_second": batch * (len(stamps) - 1) / seconds, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4 * batch}


def device_prefill(model, tokens, repeats=3):
    import torch

    from models_b200.engine import StepEntry

    engine = model.engine
    prompt = random_prompts(1, tokens, engine.spec.vocab_size, 3)[0]
    times = []
    for _ in range(repeats + 2):
        slot = engine.open_slot()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(slot, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
        engine.release_slot(slot)
    return statistics.median(times[2:])


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)  # the workload's 256 generated tokens
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=LLAMA_3_2_1B["num_hidden_layers"])
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 decode points and the prefill")
    parser.add_argument("--only-prefill", action="store_true",
                        help="run the 2,048-token prefill alone and print its figures (for profiling)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": (
            "integrallis/models is a Java 25 / Gradle library with a Rust crate and no Python package: pip cannot "
            "install it, and no JVM, Gradle or cargo is in this image")}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library runs on a single GPU and --gpus {args.gpus} is not built")
        return 2
    warmup = max(args.warmup, 3)

    import torch

    config = dict(LLAMA_3_2_1B, num_hidden_layers=args.layers)
    peak = peaks()
    model = make_model(config, args.batch if (args.no_points or args.only_prefill) else max(64, args.batch))
    if args.only_prefill:
        ms = device_prefill(model, PREFILL_TOKENS, repeats=1)
        print(json.dumps({"prefill_ms": ms, "tokens": PREFILL_TOKENS}))
        return 0
    main_run = device_decode(model, args.batch, args.steps, warmup, sample_clocks=True)
    e2e = e2e_decode(model, args.batch, args.steps, warmup)
    bytes_per_step = decode_bytes(config, args.layers, main_run["kv_tokens_per_step"])
    achieved = bytes_per_step / (main_run["ms_per_step"] / 1e3) / 1e9

    line = {
        "metric": "decode tok/s @ batch 8 (Llama 3.2 1B, bf16)",
        "value": main_run["tokens_per_second"],
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": "Llama 3.2 1B (LlamaForCausalLM)",
            "layers": args.layers,
            "layers_of_model": LLAMA_3_2_1B["num_hidden_layers"],
            "hidden_size": config["hidden_size"],
            "heads": config["num_attention_heads"],
            "kv_heads": config["num_key_value_heads"],
            "head_dim": config["head_dim"],
            "intermediate_size": config["intermediate_size"],
            "vocab_size": config["vocab_size"],
            "tied_embeddings": True,
            "global_batch": args.batch,
            "context_len": CONTEXT,
            "prompt_len": PROMPT_TOKENS,
            "seq_len": PROMPT_TOKENS + warmup + args.steps,
            "parallelism": "single GPU",
            "sampling": "greedy",
            "cache": "paged, 64 positions per page, bf16",
            "l2": "each step reads ~2.5 GB of weights (> 126 MB L2); no flush needed",
            "peaks": peak["source"],
        },
        "e2e": {"value": e2e["tokens_per_second"], "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"]},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": bytes_per_step},
    }
    if not args.no_points:
        ms = device_prefill(model, PREFILL_TOKENS)
        flops = prefill_flops(config, args.layers, PREFILL_TOKENS)
        line["prefill"] = {"value": PREFILL_TOKENS / (ms / 1e3), "tokens": PREFILL_TOKENS, "ms": ms,
                           "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
        points = {}
        for b in (1, 64):
            points[f"decode_b{b}"] = device_decode(model, b, min(args.steps, 64), warmup)["tokens_per_second"]
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
