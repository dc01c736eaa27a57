#!/usr/bin/env python3
"""Benchmark of models_b200 on one B200: decode tokens per second of Llama 3.2 1B (bfloat16, random
weights, synthetic token ids), with prefill and roofline figures on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model 1b|3b|8b] [--batch B] [--layers L] [--impl ours|reference]

A "step" is one decode step of the whole batch.  `value` is device-timed (CUDA events around K
steps); `e2e` is the same rate through the Python entry point (`generate_batch`: host token ids in,
host token ids out, every step's indices copied to the device and its sampled ids copied back).
Each decode step reads about 2.5 GB of weights, far more than the 126 MB L2, so successive steps
do not find their inputs in the cache.
"""

from __future__ import annotations

import argparse
import hashlib
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

# The other two workloads of the baseline file (--model 3b / 8b); the default run is the 1B one.
LLAMA_3_2_3B = dict(LLAMA_3_2_1B, num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8,
                    head_dim=128, intermediate_size=8192)
LLAMA_3_1_8B = dict(LLAMA_3_2_1B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                    head_dim=128, intermediate_size=14336, tie_word_embeddings=False,
                    rope_scaling=dict(LLAMA_3_2_1B["rope_scaling"], factor=8.0))
WORKLOADS = {
    # prompt: a length, or (shortest, longest) for unequal prompts; context: positions per sequence the cache is sized for
    "1b": {"config": LLAMA_3_2_1B, "name": "Llama 3.2 1B (LlamaForCausalLM)", "batch": 8, "prompt": PROMPT_TOKENS,
           "context": CONTEXT, "steps": 256, "prefill": PREFILL_TOKENS, "points": (1, 64)},
    "3b": {"config": LLAMA_3_2_3B, "name": "Llama 3.2 3B (LlamaForCausalLM)", "batch": 16, "prompt": (128, 2048),
           "context": 2048 + 192, "steps": 128, "prefill": PREFILL_TOKENS, "points": ()},
    "8b": {"config": LLAMA_3_1_8B, "name": "Llama 3.1 8B-shaped (LlamaForCausalLM)", "batch": 64, "prompt": 1024,
           "context": 1024 + 320, "steps": 256, "prefill": 16384, "points": ()},
}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    """The roofline denominators: the driver's measured copy bandwidth and cuBLAS bf16 throughput (burst) when
    MEASURED_PEAKS.json is there, else the stated fallback figures."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")

    def number(raw, names, scale=1.0):
        for name in names:
            value = raw.get(name)
            if isinstance(value, dict):
                value = value.get("value", value.get("measured"))
            if isinstance(value, (int, float)) and value > 0:
                return float(value) * scale
        return None

    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            hbm = number(raw, ("hbm_gbs", "hbm_gb_s", "hbm_gbps")) or number(raw, ("hbm_tbs", "hbm_tb_s"), 1000.0)
            bf16 = number(raw, ("bf16_tflops", "bf16_tflops_burst")) or number(raw, ("bf16_pflops",), 1000.0)
            if hbm and bf16:
                return {"hbm_gbs": hbm, "bf16_tflops": bf16, "source": "measured"}
        except (OSError, ValueError, TypeError, AttributeError):
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


def make_model(config, max_batch, context=CONTEXT):
    import models_b200

    return models_b200.load_model(config=config, seed=0, dtype="bfloat16", max_batch=max_batch, context=context)


def random_prompts(n, length, vocab, seed):
    """n prompts of `length` tokens each, or of lengths drawn from (shortest, longest)."""
    import numpy as np

    rng = np.random.default_rng(seed)
    lengths = [length] * n if isinstance(length, int) else [int(x) for x in rng.integers(length[0], length[1] + 1, size=n)]
    return [[int(t) for t in rng.integers(0, vocab, size=m)] for m in lengths]


def device_decode(model, batch, steps, warmup, sample_clocks=False, prompt=PROMPT_TOKENS):
    """K decode steps of `batch` sequences after their prompts (512 tokens each in the default run), greedy, timed on the device.
    As in generation, a step is queued with the ids of the step before it still on the device, and
    the host reads every step's ids while the next step runs."""
    import torch

    from models_b200 import SamplingOptions
    from models_b200.engine.stepper import EngineStepper
    from models_b200.kernels import ops
    from models_b200.sampling.sampler import RequestSampling

    engine = model.engine
    vocab = engine.spec.vocab_size
    prompts = random_prompts(batch, prompt, vocab, 1)
    stepper = EngineStepper(engine)
    greedy = [RequestSampling(SamplingOptions(temperature=0.0), p) for p in prompts]
    rows = list(range(batch))
    slots = [stepper.open_slot() for _ in range(batch)]
    pending = stepper.sample_start(stepper.prefill(slots, prompts), greedy)
    for _ in range(warmup):
        logits = stepper.decode_pending(slots, pending, rows)
        pending.result()
        pending = stepper.sample_start(logits, greedy)
    graphs = engine.decode_graphs
    if graphs is not None and batch <= graphs.max_batch:
        # part of the warm-up: the captures of every class of context length that the timed steps will meet (a
        # sequence that crosses such a boundary would otherwise pay for a capture inside the timed region)
        longest = max(engine.length(s) for s in slots)
        for kv in range(longest + 1, longest + steps + 2):
            graphs.prepare(graphs.rung(batch), kv)
    sampler = ClockSampler() if sample_clocks else None
    if sampler:
        sampler.start()
    kv_total = 0
    launches_before = ops.launch_count()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]  # one after every step, on the step's stream
    torch.cuda.synchronize()
    marks[0].record()
    for step in range(steps):
        kv_total += sum(engine.length(s) + 1 for s in slots)
        logits = stepper.decode_pending(slots, pending, rows)
        pending.result()
        pending = stepper.sample_start(logits, greedy)
        marks[step + 1].record()
    torch.cuda.synchronize()
    seconds = marks[0].elapsed_time(marks[-1]) / 1e3
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    launches = ops.launch_count() - launches_before
    clocks = sampler.stop() if sampler else None
    # which form of each product the step ran: the launchers' names of the last capture this batch size replayed
    kernels = {}
    if graphs is not None and batch <= graphs.max_batch:
        key = (graphs.rung(batch), graphs.launch_class(graphs.rung(batch), max(engine.length(s) for s in slots)))
        for name in getattr(graphs.captured.get(key), "kernel_names", []):
            kernels[name] = kernels.get(name, 0) + 1
    for s in slots:
        engine.release_slot(s)
    return {"seconds": seconds, "kernels": kernels, "tokens_per_second": batch * steps / seconds, "ms_per_step": 1e3 * seconds / steps,
            "ms_per_step_p50": percentile(per_step, 0.50), "ms_per_step_p95": percentile(per_step, 0.95),
            "kv_tokens_per_step": kv_total / steps, "launches": launches, "clocks": clocks}


def percentile(ordered, fraction):
    """Nearest-rank percentile of an ascending list (integrallis/models, models-bench/.../BenchmarkStatistics.java:35-59)."""
    if not ordered:
        return None
    rank = max(1, -(-int(round(fraction * 1000)) * len(ordered) // 1000))
    return ordered[min(len(ordered), rank) - 1]


def e2e_decode(model, batch, steps, warmup, prompt=PROMPT_TOKENS):
    """The same through generate_batch: host ids in, host ids out; rate over the decode steps
    (tokens after each request's first, as integrallis/models' TrialMeasurement counts them)."""
    from models_b200 import SamplingOptions

    vocab = model.metadata.vocab_size
    prompts = random_prompts(batch, prompt, vocab, 2)
    stamps = []

    def on_token(index, token):
        if index == 0:
            stamps.append(time.perf_counter())

    first = model.generate_batch(prompts, SamplingOptions(temperature=0.0, max_tokens=warmup + 1))  # warm-up
    results = model.generate_batch(prompts, SamplingOptions(temperature=0.0, max_tokens=steps + 1), on_token=on_token)
    seconds = stamps[-1] - stamps[0]
    # what was generated, as a hash (integrallis/models prints one per run, models-bench/.../SessionBatchProfileCli.java:287-293),
    # and whether the warm-up run -- the same prompts, fewer tokens -- produced the same ids as far as it went
    digest = hashlib.sha256()
    for result in results:
        digest.update(",".join(str(t) for t in result.tokens).encode() + b";")
    repeated = all(a.tokens == b.tokens[: len(a.tokens)] for a, b in zip(first, results))
    graphs = model.engine.decode_graphs
    h2d = 0  # the step's indices; the ids themselves stay on the device
    if graphs and graphs.captured:
        layout = next(c for (size, _), c in graphs.captured.items() if size == graphs.rung(batch)).layout
        h2d = 4 * (layout.total - layout.tokens)
    return {"tokens_per_second": batch * (len(stamps) - 1) / seconds, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4 * batch, "tokens_hash": digest.hexdigest()[:16], "repeated": repeated}


def device_prefill(model, tokens, repeats=5):
    import torch

    from models_b200.engine import StepEntry

    engine = model.engine
    prompt = random_prompts(1, tokens, engine.spec.vocab_size, 3)[0]
    times = []
    warm = 4  # (a class of prompt steps is captured when it comes up for the third time: that run is part of the warm-up)
    for _ in range(repeats + warm):
        slot = engine.open_slot()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(slot, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
        engine.release_slot(slot)
    return statistics.median(times[warm:])


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None, help="decode steps timed (default: the workload's generated tokens)")
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--model", default="1b", choices=sorted(WORKLOADS),
                        help="1b: the default run; 3b, 8b: the other two workloads of the baseline file")
    parser.add_argument("--batch", type=int, default=None, help="sequences decoded together (default: the workload's)")
    parser.add_argument("--prompt", type=int, default=None,
                        help="prompt tokens per sequence (default: the workload's); the context grows to hold them")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (both counts are reported)")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 decode points and the prefill")
    parser.add_argument("--only-prefill", action="store_true",
                        help="run the workload's prefill alone and print its figures (for profiling)")
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
    work = WORKLOADS[args.model]
    batch = args.batch or work["batch"]
    steps = args.steps or work["steps"]
    layers = args.layers or work["config"]["num_hidden_layers"]
    prompt, context, prefill_tokens = work["prompt"], work["context"], work["prefill"]
    if args.prompt:
        prompt, context = args.prompt, max(context, args.prompt + warmup + steps + 64)
    longest_prompt = prompt if isinstance(prompt, int) else prompt[1]
    if longest_prompt + warmup + steps + 1 > context:
        print(f"bench.py: {longest_prompt} prompt tokens + {warmup} + {steps} steps do not fit the context of {context}")
        return 2

    import torch

    config = dict(work["config"], num_hidden_layers=layers)
    peak = peaks()
    if args.only_prefill:
        model = make_model(config, 1, max(context, prefill_tokens + 64))
        ms = device_prefill(model, prefill_tokens, repeats=1)
        print(json.dumps({"prefill_ms": ms, "tokens": prefill_tokens}))
        return 0
    with_points = not args.no_points
    # the prefill fits the decode cache when it is no longer than a sequence's context; else it gets a model of its own
    prefill_fits = prefill_tokens + 64 <= context
    sequences = max([batch] + (list(work["points"]) if with_points else []))
    model = make_model(config, sequences, context)
    main_run = device_decode(model, batch, steps, warmup, sample_clocks=True, prompt=prompt)
    e2e = e2e_decode(model, batch, steps, warmup, prompt=prompt)
    bytes_per_step = decode_bytes(config, layers, main_run["kv_tokens_per_step"])
    achieved = bytes_per_step / (main_run["ms_per_step"] / 1e3) / 1e9
    weights_gb = decode_bytes(config, layers, 0) / 1e9

    line = {
        "metric": f"decode tok/s @ batch {batch} ({work['name'].split(' (')[0]}, bf16)",
        "value": main_run["tokens_per_second"],
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"],
        "ms_per_step_p50": main_run["ms_per_step_p50"],
        "ms_per_step_p95": main_run["ms_per_step_p95"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "gpu": torch.cuda.get_device_name(0),
        "tokens_hash": e2e["tokens_hash"],
        "tokens_repeat_the_warmup_run": e2e["repeated"],
        "config": {
            "model": work["name"],
            "layers": layers,
            "layers_of_model": work["config"]["num_hidden_layers"],
            "hidden_size": config["hidden_size"],
            "heads": config["num_attention_heads"],
            "kv_heads": config["num_key_value_heads"],
            "head_dim": config["head_dim"],
            "intermediate_size": config["intermediate_size"],
            "vocab_size": config["vocab_size"],
            "tied_embeddings": bool(config["tie_word_embeddings"]),
            "global_batch": batch,
            "context_len": context,
            "prompt_len": prompt if isinstance(prompt, int) else f"{prompt[0]}..{prompt[1]} (unequal)",
            "seq_len": longest_prompt + warmup + steps,
            "parallelism": "single GPU",
            "sampling": "greedy",
            "cache": "paged, 64 positions per page, bf16",
            "l2": f"each step reads ~{weights_gb:.1f} GB of weights (> 126 MB L2); no flush needed",
            "peaks": peak["source"],
        },
        "e2e": {"value": e2e["tokens_per_second"], "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"]},
        "gpu_launches": main_run["launches"],
        "kernels": main_run["kernels"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": bytes_per_step},
    }
    if with_points:
        points = {}
        for b in work["points"]:
            points[f"decode_b{b}"] = device_decode(model, b, min(steps, 64), warmup, prompt=prompt)["tokens_per_second"]
        if points:
            line["points"] = points
        if not prefill_fits:
            model.close()
            del model
            torch.cuda.empty_cache()
            model = make_model(config, 1, prefill_tokens + 64)
        ms = device_prefill(model, prefill_tokens)
        flops = prefill_flops(config, layers, prefill_tokens)
        line["prefill"] = {"value": prefill_tokens / (ms / 1e3), "tokens": prefill_tokens, "ms": ms,
                           "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12)}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
