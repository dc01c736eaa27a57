"""Whole models at 16 to 64 sequences against the plain implementation, with CUDA graphs, one batch
after another.

A step of 9 to 128 rows takes other matrix products than a step of a few rows or of a long prompt
(the wide tcgen05 forms, K split over blocks, a library product where a width is no multiple of 8),
decode captures of 16, 32 and 64 sequences pad a smaller batch up to their size, and a vocabulary of
19,000 puts the wide tcgen05 product under the output matrix of a real step.  Every row of every
step is compared: unequal prompts of 1 to 200 tokens in one step, decoding with requests that end at
different steps, then the next batch on the slots and pages that were given back.  The reference's
own form of this test is batch == alone
(backend-java/src/test/.../llama/LlamaForwardPassTest.java:1573-1676).
"""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tiny import MID_D, MID_E, TINY_B, TOLERANCE, make_folder, plain_logits, random_tokens, scaled_error

pytestmark = pytest.mark.gpu

# a vocabulary wide enough for a row tile of the output matrix per multiprocessor (128 x 148 = 18,944)
WIDE_V = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 256,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "intermediate_size": 640,
    "vocab_size": 19000,
    "rope_theta": 10000.0,
    "rope_scaling": None,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
}

CONFIGS = {"B": TINY_B, "D": MID_D, "E": MID_E, "V": WIDE_V}
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("wide_models")
    return {name: make_folder(raw, seed=61 + i, tmp_path=root, std=0.04) for i, (name, raw) in enumerate(CONFIGS.items())}


def unequal_batch(vocab, count, seed, longest=200, most_decodes=10):
    """`count` sequences: prompt lengths 1...longest (the ends and a page boundary among them), and how
    many tokens each decodes (1...most_decodes, so they end at different steps)."""
    rng = np.random.default_rng(seed)
    prompts = [int(n) for n in rng.integers(1, longest + 1, size=count)]
    prompts[0], prompts[1], prompts[-1] = 1, longest, 64
    decodes = [int(n) for n in rng.integers(1, most_decodes + 1, size=count)]
    decodes[1] = most_decodes
    sequences = [random_tokens(vocab, p + d, seed * 1000 + i) for i, (p, d) in enumerate(zip(prompts, decodes))]
    return prompts, decodes, sequences


def run_batch(engine, folder, prompts, decodes, sequences, dtype, what):
    from models_b200.engine import StepEntry

    tolerance = TOLERANCE[dtype]
    expected = [plain_logits(folder, s) for s in sequences]
    slots = [engine.open_slot() for _ in prompts]
    out = engine.step([StepEntry(slot, s[:p], [p - 1]) for slot, s, p in zip(slots, sequences, prompts)])
    assert out.shape[0] == len(prompts)
    for i, p in enumerate(prompts):
        err = scaled_error(out[i], expected[i][p - 1])
        assert err < tolerance, (what, "prompt", i, p, err)
    live = list(range(len(slots)))
    for step in range(max(decodes)):
        live = [i for i in live if step < decodes[i]]
        out = engine.decode([slots[i] for i in live], [sequences[i][prompts[i] + step] for i in live])
        assert out.shape[0] == len(live)
        for row, i in enumerate(live):
            err = scaled_error(out[row], expected[i][prompts[i] + step])
            assert err < tolerance, (what, "decode step", step, "sequence", i, "of", len(live), err)
        for i in live:
            if step + 1 == decodes[i]:
                engine.release_slot(slots[i])
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D", "E", "V"])
def test_batches_of_33_64_and_16_one_after_another(cuda_device, folders, name, dtype):
    import models_b200

    raw = CONFIGS[name]
    model = models_b200.load_model(folders[name], dtype=dtype, max_batch=64, context=256)
    engine = model.engine
    assert engine.decode_graphs is not None
    for round_index, count in enumerate((33, 64, 16)):
        prompts, decodes, sequences = unequal_batch(raw["vocab_size"], count, 7 * round_index + len(name))
        run_batch(engine, folders[name], prompts, decodes, sequences, dtype, f"{name} round {round_index} of {count}")
    assert engine.cache.slots.held == 0 and all(g.pages.held == 0 for g in engine.cache.groups)
    sizes = {size for size, _ in engine.decode_graphs.captured}
    assert {64, 32, 16} <= sizes, sizes  # the large captures ran, with smaller batches padded up to them
    if dtype == "bfloat16":
        from models_b200.kernels import ops

        assert ops.gemm_tcgen05_status() == 0
    model.close()


def test_which_product_takes_how_many_rows(cuda_device, folders):
    """What the tests above rely on: 1 to 8 rows take the narrow decode product, 9 to 128 the wide tcgen05
    product (every matrix of a layer and the output matrix), more the prefill tcgen05 product."""
    import torch

    from models_b200.kernels import ops

    wide = torch.empty((WIDE_V["vocab_size"], WIDE_V["hidden_size"]), dtype=torch.bfloat16, device="cuda")
    narrow = torch.empty((MID_D["vocab_size"], MID_D["hidden_size"]), dtype=torch.bfloat16, device="cuda")
    for weight in (wide, narrow):
        assert ops.skinny_pays(weight, 8) and not ops.skinny_pays(weight, 9)
        assert not ops.gemm_tcgen05_takes(weight, ops.EPI_F32, rows=8)
        assert all(ops.gemm_tcgen05_takes(weight, ops.EPI_F32, rows=rows) for rows in (9, 33, 64, 128, 129, 2048))
    odd = torch.empty((203, 136), dtype=torch.bfloat16, device="cuda")  # a vocabulary that is no multiple of 8: a library product
    assert not ops.gemm_tcgen05_takes(odd, ops.EPI_F32, rows=64)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_with_graphs_in_unequal_batches(cuda_device, folders, dtype, tmp_path):
    """bin/trace_run as generation runs: decode steps replayed from captures, two batches one after
    the other on the same slots, every sequence over several pages, shorter requests ending earlier."""
    name = "D"
    raw = CONFIGS[name]
    vocab = raw["vocab_size"]
    steps, checks, number = [], [], 0
    for batch_index, lengths in enumerate([((70, 9), (130, 4), (100, 12), (5, 7), (64, 1)), ((70, 12), (130, 9), (100, 4))]):
        ids = [f"r{batch_index}_{i}" for i in range(len(lengths))]
        sequences = [random_tokens(vocab, p + d, 900 + 10 * batch_index + i) for i, (p, d) in enumerate(lengths)]
        steps.append({"step": number, "entries": [{"id": rid, "tokens": s[:p], "want": [0, p - 1]}
                                                  for rid, s, (p, _) in zip(ids, sequences, lengths)], "end": []})
        checks.append((sequences, [(i, place) for i, (p, _) in enumerate(lengths) for place in (0, p - 1)]))
        number += 1
        for step in range(max(d for _, d in lengths)):
            live = [i for i, (_, d) in enumerate(lengths) if step < d]
            steps.append({"step": number,
                          "entries": [{"id": ids[i], "tokens": [sequences[i][lengths[i][0] + step]], "want": [0]} for i in live],
                          "end": [ids[i] for i in live if step + 1 == lengths[i][1]]})
            checks.append((sequences, [(i, lengths[i][0] + step) for i in live]))
            number += 1
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    # five requests of up to 3 pages each are live at most
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folders[name]), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(64 * 12)],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(number)]
    cache = {}
    for step, (sequences, rows) in enumerate(checks):
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), vocab)
        for row, (i, place) in enumerate(rows):
            key = tuple(sequences[i])
            if key not in cache:
                cache[key] = plain_logits(folders[name], sequences[i])
            err = scaled_error(got[row], cache[key][place])
            assert err < TOLERANCE[dtype], (step, i, place, err)
