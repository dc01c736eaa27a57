"""The engine against the plain implementation: whole prompts, token by token, unequal batches."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tiny import MID, TINY, TOLERANCE, make_folder, plain_logits, random_tokens, scaled_error

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def _engine(folder, dtype, max_tokens=1024):
    from models_b200.engine.loading import engine_from_folder

    return engine_from_folder(folder, dtype, max_tokens)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: make_folder(raw, seed=11 + i, tmp_path=root) for i, (name, raw) in enumerate(TINY.items())}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_every_position(cuda_device, folders, name, dtype):
    # 1 and 7 tokens take the decode kernels, 70 the library product, 128 and more the tcgen05 product
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    for n, seed in ((1, 1), (7, 2), (70, 3), ({"A": 128, "B": 200, "C": 300}[name], 4)):
        tokens = random_tokens(TINY[name]["vocab_size"], n, seed)
        slot = engine.open_slot()
        logits = engine.step([StepEntry(slot, tokens, list(range(n)))])
        engine.release_slot(slot)
        expected = plain_logits(folders[name], tokens)
        assert scaled_error(logits, expected) < TOLERANCE[dtype], (name, dtype, n)
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(cuda_device, folders, name, dtype):
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    n = 100
    tokens = random_tokens(TINY[name]["vocab_size"], n, 5)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    head = n - 32
    rows = [engine.step([StepEntry(slot, tokens[:head], [head - 1])])]
    for i in range(head, n):
        rows.append(engine.step([StepEntry(slot, [tokens[i]], [0])]))
    got = torch.cat(rows)
    errors = [scaled_error(got[i], expected[head - 1 + i]) for i in range(got.shape[0])]
    worst = int(np.argmax(errors))
    assert errors[worst] < TOLERANCE[dtype], f"first wrong row {next(i for i, e in enumerate(errors) if e >= TOLERANCE[dtype])}, worst {worst}: {errors[worst]}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_one_after_another(cuda_device, folders, name, dtype):
    """Prompts of unequal lengths start together, decode together, the shorter requests end earlier,
    and the next batch takes the slots (and pages) the first one gave back."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=4 * 128)
    vocab = TINY[name]["vocab_size"]
    for round_index, (lengths, decodes) in enumerate([((5, 11, 17), (8, 3, 6)), ((1, 7, 30, 64), (12, 5, 1, 9)),
                                                      ((64, 2, 33), (4, 4, 20))]):
        full = [random_tokens(vocab, p + d, 100 * round_index + i) for i, (p, d) in enumerate(zip(lengths, decodes))]
        expected = [plain_logits(folders[name], t) for t in full]
        slots = [engine.open_slot() for _ in lengths]
        out = engine.step([StepEntry(s, t[:p], [p - 1]) for s, t, p in zip(slots, full, lengths)])
        for i, p in enumerate(lengths):
            assert scaled_error(out[i], expected[i][p - 1]) < TOLERANCE[dtype], (round_index, "prefill", i)
        live = list(range(len(lengths)))
        for step in range(max(decodes)):
            live = [i for i in live if step < decodes[i]]
            out = engine.step([StepEntry(slots[i], [full[i][lengths[i] + step]], [0]) for i in live])
            for row, i in enumerate(live):
                err = scaled_error(out[row], expected[i][lengths[i] + step])
                assert err < TOLERANCE[dtype], (round_index, "decode", step, i, err)
            for i in live:
                if step + 1 == decodes[i]:
                    engine.release_slot(slots[i])
            engine.cache.check()
    assert engine.cache.slots.held == 0
    assert all(g.pages.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(cuda_device, folders, dtype, tmp_path):
    """bin/trace_run as a user calls it: whole prompt, then one token at a time, in a batch of two."""
    name = "B"
    vocab = TINY[name]["vocab_size"]
    a, b = random_tokens(vocab, 40, 1), random_tokens(vocab, 9, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]},
                                     {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for i in range(10):
        entries = [{"id": "a", "tokens": [a[30 + i]], "want": [0]}]
        end = []
        if i < 4:
            entries.append({"id": "b", "tokens": [b[5 + i]], "want": [0]})
            if i == 3:
                end.append("b")
        if i == 9:
            end.append("a")
        steps.append({"step": i + 1, "entries": entries, "end": end})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folders[name]), "--dtype", dtype,
         "--out", str(out), "--max-tokens", "128"],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(11)]
    ea, eb = plain_logits(folders[name], a), plain_logits(folders[name], b)
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, vocab)
    assert scaled_error(first[0], ea[0]) < TOLERANCE[dtype]
    assert scaled_error(first[1], ea[29]) < TOLERANCE[dtype]
    assert scaled_error(first[2], eb[4]) < TOLERANCE[dtype]
    for i in range(10):
        got = np.fromfile(out / f"{i + 1}.f32", dtype="<f4").reshape(-1, vocab)
        assert scaled_error(got[0], ea[30 + i]) < TOLERANCE[dtype], i
        if i < 4:
            assert scaled_error(got[1], eb[5 + i]) < TOLERANCE[dtype], i


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "E"])
def test_mid_size_models_all_ways(cuda_device, tmp_path, name, dtype):
    """At sizes where the tensor-core kernels run their real tilings: a whole prompt of 300 (tcgen05
    products, tiled prefill attention), the same prompt cut at 200 with the rest one by one (decode
    products with K split over clusters, cluster-combined attention), and an unequal batch."""
    from models_b200.engine import StepEntry
    from models_b200.kernels import ops

    raw = MID[name]
    folder = make_folder(raw, seed=31, tmp_path=tmp_path, std=0.03)
    engine = _engine(folder, dtype, max_tokens=2048)
    vocab = raw["vocab_size"]
    a, b, c = random_tokens(vocab, 300, 1), random_tokens(vocab, 140, 2), random_tokens(vocab, 17, 3)
    ea, eb, ec = (plain_logits(folder, t) for t in (a, b, c))
    tol = TOLERANCE[dtype]
    slot = engine.open_slot()
    out = engine.step([StepEntry(slot, a, [0, 63, 64, 150, 299])])
    for row, place in enumerate([0, 63, 64, 150, 299]):
        assert scaled_error(out[row], ea[place]) < tol, ("whole", place)
    engine.release_slot(slot)
    slot = engine.open_slot()
    out = engine.step([StepEntry(slot, a[:200], [199])])
    assert scaled_error(out[0], ea[199]) < tol
    for i in range(200, 232):
        out = engine.step([StepEntry(slot, [a[i]], [0])])
        assert scaled_error(out[0], ea[i]) < tol, ("one by one", i)
    engine.release_slot(slot)
    slots = [engine.open_slot() for _ in range(3)]
    out = engine.step([StepEntry(slots[0], a[:130], [129]), StepEntry(slots[1], b[:129], [0, 128]), StepEntry(slots[2], c[:5], [4])])
    for row, (expected, place) in enumerate(((ea, 129), (eb, 0), (eb, 128), (ec, 4))):
        assert scaled_error(out[row], expected[place]) < tol, ("batch prefill", row)
    for i in range(11):
        live = [(slots[0], a, 130), (slots[1], b, 129)] + ([(slots[2], c, 5)] if i < 9 else [])
        out = engine.decode([s for s, _, _ in live], [t[p + i] for _, t, p in live])
        for row, (_, t, p) in enumerate(live):
            expected = {id(a): ea, id(b): eb, id(c): ec}[id(t)]
            assert scaled_error(out[row], expected[p + i]) < tol, ("batch decode", i, row)
        if i == 8:
            engine.release_slot(slots[2])
    if dtype == "bfloat16":
        assert ops.gemm_tcgen05_status() == 0
    engine.cache.check()


def test_the_same_prompt_gives_the_same_bits_every_time(cuda_device, tmp_path):
    """A prompt of 256 tokens (the size at which the residual products split K over blocks) five times,
    alone and next to another prompt, in bfloat16: every run's logits are equal bit for bit
    (integrallis/models gates on exact-logit repeatability, models-bench/.../DeterminismAuditCli.java:115-140)."""
    from models_b200.engine import StepEntry

    raw = MID["D"]
    folder = make_folder(raw, seed=33, tmp_path=tmp_path, std=0.03)
    engine = _engine(folder, "bfloat16", max_tokens=4096)
    tokens, other = random_tokens(raw["vocab_size"], 256, 9), random_tokens(raw["vocab_size"], 100, 10)
    runs = []
    for i in range(5):
        slot = engine.open_slot()
        runs.append(engine.step([StepEntry(slot, tokens, [0, 100, 255])]))
        engine.release_slot(slot)
    for other_run in runs[1:]:
        assert torch.equal(runs[0], other_run)
    assert scaled_error(runs[0][2], plain_logits(folder, tokens)[255]) < TOLERANCE["bfloat16"]
    pairs = []
    for i in range(3):
        slots = [engine.open_slot(), engine.open_slot()]
        pairs.append(engine.step([StepEntry(slots[0], other, [99]), StepEntry(slots[1], tokens, [255])]))
        for slot in slots:
            engine.release_slot(slot)
    assert torch.equal(pairs[0], pairs[1]) and torch.equal(pairs[0], pairs[2])
