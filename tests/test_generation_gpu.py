"""Generation through the Python entry point, sampling kernels, CUDA-graph decode, long decoding."""

import numpy as np
import pytest
import torch

from plain import plain_llama
from tiny import TINY, TOLERANCE, make_folder, plain_logits, random_tokens, scaled_error

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen_models")
    # larger weights than N(0, 0.02) so that logits are spread and greedy choices are not near-ties
    return {name: make_folder(raw, seed=21 + i, tmp_path=root, std=0.08) for i, (name, raw) in enumerate(TINY.items())}


def plain_greedy(folder, prompt, max_tokens, stop_ids=()):
    """Greedy generation with the plain implementation; also the smallest top-2 margin met."""
    config, weights = plain_llama.read_model_folder(folder)
    tokens, out, margins = list(prompt), [], []
    for _ in range(max_tokens):
        logits = plain_llama.forward(config, weights, tokens)[-1]
        top2 = torch.topk(logits, 2).values
        margins.append(float(top2[0] - top2[1]))
        nxt = plain_llama.plain_argmax(logits)
        if nxt in stop_ids:
            break
        out.append(nxt)
        tokens.append(nxt)
    return out, margins


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(cuda_device, folders, name, dtype):
    import models_b200
    from models_b200 import SamplingOptions

    raw = TINY[name]
    model = models_b200.load_model(folders[name], dtype=dtype, max_batch=4, context=128)
    prompts = [random_tokens(raw["vocab_size"], n, 30 + n) for n in (3, 17, 1, 40, 9)]
    options = SamplingOptions(temperature=0.0, max_tokens=12)
    results = model.generate_batch(prompts, options)  # five requests, batches of four: slots are used again
    for prompt, result in zip(prompts, results):
        expected, margins = plain_greedy(folders[name], prompt, 12, model.engine.spec.stop_token_ids)
        got = result.tokens
        if dtype == "float32":
            assert got == expected
        else:
            # bfloat16 may pick the other token only where the plain top-2 margin is within rounding
            for i, (g, e) in enumerate(zip(got, expected)):
                if g != e:
                    assert margins[i] < 0.05, (i, margins[i])
                    break
        assert result.usage.prompt_tokens == len(prompt)
    alone = model.generate(prompts[1], options)
    if dtype == "float32":
        assert alone == results[1].tokens  # batch or alone: the same tokens
    streamed = []
    done = []
    model.generate(prompts[1], options, models_b200.CallbackStream(streamed.append, done.append, done.append))
    assert streamed == alone and len(done) == 1 and done[0].completion_tokens == len(alone)
    assert list(model.stream(prompts[1], options)) == alone
    abandoned = model.stream(prompts[1], options)  # read two tokens, then drop the iterator: the generation stops
    assert [next(abandoned), next(abandoned)] == alone[:2]
    abandoned.close()
    assert model.engine.cache.slots.held == 0
    errors = []
    model.generate([], options, models_b200.CallbackStream(on_error=errors.append))
    assert len(errors) == 1 and "empty" in str(errors[0])
    model.engine.cache.check()
    assert model.engine.cache.slots.held == 0
    model.close()
    model.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_graphs_matches_plain(cuda_device, folders, dtype):
    """Three prompt tokens, then 200 tokens one at a time across several cache pages, in a batch with
    a second sequence that ends early; decode steps replay CUDA graphs."""
    import models_b200

    name = "B"
    vocab = TINY[name]["vocab_size"]
    model = models_b200.load_model(folders[name], dtype=dtype, max_batch=2, context=256)
    engine = model.engine
    a, b = random_tokens(vocab, 203, 1), random_tokens(vocab, 40, 2)
    ea, eb = plain_logits(folders[name], a), plain_logits(folders[name], b)
    sa, sb = engine.open_slot(), engine.open_slot()
    from models_b200.engine import StepEntry

    out = engine.step([StepEntry(sa, a[:3], [2]), StepEntry(sb, b[:10], [9])])
    assert scaled_error(out[0], ea[2]) < TOLERANCE[dtype] and scaled_error(out[1], eb[9]) < TOLERANCE[dtype]
    for i in range(200):
        if i < 30:
            out = engine.decode([sa, sb], [a[3 + i], b[10 + i]])
            assert scaled_error(out[1], eb[10 + i]) < TOLERANCE[dtype], ("b", i)
            if i == 29:
                engine.release_slot(sb)
        else:
            out = engine.decode([sa], [a[3 + i]])
        assert scaled_error(out[0], ea[3 + i]) < TOLERANCE[dtype], ("a", i)
    assert engine.decode_graphs is not None and sorted(size for size, _ in engine.decode_graphs.captured) == [1, 2]
    engine.release_slot(sa)
    engine.cache.check()


def test_graph_decoding_across_a_context_class(cuda_device, tmp_path):
    """A sequence grows from 2,040 to 2,060 positions while it decodes with CUDA graphs: past 2,048 its
    keys are split over more blocks than a cluster holds, which takes a capture of its own; every
    step's logits are compared with the plain implementation."""
    import models_b200
    from models_b200.engine import StepEntry
    from models_b200.kernels import ops
    from tiny import TINY_B

    raw = dict(TINY_B, max_position_embeddings=4096)
    folder = make_folder(raw, seed=77, tmp_path=tmp_path, std=0.08)
    tokens = random_tokens(raw["vocab_size"], 2061, 5)
    expected = plain_logits(folder, tokens)
    model = models_b200.load_model(folder, dtype="bfloat16", max_batch=1, context=2112)
    engine = model.engine
    slot = engine.open_slot()
    out = engine.step([StepEntry(slot, tokens[:2040], [2039])])
    assert scaled_error(out[0], expected[2039]) < TOLERANCE["bfloat16"]
    for i in range(2040, 2061):
        out = engine.decode([slot], [tokens[i]])
        assert scaled_error(out[0], expected[i]) < TOLERANCE["bfloat16"], i
    spans = {capture.span for capture in engine.decode_graphs.captured.values()}
    assert spans == {ops.decode_span(2041), ops.decode_span(2049)} == {2048, 4096}
    assert ops.decode_splits(1, raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], 2049) > 8
    engine.release_slot(slot)
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_prompt_steps_replayed_from_captures_match_plain(cuda_device, folders, name, dtype):
    """Batches of unequal prompts, one after another so that slots are used again; from the third
    step of a class on, the step is a replayed capture with empty sequences and spare rows as
    padding.  Every wanted row is compared with the plain implementation, and a prompt that
    arrives in two pieces continues on what the first piece left."""
    import models_b200
    from models_b200.engine import StepEntry

    vocab = TINY[name]["vocab_size"]
    model = models_b200.load_model(folders[name], dtype=dtype, max_batch=4, context=128)
    engine = model.engine
    assert engine.prompt_graphs is not None
    seed = 0
    for round_ in range(6):
        lengths = [(5, 9, 4), (11, 3, 8), (7, 7, 7, 1), (12, 2, 9), (2, 25, 4), (19, 6, 5)][round_]  # 17 to 32 tokens
        prompts = []
        for n in lengths:
            seed += 1
            prompts.append(random_tokens(vocab, n, 100 + seed))
        slots = [engine.open_slot() for _ in prompts]
        # the last row of every prompt, and where a row of logits is to spare the first prompt's first row
        wants = [[len(p) - 1] for p in prompts]
        if len(prompts) < 4:
            wants[0] = [0, len(prompts[0]) - 1]
        out = engine.step([StepEntry(s, p, w) for s, p, w in zip(slots, prompts, wants)])
        assert out.shape[0] == sum(len(w) for w in wants)
        if len(prompts) < 4:
            assert scaled_error(out[0], plain_logits(folders[name], prompts[0])[0]) < TOLERANCE[dtype], round_
            out = out[1:]
        for b, p in enumerate(prompts):
            assert scaled_error(out[b], plain_logits(folders[name], p)[-1]) < TOLERANCE[dtype], (round_, b)
        # the first sequence goes on with four more tokens, alone
        more = random_tokens(vocab, 4, 500 + round_)
        out2 = engine.step([StepEntry(slots[0], more, [3])])
        expected = plain_logits(folders[name], prompts[0] + more)
        assert scaled_error(out2[0], expected[-1]) < TOLERANCE[dtype], round_
        # what the first step returned was a copy: the second step did not rewrite it
        assert scaled_error(out[0], plain_logits(folders[name], prompts[0])[-1]) < TOLERANCE[dtype]
        for s in slots:
            engine.release_slot(s)
    engine.cache.check()
    captured = set(engine.prompt_graphs.captured)
    assert captured == {(4, 32, 2), (1, 16, 2)}, captured  # the classes that came up more than twice


def test_long_prompt_steps_replayed_from_captures_match_the_launched_ones(cuda_device, tmp_path):
    """Prompt steps of several hundred tokens (the larger classes of captures, many pages per sequence, two
    sequences of unequal length): the replayed step's logits against the same step launched kernel by kernel
    on an engine without captures, in bfloat16 bit for bit (the kernels and their launch shapes are the same),
    then a few decoded tokens on top."""
    import models_b200
    from models_b200.engine import StepEntry

    from tiny import MID, make_folder

    raw = MID["D"]  # heads of 64: the tcgen05 products and attention of a real prompt step
    folder = make_folder(raw, seed=41, tmp_path=tmp_path, std=0.03)
    vocab = raw["vocab_size"]
    fast = models_b200.load_model(folder, dtype="bfloat16", max_batch=2, context=1024)
    slow = models_b200.load_model(folder, dtype="bfloat16", max_batch=2, context=1024, cuda_graphs=False)
    for round_ in range(4):  # the third and fourth rounds are replays
        prompts = [random_tokens(vocab, 430 + 7 * round_, 900 + round_), random_tokens(vocab, 200 - 3 * round_, 950 + round_)]
        outs = []
        for model in (fast, slow):
            engine = model.engine
            slots = [engine.open_slot() for _ in prompts]
            rows = [engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])]
            for step in range(3):
                rows.append(engine.decode(slots, [5 + step, 9 + step]).clone())
            outs.append(torch.cat(rows))
            for s in slots:
                engine.release_slot(s)
        assert torch.equal(outs[0], outs[1]), round_
    assert any(tokens == 640 for _, tokens, _ in fast.engine.prompt_graphs.captured), fast.engine.prompt_graphs.captured
    fast.close()
    slow.close()


def test_prompt_captures_leave_large_and_unwanted_steps_alone(cuda_device, folders):
    """Steps beyond the largest class, steps that want no logits and steps that want more rows than
    they have sequences run launch by launch."""
    import models_b200
    from models_b200.engine import StepEntry
    from models_b200.engine.decode_graph import PROMPT_TOKENS

    name = "B"
    model = models_b200.load_model(folders[name], dtype="bfloat16", max_batch=2, context=1024)
    engine = model.engine
    graphs = engine.prompt_graphs
    slot = engine.open_slot()
    assert graphs.bucket([(slot, [1] * (PROMPT_TOKENS[-1] + 1), [0])]) is None
    assert graphs.bucket([(slot, [1] * 8, [])]) is None
    assert graphs.bucket([(slot, [1] * 8, [0, 1, 2])]) is None
    assert graphs.bucket([(slot, [1] * 8, [7])]) == (1, 16, 4)
    assert graphs.bucket([(slot, [1] * 17, [0])]) == (1, 32, 4)
    engine.release_slot(slot)


def test_graph_and_eager_decode_agree(cuda_device, folders):
    import models_b200
    from models_b200.engine import StepEntry

    name = "A"
    vocab = TINY[name]["vocab_size"]
    tokens = [random_tokens(vocab, 30, s) for s in range(3)]
    outs = []
    for graphs in (True, False):
        model = models_b200.load_model(folders[name], dtype="bfloat16", max_batch=4, context=128, cuda_graphs=graphs)
        engine = model.engine
        slots = [engine.open_slot() for _ in tokens]
        engine.step([StepEntry(s, t[:20], []) for s, t in zip(slots, tokens)])
        rows = []
        for i in range(20, 30):
            rows.append(engine.decode(slots, [t[i] for t in tokens]).clone())
        outs.append(torch.stack(rows))
    assert torch.equal(outs[0], outs[1])  # three live rows in a graph of four: padding changes nothing


def expected_draw(logits, previous, options, u):
    ids, probs = plain_llama.plain_candidates(logits, previous, options.temperature, options.top_k, options.top_p,
                                              options.repetition_penalty)
    total = np.float32(0)
    for p in probs:
        total += np.float32(p)
    target = np.float32(u) * total
    acc = np.float32(0)
    for i, p in zip(ids, probs):
        acc += np.float32(p)
        if acc >= target:
            return i, ids
    return ids[-1], ids


@pytest.mark.parametrize("vocab", [203, 5003])
def test_sampling_kernel_follows_the_reference_pipeline(cuda_device, vocab):
    from models_b200.sampling import BatchSampler, RequestSampling, SamplingOptions, philox_uniform

    g = torch.Generator().manual_seed(vocab)
    sampler = BatchSampler(vocab, "cuda:0")
    cases = [
        SamplingOptions(temperature=1.0, top_k=40, top_p=0.9, seed=1),
        SamplingOptions(temperature=0.7, top_k=5, top_p=1.0, seed=2),
        SamplingOptions(temperature=1.3, top_k=1000, top_p=0.5, seed=3),
        SamplingOptions(temperature=0.0, repetition_penalty=1.5, seed=4),
        SamplingOptions(temperature=0.9, top_k=vocab, top_p=1.0, seed=5),
        SamplingOptions(temperature=1.0, top_k=12, top_p=0.8, repetition_penalty=1.3, seed=6),
        SamplingOptions(temperature=0.0, seed=7),
    ]
    prompt = [int(t) for t in torch.randint(0, vocab, (25,), generator=g)] + [3, 3, 3]
    requests = [RequestSampling(o, prompt) for o in cases]
    first_arrays = {}
    for step in range(6):
        logits = torch.randn(len(cases), vocab, generator=g) * 3
        logits[:, 3] = 6.0  # a likely token that the history penalises three times
        logits[0, 10] = logits[0, 11] = logits[0, 12] = 5.0  # ties inside the top-k
        draws = [r.draws for r in requests]
        got = sampler.sample(logits.cuda(), requests).tolist()
        for row, (o, r) in enumerate(zip(cases, requests)):
            if o.temperature == 0.0:
                adjusted = logits[row].clone()
                if o.repetition_penalty > 1.0:
                    for t in r.history:
                        adjusted[t] = adjusted[t] / o.repetition_penalty if adjusted[t] > 0 else adjusted[t] * o.repetition_penalty
                assert got[row] == plain_llama.plain_argmax(adjusted), (step, row)
                continue
            u = philox_uniform(r.seed, draws[row])
            want, ids = expected_draw(logits[row].numpy(), r.history or [], o, u)
            if min(o.top_k, vocab) > 1024:
                assert got[row] in ids, (step, row)  # drawn in id order: same distribution, other token
            else:
                assert got[row] == want, (step, row, got[row], want)
        BatchSampler.record(requests, got)
        # the history lives on the device: sent once, then grown there by the kernel itself
        for r in requests:
            if r.history is not None:
                if step == 0:
                    first_arrays[id(r)] = r.history_device
                assert r.history_device is first_arrays[id(r)]
                assert r.history_device[: len(r.history)].tolist() == r.history
    with pytest.raises(ValueError, match="top_p"):
        BatchSampler(5003, "cuda:0").check(SamplingOptions(top_k=2000, top_p=0.9))


@pytest.mark.parametrize("vocab", [5003, 128256])
def test_sampling_over_a_cluster_follows_the_reference_pipeline(cuda_device, vocab):
    """Rows that keep at most 1,024 candidates are spread over a cluster of blocks: the same pipeline,
    at vocabularies that do not divide by the cluster size, with more tokens tied at the k-th
    probability than fit (the lower ids go in; they straddle two blocks' id ranges), a penalised
    history, and greedy rows in the same batch."""
    from models_b200.sampling import BatchSampler, RequestSampling, SamplingOptions, philox_uniform

    g = torch.Generator().manual_seed(vocab + 1)
    sampler = BatchSampler(vocab, "cuda:0")
    cases = [
        SamplingOptions(temperature=1.0, top_k=40, top_p=0.9, seed=1),
        SamplingOptions(temperature=0.7, top_k=5, top_p=1.0, seed=2),
        SamplingOptions(temperature=1.3, top_k=1000, top_p=0.5, seed=3),
        SamplingOptions(temperature=0.0, repetition_penalty=1.5, seed=4),
        SamplingOptions(temperature=1.1, top_k=50, top_p=1.0, seed=5),    # the row with the wide tie
        SamplingOptions(temperature=1.0, top_k=12, top_p=0.8, repetition_penalty=1.3, seed=6),
        SamplingOptions(temperature=0.0, seed=7),
        SamplingOptions(temperature=0.6, top_k=1024, top_p=0.97, seed=8),
        SamplingOptions(temperature=0.9, top_k=vocab, top_p=1.0, seed=9),  # nothing cut: drawn in id order
    ]
    prompt = [int(t) for t in torch.randint(0, vocab, (25,), generator=g)] + [3, 3, 3]
    requests = [RequestSampling(o, prompt) for o in cases]
    boundary = -(-vocab // 8)  # the first id of the second block
    for step in range(5):
        logits = torch.randn(len(cases), vocab, generator=g) * 3
        logits[:, 3] = 6.0
        logits[0, 10] = logits[0, 11] = logits[0, 12] = 5.0
        logits[4, :] = torch.randn(vocab, generator=g).clamp(max=2.0)
        logits[4, 7:37] = 9.0 + torch.arange(30).float() * 0.01  # 30 clear leaders ...
        logits[4, boundary - 40:boundary + 40] = 8.0                # ... and 80 tokens tied for the other 20 places
        draws = [r.draws for r in requests]
        got = sampler.sample(logits.cuda(), requests).tolist()
        for row, (o, r) in enumerate(zip(cases, requests)):
            if o.temperature == 0.0:
                adjusted = logits[row].clone()
                if o.repetition_penalty > 1.0:
                    for t in r.history:
                        adjusted[t] = adjusted[t] / o.repetition_penalty if adjusted[t] > 0 else adjusted[t] * o.repetition_penalty
                assert got[row] == plain_llama.plain_argmax(adjusted), (step, row)
                continue
            u = philox_uniform(r.seed, draws[row])
            want, ids = expected_draw(logits[row].numpy(), r.history or [], o, u)
            if row == 4:
                assert sorted(ids)[30:] == list(range(boundary - 40, boundary - 20)), "the plain pipeline keeps the lower ids"
            if o.top_k >= vocab:
                # the walk in id order: the token at which the running mass (ascending id) reaches u
                p = torch.softmax(logits[row].double() / o.temperature, 0)
                running = torch.cumsum(p, 0)
                at = int(torch.searchsorted(running, torch.tensor(float(u), dtype=torch.float64)))
                assert abs(got[row] - at) <= 1 or abs(float(running[got[row]]) - float(u)) < 1e-4, (step, row, got[row], at)
                continue
            assert got[row] == want, (step, row, got[row], want)
        BatchSampler.record(requests, got)
    # the full-vocabulary draw follows the distribution
    few = torch.full((1, vocab), -40.0)
    few[0, [5, boundary + 3, vocab - 1]] = torch.tensor([1.0, 2.0, 0.0])
    request = RequestSampling(SamplingOptions(temperature=1.0, top_k=vocab, top_p=1.0, seed=21), [0])
    drawn = torch.tensor([sampler.sample(few.cuda(), [request]).item() for _ in range(600)])
    expected = torch.softmax(torch.tensor([1.0, 2.0, 0.0]), 0)
    seen = torch.tensor([(drawn == 5).sum(), (drawn == boundary + 3).sum(), (drawn == vocab - 1).sum()]).float() / 600
    assert float(seen.sum()) == 1.0 and float((seen - expected).abs().max()) < 0.07, seen


def test_sampling_is_reproducible_and_follows_the_distribution(cuda_device):
    import models_b200
    from models_b200.sampling import BatchSampler, RequestSampling, SamplingOptions

    vocab = 64
    logits = torch.zeros(1, vocab)
    logits[0, :4] = torch.tensor([2.0, 1.0, 0.0, -1.0])
    logits[0, 4:] = -30.0
    sampler = BatchSampler(vocab, "cuda:0")
    device_logits = logits.cuda()

    def run(seed, top_k):
        request = RequestSampling(SamplingOptions(temperature=1.0, top_k=top_k, top_p=1.0, seed=seed), [0])
        return [sampler.sample(device_logits, [request]).item() for _ in range(400)]

    first = run(11, 4)
    assert first == run(11, 4) and first != run(12, 4)
    expected = torch.softmax(logits[0, :4], 0)
    for top_k in (4, 64):
        draws = run(13, top_k)
        counts = torch.bincount(torch.tensor(draws), minlength=vocab)[:4].float() / len(draws)
        assert float((counts - expected).abs().max()) < 0.08, (top_k, counts)


def test_temperature_generation_through_the_entry_point(cuda_device, folders):
    import models_b200
    from models_b200 import SamplingOptions

    # float32: a row's logits are bit-identical alone and in a batch, so the draws are too
    model = models_b200.load_model(folders["B"], dtype="float32", max_batch=4, context=128)
    prompts = [[1, 2, 3], [9] * 20, [4]]
    options = SamplingOptions(temperature=0.8, top_k=20, top_p=0.95, max_tokens=10, seed=5, repetition_penalty=1.1)
    a = model.generate_batch(prompts, options)
    b = model.generate_batch(prompts, options)
    assert [r.tokens for r in a] == [r.tokens for r in b]  # same seed, same tokens
    c = model.generate_batch(prompts, SamplingOptions(temperature=0.8, top_k=20, top_p=0.95, max_tokens=10, seed=6))
    assert [r.tokens for r in a] != [r.tokens for r in c]
    assert all(0 <= t < 320 for r in a for t in r.tokens)
    assert model.generate_batch([[1, 2, 3]], options)[0].tokens == a[0].tokens  # alone or in a batch


def test_command_line_generate_and_profiles(cuda_device, folders, tmp_path):
    """`python -m models_b200 ...` as a user types it: generate (greedy, two prompts from a file), a
    random model folder, and the decode / sessions profiles."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(*args):
        proc = subprocess.run([sys.executable, "-m", "models_b200", *args], cwd=root, capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        return proc.stdout

    prompts = tmp_path / "prompts.txt"
    prompts.write_text("1 2 3 4\n9,8,7\n")
    report = json.loads(run("generate", "--model", str(folders["B"]), "--prompt-file", str(prompts), "--max-tokens", "6",
                            "--temperature", "0", "--dtype", "float32", "--context", "128"))
    assert len(report["results"]) == 2
    for prompt, result in zip(([1, 2, 3, 4], [9, 8, 7]), report["results"]):
        expected, _ = plain_greedy(folders["B"], prompt, 6, (5, 7))
        assert result["tokens"] == expected and result["prompt_tokens"] == len(prompt)
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY["A"]))
    made = run("random-model", "--config", str(config), "--seed", "4", "--output", str(tmp_path / "made")).strip()
    assert sorted(os.listdir(made)) == ["config.json", "model.safetensors"]
    out = json.loads(run("profile-decode", "--model", made, "--prompt-tokens", "20", "--measure-tokens", "8", "--context", "128"))
    assert out["measured_tokens"] == 8 and out["decode_tokens_per_second"] > 0
    out = json.loads(run("profile-sessions", "--model", made, "--prompt-tokens", "10", "--concurrency", "3", "--measure-steps",
                         "4", "--context", "128"))
    assert out["aggregate_tokens_per_second"] > 0
    out = json.loads(run("profile-prefill", "--config", str(config), "--random-seed", "1", "--prompt-tokens", "100",
                         "--context", "128", "--iterations", "2"))
    assert out["prompt_tokens"] == 100
    bad = subprocess.run([sys.executable, "-m", "models_b200", "generate", "--model", made, "--bogus", "1"], cwd=root,
                         capture_output=True, text=True)
    assert bad.returncode == 2 and "unknown option: --bogus" in bad.stderr


class OneAtATime:
    """An engine stepper without the step-ahead interface: the loop then waits for every step's ids."""

    def __init__(self, stepper):
        self._stepper = stepper
        self.page_size, self.capacity_tokens, self.max_positions = stepper.page_size, stepper.capacity_tokens, stepper.max_positions
        for name in ("open_slot", "release_slot", "check_options", "prefill", "decode", "sample"):
            setattr(self, name, getattr(stepper, name))


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stepping_ahead_of_the_sampled_ids_changes_no_token(cuda_device, folders, dtype, graphs):
    """The loop queues the next decode step before the last ids have reached the host.  The tokens,
    the finish reasons and the slots are those of the loop that waits, for greedy and for seeded
    sampling, with requests that stop early (a stop id chosen among the tokens they produce).  Two
    prompts span several cache pages and the six requests run as two batches, so pages grow and
    slots are used again inside the test.  In float32 (whose kernels give a row the same bits in any
    batch) the loop that waits runs on a second model without CUDA graphs, so a fault of the captures
    cannot hide in both arms; in both precisions the greedy tokens are checked against the plain
    implementation."""
    import models_b200
    from models_b200 import SamplingOptions
    from models_b200.engine.generation import GenerationLoop

    raw = TINY["B"]
    model = models_b200.load_model(folders["B"], dtype=dtype, max_batch=4, context=256, cuda_graphs=graphs)
    other = model
    if dtype == "float32" and graphs:
        other = models_b200.load_model(folders["B"], dtype=dtype, max_batch=4, context=256, cuda_graphs=False)
    prompts = [random_tokens(raw["vocab_size"], n, 70 + n) for n in (5, 1, 70, 12, 130, 31)]
    waiting = GenerationLoop(OneAtATime(other._stepper), 4, model.engine.spec.stop_token_ids)
    for base in (SamplingOptions(temperature=0.0, max_tokens=24),
                 SamplingOptions(temperature=0.9, top_k=30, top_p=0.9, max_tokens=24, seed=11),
                 SamplingOptions(temperature=0.7, top_k=12, top_p=1.0, max_tokens=24, seed=3, repetition_penalty=1.2)):
        free_run = waiting.run(prompts, base)
        if base.temperature == 0.0:
            for prompt, result in zip(prompts, free_run):
                expected, margins = plain_greedy(folders["B"], prompt, 24, model.engine.spec.stop_token_ids)
                for i, (g, e) in enumerate(zip(result.tokens, expected)):
                    if g != e:
                        assert dtype == "bfloat16" and margins[i] < 0.05, (len(prompt), i, margins[i])
                        break
        # stop ids that occur: the 4th token of one request, the 9th of another; and unequal limits
        stops = (free_run[0].tokens[3], free_run[2].tokens[8])
        options = [SamplingOptions(temperature=base.temperature, top_k=base.top_k, top_p=base.top_p, seed=base.seed,
                                   repetition_penalty=base.repetition_penalty, max_tokens=limit, stop_token_ids=stops)
                   for limit in (24, 3, 24, 1, 17, 10)]
        expected = waiting.run(prompts, options)
        got = model.generate_batch(prompts, options)
        assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in expected]
        assert any(r.finish_reason == "stop" for r in got)
        model.engine.cache.check()
        assert model.engine.cache.slots.held == 0
    model.close()


def test_graph_capture_is_not_disturbed_by_garbage_collection(cuda_device, folders):
    """Cyclic garbage that owns device and pinned memory, and a collector set to run at every
    opportunity: collecting it inside a graph capture would free memory there, which a capture
    forbids.  Generation (which captures at its first decode step) must work all the same."""
    import gc

    import models_b200
    from models_b200 import SamplingOptions

    class Knot:
        def __init__(self):
            self.me = self
            self.device = torch.empty(1 << 18, device="cuda")
            self.pinned = torch.empty(1 << 12).pin_memory()

    old_model = models_b200.load_model(folders["A"], dtype="bfloat16", max_batch=2, context=64)
    old_model.generate([1, 2, 3], SamplingOptions(temperature=0.0, max_tokens=4))
    old_model.me = old_model  # an older model that nobody closed, reachable only from itself
    del old_model
    for _ in range(20):
        Knot()
    before = gc.get_threshold()
    gc.set_threshold(1, 1, 1)
    try:
        model = models_b200.load_model(folders["B"], dtype="float32", max_batch=2, context=64)
        got = model.generate([4, 5, 6], SamplingOptions(temperature=0.0, max_tokens=6))
        assert gc.isenabled()
    finally:
        gc.set_threshold(*before)
    expected, _ = plain_greedy(folders["B"], [4, 5, 6], 6, model.engine.spec.stop_token_ids)
    assert got == expected
    model.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_next_request_goes_on_from_the_prefix_it_shares_with_the_last(cuda_device, folders, dtype):
    """Prompt-prefix reuse between requests (models-runtime/.../GenerationLoop.java:217-248): a second turn that
    repeats the first prompt and its reply runs only what is new; a prompt that parts from the kept sequence inside
    its first page cuts the sequence back across a page; tokens are those of the plain implementation each time."""
    import models_b200
    from models_b200 import PromptCacheMetrics, SamplingOptions

    raw = TINY["B"]
    model = models_b200.load_model(folders["B"], dtype=dtype, max_batch=4, context=256, reuse_prefix=True)
    stops = model.engine.spec.stop_token_ids
    options = SamplingOptions(temperature=0.0, max_tokens=12)

    def agrees(prompt, got):
        expected, margins = plain_greedy(folders["B"], prompt, 12, stops)
        if dtype == "float32":
            assert got == expected
        else:
            for i, (g, e) in enumerate(zip(got, expected)):
                if g != e:
                    assert margins[i] < 0.05, (i, margins[i])
                    break

    first = random_tokens(raw["vocab_size"], 100, 5)
    reply = model.generate(first, options)
    agrees(first, reply)
    assert model.last_prompt_cache == PromptCacheMetrics(True, 100, 0, 100)
    held = model.engine.cache.slots.held
    assert held == 1
    second = first + reply + random_tokens(raw["vocab_size"], 9, 6)
    agrees(second, model.generate(second, options))
    # all of the first prompt and every reply token that went through the model (the last one did not, unless a stop
    # token followed it)
    reused = model.last_prompt_cache.cache_read_input_tokens
    assert reused in (100 + len(reply) - 1, 100 + len(reply)) and model.last_prompt_cache.cache_write_input_tokens == len(second) - reused
    third = first[:30] + random_tokens(raw["vocab_size"], 50, 7)
    agrees(third, model.generate(third, options))
    assert model.last_prompt_cache == PromptCacheMetrics(True, 80, 30, 50)
    model.engine.cache.check()
    # a batch in between gives the kept sequence back; so does closing the model
    model.generate_batch([first[:20], first[:33]], options)
    assert model.engine.cache.slots.held == 0 and model.last_prompt_cache.supported is False
    agrees(third, model.generate(third, options))
    assert model.engine.cache.slots.held == 1
    model.close()
    assert model.engine.cache.slots.held == 0
    model.engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_waiting_requests_join_the_running_ones(cuda_device, folders, dtype):
    """Continuous batching through the entry point: five requests of unequal prompts and lengths, two at a time; a
    request that waits starts as soon as another ends (its prompt as a step of its own between two decode steps of
    the others, slots used again at once).  Every request's tokens are those of the plain implementation."""
    import models_b200
    from models_b200 import SamplingOptions

    raw = TINY["B"]
    model = models_b200.load_model(folders["B"], dtype=dtype, max_batch=2, context=256, continuous=True)
    stops = model.engine.spec.stop_token_ids
    prompts = [random_tokens(raw["vocab_size"], n, 50 + n) for n in (70, 5, 130, 33, 64)]
    lengths = [4, 19, 9, 3, 12]
    options = [SamplingOptions(temperature=0.0, max_tokens=n) for n in lengths]
    prefills = []
    real = model._stepper.prefill
    model._stepper.prefill = lambda slots, ps: (prefills.append([len(p) for p in ps]), real(slots, ps))[1]
    results = model.generate_batch(prompts, options)
    assert prefills[0] == [70, 5] and sorted(n for step in prefills[1:] for n in step) == [33, 64, 130]
    assert len(prefills) >= 3  # the others came in as places became free, not as one second batch
    for prompt, limit, result in zip(prompts, lengths, results):
        expected, margins = plain_greedy(folders["B"], prompt, limit, stops)
        if dtype == "float32":
            assert result.tokens == expected
        else:
            for i, (g, e) in enumerate(zip(result.tokens, expected)):
                if g != e:
                    assert margins[i] < 0.05, (i, margins[i])
                    break
        assert result.usage.prompt_tokens == len(prompt)
    model.engine.cache.check()
    assert model.engine.cache.slots.held == 0
    model.close()
