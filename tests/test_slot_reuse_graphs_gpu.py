"""Slots and pages that are used again while decode steps replay CUDA graphs.

A request that ends gives its slot and its pages back; the next request may get the same slot, at
the same row of the batch, with as many pages as the old one ended with -- but other pages, or the
same pages in another order.  Every sequence here spans several pages, so a page table that a
capture kept from the earlier tenant shows as wrong logits.  integrallis/models asks the same of
its own cache: reset and reuse reproduce results exactly
(backend-java/src/test/.../llama/LlamaForwardPassTest.java:1948-1969), and a batch equals each
request alone, cache included (:1573-1676).
"""

import pytest
import torch

from plain import plain_llama
from tiny import TINY_A, TINY_B, TOLERANCE, make_folder, plain_logits, random_tokens, scaled_error

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CONFIGS = {"A": dict(TINY_A, max_position_embeddings=512), "B": dict(TINY_B, max_position_embeddings=512)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("reuse_models")
    # wide weights: logits are spread, so greedy choices are no near-ties and a wrong page shows
    return {name: make_folder(raw, seed=41 + i, tmp_path=root, std=0.08) for i, (name, raw) in enumerate(CONFIGS.items())}


def plain_greedy(folder, prompt, max_tokens, stop_ids=()):
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


def assert_greedy(got, expected, margins, dtype, what):
    if dtype == "float32":
        assert got == expected, what
        return
    for i, (g, e) in enumerate(zip(got, expected)):
        if g != e:  # bfloat16 may pick the other token only where the plain top-2 margin is within rounding
            assert margins[i] < 0.05, (what, i, margins[i])
            return
    assert len(got) == len(expected), what


def decode_and_compare(engine, folder, slots, sequences, prompt_lengths, decode_counts, dtype, what):
    """Teacher-forced: the prompts in one step, then `decode_counts[i]` tokens of sequence i one at a
    time through Engine.decode; a sequence that has had its count is released at once.  Every row of
    logits is compared with the plain implementation."""
    from models_b200.engine import StepEntry

    expected = [plain_logits(folder, s) for s in sequences]
    out = engine.step([StepEntry(slot, s[:p], [p - 1]) for slot, s, p in zip(slots, sequences, prompt_lengths)])
    for i, p in enumerate(prompt_lengths):
        assert scaled_error(out[i], expected[i][p - 1]) < TOLERANCE[dtype], (what, "prompt", i)
    live = list(range(len(slots)))
    for step in range(max(decode_counts)):
        live = [i for i in live if step < decode_counts[i]]
        out = engine.decode([slots[i] for i in live], [sequences[i][prompt_lengths[i] + step] for i in live])
        for row, i in enumerate(live):
            err = scaled_error(out[row], expected[i][prompt_lengths[i] + step])
            assert err < TOLERANCE[dtype], (what, "decode step", step, "sequence", i, err)
        for i in live:
            if step + 1 == decode_counts[i]:
                engine.release_slot(slots[i])
        engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_the_same_long_prompt_twice(cuda_device, folders, name, dtype):
    """model.generate twice with one prompt of 100 tokens: the second call gets the first call's slot and
    its two pages, in the other order."""
    import models_b200
    from models_b200 import SamplingOptions

    model = models_b200.load_model(folders[name], dtype=dtype, max_batch=2, context=256)
    assert model.engine.decode_graphs is not None
    prompt = random_tokens(CONFIGS[name]["vocab_size"], 100, 3)
    options = SamplingOptions(temperature=0.0, max_tokens=20)
    expected, margins = plain_greedy(folders[name], prompt, 20, model.engine.spec.stop_token_ids)
    for call in range(3):
        assert_greedy(model.generate(prompt, options), expected, margins, dtype, f"call {call}")
    model.engine.cache.check()
    assert model.engine.cache.slots.held == 0
    model.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_batches_of_three_on_the_same_slots(cuda_device, folders, name, dtype):
    """Three sequences of two to four pages, then three others of the same page counts on the slots
    and pages the first three gave back (an odd count keeps the middle slot at its row), then a batch
    whose requests end at different steps followed by one more."""
    import models_b200

    vocab = CONFIGS[name]["vocab_size"]
    model = models_b200.load_model(folders[name], dtype=dtype, max_batch=4, context=320)
    engine = model.engine
    rounds = [
        ((70, 130, 100), (12, 12, 12)),
        ((70, 130, 100), (12, 12, 12)),   # the same page counts on recycled slots
        ((100, 66, 190), (5, 30, 17)),    # ends at different steps
        ((120, 70, 129, 10), (9, 9, 20, 70)),
        ((70,), (60,)),
    ]
    for r, (prompts, decodes) in enumerate(rounds):
        sequences = [random_tokens(vocab, p + d, 1000 * r + i) for i, (p, d) in enumerate(zip(prompts, decodes))]
        slots = [engine.open_slot() for _ in prompts]
        decode_and_compare(engine, folders[name], slots, sequences, prompts, decodes, dtype, f"round {r}")
    assert engine.cache.slots.held == 0 and all(g.pages.held == 0 for g in engine.cache.groups)
    assert {size for size, _ in engine.decode_graphs.captured} == {1, 2, 4}


@pytest.mark.parametrize("dtype", DTYPES)
def test_rewind_across_a_page_while_another_sequence_takes_it(cuda_device, folders, dtype):
    """A sequence decodes into its third page and is rewound into its second; the page it gave back goes
    to another sequence; both then decode from graphs.  The first one's third page is a new one."""
    import models_b200
    from models_b200.engine import StepEntry

    name = "B"
    vocab = CONFIGS[name]["vocab_size"]
    model = models_b200.load_model(folders[name], dtype=dtype, max_batch=2, context=320)
    engine = model.engine
    a = random_tokens(vocab, 140, 7)
    sa = engine.open_slot()
    engine.step([StepEntry(sa, a[:120], [])])
    ea = plain_logits(folders[name], a)
    for i in range(120, 135):  # into the third page (positions 128...)
        out = engine.decode([sa], [a[i]])
        assert scaled_error(out[0], ea[i]) < TOLERANCE[dtype], i
    engine.rewind(sa, 100)
    b = random_tokens(vocab, 90, 8)
    sb = engine.open_slot()
    engine.step([StepEntry(sb, b[:60], [])])  # takes the page the rewind freed
    a2 = a[:100] + random_tokens(vocab, 60, 9)
    ea2, eb = plain_logits(folders[name], a2), plain_logits(folders[name], b)
    for i in range(30):
        out = engine.decode([sa, sb], [a2[100 + i], b[60 + i]])
        assert scaled_error(out[0], ea2[100 + i]) < TOLERANCE[dtype], ("a", i)
        assert scaled_error(out[1], eb[60 + i]) < TOLERANCE[dtype], ("b", i)
    engine.release_slot(sb)
    for i in range(30, 60):
        out = engine.decode([sa], [a2[100 + i]])
        assert scaled_error(out[0], ea2[100 + i]) < TOLERANCE[dtype], ("a", i)
    engine.release_slot(sa)
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_pipeline_calls_after_reset_context(cuda_device, folders, dtype):
    """prefill / forward / reset_context / prefill / forward on the default sequence: the second
    context has the first one's slot and page count."""
    import models_b200

    name = "A"
    vocab = CONFIGS[name]["vocab_size"]
    model = models_b200.load_model(folders[name], dtype=dtype, max_batch=1, context=256)
    for call in range(3):
        tokens = random_tokens(vocab, 120, 50 + call)
        expected = plain_logits(folders[name], tokens)
        first = model.prefill(tokens[:100])
        assert scaled_error(first, expected[99]) < TOLERANCE[dtype], call
        kept = []
        for i in range(100, 120):
            kept.append(model.forward(tokens[i]))
        for i, row in enumerate(kept):  # every result is the caller's own: a later call does not rewrite it
            assert scaled_error(row, expected[100 + i]) < TOLERANCE[dtype], (call, i)
        model.reset_context()
    model.close()
