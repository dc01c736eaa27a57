"""The layer sizes of the benchmark model (Llama 3.2 1B: width 2048, 32 query and 8 key/value heads of
64, feed-forward 8192, vocabulary 128,256, llama3 rope scaling by 32), two layers of them, random
weights: the bfloat16 path that bench.py times against the float32 path of the same engine.

The plain implementation is too slow for these sizes beyond a short prompt, so it anchors the
float32 path once (40 tokens), and the float32 path -- whose kernels give a row the same bits in any
batch -- is the oracle for everything else: a whole prompt of 300 and of 2,048 tokens, the last 32
tokens one by one, and decoding at 1, 8 and 64 sequences.  Reported for every cut: the largest
scaled error and how often the greedy token agrees; where it does not, the float32 top-2 margin has
to be within the error bound (a near-tie that rounding may turn), never beyond it.  The reference's
own form of this test is equality of every fast path with its plainest path
(backend-java/src/test/.../llama/LlamaForwardPassTest.java:602-1570).
"""

import pytest
import torch

from plain import plain_llama
from tiny import TOLERANCE, random_tokens, scaled_error

pytestmark = pytest.mark.gpu

SIZES_1B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
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
SEED = 5
VOCAB = SIZES_1B["vocab_size"]


@pytest.fixture(scope="module")
def engines(cuda_device):
    """The same random model -- bfloat16 weights drawn on the device, the same bits for both -- as a
    float32 engine (the weights widened, everything computed in 32-bit) and as the bfloat16 model that
    generation uses, CUDA graphs on."""
    import models_b200
    from models_b200.config import config_from_dict
    from models_b200.engine import Engine, parameter_requests
    from models_b200.weights import random_tensors

    spec = config_from_dict(SIZES_1B).model_spec()
    tensors = random_tensors(parameter_requests(spec), SEED, dtype=torch.bfloat16, device="cuda")
    exact = Engine(spec, tensors, "float32", max_tokens=64 * 320, max_sequence=2304)
    del tensors
    model = models_b200.load_model(config=SIZES_1B, seed=SEED, dtype="bfloat16", max_batch=64, context=2304)
    assert torch.equal(model.engine.model.embedding.weight.float(), exact.model.embedding.weight)
    yield exact, model.engine
    model.close()


def compare(got, expected, what, report):
    """Rows of bfloat16-path logits against float32-path logits: scaled error within the bfloat16
    tolerance; the greedy token may differ only where the float32 top-2 margin is inside the bound."""
    got, expected = got.float().cpu(), expected.float().cpu()
    assert got.shape == expected.shape, (what, got.shape, expected.shape)
    size = float(expected.abs().max())
    worst, agree = 0.0, 0
    for row in range(expected.shape[0]):
        err = float((got[row] - expected[row]).abs().max()) / size
        worst = max(worst, err)
        top2 = torch.topk(expected[row], 2)
        if int(got[row].argmax()) == int(top2.indices[0]):
            agree += 1
        else:
            margin = float(top2.values[0] - top2.values[1])
            assert margin <= 2 * TOLERANCE["bfloat16"] * size, (what, row, "greedy token differs at a margin of", margin)
    report.append(f"{what}: rows {expected.shape[0]}, scaled error {worst:.2e}, greedy agreement {agree}/{expected.shape[0]}")
    assert worst < TOLERANCE["bfloat16"], (what, worst)


def test_the_float32_path_agrees_with_the_plain_implementation_at_these_widths(engines):
    from models_b200.engine import StepEntry, parameter_requests
    from models_b200.weights import random_tensors

    exact, _ = engines
    weights = {name: t.cpu() for name, t in random_tensors(parameter_requests(exact.spec), SEED, dtype=torch.bfloat16,
                                                            device="cuda").items()}
    tokens = random_tokens(VOCAB, 40, 1)
    expected = plain_llama.forward(SIZES_1B, weights, tokens)
    slot = exact.open_slot()
    got = exact.step([StepEntry(slot, tokens, list(range(40)))])
    exact.release_slot(slot)
    assert scaled_error(got, expected) < TOLERANCE["float32"]


def test_bfloat16_against_float32_whole_prompts_and_one_by_one(engines):
    from models_b200.engine import StepEntry

    exact, fast = engines
    report = []
    for length, places in ((300, [0, 63, 64, 150, 299]), (2048, [0, 1000, 2047])):
        tokens = random_tokens(VOCAB, length, length)
        outs = []
        for engine in (exact, fast):
            slot = engine.open_slot()
            outs.append(engine.step([StepEntry(slot, tokens, places)]))
            engine.release_slot(slot)
        compare(outs[1], outs[0], f"whole prompt of {length}", report)
    tokens = random_tokens(VOCAB, 300, 7)
    slot = exact.open_slot()
    expected = exact.step([StepEntry(slot, tokens, list(range(267, 300)))])
    exact.release_slot(slot)
    slot = fast.open_slot()
    rows = [fast.step([StepEntry(slot, tokens[:268], [267])])]
    for i in range(268, 300):
        rows.append(fast.decode([slot], [tokens[i]]).clone())
    fast.release_slot(slot)
    compare(torch.cat(rows), expected, "last 32 one by one", report)
    print("\n".join(report))


@pytest.mark.parametrize("batch", [1, 8, 64])
def test_bfloat16_against_float32_decoding(engines, batch):
    """`batch` sequences of unequal prompts (20 to 200 tokens) in one step, then six tokens each."""
    import numpy as np

    from models_b200.engine import StepEntry

    exact, fast = engines
    rng = np.random.default_rng(batch)
    lengths = [int(n) for n in rng.integers(20, 201, size=batch)]
    steps = 6
    sequences = [random_tokens(VOCAB, n + steps, 100 * batch + i) for i, n in enumerate(lengths)]
    report = []
    outs = {}
    for name, engine in (("exact", exact), ("fast", fast)):
        slots = [engine.open_slot() for _ in range(batch)]
        rows = [engine.step([StepEntry(s, seq[:n], [n - 1]) for s, seq, n in zip(slots, sequences, lengths)])]
        for step in range(steps):
            rows.append(engine.decode(slots, [seq[n + step] for seq, n in zip(sequences, lengths)]).clone())
        for s in slots:
            engine.release_slot(s)
        outs[name] = rows
    compare(outs["fast"][0], outs["exact"][0], f"batch {batch}: prompts", report)
    compare(torch.cat(outs["fast"][1:]), torch.cat(outs["exact"][1:]), f"batch {batch}: {steps} decode steps", report)
    assert {size for size, _ in fast.decode_graphs.captured} >= {batch}
    print("\n".join(report))
