"""The plain implementation checked against hand-computable cases, mirroring integrallis/models' own
primitive tests (backend-java/src/test/.../ops/TensorOpsTest.java:40-69,1368-1455,1457-1605 and
ops/RotaryTableTest.java:29-101) and its structural equalities."""

import math
import os

import numpy as np
import pytest
import torch

from plain import plain_llama as P
from tiny import TINY_A, TINY_B, make_folder, random_tokens


def test_rms_norm_identity_and_weight():
    x = torch.tensor([[3.0, 4.0]])
    out = P.rms_norm(x, torch.ones(2), 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, x / rms)
    assert torch.allclose(P.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0), x / rms * torch.tensor([2.0, 0.5]))
    assert torch.allclose(P.rms_norm(torch.zeros(1, 4), torch.ones(4), 1e-5), torch.zeros(1, 4))


def test_linear_known_product():
    w = torch.tensor([[1.0, 2.0, 3.0], [0.0, -1.0, 1.0]])
    assert P.linear(torch.tensor([[1.0, 1.0, 1.0]]), w).tolist() == [[6.0, 0.0]]
    assert P.linear(torch.tensor([[1.0, 1.0, 1.0]]), w, torch.tensor([1.0, 1.0])).tolist() == [[7.0, 1.0]]


def test_swiglu_known_values():
    out = P.swiglu(torch.tensor([0.0, 1.0, -1.0]), torch.tensor([5.0, 2.0, 2.0]))
    assert out[0] == 0.0
    assert out[1] == pytest.approx(2.0 / (1 + math.exp(-1.0)), rel=1e-6)
    assert out[2] == pytest.approx(-2.0 / (1 + math.exp(1.0)), rel=1e-6)


def test_rope_position_zero_is_identity_and_norm_is_kept():
    freqs = P.rope_pair_frequencies(8, 10000.0)
    assert freqs[0] == 1.0 and freqs[1] == pytest.approx(10000.0 ** (-2 / 8), rel=1e-6)
    x = torch.randn(3, 2, 8, generator=torch.Generator().manual_seed(0))
    cos, sin = P.rope_cos_sin(torch.tensor([0, 0, 0]), freqs, None)
    assert torch.equal(P.rope_rotate_split_half(x, cos, sin), x)
    cos, sin = P.rope_cos_sin(torch.tensor([1, 17, 400]), freqs, None)
    rotated = P.rope_rotate_split_half(x, cos, sin)
    assert torch.allclose(rotated.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    # pair i is (x[i], x[i + 4]): rotating by angle 1 * freq_0 = 1 rad
    v = torch.zeros(1, 1, 8)
    v[0, 0, 0] = 1.0
    c1, s1 = P.rope_cos_sin(torch.tensor([1]), freqs, None)
    r = P.rope_rotate_split_half(v, c1, s1)
    assert r[0, 0, 0] == pytest.approx(math.cos(1.0), rel=1e-6) and r[0, 0, 4] == pytest.approx(math.sin(1.0), rel=1e-6)


def test_rope_divisors_and_frequency_scale():
    freqs = P.rope_pair_frequencies(4, 100.0)
    plain_c, _ = P.rope_cos_sin(torch.tensor([6]), freqs, None)
    halved_c, _ = P.rope_cos_sin(torch.tensor([12]), freqs, torch.tensor([2.0, 2.0]))
    scaled_c, _ = P.rope_cos_sin(torch.tensor([12]), freqs, None, frequency_scale=0.5)
    assert torch.allclose(plain_c, halved_c) and torch.allclose(plain_c, scaled_c)


def test_llama3_divisors_have_three_bands():
    s = TINY_B["rope_scaling"]
    freqs = P.rope_pair_frequencies(32, 500000.0)
    d = P.llama3_pair_divisors(freqs, s["factor"], s["low_freq_factor"], s["high_freq_factor"],
                               s["original_max_position_embeddings"])
    assert d[0] == 1.0 and d[-1] == 8.0
    middle = [float(v) for v in d if 1.0 < v < 8.0]
    assert middle and middle == sorted(middle)
    wavelengths = 2 * math.pi / freqs.double()
    assert all((w < 16) == (v == 1.0) for w, v in zip(wavelengths.tolist(), d.tolist()))


def test_attention_one_key_uniform_and_window():
    q = torch.randn(4, 2, 8, generator=torch.Generator().manual_seed(1))
    k = torch.zeros(4, 1, 8)
    v = torch.arange(4.0).reshape(4, 1, 1).expand(4, 1, 8).contiguous()
    out = P.causal_gqa_attention(q, k, v).reshape(4, 2, 8)
    # equal scores: position t averages values 0..t
    assert torch.allclose(out[:, 0, 0], torch.tensor([0.0, 0.5, 1.0, 1.5]))
    windowed = P.causal_gqa_attention(q, k, v, window=2).reshape(4, 2, 8)
    assert torch.allclose(windowed[:, 1, 0], torch.tensor([0.0, 0.5, 1.5, 2.5]))
    # consecutive query heads share a kv head: head / (heads / kv_heads)
    k2 = torch.randn(4, 2, 8, generator=torch.Generator().manual_seed(2))
    v2 = torch.randn(4, 2, 8, generator=torch.Generator().manual_seed(3))
    q4 = torch.randn(4, 4, 8, generator=torch.Generator().manual_seed(4))
    both = P.causal_gqa_attention(q4, k2, v2).reshape(4, 4, 8)
    first = P.causal_gqa_attention(q4[:, :2], k2[:, :1], v2[:, :1]).reshape(4, 2, 8)
    assert torch.allclose(both[:, :2], first)


def test_prefix_of_a_sequence_gives_the_same_logits(tmp_path):
    """Causality: the logits at a position do not depend on later tokens (the reference's
    'prefill == token at a time', backend-java/src/test/.../LlamaForwardPassTest.java:461-486)."""
    for raw in (TINY_A, TINY_B):
        folder = make_folder(raw, 3, tmp_path / raw["model_type"] / str(raw["hidden_size"]))
        config, weights = P.read_model_folder(folder)
        tokens = random_tokens(raw["vocab_size"], 20, 0)
        whole = P.forward(config, weights, tokens)
        assert whole.shape == (20, raw["vocab_size"])
        for n in (1, 7, 19):
            assert torch.allclose(P.forward(config, weights, tokens[:n]), whole[:n], atol=1e-6)
        assert not torch.allclose(whole[3], whole[4])
        double = P.forward(config, weights, tokens, dtype=torch.float64)
        assert float((double - whole.double()).abs().max()) < 1e-5


def test_golden_logits_of_the_plain_implementation():
    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "plain_tiny_logits.npz"))
    from golden.make_golden import compute

    for key, value in compute().items():
        assert np.allclose(golden[key], value, atol=1e-6), key


def test_plain_sampling_candidates():
    logits = [1.0, 3.0, 3.0, 0.0, 2.0]
    ids, probs = P.plain_candidates(logits, [], 1.0, 3, 1.0, 1.0)
    assert ids == [1, 2, 4]  # ties to the lower id
    ids, _ = P.plain_candidates(logits, [], 1.0, 5, 0.5, 1.0)
    assert ids == [1, 2]  # the token that crosses top_p is kept
    ids, _ = P.plain_candidates(logits, [1, 1], 1.0, 1, 1.0, 2.0)
    assert ids == [2]  # token 1 was penalised twice: 3 / 2 / 2
    assert P.plain_argmax([1.0, 5.0, 5.0]) == 1
