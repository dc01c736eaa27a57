"""Sampling options, the host twin of the device generator, and the command line's parsing (no GPU)."""

import pytest

from models_b200.cli import CliError, OPTIONS, parse_options, token_list
from models_b200.sampling import SamplingOptions, philox_uniform


def test_defaults_are_the_references():
    o = SamplingOptions.builder().build()
    assert (o.temperature, o.top_p, o.top_k, o.max_tokens, o.seed, o.repetition_penalty) == (1.0, 0.9, 40, 256, None, 1.0)
    assert SamplingOptions.builder().temperature(0).top_k(5).stop_token_id(3).build().stop_token_ids == (3,)


@pytest.mark.parametrize("kwargs,message", [
    ({"temperature": -0.1}, "temperature must be finite and >= 0"),
    ({"temperature": float("inf")}, "temperature"),
    ({"top_p": 0.0}, "topP must be finite and in"),
    ({"top_p": 1.5}, "topP"),
    ({"top_k": 0}, "topK must be > 0"),
    ({"max_tokens": 0}, "maxTokens must be > 0"),
    ({"repetition_penalty": 0.9}, "repetitionPenalty must be finite and >= 1.0"),
])
def test_option_checks(kwargs, message):
    with pytest.raises(ValueError, match=message):
        SamplingOptions(**kwargs)


def test_greedy_fast_path_condition():
    assert SamplingOptions(temperature=0.0).greedy
    assert not SamplingOptions(temperature=0.0, repetition_penalty=1.2).greedy
    assert not SamplingOptions(temperature=0.7).greedy


def test_philox_is_a_function_of_seed_and_counter():
    a = [philox_uniform(7, i) for i in range(200)]
    assert a == [philox_uniform(7, i) for i in range(200)]
    assert all(0.0 <= u < 1.0 for u in a)
    assert len(set(a)) > 190 and a != [philox_uniform(8, i) for i in range(200)]
    assert abs(sum(a) / len(a) - 0.5) < 0.08


def test_strict_name_value_parsing():
    allowed = OPTIONS["generate"]
    assert parse_options(["--model", "m", "--max-tokens", "4"], allowed) == {"model": "m", "max-tokens": "4"}
    with pytest.raises(CliError, match="pairs"):
        parse_options(["--model"], allowed)
    with pytest.raises(CliError, match="unknown option: --bogus"):
        parse_options(["--bogus", "1"], allowed)
    with pytest.raises(CliError, match="duplicate option: --model"):
        parse_options(["--model", "a", "--model", "b"], allowed)
    with pytest.raises(CliError, match="expected option"):
        parse_options(["model", "a"], allowed)
    assert token_list("1, 2 3", "--prompt") == [1, 2, 3]
    with pytest.raises(CliError):
        token_list("1,x", "--prompt")
