"""The generation loop's decisions, with a scripted stepper in place of a model (no GPU).
The rules are integrallis/models' (models-runtime/.../GenerationLoop.java:250-279; its own tests:
models-runtime/src/test/.../GenerationLoopTest.java:92-133,189-236)."""

import pytest

from models_b200.engine.generation import GenerationLoop
from models_b200.sampling import SamplingOptions


class ScriptedStepper:
    """Each request 'generates' the tokens of its script, found by its prompt's first id."""

    page_size = 64
    max_positions = 4096

    def __init__(self, scripts, capacity_tokens=64 * 64, max_slots=64):
        self.scripts = scripts
        self.capacity_tokens = capacity_tokens
        self.free = list(range(max_slots - 1, -1, -1))
        self.held = {}  # slot -> [script key, tokens seen]
        self.calls = []

    def open_slot(self):
        slot = self.free.pop()
        self.held[slot] = None
        return slot

    def release_slot(self, slot):
        assert slot in self.held, "released twice"
        del self.held[slot]
        self.free.append(slot)

    def check_options(self, options):
        pass

    def prefill(self, slots, prompts):
        self.calls.append(("prefill", list(slots), [list(p) for p in prompts]))
        for s, p in zip(slots, prompts):
            self.held[s] = [p[0], 0]
        return list(slots)

    def decode(self, slots, tokens):
        self.calls.append(("decode", list(slots), list(tokens)))
        for s, t in zip(slots, tokens):
            key, n = self.held[s]
            assert t == self.scripts[key][n], "the token fed back is the one sampled"
            self.held[s][1] += 1
        return list(slots)

    def sample(self, logits, requests):
        return [self.scripts[self.held[s][0]][self.held[s][1]] for s in logits]


EOS = 99


def test_stops_at_eos_without_emitting_it_and_counts_usage():
    stepper = ScriptedStepper({1: [10, 11, 12, EOS, 13]})
    loop = GenerationLoop(stepper, 4, [EOS])
    result = loop.run([[1, 2, 3]], SamplingOptions(temperature=0.0, max_tokens=50))[0]
    assert result.tokens == [10, 11, 12] and result.finish_reason == "stop"
    assert (result.usage.prompt_tokens, result.usage.completion_tokens) == (3, 3)
    assert [c[0] for c in stepper.calls] == ["prefill", "decode", "decode", "decode"]
    assert not stepper.held


def test_max_tokens_and_the_last_token_is_not_fed_back():
    stepper = ScriptedStepper({1: [10, 11, 12, 13, 14]})
    result = GenerationLoop(stepper, 4, [EOS]).run([[1]], SamplingOptions(temperature=0.0, max_tokens=3))[0]
    assert result.tokens == [10, 11, 12] and result.finish_reason == "length"
    assert [c[0] for c in stepper.calls] == ["prefill", "decode", "decode"]  # 3 tokens, 2 model runs after prefill


def test_any_stop_id_ends_and_request_stop_ids_add_to_the_models():
    stepper = ScriptedStepper({1: [10, 55, 11], 2: [10, 77, 11]})
    loop = GenerationLoop(stepper, 4, [55])
    a, b = loop.run([[1], [2]], [SamplingOptions(temperature=0.0), SamplingOptions(temperature=0.0, stop_token_ids=(77,))])
    assert a.tokens == [10] and b.tokens == [10] and a.finish_reason == b.finish_reason == "stop"


def test_unequal_prompts_start_together_and_shorter_requests_end_earlier():
    scripts = {1: [10, EOS], 2: [20, 21, 22, 23, EOS], 3: [30, 31, EOS]}
    stepper = ScriptedStepper(scripts)
    streamed = []
    results = GenerationLoop(stepper, 8, [EOS]).run(
        [[1, 0, 0, 0, 0], [2], [3, 0]], SamplingOptions(temperature=0.0, max_tokens=10),
        on_token=lambda i, t: streamed.append((i, t)))
    assert [r.tokens for r in results] == [[10], [20, 21, 22, 23], [30, 31]]
    kinds = [(c[0], len(c[1])) for c in stepper.calls]
    assert kinds == [("prefill", 3), ("decode", 3), ("decode", 2), ("decode", 1), ("decode", 1)]
    assert [t for i, t in streamed if i == 1] == [20, 21, 22, 23]  # in token order per request
    assert not stepper.held


def test_batches_follow_one_another_and_slots_are_used_again():
    scripts = {i: [100 + i, EOS] for i in range(1, 8)}
    stepper = ScriptedStepper(scripts, max_slots=3)
    results = GenerationLoop(stepper, 3, [EOS]).run([[i] for i in range(1, 8)], SamplingOptions(temperature=0.0))
    assert [r.tokens for r in results] == [[100 + i] for i in range(1, 8)]
    prefills = [c for c in stepper.calls if c[0] == "prefill"]
    assert [len(c[1]) for c in prefills] == [3, 3, 1]
    assert all(set(c[1]) <= {0, 1, 2} for c in prefills)


def test_cache_budget_splits_batches_and_refuses_what_never_fits():
    stepper = ScriptedStepper({1: [5] * 200, 2: [6] * 200}, capacity_tokens=4 * 64)
    loop = GenerationLoop(stepper, 8, [EOS])
    # each request may grow to 100 + 100 - 1 positions = 4 pages: one per batch
    assert loop.plan_batches([[1] * 100, [2] * 100], [100, 100]) == [[0], [1]]
    assert loop.plan_batches([[1] * 10, [2] * 10], [100, 100]) == [[0, 1]]
    with pytest.raises(ValueError, match="cache pages"):
        loop.run([[1] * 300], SamplingOptions(temperature=0.0, max_tokens=10))


def test_empty_prompt_and_mismatched_options_are_refused_before_anything_runs():
    stepper = ScriptedStepper({})
    loop = GenerationLoop(stepper, 2, [EOS])
    with pytest.raises(ValueError, match="prompt must not be empty"):
        loop.run([[]], SamplingOptions())
    with pytest.raises(ValueError, match="2 prompts but 1"):
        loop.run([[1], [2]], [SamplingOptions()])
    assert stepper.calls == []


def test_context_limit_caps_the_generated_tokens():
    stepper = ScriptedStepper({1: list(range(10, 40))})
    stepper.max_positions = 8
    result = GenerationLoop(stepper, 2, [EOS]).run([[1, 0, 0, 0, 0]], SamplingOptions(temperature=0.0, max_tokens=20))[0]
    # positions 5, 6, 7 take three generated tokens; the fourth is sampled but never stored
    assert len(result.tokens) == 4 and result.finish_reason == "length"


def test_a_failing_step_gives_the_slots_back():
    class Failing(ScriptedStepper):
        def decode(self, slots, tokens):
            raise RuntimeError("boom")

    stepper = Failing({1: [10, 11], 2: [20, 21]})
    with pytest.raises(RuntimeError, match="boom"):
        GenerationLoop(stepper, 4, [EOS]).run([[1], [2]], SamplingOptions(temperature=0.0))
    assert not stepper.held


class AheadStepper(ScriptedStepper):
    """The same scripted model with the two-halves interface: ids that are 'still on the device'
    until result() is called, and a decode step that takes them from there."""

    class Pending:
        def __init__(self, values, log):
            self.values, self.log, self.count = values, log, len(values)

        def result(self):
            self.log.append(("result",))
            return self.values

    def sample_start(self, logits, requests):
        # rows of requests that have just ended may still be among the logits; their ids are never read
        values = [self.scripts[self.held[s][0]][self.held[s][1]] if s in self.held else -1 for s in logits]
        return self.Pending(values, self.calls)

    def decode_pending(self, slots, pending, rows):
        return self.decode(slots, [pending.values[i] for i in rows])

    def decode(self, slots, tokens):
        # a step ahead may carry a stop token for a request that is about to end: the script allows it
        self.calls.append(("decode", list(slots), list(tokens)))
        for s, t in zip(slots, tokens):
            key, n = self.held[s]
            assert t == self.scripts[key][n], "the token fed back is the one sampled"
            self.held[s][1] += 1
        return list(slots)


def test_the_loop_that_runs_a_step_ahead_decides_the_same():
    scripts = {1: [10, 11, 12, EOS, 13], 2: [20, EOS, 5, 5, 5, 5, 5], 3: [30, 31, 32, 33, 34, 35, 36], 4: [EOS, 1, 1, 1],
               5: [50, 51, 77, 52, 53, 54, 55]}
    prompts = [[1, 7], [2], [3, 3, 3], [4], [5, 5]]
    options = [SamplingOptions(temperature=0.0, max_tokens=6), SamplingOptions(temperature=0.0, max_tokens=6),
               SamplingOptions(temperature=0.0, max_tokens=4), SamplingOptions(temperature=0.0, max_tokens=1),
               SamplingOptions(temperature=0.0, max_tokens=6, stop_token_ids=(77,))]
    seen = {}
    for kind in (ScriptedStepper, AheadStepper):
        stepper = kind(scripts)
        emitted = []
        results = GenerationLoop(stepper, 3, [EOS]).run(prompts, options, on_token=lambda i, t: emitted.append((i, t)))
        seen[kind] = ([(r.tokens, r.finish_reason, r.usage.prompt_tokens, r.usage.completion_tokens) for r in results], emitted)
        assert not stepper.held and len(stepper.free) == 64 and len(set(stepper.free)) == 64
    assert seen[ScriptedStepper] == seen[AheadStepper]
    assert [r[0] for r in seen[AheadStepper][0]] == [[10, 11, 12], [20], [30, 31, 32, 33], [], [50, 51]]
    # the step ahead is queued before the ids are read, and never for a request at its limit
    calls = AheadStepper(scripts)
    GenerationLoop(calls, 3, [EOS]).run([[3, 3, 3]], SamplingOptions(temperature=0.0, max_tokens=3))
    kinds = [c[0] for c in calls.calls]
    assert kinds == ["prefill", "decode", "result", "decode", "result", "result"]


def test_a_failing_step_ahead_gives_the_slots_back():
    class Failing(AheadStepper):
        def decode_pending(self, slots, pending, rows):
            raise RuntimeError("boom")

    stepper = Failing({1: [10, 11], 2: [20, 21]})
    with pytest.raises(RuntimeError, match="boom"):
        GenerationLoop(stepper, 4, [EOS]).run([[1], [2]], SamplingOptions(temperature=0.0))
    assert not stepper.held


# ------------------------------------------------------------------ prompt-prefix reuse between requests
# (the cases of models-runtime/src/test/.../GenerationLoopTest.java:563-617, and what batching adds to them)

class RewindableStepper(ScriptedStepper):
    """Keeps, per slot, the tokens it holds; every request 'generates' token 7."""

    def __init__(self, **more):
        super().__init__({}, **more)
        self.tokens = {}
        self.prefills, self.rewinds, self.releases = [], [], 0
        self.refuse_rewind = False

    def open_slot(self):
        slot = super().open_slot()
        self.tokens[slot] = []
        return slot

    def release_slot(self, slot):
        super().release_slot(slot)
        del self.tokens[slot]
        self.releases += 1

    def rewind(self, slot, length):
        if self.refuse_rewind:
            raise ValueError("this cache cannot be cut back")
        assert 0 <= length <= len(self.tokens[slot])
        self.rewinds.append(length)
        del self.tokens[slot][length:]

    def prefill(self, slots, prompts):
        for s, p in zip(slots, prompts):
            self.prefills.append((len(self.tokens[s]), list(p)))
            self.tokens[s].extend(p)
        return list(slots)

    def decode(self, slots, tokens):
        for s, t in zip(slots, tokens):
            self.tokens[s].append(t)
        return list(slots)

    def sample(self, logits, requests):
        return [7 for _ in logits]


def test_the_longest_shared_prefix_is_kept_and_only_the_rest_runs():
    from models_b200.engine.generation import PromptCacheMetrics

    stepper = RewindableStepper()
    loop = GenerationLoop(stepper, 4, [EOS], reuse_prefix=True)
    one = SamplingOptions(temperature=0.0, max_tokens=1)
    assert loop.run([[2, 3, 4]], one)[0].tokens == [7]
    assert loop.last_prompt_cache == PromptCacheMetrics(True, 3, 0, 3)
    assert loop.run([[2, 3, 4, 5]], one)[0].tokens == [7]
    assert stepper.prefills == [(0, [2, 3, 4]), (3, [5])] and stepper.rewinds == [3]
    assert loop.last_prompt_cache == PromptCacheMetrics(True, 4, 3, 1) and loop.last_prompt_cache.hit_rate == 0.75
    assert len(stepper.held) == 1 and stepper.releases == 0  # the one sequence is still there, nothing was given back
    loop.drop_kept()
    assert not stepper.held


def test_nothing_shared_starts_from_nothing_and_an_identical_prompt_runs_its_last_token_again():
    from models_b200.engine.generation import PromptCacheMetrics

    stepper = RewindableStepper()
    loop = GenerationLoop(stepper, 4, [EOS], reuse_prefix=True)
    one = SamplingOptions(temperature=0.0, max_tokens=1)
    loop.run([[2, 3, 4]], one)
    loop.run([[5]], one)
    assert stepper.prefills == [(0, [2, 3, 4]), (0, [5])] and stepper.rewinds == [] and stepper.releases == 1
    assert loop.last_prompt_cache == PromptCacheMetrics(True, 1, 0, 1)
    loop.run([[5]], one)
    assert stepper.prefills[-1] == (0, [5]) and stepper.releases == 2  # a prompt of one token has no prefix to keep
    loop.run([[2, 3, 4]], one)
    loop.run([[2, 3, 4]], one)
    assert stepper.prefills[-1] == (2, [4]) and stepper.rewinds == [2]
    assert loop.last_prompt_cache == PromptCacheMetrics(True, 3, 2, 1)
    assert len(stepper.held) == 1


def test_generated_tokens_that_went_through_the_model_count_as_held():
    stepper = RewindableStepper()
    loop = GenerationLoop(stepper, 4, [EOS], reuse_prefix=True)
    result = loop.run([[2, 3]], SamplingOptions(temperature=0.0, max_tokens=3))[0]
    assert result.tokens == [7, 7, 7] and result.finish_reason == "length"
    slot = next(iter(stepper.tokens))
    assert stepper.tokens[slot] == [2, 3, 7, 7]  # the last emitted token never ran
    # the next turn of a conversation: the old prompt, the whole reply, and something new
    loop.run([[2, 3, 7, 7, 7, 9]], SamplingOptions(temperature=0.0, max_tokens=1))
    assert stepper.rewinds == [4] and stepper.prefills[-1] == (4, [7, 9])
    assert loop.last_prompt_cache.cache_read_input_tokens == 4


def test_batches_and_refused_rewinds_give_the_kept_sequence_back():
    from models_b200.engine.generation import PromptCacheMetrics

    stepper = RewindableStepper()
    loop = GenerationLoop(stepper, 4, [EOS], reuse_prefix=True)
    one = SamplingOptions(temperature=0.0, max_tokens=1)
    loop.run([[2, 3, 4]], one)
    loop.run([[2, 3, 4], [2, 3, 5]], one)  # two requests together: no reuse, and the kept slot goes back first
    assert not stepper.held and stepper.rewinds == []
    assert loop.last_prompt_cache == PromptCacheMetrics(False, 6, 0, 0)
    loop.run([[2, 3, 4]], one)
    stepper.refuse_rewind = True
    loop.run([[2, 3, 4, 5]], one)
    assert stepper.prefills[-1] == (0, [2, 3, 4, 5]) and len(stepper.held) == 1
    assert loop.last_prompt_cache == PromptCacheMetrics(True, 4, 0, 4)
    # a loop that was not asked to, or a stepper that cannot cut a sequence back, keeps nothing
    plain = GenerationLoop(RewindableStepper(), 4, [EOS])
    plain.run([[2, 3, 4]], one)
    assert not plain.stepper.held and plain.last_prompt_cache.supported is False
    assert GenerationLoop(ScriptedStepper({}), 4, [EOS], reuse_prefix=True).reuse_prefix is False
    with pytest.raises(ValueError):
        PromptCacheMetrics(False, 3, 1, 0)


def test_a_failing_step_gives_a_resumed_sequence_back_too():
    class Failing(RewindableStepper):
        fail = False

        def prefill(self, slots, prompts):
            if self.fail:
                raise RuntimeError("device lost")
            return super().prefill(slots, prompts)

    stepper = Failing()
    loop = GenerationLoop(stepper, 4, [EOS], reuse_prefix=True)
    one = SamplingOptions(temperature=0.0, max_tokens=1)
    loop.run([[2, 3, 4]], one)
    stepper.fail = True
    with pytest.raises(RuntimeError):
        loop.run([[2, 3, 4, 5]], one)
    assert not stepper.held
    stepper.fail = False
    loop.run([[2, 3, 4, 5]], one)
    assert stepper.prefills[-1] == (0, [2, 3, 4, 5])


def test_the_loop_that_runs_a_step_ahead_keeps_a_prefix_of_what_the_cache_holds():
    class AheadRewindable(RewindableStepper):
        """Generates 7, 7, then a stop token; ids are read a step late."""

        def script(self, slot):
            return [7, 7, EOS, 1, 1][self.generated[slot]]

        def open_slot(self):
            slot = super().open_slot()
            self.generated = getattr(self, "generated", {})
            self.generated[slot] = 0
            return slot

        def prefill(self, slots, prompts):
            for s in slots:
                self.generated[s] = 0
            return super().prefill(slots, prompts)

        def sample_start(self, logits, requests):
            return AheadStepper.Pending([self.script(s) if s in self.held else -1 for s in logits], self.calls)

        def decode_pending(self, slots, pending, rows):
            for s in slots:
                self.generated[s] += 1
            return self.decode(slots, [pending.values[i] for i in rows])

    stepper = AheadRewindable()
    loop = GenerationLoop(stepper, 4, [EOS], reuse_prefix=True)
    result = loop.run([[2, 3]], SamplingOptions(temperature=0.0, max_tokens=8))[0]
    assert result.tokens == [7, 7] and result.finish_reason == "stop"
    slot = next(iter(stepper.tokens))
    assert stepper.tokens[slot] == [2, 3, 7, 7, EOS]  # the step ahead carried the stop token through the model
    loop.run([[2, 3, 7, 7, 9, 9]], SamplingOptions(temperature=0.0, max_tokens=1))
    assert stepper.rewinds == [4] and stepper.prefills[-1] == (4, [9, 9])  # the stop token's position is cut off
    assert stepper.tokens[slot][:6] == [2, 3, 7, 7, 9, 9]


# ------------------------------------------------------------------ continuous batching

class JoiningStepper(ScriptedStepper):
    def concat(self, first, second):
        return list(first) + list(second)

    def prefill(self, slots, prompts):
        self.most_held = max(getattr(self, "most_held", 0), len(self.held))
        return super().prefill(slots, prompts)


class JoiningAheadStepper(AheadStepper, JoiningStepper):
    pass


@pytest.mark.parametrize("kind", [JoiningStepper, JoiningAheadStepper])
def test_a_waiting_request_joins_as_soon_as_another_ends(kind):
    scripts = {1: [10, EOS], 2: [20, 21, 22, 23, 24, 25, EOS], 3: [30, 31, EOS], 4: [40, EOS], 5: [50, 51, 52, EOS]}
    prompts = [[1, 0], [2], [3, 0, 0], [4], [5]]
    options = SamplingOptions(temperature=0.0, max_tokens=10)
    one_after_another = GenerationLoop(kind(scripts), 2, [EOS]).run(prompts, options)
    stepper = kind(scripts)
    emitted = []
    results = GenerationLoop(stepper, 2, [EOS], continuous=True).run(prompts, options, on_token=lambda i, t: emitted.append((i, t)))
    assert [(r.tokens, r.finish_reason, r.usage) for r in results] == [(r.tokens, r.finish_reason, r.usage) for r in one_after_another]
    assert [r.tokens for r in results] == [[10], [20, 21, 22, 23, 24, 25], [30, 31], [40], [50, 51, 52]]
    assert [t for i, t in emitted if i == 1] == [20, 21, 22, 23, 24, 25]
    prefills = [c[2] for c in stepper.calls if c[0] == "prefill"]
    # the first two start together; each of the others comes alone, in order, while request 1 is still running
    assert prefills == [[[1, 0], [2]], [[3, 0, 0]], [[4]], [[5]]]
    assert stepper.most_held <= 2 and not stepper.held and sorted(stepper.free) == list(range(64))
    kinds = [c[0] for c in stepper.calls if c[0] != "result"]
    assert kinds.index("prefill", 1) < len(kinds) - 1 and "decode" in kinds[kinds.index("prefill", 1):]  # decoding goes on after a join
    # without the option (or with a stepper that cannot put two steps' logits together) batches follow one another
    plain = kind(scripts)
    GenerationLoop(plain, 2, [EOS]).run(prompts, options)
    assert [c[2] for c in plain.calls if c[0] == "prefill"] == [[[1, 0], [2]], [[3, 0, 0], [4]], [[5]]]
    assert GenerationLoop(ScriptedStepper(scripts), 2, [EOS], continuous=True).continuous is False


def test_joiners_wait_for_pages_and_none_overtakes_another():
    # three pages in all; request 2 needs two of them, request 3 one: 3 could run beside 1, but waits behind 2
    scripts = {1: [10, 11, 12, EOS], 2: [20, EOS], 3: [30, EOS]}
    stepper = JoiningStepper(scripts, capacity_tokens=3 * 64)
    prompts = [[1] * 70, [2] * 100, [3]]
    results = GenerationLoop(stepper, 4, [EOS], continuous=True).run(prompts, SamplingOptions(temperature=0.0, max_tokens=8))
    assert [r.tokens for r in results] == [[10, 11, 12], [20], [30]]
    prefills = [[p[0] for p in c[2]] for c in stepper.calls if c[0] == "prefill"]
    assert prefills == [[1], [2, 3]]  # request 1 alone (2 pages of 3); when it ends, 2 and 3 start together
    assert not stepper.held


@pytest.mark.parametrize("kind", [JoiningStepper, JoiningAheadStepper])
def test_a_failing_join_gives_every_slot_back(kind):
    class Failing(kind):
        def prefill(self, slots, prompts):
            if any(p[0] == 3 for p in prompts):
                raise RuntimeError("boom")
            return super().prefill(slots, prompts)

    stepper = Failing({1: [10, EOS], 2: [20, 21, 22, 23, EOS], 3: [30, EOS]})
    with pytest.raises(RuntimeError, match="boom"):
        GenerationLoop(stepper, 2, [EOS], continuous=True).run([[1], [2], [3]], SamplingOptions(temperature=0.0, max_tokens=8))
    assert not stepper.held and sorted(stepper.free) == list(range(64))
