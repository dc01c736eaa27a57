"""Each part alone, models put together from specs that no architecture here uses (a window in one
layer only, a layer named twice, a run that reads another run's cache), and a toy mixer with state
of its own that is defined here and registered without touching the package."""

import math

import pytest
import torch

from plain import plain_llama as P
from tiny import TOLERANCE, scaled_error

pytestmark = pytest.mark.gpu


def _specs(hidden=80, heads=4, kv_heads=2, head_dim=16, inter=136, vocab=203, windows=(None, 24), theta=5000.0,
           eps=2e-6, schedule=None):
    from models_b200.config.specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedFeedForwardSpec, HeadSpec, ModelSpec,
                                          NormSpec, RopeSpec, ScheduleEntry)

    rope = RopeSpec(rotary_dim=head_dim, theta=theta, pairing="half")
    layers = []
    for i, window in enumerate(windows):
        p = f"layers.{i}."
        layers.append(BlockSpec(
            mixer=AttentionSpec(hidden, heads, kv_heads, head_dim, 1.0 / math.sqrt(head_dim), rope, window, False,
                                {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}),
            feed_forward=GatedFeedForwardSpec(hidden, inter, "silu", False, {"gate": p + "gate", "up": p + "up", "down": p + "down"}),
            mixer_norm=NormSpec(hidden, eps, {"weight": p + "norm1"}),
            feed_forward_norm=NormSpec(hidden, eps, {"weight": p + "norm2"})))
    schedule = schedule or [ScheduleEntry(i) for i in range(len(layers))]
    return ModelSpec("test-only", vocab, hidden, 512, EmbeddingSpec(vocab, hidden, 1.0, {"weight": "embed"}), tuple(layers),
                     tuple(schedule), NormSpec(hidden, eps, {"weight": "final_norm"}), HeadSpec(vocab, hidden, False, {"weight": "head"}))


def _plain_forward(spec, tensors, tokens):
    """The plain functions put together the way `spec` says, whole sequence, float32."""
    w = {k: v.float() for k, v in tensors.items()}
    T = len(tokens)
    x = P.embed(w["embed"], torch.tensor(tokens))
    kv_of_run = {}
    for run, entry in enumerate(spec.schedule):
        layer = spec.layers[entry.layer]
        m, names = layer.mixer, layer.mixer.weights
        xn = P.rms_norm(x, w[layer.mixer_norm.weights["weight"]], layer.mixer_norm.eps)
        freqs = P.rope_pair_frequencies(m.position.rotary_dim, m.position.theta)
        cos, sin = P.rope_cos_sin(torch.arange(T), freqs, None)
        q = P.rope_rotate_split_half(P.linear(xn, w[names["q"]]).reshape(T, m.num_heads, m.head_dim), cos, sin)
        if entry.cache_from is None:
            k = P.rope_rotate_split_half(P.linear(xn, w[names["k"]]).reshape(T, m.num_kv_heads, m.head_dim), cos, sin)
            v = P.linear(xn, w[names["v"]]).reshape(T, m.num_kv_heads, m.head_dim)
            kv_of_run[run] = (k, v)
        else:
            k, v = kv_of_run[entry.cache_from]
        x = x + P.linear(P.causal_gqa_attention(q, k, v, m.window), w[names["o"]])
        f = layer.feed_forward.weights
        xn = P.rms_norm(x, w[layer.feed_forward_norm.weights["weight"]], layer.feed_forward_norm.eps)
        x = x + P.feed_forward(xn, w[f["gate"]], w[f["up"]], w[f["down"]])
    return P.linear(P.rms_norm(x, w["final_norm"], spec.final_norm.eps), w["head"])


def _engine(spec, dtype, seed=1, max_tokens=1024):
    from models_b200.engine import Engine, parameter_requests
    from models_b200.weights import random_tensors

    tensors = random_tensors(parameter_requests(spec), seed, std=0.05)
    return Engine(spec, tensors, dtype, max_tokens), tensors


def _tokens(n, vocab, seed):
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_different_mixers_in_different_layers(cuda_device, dtype):
    """Layer 0 sees all keys, layer 1 a window of 24: two cache groups, each with storage of its own;
    whole prompts, then token by token across the window's edge and across pages."""
    from models_b200.engine import StepEntry

    spec = _specs(windows=(None, 24))
    engine, tensors = _engine(spec, dtype)
    assert len(engine.cache.groups) == 2
    tokens = _tokens(150, spec.vocab_size, 0)
    expected = _plain_forward(spec, tensors, tokens)
    slot = engine.open_slot()
    out = engine.step([StepEntry(slot, tokens[:100], list(range(100)))])
    assert scaled_error(out, expected[:100]) < TOLERANCE[dtype]
    for i in range(100, 150):
        out = engine.step([StepEntry(slot, [tokens[i]], [0])])
        assert scaled_error(out[0], expected[i]) < TOLERANCE[dtype], i
    full, windowed = engine.cache.groups
    assert sum(p >= 0 for p in full.tables[slot]) == 3 and sum(p >= 0 for p in windowed.tables[slot]) == 2
    engine.release_slot(slot)
    engine.cache.check()


@pytest.mark.parametrize("head_dim,heads,kv_heads", [(64, 4, 2), (128, 3, 1)])
def test_a_windowed_layer_at_the_head_sizes_of_the_tcgen05_kernels(cuda_device, head_dim, heads, kv_heads):
    """The same mix -- one layer sees everything, the other a window of 100 -- at head sizes 64 and 128
    in bfloat16, where a prompt takes the tcgen05 attention and the folded q/k/v product: a prompt in
    two pieces (the second on top of cached positions whose early pages the window group has already
    given back), then token by token across a page boundary."""
    from models_b200.engine import StepEntry

    spec = _specs(hidden=256, heads=heads, kv_heads=kv_heads, head_dim=head_dim, inter=328, vocab=331, windows=(None, 100))
    engine, tensors = _engine(spec, "bfloat16", seed=7, max_tokens=2048)
    assert len(engine.cache.groups) == 2
    tokens = _tokens(470, spec.vocab_size, 5)
    expected = _plain_forward(spec, tensors, tokens)
    slot = engine.open_slot()
    out = engine.step([StepEntry(slot, tokens[:260], [0, 99, 100, 259])])
    assert scaled_error(out, expected[[0, 99, 100, 259]]) < TOLERANCE["bfloat16"]
    out = engine.step([StepEntry(slot, tokens[260:440], [0, 60, 179])])  # 180 more on top of 260 cached
    assert scaled_error(out, expected[[260, 320, 439]]) < TOLERANCE["bfloat16"]
    full, windowed = engine.cache.groups
    assert sum(p >= 0 for p in full.tables[slot]) == 7 and sum(p >= 0 for p in windowed.tables[slot]) <= 3
    for i in range(440, 470):
        out = engine.step([StepEntry(slot, [tokens[i]], [0])])
        assert scaled_error(out[0], expected[i]) < TOLERANCE["bfloat16"], i
    engine.release_slot(slot)
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_names_a_layer_twice_and_shares_a_cache(cuda_device, dtype):
    from models_b200.config.specs import ScheduleEntry
    from models_b200.engine import StepEntry

    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_from=1)]
    spec = _specs(windows=(None, None), schedule=schedule, heads=3, kv_heads=1, head_dim=32, hidden=96)
    engine, tensors = _engine(spec, dtype, seed=2)
    assert engine.cache.groups[0].runs == [0, 1, 2]  # run 3 owns no storage
    a, b = _tokens(70, spec.vocab_size, 1), _tokens(9, spec.vocab_size, 2)
    ea, eb = _plain_forward(spec, tensors, a), _plain_forward(spec, tensors, b)
    sa, sb = engine.open_slot(), engine.open_slot()
    out = engine.step([StepEntry(sa, a[:60], [0, 59]), StepEntry(sb, b[:5], [4])])
    assert scaled_error(out[0], ea[0]) < TOLERANCE[dtype] and scaled_error(out[1], ea[59]) < TOLERANCE[dtype]
    assert scaled_error(out[2], eb[4]) < TOLERANCE[dtype]
    for i in range(4):
        out = engine.step([StepEntry(sa, [a[60 + i]], [0]), StepEntry(sb, [b[5 + i]], [0])])
        assert scaled_error(out[0], ea[60 + i]) < TOLERANCE[dtype] and scaled_error(out[1], eb[5 + i]) < TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parts_alone(cuda_device, dtype):
    """Norm, position tables, feed-forward and the attention mixer, each built from its spec alone."""
    from models_b200.cache import KvCache
    from models_b200.config.specs import RopeScalingSpec, RopeSpec
    from models_b200.engine.batch import build_step_batch
    from models_b200.parts import RunContext, Runtime, build_part
    from models_b200.weights import random_tensors

    runtime = Runtime(torch.device("cuda:0"), dtype, max_positions=300)
    compute = runtime.compute_dtype
    spec = _specs(windows=(None,), hidden=72, heads=6, kv_heads=2, head_dim=48, inter=200)
    layer = spec.layers[0]
    tol = TOLERANCE[dtype]
    g = torch.Generator().manual_seed(5)

    # norm (with the add that precedes it)
    norm = build_part("norm", layer.mixer_norm, runtime)
    tensors = random_tensors({r.name: r for r in norm.parameters()}, 1)
    norm.load(tensors)
    x = torch.randn(9, 72, generator=g)
    delta = torch.randn(9, 72, generator=g).to(compute)
    xd = x.cuda()
    out = norm.forward(xd, delta.cuda())
    gain = tensors["layers.0.norm1"].float()
    assert scaled_error(out, P.rms_norm(x + delta.float(), gain, layer.mixer_norm.eps)) < tol
    assert scaled_error(xd, x + delta.float()) < 1e-6

    # position tables: llama3 scaling, linear scaling, plain
    for scaling in (None, RopeScalingSpec("linear", 4.0), RopeScalingSpec("llama3", 8.0, 1.0, 4.0, 64)):
        rope = build_part("position", RopeSpec(32, 500000.0, "half", scaling), runtime)
        freqs = P.rope_pair_frequencies(32, 500000.0)
        divisors, scale = None, 1.0
        if scaling is not None and scaling.kind == "llama3":
            divisors = P.llama3_pair_divisors(freqs, 8.0, 1.0, 4.0, 64)
        if scaling is not None and scaling.kind == "linear":
            scale = 0.25
        cos, sin = P.rope_cos_sin(torch.arange(300), freqs, divisors, scale)
        assert torch.equal(rope.cos.cpu(), cos) and torch.equal(rope.sin.cpu(), sin)

    # feed-forward
    ffn = build_part("feed_forward", layer.feed_forward, runtime)
    tensors = random_tensors({r.name: r for r in ffn.parameters()}, 2, std=0.1)
    ffn.load(tensors)
    xn = torch.randn(9, 72, generator=g).to(compute)
    w = {k: v.float() for k, v in tensors.items()}
    expected = P.feed_forward(xn.float(), w["layers.0.gate"], w["layers.0.up"], w["layers.0.down"])
    assert scaled_error(ffn.forward(xn.cuda()), expected) < tol

    # attention mixer over a cache of its own: a prompt of 70, then 3 single tokens
    mixer = build_part("mixer", layer.mixer, runtime)
    tensors = random_tensors({r.name: r for r in mixer.parameters()}, 3, std=0.1)
    mixer.load(tensors)
    w = {k: v.float() for k, v in tensors.items()}
    cache = KvCache([mixer.kv_request()], [None], 256)
    cache.allocate_storage(lambda shape: torch.zeros(shape, dtype=compute, device="cuda:0"))
    group, k_pool, v_pool = cache.pools(0)
    run = RunContext(0, group, k_pool, v_pool, True, None)
    slot = cache.open_slot()
    T = 73
    xn = torch.randn(T, 72, generator=g).to(compute)
    m = layer.mixer
    cos, sin = P.rope_cos_sin(torch.arange(T), P.rope_pair_frequencies(48, m.position.theta), None)
    q = P.rope_rotate_split_half(P.linear(xn.float(), w["layers.0.q"]).reshape(T, 6, 48), cos, sin)
    k = P.rope_rotate_split_half(P.linear(xn.float(), w["layers.0.k"]).reshape(T, 2, 48), cos, sin)
    v = P.linear(xn.float(), w["layers.0.v"]).reshape(T, 2, 48)
    expected = P.linear(P.causal_gqa_attention(q, k, v), w["layers.0.o"])
    rows = []
    for begin, end in ((0, 70), (70, 71), (71, 72), (72, 73)):
        cache.append([(slot, end - begin)])
        batch = build_step_batch(cache, [(slot, [0] * (end - begin), [])], "cuda:0")
        rows.append(mixer.forward(xn[begin:end].cuda(), batch, run))
        cache.commit([(slot, end - begin)])
    assert scaled_error(torch.cat(rows), expected) < tol


class RunningMeanMixer:
    """A toy mixer with state of its own and no keys or values: it returns, for every token, the mean
    of all inputs of its sequence so far, times a learned gain.  Per sequence it keeps the running sum
    and the count in the state area.  It exists only in this test."""

    def __init__(self, spec, runtime):
        self.spec, self.runtime = spec, runtime

    def parameters(self):
        from models_b200.weights import ParamRequest

        return [ParamRequest(self.spec.weights["gain"], (self.spec.hidden_size,), "gain")]

    def load(self, tensors):
        self.gain = self.runtime.vector(tensors[self.spec.weights["gain"]])

    def kv_request(self):
        return None

    def state_request(self):
        from models_b200.cache import StateRequest

        return StateRequest((self.spec.hidden_size + 1,), torch.float32)

    def forward(self, xn, batch, run):
        out = torch.empty_like(xn)
        slots = batch.slots.tolist()
        cu = batch.cu_q.tolist()
        for b in range(batch.num_sequences):
            state = run.state[slots[b]]
            rows = xn[cu[b]:cu[b + 1]].float()
            sums = state[:-1] + rows.cumsum(0)
            counts = state[-1] + torch.arange(1, rows.shape[0] + 1, device=xn.device)
            out[cu[b]:cu[b + 1]] = (sums / counts[:, None] * self.gain).to(xn.dtype)
            state[:-1] = sums[-1]
            state[-1] = counts[-1]
        return out


def test_a_toy_mixer_with_its_own_state_registers_builds_and_steps(cuda_device):
    from dataclasses import dataclass, field

    from models_b200.config.specs import BlockSpec, ModelSpec, ScheduleEntry
    from models_b200.engine import StepEntry
    from models_b200.parts import register_part, unregister_part

    @dataclass(frozen=True)
    class RunningMeanSpec:
        hidden_size: int
        weights: dict = field(default_factory=dict, hash=False, compare=False)
        kind: str = "test_running_mean"

    register_part("mixer", "test_running_mean", RunningMeanMixer)
    try:
        base = _specs(windows=(None, None))
        toy = BlockSpec(RunningMeanSpec(base.hidden_size, {"gain": "layers.1.mean_gain"}), base.layers[1].feed_forward,
                        base.layers[1].mixer_norm, base.layers[1].feed_forward_norm)
        spec = ModelSpec(base.architecture, base.vocab_size, base.hidden_size, base.max_positions, base.embedding,
                         (base.layers[0], toy), (ScheduleEntry(0), ScheduleEntry(1)), base.final_norm, base.head)
        engine, tensors = _engine(spec, "float32", seed=4, max_tokens=512)
        assert engine.state.of_run(1).shape == (engine.cache.max_slots + 1, base.hidden_size + 1)
        assert engine.state.of_run(0) is None and len(engine.cache.groups) == 1

        def plain(tokens):
            w = {k: v.float() for k, v in tensors.items()}
            T = len(tokens)
            x = P.embed(w["embed"], torch.tensor(tokens))
            l0 = spec.layers[0]
            m = l0.mixer
            xn = P.rms_norm(x, w["layers.0.norm1"], l0.mixer_norm.eps)
            cos, sin = P.rope_cos_sin(torch.arange(T), P.rope_pair_frequencies(m.head_dim, m.position.theta), None)
            q = P.rope_rotate_split_half(P.linear(xn, w["layers.0.q"]).reshape(T, m.num_heads, m.head_dim), cos, sin)
            k = P.rope_rotate_split_half(P.linear(xn, w["layers.0.k"]).reshape(T, m.num_kv_heads, m.head_dim), cos, sin)
            v = P.linear(xn, w["layers.0.v"]).reshape(T, m.num_kv_heads, m.head_dim)
            x = x + P.linear(P.causal_gqa_attention(q, k, v), w["layers.0.o"])
            x = x + P.feed_forward(P.rms_norm(x, w["layers.0.norm2"], l0.feed_forward_norm.eps), w["layers.0.gate"],
                                   w["layers.0.up"], w["layers.0.down"])
            xn = P.rms_norm(x, w["layers.1.norm1"], toy.mixer_norm.eps)
            x = x + xn.cumsum(0) / torch.arange(1, T + 1)[:, None] * w["layers.1.mean_gain"]
            x = x + P.feed_forward(P.rms_norm(x, w["layers.1.norm2"], toy.feed_forward_norm.eps), w["layers.1.gate"],
                                   w["layers.1.up"], w["layers.1.down"])
            return P.linear(P.rms_norm(x, w["final_norm"], spec.final_norm.eps), w["head"])

        for round_index in range(2):  # the second round takes the first one's slots: the state starts at zero again
            a, b = _tokens(20, spec.vocab_size, 10 + round_index), _tokens(7, spec.vocab_size, 20 + round_index)
            ea, eb = plain(a), plain(b)
            sa, sb = engine.open_slot(), engine.open_slot()
            out = engine.step([StepEntry(sa, a[:12], [11]), StepEntry(sb, b[:3], [2])])
            assert scaled_error(out[0], ea[11]) < 1e-4 and scaled_error(out[1], eb[2]) < 1e-4
            for i in range(4):
                out = engine.step([StepEntry(sa, [a[12 + i]], [0]), StepEntry(sb, [b[3 + i]], [0])])
                assert scaled_error(out[0], ea[12 + i]) < 1e-4 and scaled_error(out[1], eb[3 + i]) < 1e-4
            engine.release_slot(sa)
            engine.release_slot(sb)
    finally:
        unregister_part("mixer", "test_running_mean")


class LinearAnglePosition:
    """A toy position encoding: pair i of position p is rotated by p * step * (i + 1).  It offers what
    the attention mixer asks of any position part: rotary_dim, interleaved, and cos / sin tables."""

    def __init__(self, spec, runtime):
        self.spec, self.runtime = spec, runtime
        self.rotary_dim, self.interleaved = spec.rotary_dim, False
        angle = (torch.arange(max(1, runtime.max_positions), dtype=torch.float64)[:, None] * spec.step *
                 torch.arange(1, spec.rotary_dim // 2 + 1, dtype=torch.float64)[None, :])
        self.cos = torch.cos(angle).float().contiguous().to(runtime.device)
        self.sin = torch.sin(angle).float().contiguous().to(runtime.device)

    def parameters(self):
        return []

    def load(self, tensors):
        pass


class TopOneExperts:
    """A toy feed-forward with routing: router logits in 32-bit, the best expert's gated feed-forward
    for each token (the first of equal logits).  Plain tensor code: it shows the interface, not speed."""

    def __init__(self, spec, runtime):
        self.spec, self.runtime = spec, runtime

    def parameters(self):
        from models_b200.weights import ParamRequest

        s, n = self.spec, self.spec.weights
        out = [ParamRequest(n["router"], (s.experts, s.hidden_size))]
        for e in range(s.experts):
            out += [ParamRequest(n["gate"].format(e), (s.intermediate_size, s.hidden_size)),
                    ParamRequest(n["up"].format(e), (s.intermediate_size, s.hidden_size)),
                    ParamRequest(n["down"].format(e), (s.hidden_size, s.intermediate_size))]
        return out

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        self.router = rt.vector(tensors[n["router"]])  # read as 32-bit in both modes, like a norm's gain
        self.experts = [tuple(rt.matrix(tensors[n[k].format(e)]).float() for k in ("gate", "up", "down"))
                        for e in range(self.spec.experts)]

    def forward(self, xn):
        x = xn.float()
        choice = torch.argmax(x @ self.router.t(), dim=1)
        out = torch.zeros_like(x)
        for e, (gate, up, down) in enumerate(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                h = x[rows]
                out[rows] = (torch.nn.functional.silu(h @ gate.t()) * (h @ up.t())) @ down.t()
        return out.to(xn.dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_register_and_run(cuda_device, dtype):
    """Layer 0: the package's attention with a position encoding defined here; layer 1: the package's
    attention and a feed-forward with routing defined here.  Both are registered from outside, built
    from specs, loaded by tensor name and stepped (whole, then token by token) against plain code."""
    from dataclasses import dataclass, field, replace

    from models_b200.config.specs import BlockSpec, ModelSpec
    from models_b200.engine import StepEntry
    from models_b200.parts import register_part, unregister_part

    @dataclass(frozen=True)
    class LinearAngleSpec:
        rotary_dim: int
        step: float
        kind: str = "test_linear_angles"

    @dataclass(frozen=True)
    class TopOneSpec:
        hidden_size: int
        intermediate_size: int
        experts: int
        weights: dict = field(default_factory=dict, hash=False, compare=False)
        kind: str = "test_top1_experts"

    register_part("position", "test_linear_angles", LinearAnglePosition)
    register_part("feed_forward", "test_top1_experts", TopOneExperts)
    try:
        base = _specs(windows=(None, None))
        toy_position = LinearAngleSpec(base.layers[0].mixer.head_dim, 0.013)
        layer0 = replace(base.layers[0], mixer=replace(base.layers[0].mixer, position=toy_position))
        toy_ffn = TopOneSpec(base.hidden_size, 72, 3, {"router": "layers.1.router", "gate": "layers.1.expert{}.gate",
                                                        "up": "layers.1.expert{}.up", "down": "layers.1.expert{}.down"})
        layer1 = replace(base.layers[1], feed_forward=toy_ffn)
        spec = ModelSpec(base.architecture, base.vocab_size, base.hidden_size, base.max_positions, base.embedding,
                         (layer0, layer1), base.schedule, base.final_norm, base.head)
        engine, tensors = _engine(spec, dtype, seed=6, max_tokens=512)
        assert "layers.1.expert2.down" in tensors and "layers.1.router" in tensors

        def plain(tokens):
            w = {k: v.float() for k, v in tensors.items()}
            T = len(tokens)
            x = P.embed(w["embed"], torch.tensor(tokens))
            for i, layer in enumerate(spec.layers):
                m, names = layer.mixer, layer.mixer.weights
                xn = P.rms_norm(x, w[layer.mixer_norm.weights["weight"]], layer.mixer_norm.eps)
                if i == 0:
                    angle = (torch.arange(T, dtype=torch.float64)[:, None] * toy_position.step *
                             torch.arange(1, m.head_dim // 2 + 1, dtype=torch.float64)[None, :])
                    cos, sin = torch.cos(angle).float(), torch.sin(angle).float()
                else:
                    cos, sin = P.rope_cos_sin(torch.arange(T), P.rope_pair_frequencies(m.head_dim, m.position.theta), None)
                q = P.rope_rotate_split_half(P.linear(xn, w[names["q"]]).reshape(T, m.num_heads, m.head_dim), cos, sin)
                k = P.rope_rotate_split_half(P.linear(xn, w[names["k"]]).reshape(T, m.num_kv_heads, m.head_dim), cos, sin)
                v = P.linear(xn, w[names["v"]]).reshape(T, m.num_kv_heads, m.head_dim)
                x = x + P.linear(P.causal_gqa_attention(q, k, v), w[names["o"]])
                xn = P.rms_norm(x, w[layer.feed_forward_norm.weights["weight"]], layer.feed_forward_norm.eps)
                if i == 0:
                    f = layer.feed_forward.weights
                    x = x + P.feed_forward(xn, w[f["gate"]], w[f["up"]], w[f["down"]])
                else:
                    router_logits = xn @ w["layers.1.router"].t()
                    choice = torch.argmax(router_logits, dim=1)
                    top2 = torch.topk(router_logits, 2, dim=1).values
                    margins.append(top2[:, 0] - top2[:, 1])
                    delta = torch.zeros_like(x)
                    for t in range(T):
                        e = int(choice[t])
                        delta[t] = P.feed_forward(xn[t:t + 1], w[f"layers.1.expert{e}.gate"], w[f"layers.1.expert{e}.up"],
                                                  w[f"layers.1.expert{e}.down"])[0]
                    x = x + delta
            return P.linear(P.rms_norm(x, w["final_norm"], spec.final_norm.eps), w["head"])

        tokens = _tokens(40, spec.vocab_size, 31)
        margins = []
        expected = plain(tokens)
        # Routing is a discrete choice: where the two best router logits are closer than bfloat16's
        # rounding of the inputs can move them, either expert is a right answer and the row is not
        # compared (the routed layer is the last one, so such a row touches no other row).
        clear = margins[0] > (0.0 if dtype == "float32" else 0.02)
        assert int(clear.sum()) >= 30
        tol = max(TOLERANCE[dtype], 1e-4)
        slot = engine.open_slot()
        out = engine.step([StepEntry(slot, tokens[:30], list(range(30)))])
        assert scaled_error(out[clear[:30].cuda()], expected[:30][clear[:30]]) < tol
        for i in range(30, 40):
            out = engine.step([StepEntry(slot, [tokens[i]], [0])])
            if clear[i]:
                assert scaled_error(out[0], expected[i]) < tol, i
        engine.release_slot(slot)
    finally:
        unregister_part("position", "test_linear_angles")
        unregister_part("feed_forward", "test_top1_experts")


def test_missing_kind_and_cpu_tensors_fail_loudly(cuda_device):
    from models_b200.kernels import ops
    from models_b200.parts import Runtime, build_part

    with pytest.raises(ValueError, match="no mixer of kind 'nope'"):
        build_part("mixer", type("S", (), {"kind": "nope"})(), Runtime(torch.device("cuda:0"), "float32"))
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.swiglu(torch.zeros(2, 4))


class HalvedEvenLogitsHead:
    """A toy output head, defined here and registered from outside the package: the package's linear
    head, after which every even-numbered token's logit is halved.  It offers what the model asks of
    any head: parameters(), load(tensors, tied_to), forward(x, pending, norm, want_rows)."""

    def __init__(self, spec, runtime):
        from models_b200.parts.head import LinearHead

        self.spec, self.inner = spec, LinearHead(spec, runtime)

    def parameters(self):
        return self.inner.parameters()

    def load(self, tensors, tied_to=None):
        self.inner.load(tensors, tied_to)

    def forward(self, x, pending, norm, want_rows):
        logits = self.inner.forward(x, pending, norm, want_rows)
        logits[:, ::2] *= 0.5
        return logits


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_with_a_logit_epilogue_and_a_toy_head_from_outside(cuda_device, dtype):
    """The output head is a part like the others: its logit scale and softcap are fields of its spec,
    and another kind of head is registered without a change to the package."""
    import dataclasses

    from models_b200.engine import StepEntry
    from models_b200.parts import register_part, unregister_part

    base = _specs(windows=(None, None))
    tokens = _tokens(40, base.vocab_size, 3)
    capped = dataclasses.replace(base, head=dataclasses.replace(base.head, logit_scale=30.0, softcap=4.0))
    register_part("head", "test_halved_even", HalvedEvenLogitsHead)
    try:
        toy = dataclasses.replace(base, head=dataclasses.replace(base.head, kind="test_halved_even"))
        for spec, name in ((base, "plain"), (capped, "capped"), (toy, "toy")):
            engine, tensors = _engine(spec, dtype, seed=6)
            expected = _plain_forward(base, tensors, tokens)
            # the cap's slope is at most 1, so it passes an error on no larger than it was: errors are
            # measured against the size of the logits that go into the cap
            size = float(expected.abs().max()) * (30.0 if name == "capped" else 1.0)
            if name == "capped":
                expected = P.softcap_logits(expected * 30.0, 4.0)
                assert size > 8.0 and float(expected.abs().max()) > 3.9  # the cap bends these logits; it is not a no-op here
            if name == "toy":
                expected[:, ::2] *= 0.5
            slot = engine.open_slot()
            out = engine.step([StepEntry(slot, tokens[:30], [0, 29])])  # two wanted rows: the folded few-row path
            for row, place in enumerate((0, 29)):
                assert float((out[row].cpu() - expected[place]).abs().max()) < TOLERANCE[dtype] * size, (name, place)
            out = engine.step([StepEntry(slot, tokens[30:], list(range(10)))])  # ten rows: norm, then the product
            assert float((out.cpu() - expected[30:]).abs().max()) < TOLERANCE[dtype] * size, name
    finally:
        unregister_part("head", "test_halved_even")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_layer_observer_sees_the_stream_after_every_run(cuda_device, tmp_path, dtype):
    """DecoderModel.observer is called once per scheduled run with the float32 residual stream after
    it, for a whole prompt (the deltas still pending are added in) and for a decode step whose norms
    and residual adds ride inside the matrix products."""
    from models_b200.engine import StepEntry
    from models_b200.engine.loading import engine_from_folder
    from tiny import TINY_B, make_folder, random_tokens

    folder = make_folder(TINY_B, 17, tmp_path, std=0.05)
    config, weights = P.read_model_folder(folder)
    tokens = random_tokens(TINY_B["vocab_size"], 31, 2)
    _, hidden = P.forward(config, weights, tokens, return_hidden=True)
    engine = engine_from_folder(folder, dtype, 256)
    seen = []
    engine.model.observer = lambda run, x: seen.append((run, x))
    slot = engine.open_slot()
    engine.step([StepEntry(slot, tokens[:30], [29])])
    assert [run for run, _ in seen] == [0, 1, 2]
    for run, x in seen:
        assert x.dtype == torch.float32 and scaled_error(x, hidden[run][:30]) < TOLERANCE[dtype], run
    seen.clear()
    engine.step([StepEntry(slot, tokens[30:], [0])])
    assert [run for run, _ in seen] == [0, 1, 2]
    for run, x in seen:
        assert scaled_error(x[0], hidden[run][30]) < TOLERANCE[dtype], run
    engine.model.observer = None


class NarrowValueMixer:
    """A toy attention with keys of one size and values of another, defined here: one head, queries and
    keys of `key_dim`, values of `value_dim`, no rotation, plain torch arithmetic over its own pages.
    It shows that the cache gives a mixer keys and values of sizes of their own."""

    def __init__(self, spec, runtime):
        self.spec, self.runtime = spec, runtime

    def parameters(self):
        from models_b200.weights import ParamRequest

        s, n = self.spec, self.spec.weights
        return [ParamRequest(n["q"], (s.key_dim, s.hidden_size)), ParamRequest(n["k"], (s.key_dim, s.hidden_size)),
                ParamRequest(n["v"], (s.value_dim, s.hidden_size)), ParamRequest(n["o"], (s.hidden_size, s.value_dim))]

    def load(self, tensors):
        n = self.spec.weights
        self.w = {name: self.runtime.matrix(tensors[n[name]]).float() for name in ("q", "k", "v", "o")}

    def kv_request(self):
        from models_b200.cache import KvRequest

        return KvRequest(1, self.spec.key_dim, None, value_dim=self.spec.value_dim)

    def state_request(self):
        return None

    def forward(self, xn, batch, run):
        s = self.spec
        x = xn.float()
        q, k, v = x @ self.w["q"].t(), x @ self.w["k"].t(), x @ self.w["v"].t()
        assert run.k_pool.shape[1:] == (1, 64, s.key_dim) and run.v_pool.shape[1:] == (1, 64, s.value_dim)
        mapping = batch.groups[run.group].slot_mapping.long()
        keep = mapping >= 0
        run.k_pool.view(-1, s.key_dim)[mapping[keep]] = k[keep].to(run.k_pool.dtype)
        run.v_pool.view(-1, s.value_dim)[mapping[keep]] = v[keep].to(run.v_pool.dtype)
        out = torch.zeros(x.shape[0], s.value_dim, device=x.device)
        cu, lens, table = batch.cu_q.tolist(), batch.kv_lens.tolist(), batch.groups[run.group].block_table
        positions = batch.positions.tolist()
        for b in range(batch.num_sequences):
            where = torch.arange(lens[b], device=x.device)
            flat = table[b][where // 64].long() * 64 + where % 64
            keys, values = run.k_pool.view(-1, s.key_dim)[flat].float(), run.v_pool.view(-1, s.value_dim)[flat].float()
            for row in range(cu[b], cu[b + 1]):
                scores = (keys[: positions[row] + 1] @ q[row]) / math.sqrt(s.key_dim)
                out[row] = torch.softmax(scores, 0) @ values[: positions[row] + 1]
        return (out @ self.w["o"].t()).to(xn.dtype)


def test_a_toy_mixer_with_keys_and_values_of_different_sizes(cuda_device):
    from dataclasses import dataclass, field

    from models_b200.config.specs import BlockSpec, ModelSpec, ScheduleEntry
    from models_b200.engine import StepEntry
    from models_b200.parts import register_part, unregister_part

    @dataclass(frozen=True)
    class NarrowValueSpec:
        hidden_size: int
        key_dim: int
        value_dim: int
        weights: dict = field(default_factory=dict, hash=False, compare=False)
        kind: str = "test_narrow_value"

    register_part("mixer", "test_narrow_value", NarrowValueMixer)
    try:
        base = _specs(windows=(None, None))
        names = {n: f"layers.1.toy_{n}" for n in ("q", "k", "v", "o")}
        toy = BlockSpec(NarrowValueSpec(base.hidden_size, 24, 8, names), base.layers[1].feed_forward,
                        base.layers[1].mixer_norm, base.layers[1].feed_forward_norm)
        spec = ModelSpec(base.architecture, base.vocab_size, base.hidden_size, base.max_positions, base.embedding,
                         (base.layers[0], toy), (ScheduleEntry(0), ScheduleEntry(1)), base.final_norm, base.head)
        engine, tensors = _engine(spec, "float32", seed=8, max_tokens=512)
        assert len(engine.cache.groups) == 2  # the toy mixer's keys and values are a group of their own
        toy_group = engine.cache.groups[1]
        assert toy_group.keys.shape[-1] == 24 and toy_group.values.shape[-1] == 8

        def plain(tokens):
            w = {k: v.float() for k, v in tensors.items()}
            T = len(tokens)
            x = P.embed(w["embed"], torch.tensor(tokens))
            l0 = spec.layers[0]
            m = l0.mixer
            xn = P.rms_norm(x, w["layers.0.norm1"], l0.mixer_norm.eps)
            cos, sin = P.rope_cos_sin(torch.arange(T), P.rope_pair_frequencies(m.head_dim, m.position.theta), None)
            q = P.rope_rotate_split_half(P.linear(xn, w["layers.0.q"]).reshape(T, m.num_heads, m.head_dim), cos, sin)
            k = P.rope_rotate_split_half(P.linear(xn, w["layers.0.k"]).reshape(T, m.num_kv_heads, m.head_dim), cos, sin)
            v = P.linear(xn, w["layers.0.v"]).reshape(T, m.num_kv_heads, m.head_dim)
            x = x + P.linear(P.causal_gqa_attention(q, k, v), w["layers.0.o"])
            x = x + P.feed_forward(P.rms_norm(x, w["layers.0.norm2"], l0.feed_forward_norm.eps), w["layers.0.gate"],
                                   w["layers.0.up"], w["layers.0.down"])
            xn = P.rms_norm(x, w["layers.1.norm1"], toy.mixer_norm.eps)
            q, k, v = (P.linear(xn, w[names[n]]) for n in ("q", "k", "v"))
            scores = (q @ k.t()) / math.sqrt(24)
            scores = scores.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            x = x + P.linear(torch.softmax(scores, -1) @ v, w[names["o"]])
            x = x + P.feed_forward(P.rms_norm(x, w["layers.1.norm2"], toy.feed_forward_norm.eps), w["layers.1.gate"],
                                   w["layers.1.up"], w["layers.1.down"])
            return P.linear(P.rms_norm(x, w["final_norm"], spec.final_norm.eps), w["head"])

        a, b = _tokens(90, spec.vocab_size, 31), _tokens(20, spec.vocab_size, 32)
        ea, eb = plain(a), plain(b)
        sa, sb = engine.open_slot(), engine.open_slot()
        out = engine.step([StepEntry(sa, a[:70], [0, 69]), StepEntry(sb, b[:5], [4])])  # across a page
        assert scaled_error(out[0], ea[0]) < 1e-4 and scaled_error(out[1], ea[69]) < 1e-4 and scaled_error(out[2], eb[4]) < 1e-4
        for i in range(15):
            out = engine.step([StepEntry(sa, [a[70 + i]], [0]), StepEntry(sb, [b[5 + i]], [0])])
            assert scaled_error(out[0], ea[70 + i]) < 1e-4 and scaled_error(out[1], eb[5 + i]) < 1e-4
        engine.release_slot(sa)
        engine.release_slot(sb)
        engine.cache.check()
    finally:
        unregister_part("mixer", "test_narrow_value")


def test_a_window_layer_with_a_budget_of_its_own_and_other_page_sizes(cuda_device):
    """With the longest step stated, the layer that keeps a window of 24 positions gets pages for its
    window only, and a sequence still decodes far past what those pages hold.  A step longer than stated
    is refused.  Pages of 32 positions run in float32 (the plain-arithmetic attention takes any page
    size); bfloat16, whose tensor-core kernels tile pages of 64, refuses them by name."""
    from models_b200.engine import Engine, StepEntry, StepError, parameter_requests
    from models_b200.weights import random_tensors

    spec = _specs(windows=(None, 24))
    tensors = random_tensors(parameter_requests(spec), 12, std=0.05)
    tokens = _tokens(400, spec.vocab_size, 41)
    expected = _plain_forward(spec, tensors, tokens)
    for dtype, page_size in (("float32", 64), ("bfloat16", 64), ("float32", 32)):
        engine = Engine(spec, tensors, dtype, max_tokens=1024, max_slots=2, max_step_tokens=40, page_size=page_size)
        full, windowed = engine.cache.groups
        per_slot = -(-(24 - 1 + 40) // page_size) + 1
        assert full.num_pages == 1024 // page_size and windowed.num_pages == 2 * per_slot
        slot = engine.open_slot()
        with pytest.raises(StepError, match="max_step_tokens"):
            engine.step([StepEntry(slot, tokens[:41], [40])])
        assert engine.length(slot) == 0
        at = 0
        while at < 400:  # prompts of 40, then single tokens: 400 positions through a window group of a few pages
            n = 40 if at < 200 else 1
            out = engine.step([StepEntry(slot, tokens[at:at + n], [n - 1])])
            assert scaled_error(out[0], expected[at + n - 1]) < TOLERANCE[dtype], (dtype, page_size, at)
            at += n
        assert sum(p >= 0 for p in windowed.tables[slot]) <= per_slot
        engine.release_slot(slot)
        engine.cache.check()
    with pytest.raises(ValueError, match="pages of 64"):
        Engine(spec, tensors, "bfloat16", max_tokens=1024, page_size=32)


@pytest.mark.parametrize("shape", ["heads of 16, a window, a wide feed-forward", "heads of 128", "heads of 64, four to a kv head"])
def test_the_fused_decode_step_against_the_part_by_part_path_and_plain(cuda_device, shape):
    """Steps of one token for each of 1 to 8 sequences can run as one kernel where the model's parts allow it
    (it is off unless asked for).  The same engine runs the same steps part by part: both must agree with the
    plain functions and with each other within rounding.  The first model has a windowed layer (two cache
    groups, each with page tables of its own), a feed-forward wider than a block can stage at once (the
    down product then runs as column ranges one after the other) and sizes that fill no tile; the others
    have the head sizes whose attention warps are laid out differently."""
    from models_b200.engine import StepEntry

    spec = {
        "heads of 16, a window, a wide feed-forward":
            _specs(hidden=72, heads=6, kv_heads=2, head_dim=16, inter=4200, vocab=203, windows=(None, 24, None)),
        "heads of 128": _specs(hidden=264, heads=2, kv_heads=1, head_dim=128, inter=520, vocab=331, windows=(None, None)),
        "heads of 64, four to a kv head": _specs(hidden=136, heads=8, kv_heads=2, head_dim=64, inter=264, vocab=203, windows=(None, 70)),
    }[shape]
    engine, tensors = _engine(spec, "bfloat16", seed=21, max_tokens=2048)
    fused = engine.model.fused_decode
    assert fused is not None and fused.why_not is None and not fused.enabled
    lengths = [90, 1, 64, 30, 127, 5, 70, 12]
    sequences = [_tokens(n + 10, spec.vocab_size, 300 + i) for i, n in enumerate(lengths)]
    expected = [_plain_forward(spec, tensors, s) for s in sequences]
    for batch in (1, 3, 8):
        results = {}
        for mode in ("one kernel", "part by part"):
            fused.enabled = mode == "one kernel"
            slots = [engine.open_slot() for _ in range(batch)]
            engine.step([StepEntry(slots[b], sequences[b][:lengths[b]], []) for b in range(batch)])
            rows = []
            for i in range(10):
                out = engine.step([StepEntry(slots[b], [sequences[b][lengths[b] + i]], [0]) for b in range(batch)])
                for b in range(batch):
                    err = scaled_error(out[b], expected[b][lengths[b] + i])
                    assert err < TOLERANCE["bfloat16"], (mode, batch, i, b, err)
                rows.append(out)
            results[mode] = torch.stack(rows)
            for slot in slots:
                engine.release_slot(slot)
        assert scaled_error(results["one kernel"], results["part by part"]) < 1e-2, batch
    assert fused.phases is not None and fused.status() == 0
    layers = len(spec.layers)
    down_ranges = 2 if shape.startswith("heads of 16") else 1
    assert fused.num_phases == 1 + layers * (4 + down_ranges) + 1  # embed; per layer q/k/v, attention, output, gate/up, down; head
    engine.cache.check()


def test_what_the_fused_decode_step_leaves_to_the_parts(cuda_device, tmp_path):
    """Biases, float32 and parts of another kind keep the part-by-part path, and say why."""
    from models_b200.engine.loading import engine_from_folder
    from tiny import TINY_A, TINY_C, make_folder

    biased = engine_from_folder(make_folder(TINY_C, 1, tmp_path), "bfloat16", 256)
    assert "biases" in biased.model.fused_decode.why_not
    exact = engine_from_folder(make_folder(TINY_A, 2, tmp_path), "float32", 256)
    assert exact.model.fused_decode is None
    plain = engine_from_folder(make_folder(TINY_A, 2, tmp_path), "bfloat16", 256)
    assert plain.model.fused_decode.why_not is None
