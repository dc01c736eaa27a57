"""Architecture-neutral descriptions of a decoder: what each part is and which sizes it has.

An architecture's typed configuration (for instance `LlamaConfig`) is translated once into a
`ModelSpec`.  Everything below the configuration layer -- parts, cache, step function -- reads
only these records, so no part knows which model it is in.  Every size and constant is a field;
nothing here has a default that stands for a particular model.

The per-layer questions integrallis/models answers with predicates on its config
(`usesRope(layer)`, `usesSlidingWindow(layer)`, `ropeTheta(layer)`;
backend-java/.../llama/LlamaConfig.java:129-173) become per-layer records here: each
`BlockSpec` carries its own mixer, feed-forward and norms, so one model may mix kinds.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


@dataclass(frozen=True)
class RopeScalingSpec:
    """How pair frequencies are stretched.  kind: "linear" (angle * 1/factor) or "llama3"."""

    kind: str
    factor: float
    low_freq_factor: float = 0.0
    high_freq_factor: float = 0.0
    original_max_position: int = 0


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the first `rotary_dim` coordinates of a head.

    pairing "half": pair i is (x[i], x[i + rotary_dim/2]); "interleaved": (x[2i], x[2i+1]).
    Mirrors RotaryTable(rotaryDim, theta, frequencyScale, frequencyFactors) plus its neox flag
    (backend-java/.../ops/RotaryTable.java:48-75,91-100).
    """

    rotary_dim: int
    theta: float
    pairing: str
    scaling: Optional[RopeScalingSpec] = None
    kind: str = "rope"


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a cache.  `window` None: all earlier keys; n: the n
    positions that end at the query.  `scale` multiplies each dot product."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: Optional[RopeSpec]
    window: Optional[int]
    bias: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "attention"


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    """down(act(gate(x)) * up(x)), dense."""

    hidden_size: int
    intermediate_size: int
    activation: str
    bias: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "gated"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which mixer, which feed-forward, which norms, and how they are arranged.

    kind "prenorm": x += mixer(norm(x)); x += feed_forward(norm(x))
    (backend-java/.../llama/LlamaForwardPass.java:1028-1182).
    """

    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object
    kind: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  The order in which layers run is a list of these: a layer may be
    named twice (its weights are shared, each run has a cache of its own) and a run may read the
    cache that an earlier run wrote (`cache_from` is that run's index in the schedule) instead of
    writing one."""

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "embedding"


@dataclass(frozen=True)
class HeadSpec:
    """Output projection to the vocabulary.  `tied`: it uses the embedding table and owns no
    tensor (backend-java/.../llama/LlamaWeights.java:83-89).  The logits are multiplied by
    `logit_scale`, then with `softcap` c != 0 become c * tanh(logits / c)
    (backend-java/.../llama/LlamaForwardPass.java:1751-1764)."""

    vocab_size: int
    hidden_size: int
    tied: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    logit_scale: float = 1.0
    softcap: float = 0.0
    kind: str = "linear_head"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    head: HeadSpec
    stop_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # Tensors a checkpoint of this architecture may hold that the model does not read: name patterns
    # (fnmatch) of buffers that are recomputed, and names that must repeat another tensor exactly (a
    # tied model's stored output matrix).  Anything else that is not asked for is an error.
    ignored_tensors: Tuple[str, ...] = ()
    duplicate_tensors: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)

    def __post_init__(self):
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{index}] names layer {entry.layer}, the model has {len(self.layers)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < index:
                    raise ValueError(
                        f"schedule[{index}] reads the cache of run {entry.cache_from}, which is not an earlier run")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(
                        f"schedule[{index}] reads the cache of run {entry.cache_from}, which owns none")
