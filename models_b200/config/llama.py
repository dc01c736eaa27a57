"""Typed configuration of the Llama decoder, read from the keys of its own config.json.

Counterpart of integrallis/models' `LlamaConfig` record
(backend-java/.../llama/LlamaConfig.java:21-95,239-311), which reads the same quantities from GGUF
metadata: positive sizes, `heads % kv_heads == 0`, head size defaulting to hidden/heads, rope base
defaulting to 10000, norm epsilon defaulting to 1e-5, a missing required key named in the error.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .specs import (
    AttentionSpec,
    BlockSpec,
    EmbeddingSpec,
    GatedFeedForwardSpec,
    HeadSpec,
    ModelSpec,
    NormSpec,
    RopeScalingSpec,
    RopeSpec,
    ScheduleEntry,
)


class ConfigError(ValueError):
    """A config.json that cannot describe a model this library builds."""


_MISSING = object()


def _require(raw: Mapping[str, Any], key: str):
    value = raw.get(key, _MISSING)
    if value is _MISSING or value is None:
        raise ConfigError(f"config.json: missing required key {key!r}")
    return value


def _positive_int(raw: Mapping[str, Any], key: str, default=_MISSING) -> int:
    value = raw.get(key)
    if value is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing required key {key!r}")
        value = default
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer, got {value!r}")
    return value


def _positive_float(value, key: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or value <= 0:
        raise ConfigError(f"config.json: {key} must be finite and > 0, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class RopeScalingConfig:
    rope_type: str
    factor: float
    low_freq_factor: float = 0.0
    high_freq_factor: float = 0.0
    original_max_position_embeddings: int = 0


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rope_scaling: Optional[RopeScalingConfig]
    rms_norm_eps: float
    tie_word_embeddings: bool
    hidden_act: str
    attention_bias: bool
    mlp_bias: bool
    sliding_window: Optional[int]
    bos_token_id: Optional[int]
    eos_token_ids: Tuple[int, ...]

    # derived sizes, named as the reference names them (LlamaConfig.java:73-95)
    @property
    def query_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def key_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def value_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def attention_output_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "LlamaConfig":
        architectures = raw.get("architectures") or ["LlamaForCausalLM"]
        hidden = _positive_int(raw, "hidden_size")
        layers = _positive_int(raw, "num_hidden_layers")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = _positive_int(raw, "num_key_value_heads", default=heads)
        if heads % kv_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({heads}) must be a multiple of num_key_value_heads ({kv_heads})")
        if raw.get("head_dim") is None and hidden % heads != 0:
            raise ConfigError(
                f"config.json: head_dim is absent and hidden_size ({hidden}) is no multiple of "
                f"num_attention_heads ({heads})")
        head_dim = _positive_int(raw, "head_dim", default=hidden // heads)
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim must be even for rotary pairs, got {head_dim}")
        intermediate = _positive_int(raw, "intermediate_size")
        vocab = _positive_int(raw, "vocab_size")
        max_positions = _positive_int(raw, "max_position_embeddings", default=2048)

        rope_parameters = raw.get("rope_parameters") or {}
        theta = raw.get("rope_theta")
        if theta is None:
            theta = rope_parameters.get("rope_theta", 10000.0)
        theta = _positive_float(theta, "rope_theta")
        scaling_raw = raw.get("rope_scaling")
        if scaling_raw is None and rope_parameters.get("rope_type", "default") != "default":
            scaling_raw = rope_parameters
        scaling = _parse_rope_scaling(scaling_raw)

        eps = _positive_float(raw.get("rms_norm_eps", 1e-5), "rms_norm_eps")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not built; the Llama feed-forward uses 'silu'")
        window = raw.get("sliding_window")
        if window is not None:
            window = _positive_int(raw, "sliding_window")

        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: eos_token_id must be an integer or a list of integers, got {eos!r}")
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: eos_token_id {e} is outside the vocabulary of {vocab}")
        bos = raw.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            raise ConfigError(f"config.json: bos_token_id must be an integer, got {bos!r}")

        return LlamaConfig(
            architecture=str(architectures[0]),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=intermediate,
            vocab_size=vocab,
            max_position_embeddings=max_positions,
            rope_theta=theta,
            rope_scaling=scaling,
            rms_norm_eps=eps,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            hidden_act=act,
            attention_bias=bool(raw.get("attention_bias", False)),
            mlp_bias=bool(raw.get("mlp_bias", False)),
            sliding_window=window,
            bos_token_id=bos,
            eos_token_ids=eos_ids,
        )

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        out = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "torch_dtype": "bfloat16",
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            out["rope_scaling"] = {"rope_type": s.rope_type, "factor": s.factor}
            if s.rope_type == "llama3":
                out["rope_scaling"].update(
                    low_freq_factor=s.low_freq_factor,
                    high_freq_factor=s.high_freq_factor,
                    original_max_position_embeddings=s.original_max_position_embeddings,
                )
        if self.sliding_window is not None:
            out["sliding_window"] = self.sliding_window
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return out

    # ------------------------------------------------------------------ translation to parts

    def model_spec(self) -> ModelSpec:
        """The parts this configuration asks for, layer by layer, with checkpoint tensor names."""
        scaling = None
        if self.rope_scaling is not None:
            s = self.rope_scaling
            scaling = RopeScalingSpec(
                kind=s.rope_type,
                factor=s.factor,
                low_freq_factor=s.low_freq_factor,
                high_freq_factor=s.high_freq_factor,
                original_max_position=s.original_max_position_embeddings,
            )
        # Rows of q_proj/k_proj in a safetensors folder are not permuted, so pairs are split-half:
        # the reference's "NeoX" routine (backend-java/.../ops/TensorOps.java:1384-1404).
        rope = RopeSpec(rotary_dim=self.head_dim, theta=self.rope_theta, pairing="half", scaling=scaling)
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            attn_names = {
                "q": p + "self_attn.q_proj.weight",
                "k": p + "self_attn.k_proj.weight",
                "v": p + "self_attn.v_proj.weight",
                "o": p + "self_attn.o_proj.weight",
            }
            if self.attention_bias:
                attn_names.update(
                    q_bias=p + "self_attn.q_proj.bias",
                    k_bias=p + "self_attn.k_proj.bias",
                    v_bias=p + "self_attn.v_proj.bias",
                    o_bias=p + "self_attn.o_proj.bias",
                )
            ffn_names = {
                "gate": p + "mlp.gate_proj.weight",
                "up": p + "mlp.up_proj.weight",
                "down": p + "mlp.down_proj.weight",
            }
            if self.mlp_bias:
                ffn_names.update(
                    gate_bias=p + "mlp.gate_proj.bias",
                    up_bias=p + "mlp.up_proj.bias",
                    down_bias=p + "mlp.down_proj.bias",
                )
            layers.append(
                BlockSpec(
                    mixer=AttentionSpec(
                        hidden_size=self.hidden_size,
                        num_heads=self.num_attention_heads,
                        num_kv_heads=self.num_key_value_heads,
                        head_dim=self.head_dim,
                        # (float)(1/sqrt(hd)) (backend-java/.../llama/LlamaForwardPass.java:1559)
                        scale=1.0 / math.sqrt(self.head_dim),
                        position=rope,
                        window=self.sliding_window,
                        bias=self.attention_bias,
                        weights=attn_names,
                    ),
                    feed_forward=GatedFeedForwardSpec(
                        hidden_size=self.hidden_size,
                        intermediate_size=self.intermediate_size,
                        activation=self.hidden_act,
                        bias=self.mlp_bias,
                        weights=ffn_names,
                    ),
                    mixer_norm=NormSpec(self.hidden_size, self.rms_norm_eps, {"weight": p + "input_layernorm.weight"}),
                    feed_forward_norm=NormSpec(
                        self.hidden_size, self.rms_norm_eps, {"weight": p + "post_attention_layernorm.weight"}),
                )
            )
        head_names = {} if self.tie_word_embeddings else {"weight": "lm_head.weight"}
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=EmbeddingSpec(self.vocab_size, self.hidden_size, 1.0, {"weight": "model.embed_tokens.weight"}),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=NormSpec(self.hidden_size, self.rms_norm_eps, {"weight": "model.norm.weight"}),
            head=HeadSpec(self.vocab_size, self.hidden_size, self.tie_word_embeddings, head_names),
            stop_token_ids=self.eos_token_ids,
            bos_token_id=self.bos_token_id,
            # older exports store the rotation frequencies as a buffer; they are recomputed from the configuration
            ignored_tensors=("*.rotary_emb.inv_freq",),
            # a tied model whose file also stores the output matrix: fine if it repeats the embedding table, an
            # error if the two disagree (backend-java/.../llama/LlamaWeights.java:83-89 ties by absence)
            duplicate_tensors={"lm_head.weight": "model.embed_tokens.weight"} if self.tie_word_embeddings else {},
        )


def _parse_rope_scaling(raw) -> Optional[RopeScalingConfig]:
    if raw is None:
        return None
    if not isinstance(raw, Mapping):
        raise ConfigError(f"config.json: rope_scaling must be an object or null, got {raw!r}")
    kind = raw.get("rope_type", raw.get("type"))
    if kind in (None, "default"):
        return None
    if kind == "linear":
        return RopeScalingConfig("linear", _positive_float(_require(raw, "factor"), "rope_scaling.factor"))
    if kind == "llama3":
        factor = _positive_float(_require(raw, "factor"), "rope_scaling.factor")
        low = _positive_float(_require(raw, "low_freq_factor"), "rope_scaling.low_freq_factor")
        high = _positive_float(_require(raw, "high_freq_factor"), "rope_scaling.high_freq_factor")
        original = _require(raw, "original_max_position_embeddings")
        if isinstance(original, bool) or not isinstance(original, int) or original <= 0:
            raise ConfigError(
                f"config.json: rope_scaling.original_max_position_embeddings must be a positive integer, got {original!r}")
        if high <= low:
            raise ConfigError(
                f"config.json: rope_scaling.high_freq_factor ({high}) must exceed low_freq_factor ({low})")
        return RopeScalingConfig("llama3", factor, low, high, original)
    raise ConfigError(f"config.json: rope scaling type {kind!r} is not built (known: default, linear, llama3)")
