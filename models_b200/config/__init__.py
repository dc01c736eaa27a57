from .llama import ConfigError, LlamaConfig, RopeScalingConfig
from .registry import (
    config_from_dict,
    known_architectures,
    load_config,
    register_architecture,
    unregister_architecture,
)
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
