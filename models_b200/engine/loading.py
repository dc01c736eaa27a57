"""From a model folder (or a configuration and a seed) to an engine on the GPU.

The order mirrors integrallis/models' load path: read the configuration, pick the architecture
from the registry, look the tensors up by name, size the cache, build the model
(backend-java/.../PureJavaBackend.java:128-273).
"""

from __future__ import annotations

from typing import Optional

from ..config import load_config
from ..weights import load_tensors, random_tensors
from .engine import Engine, require_cuda
from .model import parameter_requests


def engine_from_folder(folder, dtype: str = "bfloat16", max_tokens: int = 4096, max_slots: Optional[int] = None,
                       device="cuda:0", max_sequence: Optional[int] = None) -> Engine:
    require_cuda(device)
    config = load_config(folder)
    spec = config.model_spec()
    tensors = load_tensors(folder, parameter_requests(spec), spec.ignored_tensors, spec.duplicate_tensors)
    engine = Engine(spec, tensors, dtype, max_tokens, max_slots, device, max_sequence)
    engine.config = config
    return engine


def engine_from_config(config, seed: int, dtype: str = "bfloat16", max_tokens: int = 4096,
                       max_slots: Optional[int] = None, device="cuda:0", std: float = 0.02,
                       gain_std: float = 0.1, max_sequence: Optional[int] = None) -> Engine:
    """Random weights drawn on the device: the values `write_random_model` writes for the same seed,
    bit for bit, without the detour through a file."""
    import torch

    device = require_cuda(device)
    spec = config.model_spec()
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = random_tensors(parameter_requests(spec), seed, std, gain_std, store, device)
    engine = Engine(spec, tensors, dtype, max_tokens, max_slots, device, max_sequence)
    engine.config = config
    return engine
