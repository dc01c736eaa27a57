"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a
seed.

integrallis/models builds such models only in its tests (a seeded nano model,
models-test/.../NanoGgufModel.java:42-49,91); here it is a product feature so that benchmarks
and tests need no checkpoint.  Each tensor's values depend on (seed, tensor name) only, not on the
order in which tensors are drawn.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from .loader import ParamRequest
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensors(requests: Mapping[str, ParamRequest], seed: int, std: float = 0.02, gain_std: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """Matrices and biases N(0, std); norm gains 1 + N(0, gain_std).  Drawn in float32, then
    rounded to `dtype`."""
    out = {}
    device = torch.device(device)
    for name, request in requests.items():
        generator = torch.Generator(device=device)
        generator.manual_seed(_tensor_seed(seed, name))
        values = torch.randn(tuple(request.shape), generator=generator, dtype=torch.float32, device=device)
        if request.kind == "gain":
            values = 1.0 + values * gain_std
        else:
            values = values * std
        out[name] = values.to(dtype)
    return out


def write_random_model(folder, config, seed: int, std: float = 0.02, gain_std: float = 0.1,
                       dtype: torch.dtype = torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors for `config` (a typed configuration of a registered
    architecture) and returns the folder."""
    from ..engine.model import parameter_requests

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    requests = parameter_requests(config.model_spec())
    tensors = random_tensors(requests, seed, std, gain_std, dtype)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return folder
