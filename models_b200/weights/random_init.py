"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a
seed.

integrallis/models builds such models only in its tests (a seeded nano model,
models-test/.../NanoGgufModel.java:42-49,91); here it is a product feature so that benchmarks
and tests need no checkpoint.  Each tensor's values depend on (seed, tensor name) only, not on the
order in which tensors are drawn nor on where (host or GPU) they are drawn.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from .loader import ParamRequest
from .philox_normal import normal_float32, tensor_key
from .safetensors_io import write_safetensors


def random_tensors(requests: Mapping[str, ParamRequest], seed: int, std: float = 0.02, gain_std: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """Matrices and biases N(0, std); norm gains 1 + N(0, gain_std).  Drawn in float32, then rounded
    to `dtype`.  Values come from a counter-based generator keyed by (seed, tensor name)
    (weights/philox_normal.py): on a CUDA device a kernel draws them in place, on the host numpy does,
    and both give the same bits."""
    out = {}
    device = torch.device(device)
    for name, request in requests.items():
        key = tensor_key(seed, name)
        mean, scale = (1.0, gain_std) if request.kind == "gain" else (0.0, std)
        shape = tuple(request.shape)
        count = 1
        for n in shape:
            count *= n
        if device.type == "cuda":
            from ..kernels import ops

            out[name] = ops.random_normal(torch.empty(shape, dtype=dtype, device=device), key, mean, scale)
        else:
            values = torch.from_numpy(normal_float32(count, key, mean, scale)).reshape(shape)
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
