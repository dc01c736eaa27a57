"""Rotary position encoding: per-position cos/sin of each pair, built once on the host.

freq_i = (float)(1 / theta^(2i/rotary_dim)) with the power in double; angle = (pos * scale) *
freq_i / divisor_i in float; cos and sin of that angle taken in double and rounded to float
(integrallis/models, backend-java/.../ops/RotaryTable.java:70-72,177-186).  "linear" scaling is the
reference's frequencyScale = 1/factor (backend-java/.../llama/LlamaConfig.java:302-311); "llama3"
scaling fills the reference's per-pair divisors: pairs whose wavelength 2*pi/freq is below
original/high are untouched, above original/low are divided by `factor`, and in between
freq' = (1-s)*freq/factor + s*freq with s = (original/wavelength - low)/(high - low).

The rotation itself runs inside the mixer's cache-write kernel, which reads these tables.
"""

from __future__ import annotations

import math

import torch

from .base import Part
from .registry import register_part


def pair_frequencies(rotary_dim: int, theta: float) -> torch.Tensor:
    pairs = rotary_dim // 2
    return torch.tensor([1.0 / math.pow(theta, (2.0 * i) / rotary_dim) for i in range(pairs)],
                        dtype=torch.float64).to(torch.float32)


def pair_divisors(frequencies: torch.Tensor, scaling) -> torch.Tensor | None:
    if scaling is None or scaling.kind == "linear":
        return None
    if scaling.kind != "llama3":
        raise ValueError(f"rope scaling {scaling.kind!r} is not built (known: linear, llama3)")
    low_wavelength = scaling.original_max_position / scaling.low_freq_factor
    high_wavelength = scaling.original_max_position / scaling.high_freq_factor
    divisors = []
    for f in frequencies.to(torch.float64).tolist():
        wavelength = 2.0 * math.pi / f
        if wavelength < high_wavelength:
            divisors.append(1.0)
        elif wavelength > low_wavelength:
            divisors.append(float(scaling.factor))
        else:
            smooth = (scaling.original_max_position / wavelength - scaling.low_freq_factor) / (
                scaling.high_freq_factor - scaling.low_freq_factor)
            divisors.append(f / ((1.0 - smooth) * f / scaling.factor + smooth * f))
    return torch.tensor(divisors, dtype=torch.float64).to(torch.float32)


class RotaryEmbedding(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        if spec.pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing must be 'half' or 'interleaved', got {spec.pairing!r}")
        self.rotary_dim = spec.rotary_dim
        self.interleaved = spec.pairing == "interleaved"
        frequencies = pair_frequencies(spec.rotary_dim, spec.theta)
        divisors = pair_divisors(frequencies, spec.scaling)
        scale = 1.0
        if spec.scaling is not None and spec.scaling.kind == "linear":
            scale = 1.0 / spec.scaling.factor
        positions = torch.arange(max(1, runtime.max_positions), dtype=torch.float32)
        scaled = positions * torch.tensor(scale, dtype=torch.float32)
        angle = scaled[:, None] * frequencies[None, :]
        if divisors is not None:
            angle = angle / divisors[None, :]
        angle = angle.to(torch.float64)
        self.cos = torch.cos(angle).to(torch.float32).contiguous().to(runtime.device)
        self.sin = torch.sin(angle).to(torch.float32).contiguous().to(runtime.device)


register_part("position", "rope", RotaryEmbedding)
