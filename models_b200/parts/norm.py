"""RMSNorm fused with the residual add that precedes it.

sumSq = sum x_i^2; rms = sqrt(sumSq/size + eps); out_i = x_i * (1/rms) * w_i
(integrallis/models, backend-java/.../ops/TensorOps.java:45-58), all in float32.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part
from .registry import register_part


class RmsNorm(Part):
    # a consumer may fold this norm into its own kernel: it reads `weight` and `spec.eps`
    foldable = True

    def parameters(self):
        return [ParamRequest(self.spec.weights["weight"], (self.spec.size,), "gain")]

    def load(self, tensors):
        self.weight = self.runtime.vector(tensors[self.spec.weights["weight"]])

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                write_x: bool = True) -> torch.Tensor:
        return ops.add_rmsnorm(x, delta, self.weight, self.spec.eps, self.runtime.compute_dtype, rows, write_x)


register_part("norm", "rmsnorm", RmsNorm)
