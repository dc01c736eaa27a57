"""Token embedding: x = E[token, :] * scale, as the float32 residual stream (integrallis/models,
backend-java/.../llama/LlamaForwardPass.java:1024-1025,1742-1749; the scale is 1 for Llama).

An embedding part offers `weight` (the [vocab, width] table as the matrix products read it), so
that an output head tied to it can use the same allocation.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part
from .registry import register_part


class TokenEmbedding(Part):
    def parameters(self):
        s = self.spec
        return [ParamRequest(s.weights["weight"], (s.vocab_size, s.hidden_size))]

    def load(self, tensors):
        self.weight = self.runtime.matrix(tensors[self.spec.weights["weight"]])

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens int32 [T] -> float32 [T, width]."""
        return ops.embed_gather(self.weight, tokens, self.spec.scale)


register_part("embedding", "embedding", TokenEmbedding)
