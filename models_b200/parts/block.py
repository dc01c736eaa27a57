"""Arrangement of a layer's parts.  "prenorm": x += mixer(norm(x)); x += feed_forward(norm(x))
(integrallis/models, backend-java/.../llama/LlamaForwardPass.java:1028-1182).

The residual stream x stays in float32.  A block does not add its last result into x itself: it
returns it as the pending delta, and whoever normalises next (the following block, or the final
norm) adds it in the same kernel that normalises.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Part, Prenormed, RunContext, as_delta
from .registry import build_part, register_part


class PreNormBlock(Part):
    takes_next_norm = True  # `forward` is told which norm reads the stream next, and may hand it a Prenormed

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.feed_forward_norm = build_part("norm", spec.feed_forward_norm, runtime)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime)
        self.parts = [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def parameters(self):
        return [p for part in self.parts for p in part.parameters()]

    def load(self, tensors):
        for part in self.parts:
            part.load(tensors)

    def forward(self, x: torch.Tensor, pending, batch, run: RunContext, next_norm=None):
        rows = x.shape[0]
        mixer_chains = getattr(self.mixer, "chains", None)
        ffn_chains = getattr(self.feed_forward, "chains", None)
        # (a single row gains nothing from prepared rows: normalising one row inside a product costs less than the parts)
        if (rows >= 2 and self.runtime.mode == "bfloat16" and mixer_chains and ffn_chains and ffn_chains(rows)
                and mixer_chains(rows, run, self.feed_forward_norm) and getattr(self.mixer_norm, "foldable", False)):
            # up to 128 rows (decode): five kernels a layer, the norms riding in the products around them
            if isinstance(pending, Prenormed) and pending.norm is self.mixer_norm:
                scaled = pending
            elif rows <= ops.SKINNY_PAYS_ROWS:
                if as_delta(pending) is not None:
                    ops.residual_add(x, as_delta(pending))
                scaled = None  # few rows: the q/k/v product normalises x itself
            else:
                scaled = self.mixer_norm.forward(x, as_delta(pending))
            half_way = self.mixer.forward_chain(x, scaled, batch, run, self.feed_forward_norm, norm=self.mixer_norm)
            return self.feed_forward.forward_chain(x, half_way, next_norm)
        pending = as_delta(pending)  # (a Prenormed means: nothing left to add)
        mixer_folds = getattr(self.mixer, "folds", None)
        ffn_folds = getattr(self.feed_forward, "folds", None)
        if (self.runtime.mode == "bfloat16" and mixer_folds and ffn_folds and mixer_folds(rows, self.mixer_norm)
                and ffn_folds(rows, self.feed_forward_norm)):
            # few rows (decode): norms ride in the products that follow them and residual adds in the
            # products that precede them, so nothing stays pending
            if pending is not None:
                ops.residual_add(x, pending)
            self.mixer.forward_residual(x, self.mixer_norm, batch, run)
            self.feed_forward.forward_residual(x, self.feed_forward_norm)
            return None
        xn = self.mixer_norm.forward(x, pending)
        mixer_adds = getattr(self.mixer, "adds", None)
        if mixer_adds and mixer_adds(xn):
            self.mixer.forward_into(x, xn, batch, run)  # the residual add rides in the mixer's last product
            mixed = None
        else:
            mixed = self.mixer.forward(xn, batch, run)
        xn = self.feed_forward_norm.forward(x, mixed)
        ffn_adds = getattr(self.feed_forward, "adds", None)
        if ffn_adds and ffn_adds(xn):
            self.feed_forward.forward_into(x, xn)
            return None
        return self.feed_forward.forward(xn)


register_part("block", "prenorm", PreNormBlock)
