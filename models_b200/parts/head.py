"""The output head: final norm, projection to the vocabulary, and what is done to the logits.

xn = norm(x); logits = Wout . xn, with Wout the embedding table when the head is tied
(integrallis/models, backend-java/.../llama/LlamaForwardPass.java:1184-1196;
backend-java/.../llama/LlamaWeights.java:83-89), for the wanted rows only (Head.LOGITS, :984-991).
Then logits *= logit_scale, and with a softcap c != 0: logits = c * tanh(logits / c) (:1751-1764).
Llama has scale 1 and no softcap; both are fields of the spec, not of this class.

A head part is built with (spec, runtime) and offers parameters(), load(tensors, tied_to) where
`tied_to` is the embedding part's `weight` when spec.tied, and
forward(x, pending, norm, want_rows) -> float32 logits [wanted, vocab].
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part, Prenormed, as_delta
from .linear import linear
from .registry import register_part


class LinearHead(Part):
    takes_prenormed = True  # `forward` may be given a Prenormed as `pending`, and is told when every row is wanted

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.softcap < 0.0:
            raise ValueError(f"logit softcap must be >= 0 (0: none), got {spec.softcap}")

    def parameters(self):
        s = self.spec
        return [] if s.tied else [ParamRequest(s.weights["weight"], (s.vocab_size, s.hidden_size))]

    def load(self, tensors, tied_to: Optional[torch.Tensor] = None):
        if self.spec.tied:
            if tied_to is None:
                raise ValueError("a tied output head needs the embedding table")
            self.weight = tied_to  # one allocation
        else:
            self.weight = self.runtime.matrix(tensors[self.spec.weights["weight"]])

    def forward(self, x: torch.Tensor, pending, norm, want_rows: torch.Tensor, every_row: bool = False) -> torch.Tensor:
        """x: the float32 residual stream, `pending` a delta not yet added into it (or None, or a Prenormed
        for `norm`); `norm` the final norm part; `want_rows` int32 rows of x whose logits are wanted
        (`every_row`: all of them, in order)."""
        rows = want_rows.numel()
        s = self.spec
        if (every_row and isinstance(pending, Prenormed) and pending.norm is norm and self.runtime.mode == "bfloat16"
                and (ops.skinny_pays(self.weight, rows, with_norm=True)
                     or (ops.SKINNY_PAYS_ROWS < rows <= ops.WIDE_ROWS and ops.gemm_tcgen05_takes(self.weight, ops.EPI_F32, rows)))):
            # the last layer prepared the final norm's rows: the output product divides by the root mean square itself
            if rows <= ops.SKINNY_PAYS_ROWS:
                logits = ops.skinny_gemm(self.weight, ops.EPI_F32, x=pending.rows, norm_parts=pending.norm_parts())
            else:
                logits = ops.wide_gemm(pending.rows, self.weight, ops.EPI_F32, norm_parts=pending.norm_parts())
            if s.logit_scale != 1.0 or s.softcap != 0.0:
                ops.logit_epilogue(logits, s.logit_scale, s.softcap)
            return logits
        pending = as_delta(pending)
        if (pending is None and self.runtime.mode == "bfloat16" and getattr(norm, "foldable", False)
                and ops.skinny_pays(self.weight, rows, with_norm=True)):
            # few wanted rows: gather, final norm and output product in one kernel
            logits = ops.skinny_gemm(self.weight, ops.EPI_F32, xf=x, gain=norm.weight, eps=norm.spec.eps, rows=want_rows)
        else:
            logits = linear(norm.forward(x, pending, rows=want_rows), self.weight, torch.float32)
        if s.logit_scale != 1.0 or s.softcap != 0.0:
            ops.logit_epilogue(logits, s.logit_scale, s.softcap)
        return logits


register_part("head", "linear_head", LinearHead)
