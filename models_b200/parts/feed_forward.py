"""Dense gated feed-forward: down(act(gate(xn)) * up(xn)) (integrallis/models,
backend-java/.../llama/LlamaForwardPass.java:1150-1178).  The activation is the spec's: "silu"
(z / (1 + exp(-z)), backend-java/.../ops/TensorOps.java:1407-1425; Llama's) or "gelu_tanh"
(:1427-1449); it is an argument of every kernel that applies it, fused or not.  gate and up are one product over row-concatenated
weights, as the reference pairs them (dualMatmulDispatch,
backend-java/.../llama/LlamaForwardPass.java:1153-1164).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part, Prenormed
from .linear import linear
from .registry import register_part


class GatedFeedForward(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"gated feed-forward activation {spec.activation!r} is not built "
                             f"(known: {', '.join(sorted(ops.ACTIVATIONS))})")
        self.gated = ops.gated_epilogue(spec.activation)  # the epilogue code of a gate/up product with this activation

    def parameters(self):
        s, n = self.spec, self.spec.weights
        out = [
            ParamRequest(n["gate"], (s.intermediate_size, s.hidden_size)),
            ParamRequest(n["up"], (s.intermediate_size, s.hidden_size)),
            ParamRequest(n["down"], (s.hidden_size, s.intermediate_size)),
        ]
        if s.bias:
            out += [
                ParamRequest(n["gate_bias"], (s.intermediate_size,), "bias"),
                ParamRequest(n["up_bias"], (s.intermediate_size,), "bias"),
                ParamRequest(n["down_bias"], (s.hidden_size,), "bias"),
            ]
        return out

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        gate, up = rt.matrix(tensors[n["gate"]]), rt.matrix(tensors[n["up"]])
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = rt.matrix(tensors[n["down"]])
        self.b_gate_up = self.b_down = None
        if self.spec.bias:
            self.b_gate_up = torch.cat([rt.vector(tensors[n["gate_bias"]]), rt.vector(tensors[n["up_bias"]])]).contiguous()
            self.b_down = rt.vector(tensors[n["down_bias"]])

    def folds(self, rows: int, norm) -> bool:
        """Whether `forward_residual` applies: bfloat16 weights, few rows, no biases, a foldable norm."""
        return (self.b_gate_up is None and self.b_down is None and getattr(norm, "foldable", False)
                and ops.skinny_pays(self.w_gate_up, rows, with_norm=True) and ops.skinny_pays(self.w_down, rows))

    def forward_residual(self, x: torch.Tensor, norm) -> None:
        """x += down(act(gate(norm(x))) * up(norm(x))) in two kernels: norm, gate/up product and
        activation in one, the down product and the residual add in the other."""
        hidden = ops.skinny_gemm(self.w_gate_up, self.gated, xf=x, gain=norm.weight, eps=norm.spec.eps)
        ops.skinny_gemm(self.w_down, ops.EPI_RESIDUAL, x=hidden, out=x)

    def adds(self, xn: torch.Tensor) -> bool:
        """Whether `forward_into` applies (any number of rows): bfloat16, no biases, and a down matrix that
        the tcgen05 product takes."""
        return (self.b_gate_up is None and self.b_down is None and xn.dtype == torch.bfloat16
                and ops.gemm_tcgen05_takes(self.w_down))

    def forward_into(self, x: torch.Tensor, xn: torch.Tensor) -> None:
        """x += down(act(gate(xn)) * up(xn)) with the activation inside the gate/up product and the residual
        add inside the down product: neither the gate/up matrix nor the down result passes through memory.
        Up to 128 rows both are the wide decode product (weights as the 128-row operand, K split over a
        cluster where the matrix has few tiles), above that the prefill product."""
        rows = xn.shape[0]
        if ops.gemm_tcgen05_takes(self.w_gate_up, ops.EPI_SWIGLU, rows):
            hidden = ops.tensor_core_gemm(xn, self.w_gate_up, self.gated)  # the wide decode form up to 128 rows, the prefill form above
        elif ops.skinny_pays(self.w_gate_up, rows):
            hidden = ops.skinny_gemm(self.w_gate_up, self.gated, x=xn)
        else:
            hidden = ops.swiglu(linear(xn, self.w_gate_up, self.runtime.compute_dtype), self.spec.activation)
        if rows < ops.TCGEN05_MIN_ROWS:
            ops.gemm_tcgen05(hidden, self.w_down, ops.EPI_RESIDUAL, out=x)
        else:
            ops.tensor_core_gemm(hidden, self.w_down, ops.EPI_RESIDUAL, out=x)

    def chains(self, rows: int) -> bool:
        """Whether `forward_chain` applies: up to 128 rows (the narrow decode products up to 8, the wide ones above),
        no biases."""
        if self.b_gate_up is not None or self.b_down is not None or rows > ops.WIDE_ROWS:
            return False
        if rows <= ops.SKINNY_PAYS_ROWS:
            return ops.skinny_pays(self.w_gate_up, rows, with_norm=True) and ops.skinny_pays(self.w_down, rows)
        return (ops.gemm_tcgen05_takes(self.w_gate_up, ops.EPI_SWIGLU, rows)
                and ops.gemm_tcgen05_takes(self.w_down, ops.EPI_RESIDUAL, rows))

    def forward_chain(self, x: torch.Tensor, scaled, next_norm):
        """x += down(act(gate(norm(x))) * up(norm(x))) for 9 to 128 rows in two kernels: `scaled` is the normalised
        rows, or a Prenormed whose division by the root mean square the gate/up product does itself; the down
        product adds into x and, given a `next_norm` whose gain it can apply, prepares that norm's rows (the
        return value; else None)."""
        rows, parts = (scaled.rows, scaled.norm_parts()) if isinstance(scaled, Prenormed) else (scaled, None)
        if x.shape[0] <= ops.SKINNY_PAYS_ROWS:
            product = lambda a, w, epilogue, **more: ops.skinny_gemm(w, epilogue, x=a, **more)  # noqa: E731
        else:
            product = ops.wide_gemm
        hidden = product(rows, self.w_gate_up, self.gated, norm_parts=parts)
        if next_norm is None or not getattr(next_norm, "foldable", False):
            product(hidden, self.w_down, ops.EPI_RESIDUAL, out=x)
            return None
        _, gained, ssq, count = product(hidden, self.w_down, ops.EPI_RESIDUAL, out=x, emit_gain=next_norm.weight)
        return Prenormed(gained, ssq, count, x.shape[1], next_norm.spec.eps, next_norm)

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        dtype = self.runtime.compute_dtype
        if self.b_gate_up is None and ops.skinny_pays(self.w_gate_up, xn.shape[0]) and xn.dtype == torch.bfloat16:
            hidden = ops.skinny_gemm(self.w_gate_up, self.gated, x=xn)
            delta = linear(hidden, self.w_down, dtype)
            if self.b_down is not None:
                ops.bias_add(delta, self.b_down)
            return delta
        if (self.b_gate_up is None and xn.dtype == torch.bfloat16
                and ops.gemm_tcgen05_takes(self.w_gate_up, ops.EPI_SWIGLU, xn.shape[0])):
            hidden = ops.tensor_core_gemm(xn, self.w_gate_up, self.gated)
        else:
            gate_up = linear(xn, self.w_gate_up, dtype)
            if self.b_gate_up is not None:
                ops.bias_add(gate_up, self.b_gate_up)
            hidden = ops.swiglu(gate_up, self.spec.activation)
        delta = linear(hidden, self.w_down, dtype)
        if self.b_down is not None:
            ops.bias_add(delta, self.b_down)
        return delta


register_part("feed_forward", "gated", GatedFeedForward)
