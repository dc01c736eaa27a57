"""What every part is given and what it must offer.

A part is built from its spec (sizes and constants) and a `Runtime` (device and precision).  It
names the checkpoint tensors it needs, receives them once, and is then called with activations.
No part sees the model's configuration or knows which model it is in.

Interfaces (duck-typed; the base classes below only document them):

  Norm          forward(x, delta, rows=None, write_x=True) -> normalised rows in the compute dtype.
                x is the float32 residual stream [T, width]; delta (or None) is added to it first.
  Position      tables(max_positions) are prepared at build; apply is fused into the mixer's
                cache-write kernel, so a position part exposes `rotary_dim`, `interleaved`,
                `cos`, `sin`.
  Mixer         kv_request() -> KvRequest | None; state_request() -> StateRequest | None;
                forward(xn, batch, run) -> delta [T, width] in the compute dtype.
  FeedForward   forward(xn) -> delta [T, width] in the compute dtype.
  Block         forward(x, pending, batch, run) -> new pending delta; adds `pending` into x first.
                A block that sets `takes_next_norm` is also given `next_norm` (the norm that will read the
                stream after it) and may then return a `Prenormed` in place of a delta.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional

import torch

from ..weights.loader import ParamRequest

MODES = ("bfloat16", "float32")


@dataclass
class Runtime:
    """Where and in which precision a model runs.

    mode "bfloat16": matrices and activations between kernels in bfloat16, accumulation, residual
    stream, norms, softmax, rotation and logits in float32 -- what serving uses.
    mode "float32": everything in true 32-bit; matrix products on the CUDA cores with float FMAs.
    """

    device: torch.device
    mode: str
    max_positions: int = 0
    shared: Dict[object, object] = field(default_factory=dict)  # parts shared between layers, by spec

    def __post_init__(self):
        if self.mode not in MODES:
            raise ValueError(f"dtype must be one of {MODES}, got {self.mode!r}")
        self.device = torch.device(self.device)

    @property
    def compute_dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.mode == "bfloat16" else torch.float32

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix as the matrix products of this mode read it: widened to float32 in the 32-bit
        mode; otherwise as stored (bfloat16 stays bfloat16, a matrix stored in 32-bit stays so
        and is multiplied in 32-bit)."""
        t = t.to(self.device)
        if self.mode == "float32":
            return t.float().contiguous()
        return t.contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """Norm gains and biases are read as float32 in both modes."""
        return t.to(self.device).float().contiguous()


@dataclass
class RunContext:
    """What one run of the schedule hands to its block: where its keys and values live, whether
    this run writes them, and its slice of the per-sequence state area."""

    run: int
    group: Optional[int] = None
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    writes_cache: bool = True
    state: Optional[torch.Tensor] = None


@dataclass
class Prenormed:
    """What a block may hand on in place of a delta that is still to be added: the residual stream is up to
    date, and the rows of the NEXT norm are half done -- `rows` holds x times that norm's gain (bfloat16) and
    `ssq` the parts of every row's sum of squares ([parts, 128] float32, `count` of them valid).  A product
    that takes them divides by the root mean square in its own epilogue, so the norm needs no kernel."""

    rows: torch.Tensor
    ssq: torch.Tensor
    count: int
    width: int
    eps: float
    norm: object  # the norm part whose gain and eps went into `rows`: only that norm's consumer may use them

    def norm_parts(self):
        return self.ssq, self.count, self.width, self.eps


def as_delta(pending):
    """The delta that is still to be added into the residual stream, or None (also for a Prenormed: the
    stream it belongs to is up to date)."""
    return None if isinstance(pending, Prenormed) else pending


class Part:
    def __init__(self, spec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime

    def parameters(self) -> List[ParamRequest]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pass


class Mixer(Part):
    def kv_request(self):
        return None

    def state_request(self):
        return None

    def forward(self, xn: torch.Tensor, batch, run: RunContext) -> torch.Tensor:
        raise NotImplementedError
