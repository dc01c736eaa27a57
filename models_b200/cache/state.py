"""Per-sequence state of fixed size, beside the keys and values.

A mixer that carries a recurrent state instead of (or besides) per-position keys and values asks
for a tensor of a fixed shape per sequence; it gets one row per slot, zeroed when the slot is
opened.  The Llama decoder asks for none; integrallis/models' only per-sequence state is
Session.nextPosition (backend-java/.../llama/LlamaForwardPass.java:50-68), which lives in the
cache's lengths here.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Sequence, Tuple


@dataclass(frozen=True)
class StateRequest:
    shape: Tuple[int, ...]
    dtype: object  # a torch dtype


class StateArea:
    """tensors[run] has shape [max_slots + 1, *request.shape]; row max_slots is the padding row."""

    def __init__(self, requests: Sequence[Optional[StateRequest]], max_slots: int,
                 allocate: Callable[[Tuple[int, ...], object], object]):
        self.max_slots = max_slots
        self.tensors: Dict[int, object] = {}
        for run, request in enumerate(requests):
            if request is not None:
                self.tensors[run] = allocate((max_slots + 1,) + tuple(request.shape), request.dtype)

    def of_run(self, run: int):
        return self.tensors.get(run)

    def reset(self, slot: int) -> None:
        if not 0 <= slot < self.max_slots:
            raise IndexError(f"slot {slot} is outside the state area of {self.max_slots} slots")
        for tensor in self.tensors.values():
            tensor[slot].zero_()

    @property
    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())
