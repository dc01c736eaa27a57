"""The decoder put together from parts, as its ModelSpec says: embedding, the scheduled runs of
blocks, final norm, output head (integrallis/models' layer order:
backend-java/.../llama/LlamaForwardPass.java:1024-1196).  Every piece, the embedding and the head
included, is built from its spec through the registry of parts; this file knows none of them.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Mapping, Optional

import torch

from ..config.specs import ModelSpec
from ..parts import RunContext, Runtime, as_delta, build_part
from ..weights.loader import ParamRequest, check_names_and_shapes


def _collect(requests: List[ParamRequest]) -> Dict[str, ParamRequest]:
    out: Dict[str, ParamRequest] = {}
    for r in requests:
        if r.name in out and tuple(out[r.name].shape) != tuple(r.shape):
            raise ValueError(f"tensor {r.name} is asked for with shapes {out[r.name].shape} and {r.shape}")
        out[r.name] = r
    return out


class DecoderModel:
    """Builds every part on `runtime.device`; `load` hands each part its tensors."""

    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.blocks = [build_part("block", layer, runtime) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.head = build_part("head", spec.head, runtime)
        # when set, called with (run index, a copy of the float32 residual stream after that run), for
        # finding the layer where two computations part (the reference's LayerObserver,
        # backend-java/.../llama/LlamaForwardPass.java:44-47,1179-1181)
        self.observer: Optional[Callable[[int, torch.Tensor], None]] = None
        self.fused_decode = None  # the whole decode step as one kernel, where the model's parts allow it (set by `load`)

    # ------------------------------------------------------------------ weights

    def parameters(self) -> Dict[str, ParamRequest]:
        requests = list(self.embedding.parameters())
        for block in self.blocks:
            requests += block.parameters()
        requests += self.final_norm.parameters()
        requests += self.head.parameters()
        return _collect(requests)

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        requests = self.parameters()
        check_names_and_shapes(requests, {n: tuple(t.shape) for n, t in tensors.items()}, "model tensors")
        self.embedding.load(tensors)
        for block in self.blocks:
            block.load(tensors)
        self.final_norm.load(tensors)
        # tied output: the embedding matrix stands in (backend-java/.../llama/LlamaWeights.java:83-89)
        self.head.load(tensors, tied_to=getattr(self.embedding, "weight", None) if self.spec.head.tied else None)
        if self.runtime.mode == "bfloat16" and self.runtime.device.type == "cuda":
            from .fused_decode import FusedDecode

            self.fused_decode = FusedDecode(self)

    # ------------------------------------------------------------------ cache needs

    def kv_requests(self):
        return [self.blocks[entry.layer].mixer.kv_request() for entry in self.spec.schedule]

    def state_requests(self):
        return [self.blocks[entry.layer].mixer.state_request() for entry in self.spec.schedule]

    # ------------------------------------------------------------------ forward

    def forward(self, batch, runs: List[RunContext]) -> Optional[torch.Tensor]:
        """Runs the tokens of `batch` through every scheduled run and returns float32 logits at
        batch.want_rows ([rows, vocab]), or None when no row is wanted."""
        if self.fused_decode is not None and self.fused_decode.takes(batch):
            logits = self.fused_decode.run(batch, runs)  # one token for each of a few sequences: the step as one kernel
            if logits is not None:
                return logits
        x = self.embedding.forward(batch.tokens)
        pending = None
        schedule = self.spec.schedule
        for index, (run, entry) in enumerate(zip(runs, schedule)):
            block = self.blocks[entry.layer]
            if getattr(block, "takes_next_norm", False):
                # the norm that reads the stream after this run: the next run's first norm, or the final one
                following = self.blocks[schedule[index + 1].layer] if index + 1 < len(schedule) else None
                next_norm = getattr(following, "mixer_norm", None) if following is not None else self.final_norm
                pending = block.forward(x, pending, batch, run, next_norm)
            else:
                pending = block.forward(x, as_delta(pending), batch, run)
            if self.observer is not None:
                delta = as_delta(pending)
                self.observer(run.run, x + delta.float() if delta is not None else x.clone())
        if batch.num_wanted == 0:
            return None
        if getattr(self.head, "takes_prenormed", False):
            every_row = batch.max_q_len == 1 and batch.num_wanted == batch.num_tokens
            return self.head.forward(x, pending, self.final_norm, batch.want_rows, every_row)
        return self.head.forward(x, as_delta(pending), self.final_norm, batch.want_rows)


def parameter_requests(spec: ModelSpec) -> Dict[str, ParamRequest]:
    """The tensors a model of this spec needs, without building anything on a device."""
    model = DecoderModel(spec, Runtime(torch.device("meta"), "float32", max_positions=1))
    return model.parameters()
