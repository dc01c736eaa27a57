"""The decoder put together from parts, as its ModelSpec says: embedding, the scheduled runs of
blocks, final norm, output projection (integrallis/models' layer order:
backend-java/.../llama/LlamaForwardPass.java:1024-1196).
"""

from __future__ import annotations

from typing import Callable, Dict, List, Mapping, Optional

import torch

from ..config.specs import ModelSpec
from ..kernels import ops
from ..parts import RunContext, Runtime, build_part
from ..parts.linear import linear
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
        self.embedding = None
        self.head_weight = None
        self.observer: Optional[Callable[[int, torch.Tensor], None]] = None

    # ------------------------------------------------------------------ weights

    def parameters(self) -> Dict[str, ParamRequest]:
        s = self.spec
        requests = [ParamRequest(s.embedding.weights["weight"], (s.embedding.vocab_size, s.embedding.hidden_size))]
        for block in self.blocks:
            requests += block.parameters()
        requests += self.final_norm.parameters()
        if not s.head.tied:
            requests.append(ParamRequest(s.head.weights["weight"], (s.head.vocab_size, s.head.hidden_size)))
        return _collect(requests)

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        requests = self.parameters()
        check_names_and_shapes(requests, {n: tuple(t.shape) for n, t in tensors.items()}, "model tensors")
        rt, s = self.runtime, self.spec
        self.embedding = rt.matrix(tensors[s.embedding.weights["weight"]])
        for block in self.blocks:
            block.load(tensors)
        self.final_norm.load(tensors)
        # tied output: the embedding matrix stands in (backend-java/.../llama/LlamaWeights.java:83-89)
        self.head_weight = self.embedding if s.head.tied else rt.matrix(tensors[s.head.weights["weight"]])

    # ------------------------------------------------------------------ cache needs

    def kv_requests(self):
        return [self.blocks[entry.layer].mixer.kv_request() for entry in self.spec.schedule]

    def state_requests(self):
        return [self.blocks[entry.layer].mixer.state_request() for entry in self.spec.schedule]

    # ------------------------------------------------------------------ forward

    def forward(self, batch, runs: List[RunContext]) -> Optional[torch.Tensor]:
        """Runs the tokens of `batch` through every scheduled run and returns float32 logits at
        batch.want_rows ([rows, vocab]), or None when no row is wanted."""
        x = ops.embed_gather(self.embedding, batch.tokens, self.spec.embedding.scale)
        pending = None
        for run, entry in zip(runs, self.spec.schedule):
            pending = self.blocks[entry.layer].forward(x, pending, batch, run)
            if self.observer is not None:
                self.observer(run.run, x + pending.float() if pending is not None else x.clone())
        if batch.num_wanted == 0:
            return None
        if (pending is None and self.runtime.mode == "bfloat16" and getattr(self.final_norm, "foldable", False)
                and ops.skinny_pays(self.head_weight, batch.num_wanted, with_norm=True)):
            # few wanted rows: gather, final norm and output product in one kernel
            return ops.skinny_gemm(self.head_weight, ops.EPI_F32, xf=x, gain=self.final_norm.weight,
                                   eps=self.final_norm.spec.eps, rows=batch.want_rows)
        xn = self.final_norm.forward(x, pending, rows=batch.want_rows)
        return linear(xn, self.head_weight, torch.float32)


def parameter_requests(spec: ModelSpec) -> Dict[str, ParamRequest]:
    """The tensors a model of this spec needs, without building anything on a device."""
    model = DecoderModel(spec, Runtime(torch.device("meta"), "float32", max_positions=1))
    return model.parameters()
